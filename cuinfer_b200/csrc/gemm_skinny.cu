// out[M, N] = act[M, K] · W[N, K]^T for a handful of rows (M <= 16): the decode-step projections, bfloat16.
//
// The reference sends these to cuBLAS one by one, with a norm kernel before and an activation kernel after
// (csrc/model/layers/attention.cpp:44-105, csrc/model/layers/mlp.cpp:21-27, csrc/ops/projection.cu:32-44).
// With few rows the product is a single pass over the weights, so this kernel is built around that stream:
//
//   * the weight matrix is the A operand of mma.sync m16n8k16 (16 output features x 16 k), the rows of the
//     batch are the B operand (k x 8 rows): "swap A/B".  Every lane reads its A fragments straight from global
//     memory as 16-byte loads (8 consecutive k of one weight row), which fixes a permutation of k inside each
//     32-k step; the activations are read from shared memory with the same permutation (one 16-byte load per
//     lane), so no shuffle or ldmatrix is needed and every weight byte is read exactly once;
//   * a CTA has 8 warps: RT tiles of 16 output features x KS slices of K (RT * KS = 8); slices are summed in
//     shared memory in a fixed order, so results do not depend on timing;
//   * optional prologue: the activations are RMSNorm(residual + pending) computed on the fly by every CTA
//     (CTA 0 also stores the new residual to a second buffer), which removes the norm kernel;
//   * optional epilogue: rows come in (gate, up) pairs and silu(gate) * up is stored, which removes the
//     activation kernel; or the result is stored in 32 bits (the output head);
//   * the first weight loads are issued before `griddepcontrol.wait`, so that with programmatic dependent
//     launch a projection starts streaming its weights while the kernel before it is still running.
#include "mma_utils.cuh"

#include <cooperative_groups.h>

namespace cib {

constexpr int kSkWarps = 8;
constexpr int kSkU = 4;           // 32-k steps whose weight loads are in flight together

enum SkinnyEpilogue : int { kStoreBf16 = 0, kStoreF32 = 1, kSiluPair = 2 };

struct SkinnyArgs {
    const __nv_bfloat16* w; int ldw; int N; int K;
    const __nv_bfloat16* act; int lda;                       // plain activations, or
    const float* res_in; const void* pending; int pending_bf16; AnyVec norm_w; float eps; float* res_out;
    void* out; int ldo; int M;
    int up_offset;                                           // kSiluPair: first row of the "up" half
    int act_stride;                                          // shared-memory row stride in elements
    const void* warm; unsigned long long warm_bytes;         // the weights of the kernel after this one (or null): fetched into L2
    int norm_w_offset;                                       // byte offset of the norm gains' copy in shared memory
    int inbox_offset;                                        // CS > 1: byte offset of the first CTA's slots for the others' sums
};

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// CS > 1: a cluster of CS CTAs shares one group of row tiles, each CTA taking 1/CS of K; the partial sums meet
// in the shared memory of the cluster's first CTA (distributed shared memory), which stores the result.
template <int MT, int RT, int KS, int EPI, int CS>
__global__ void __launch_bounds__(kSkWarps * 32)
skinny_gemm_kernel(const SkinnyArgs a) {
    namespace cg = cooperative_groups;
    const int crank = CS > 1 ? (int)(blockIdx.x % CS) : 0;
    const int tile_block = CS > 1 ? (int)(blockIdx.x / CS) : (int)blockIdx.x;
    static_assert(RT * KS == kSkWarps, "a CTA has 8 warps");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* s_act = reinterpret_cast<__nv_bfloat16*>(smem_raw);                  // [MT*8][act_stride]
    float* s_red = reinterpret_cast<float*>(smem_raw + (size_t)MT * 8 * a.act_stride * 2); // [KS][RT][16][MT*8]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = lane & 3, qrow = lane >> 2;
    const int rt = warp % RT, ks = warp / RT;
    // "this CTA runs": its shared memory may be written by the others of the cluster once all have said so
    if (CS > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

    // rows of this warp's tile
    int tile_row0;
    if (EPI == kSiluPair) tile_row0 = (rt == 0 ? 0 : a.up_offset) + tile_block * 16;
    else tile_row0 = (tile_block * RT + rt) * 16;
    const int row_limit = (EPI == kSiluPair) ? (rt == 0 ? a.up_offset : a.N) : a.N;
    const int r0 = tile_row0 + qrow, r1 = r0 + 8;
    const bool ok0 = r0 < row_limit, ok1 = r1 < row_limit;
    const __nv_bfloat16* w0 = a.w + (size_t)(ok0 ? r0 : 0) * a.ldw;
    const __nv_bfloat16* w1 = a.w + (size_t)(ok1 ? r1 : 0) * a.ldw;

    // k range of this warp's slice, in 32-k steps
    const int steps_total = (a.K + 31) / 32;
    const int steps_per = (steps_total + KS * CS - 1) / (KS * CS);
    const int step_begin = (crank * KS + ks) * steps_per;
    const int step_end = min(steps_total, step_begin + steps_per);

    // two register buffers of kSkU steps each, named apart so that every index is a compile-time constant
    uint4 waA[kSkU], wbA[kSkU], waB[kSkU], wbB[kSkU];
    auto load_chunk = [&](uint4 (&wa)[kSkU], uint4 (&wb)[kSkU], int step0) {
#pragma unroll
        for (int u = 0; u < kSkU; ++u) {
            const int k = (step0 + u) * 32 + quad * 8;
            const bool in = step0 + u < step_end && k < a.K;
            wa[u] = (in && ok0) ? ldg_stream16(w0 + k) : make_uint4(0, 0, 0, 0);
            wb[u] = (in && ok1) ? ldg_stream16(w1 + k) : make_uint4(0, 0, 0, 0);
        }
    };
    load_chunk(waA, wbA, step_begin);   // weights do not depend on the kernel before this one
    if (tid == 0) warm_l2_share(a.warm, a.warm_bytes, blockIdx.x, gridDim.x);
    // neither do the norm's gains: they wait in shared memory (read from global memory in the second pass of the norm,
    // eight dependent round trips per row, they were a third of this kernel's time)
    float* s_nw = reinterpret_cast<float*>(smem_raw + a.norm_w_offset);
    if (a.res_in != nullptr)
        for (int k = tid; k < a.K; k += kSkWarps * 32) s_nw[k] = a.norm_w[k];
    griddep_launch();
    griddep_wait();                     // from here on the previous kernel's results may be read
    if (a.res_in != nullptr) __syncthreads();      // the gains' copy is complete

    // ---- activations -> shared memory (bfloat16 rows, padded), optionally normalised on the way ----
    const int rows_pad = MT * 8;
    if (a.res_in != nullptr) {
        float* s_x = reinterpret_cast<float*>(s_red);               // un-normalised 32-bit rows [rows][K]
        for (int row = warp; row < rows_pad; row += kSkWarps) {
            float ss = 0.f;
            if (row < a.M) {
                const float* rp = a.res_in + (size_t)row * a.K;
                // eight independent 16-byte loads of the residual (and of the delta) are in flight per lane
                for (int k0 = lane * 4; k0 < a.K; k0 += 128 * 8) {
                    float4 x[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int k = k0 + u * 128;
                        x[u] = k < a.K ? *reinterpret_cast<const float4*>(rp + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    if (a.pending) {
                        if (a.pending_bf16) {
                            uint2 pv[8];
                            const __nv_bfloat16* pp = reinterpret_cast<const __nv_bfloat16*>(a.pending) + (size_t)row * a.K;
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                const int k = k0 + u * 128;
                                pv[u] = k < a.K ? *reinterpret_cast<const uint2*>(pp + k) : make_uint2(0u, 0u);
                            }
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                const __nv_bfloat162 p01 = *reinterpret_cast<const __nv_bfloat162*>(&pv[u].x);
                                const __nv_bfloat162 p23 = *reinterpret_cast<const __nv_bfloat162*>(&pv[u].y);
                                x[u].x += __low2float(p01); x[u].y += __high2float(p01);
                                x[u].z += __low2float(p23); x[u].w += __high2float(p23);
                            }
                        } else {
                            const float* pp = reinterpret_cast<const float*>(a.pending) + (size_t)row * a.K;
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                const int k = k0 + u * 128;
                                if (k < a.K) {
                                    const float4 pv = *reinterpret_cast<const float4*>(pp + k);
                                    x[u].x += pv.x; x[u].y += pv.y; x[u].z += pv.z; x[u].w += pv.w;
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int k = k0 + u * 128;
                        if (k < a.K) {
                            ss += x[u].x * x[u].x + x[u].y * x[u].y + x[u].z * x[u].z + x[u].w * x[u].w;
                            if (tile_block == 0 && a.res_out) *reinterpret_cast<float4*>(a.res_out + (size_t)row * a.K + k) = x[u];
                            *reinterpret_cast<float4*>(s_x + (size_t)row * a.K + k) = x[u];
                        }
                    }
                }
                ss = warp_sum(ss);
            }
            const float factor = row < a.M ? rsqrtf(ss / (float)a.K + a.eps) : 0.f;
            __syncwarp();
            for (int k = lane * 4; k < a.K; k += 128) {
                float4 x = row < a.M ? *reinterpret_cast<const float4*>(s_x + (size_t)row * a.K + k)
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 gw = *reinterpret_cast<const float4*>(s_nw + k);
                const float n0 = x.x * factor * gw.x, n1 = x.y * factor * gw.y;
                const float n2 = x.z * factor * gw.z, n3 = x.w * factor * gw.w;
                uint2 pk;
                pk.x = pack_bf16(n0, n1);
                pk.y = pack_bf16(n2, n3);
                *reinterpret_cast<uint2*>(s_act + (size_t)row * a.act_stride + k) = pk;
            }
        }
    } else {
        // only the k range this CTA multiplies
        const int c_begin = CS > 1 ? min(a.K / 8, crank * KS * steps_per * 4) : 0;
        const int c_end = CS > 1 ? min(a.K / 8, (crank + 1) * KS * steps_per * 4) : a.K / 8;
        const int chunks = c_end - c_begin;
        // four loads in flight per thread: one after the other they cost a round trip to the L2 each
        const int total = rows_pad * chunks;
        for (int base = tid; base < total; base += kSkWarps * 32 * 4) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = base + u * kSkWarps * 32;
                v[u] = make_uint4(0, 0, 0, 0);
                if (idx < total) {
                    const int row = idx / chunks, c = c_begin + idx % chunks;
                    if (row < a.M) v[u] = *reinterpret_cast<const uint4*>(a.act + (size_t)row * a.lda + c * 8);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = base + u * kSkWarps * 32;
                if (idx < total) {
                    const int row = idx / chunks, c = c_begin + idx % chunks;
                    *reinterpret_cast<uint4*>(s_act + (size_t)row * a.act_stride + c * 8) = v[u];
                }
            }
        }
    }
    __syncthreads();

    // ---- main loop over this warp's k slice ----
    // two accumulators per row tile, one for each half of a 32-k step: a warp's MMAs then form two chains of half the
    // length instead of one (the k slices are short, so the chain's latency is most of the loop; four chains measured
    // no better); summed at the end
    float acc[MT][4], acc2[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = acc2[i][e] = 0.f;
    }
    auto compute_chunk = [&](const uint4 (&wa)[kSkU], const uint4 (&wb)[kSkU], int step0) {
#pragma unroll
        for (int u = 0; u < kSkU; ++u) {
            if (step0 + u < step_end) {
                const int k = (step0 + u) * 32 + quad * 8;
                const uint32_t a1[4] = {wa[u].x, wb[u].x, wa[u].y, wb[u].y};
                const uint32_t a2[4] = {wa[u].z, wb[u].z, wa[u].w, wb[u].w};
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) {
                    uint4 bv = make_uint4(0, 0, 0, 0);
                    if (k < a.K) bv = *reinterpret_cast<const uint4*>(s_act + (size_t)(nt * 8 + qrow) * a.act_stride + k);
                    mma_bf16_16816(acc[nt], a1, bv.x, bv.y);
                    mma_bf16_16816(acc2[nt], a2, bv.z, bv.w);
                }
            }
        }
    };
    for (int step0 = step_begin; step0 < step_end; step0 += 2 * kSkU) {
        load_chunk(waB, wbB, step0 + kSkU);
        compute_chunk(waA, wbA, step0);
        load_chunk(waA, wbA, step0 + 2 * kSkU);
        compute_chunk(waB, wbB, step0 + kSkU);
    }
#pragma unroll
    for (int i = 0; i < MT; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] += acc2[i][e];
    }

    // ---- sum the k slices (fixed order), then the epilogue ----
    __syncthreads();                       // the activations (and the norm's scratch) are no longer needed
    constexpr int kCols = MT * 8;
    float* red = reinterpret_cast<float*>(smem_raw);                                    // [KS][RT][16][kCols]
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
        float* base = red + (((size_t)ks * RT + rt) * 16) * kCols + nt * 8 + quad * 2;
        base[(size_t)qrow * kCols] = acc[nt][0];
        base[(size_t)qrow * kCols + 1] = acc[nt][1];
        base[(size_t)(qrow + 8) * kCols] = acc[nt][2];
        base[(size_t)(qrow + 8) * kCols + 1] = acc[nt][3];
    }
    __syncthreads();
    if (CS > 1) {
        // every CTA sums its own slices; the others then write their sums into slots of the first CTA's shared memory
        // that nothing else uses (so they need not wait for the first CTA to finish its loop), say so with a release
        // and leave; the first CTA waits for them and sums in rank order
        cg::cluster_group cluster = cg::this_cluster();
        float* mine = red + (size_t)(KS + CS) * RT * 16 * kCols;          // [RT][16][kCols] sum of this CTA
        float* inbox = reinterpret_cast<float*>(smem_raw + a.inbox_offset);   // [CS - 1][RT][16][kCols], used in the first CTA
        for (int idx = tid; idx < RT * 16 * kCols; idx += kSkWarps * 32) {
            float sum = 0.f;
#pragma unroll
            for (int s = 0; s < KS; ++s) sum += red[(size_t)s * RT * 16 * kCols + idx];
            mine[idx] = sum;
        }
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");       // every CTA of the cluster runs
        if (crank != 0) {
            float* dst = cluster.map_shared_rank(inbox + (size_t)(crank - 1) * RT * 16 * kCols, 0);
            for (int idx = tid; idx < RT * 16 * kCols; idx += kSkWarps * 32) dst[idx] = mine[idx];     // each thread copies what it summed
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            return;
        }
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        __syncthreads();
        for (int idx = tid; idx < RT * 16 * kCols; idx += kSkWarps * 32) {
            const int token = idx / (RT * 16), nl = idx % (RT * 16);
            if (token >= a.M) continue;
            const int t = nl / 16, r = nl % 16;
            const size_t e = ((size_t)t * 16 + r) * kCols + token;
            float sum = mine[e];
#pragma unroll
            for (int c = 1; c < CS; ++c) sum += inbox[(size_t)(c - 1) * RT * 16 * kCols + e];
            const int n = tile_block * RT * 16 + nl;
            if (n < a.N) {
                if (EPI == kStoreF32) reinterpret_cast<float*>(a.out)[(size_t)token * a.ldo + n] = sum;
                else reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)token * a.ldo + n] = __float2bfloat16_rn(sum);
            }
        }
        return;
    }
    if (EPI == kSiluPair) {
        for (int idx = tid; idx < 16 * kCols; idx += kSkWarps * 32) {
            const int token = idx / 16, nl = idx % 16;
            if (token >= a.M) continue;
            float gsum = 0.f, usum = 0.f;
#pragma unroll
            for (int s = 0; s < KS; ++s) {
                gsum += red[(((size_t)s * RT + 0) * 16 + nl) * kCols + token];
                usum += red[(((size_t)s * RT + 1) * 16 + nl) * kCols + token];
            }
            const int n = tile_block * 16 + nl;
            if (n < a.up_offset)
                reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)token * a.ldo + n] =
                    __float2bfloat16_rn(gsum / (1.f + expf(-gsum)) * usum);
        }
    } else {
        for (int idx = tid; idx < RT * 16 * kCols; idx += kSkWarps * 32) {
            const int token = idx / (RT * 16), nl = idx % (RT * 16);
            if (token >= a.M) continue;
            const int t = nl / 16, r = nl % 16;
            float sum = 0.f;
#pragma unroll
            for (int s = 0; s < KS; ++s) sum += red[(((size_t)s * RT + t) * 16 + r) * kCols + token];
            const int n = tile_block * RT * 16 + nl;
            if (n < a.N) {
                if (EPI == kStoreF32) reinterpret_cast<float*>(a.out)[(size_t)token * a.ldo + n] = sum;
                else reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)token * a.ldo + n] = __float2bfloat16_rn(sum);
            }
        }
    }
}

static int act_stride_for(int K) {
    // row stride (elements) such that consecutive rows start 16 banks apart: 16-byte reads of two rows never collide
    const int words = K / 2;
    const int pad_words = ((16 - words % 32) % 32 + 32) % 32;
    return K + pad_words * 2;
}

template <int MT, int RT, int KS, int EPI, int CS = 1>
static int launch_skinny(SkinnyArgs& a, int grid, int use_pdl, cudaStream_t stream) {
    a.act_stride = act_stride_for(a.K);
    size_t act_bytes = (size_t)MT * 8 * a.act_stride * 2;
    size_t norm_bytes = a.res_in ? (size_t)MT * 8 * a.K * 4 : 0;         // un-normalised 32-bit rows during the prologue
    size_t red_bytes = (size_t)(KS + CS + 1) * RT * 16 * MT * 8 * 4;
    size_t smem = act_bytes + (norm_bytes > red_bytes ? norm_bytes : red_bytes);
    if (smem < red_bytes) smem = red_bytes;
    smem = (smem + 15) & ~size_t(15);
    a.norm_w_offset = (int)smem;
    if (a.res_in) smem += (size_t)a.K * 4;
    smem = (smem + 15) & ~size_t(15);
    a.inbox_offset = (int)smem;
    if (CS > 1) smem += (size_t)(CS - 1) * RT * 16 * MT * 8 * 4;
    CIB_REQUIRE(smem <= 200 * 1024, "gemm_skinny: %d rows x K=%d need %zu bytes of shared memory", a.M, a.K, smem);
    auto kernel = skinny_gemm_kernel<MT, RT, KS, EPI, CS>;
    static SmemLimit limit;
    if (int rc = raise_smem_limit(limit, kernel, 200 * 1024, "gemm_skinny")) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid * CS);
    cfg.blockDim = dim3(kSkWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (CS > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = CS;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    if (use_pdl) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, a);
    if (e != cudaSuccess) {
        set_error("gemm_skinny: launch failed: %s", cudaGetErrorString(e));
        return -2;
    }
    return 0;
}

template <int MT>
static int dispatch_skinny(SkinnyArgs& a, int epilogue, int use_pdl, cudaStream_t stream) {
    if (epilogue == kSiluPair) {
        const int grid = (a.up_offset + 15) / 16;
        return launch_skinny<MT, 2, 4, kSiluPair>(a, grid, use_pdl, stream);
    }
    // As few 16-row tiles per CTA as keep the launch within one round of CTAs (two fit on each of the 148 SMs);
    // the warps that are not needed for rows split K instead.
    const int tiles = (a.N + 15) / 16;
    if (a.res_in == nullptr && tiles <= 148 && a.K >= 2048) {
        // few output features and a long K: four CTAs of a cluster share each tile so that most SMs stream
        // (a cluster launch costs about a microsecond more, so K below 2048 stays with one CTA per tile; with more
        // tiles than SMs the split measured slower).  At K = 2048 and 64 tiles the split turned a 6.6 us launch, whose
        // warps fetched their second chunk of weights after the wait, into one whose weights are all asked for before it.
        if (epilogue == kStoreF32) return launch_skinny<MT, 1, 8, kStoreF32, 4>(a, tiles, use_pdl, stream);
        return launch_skinny<MT, 1, 8, kStoreBf16, 4>(a, tiles, use_pdl, stream);
    }
    int rt = 1;
    while (rt < 8 && (tiles + rt - 1) / rt > 296) rt *= 2;
    const int grid = (tiles + rt - 1) / rt;
#define CIB_SKINNY_CASE(RTV, KSV)                                                                         \
    if (rt == RTV) {                                                                                      \
        if (epilogue == kStoreF32) return launch_skinny<MT, RTV, KSV, kStoreF32>(a, grid, use_pdl, stream); \
        return launch_skinny<MT, RTV, KSV, kStoreBf16>(a, grid, use_pdl, stream);                          \
    }
    CIB_SKINNY_CASE(1, 8)
    CIB_SKINNY_CASE(2, 4)
    CIB_SKINNY_CASE(4, 2)
    CIB_SKINNY_CASE(8, 1)
#undef CIB_SKINNY_CASE
    return -1;
}

}  // namespace cib

using namespace cib;

// with_norm: the activations are normalised in the kernel (needs room for the 32-bit rows as well).
extern "C" int cib_gemm_skinny_supports(int M, int N, int K, int with_norm) {
    if (!(M >= 1 && M <= 16 && N >= 1 && K >= 32 && K % 8 == 0)) return 0;
    const size_t rows = M <= 8 ? 8 : 16;
    const size_t bytes = rows * (K + 64) * 2 + (with_norm ? rows * K * 4 + (size_t)K * 4 + 16 : (size_t)kSkWarps * 16 * rows * 4);
    return bytes <= 200 * 1024 && (!with_norm || K % 4 == 0);
}

// act: [M, K] bfloat16 rows (lda), or null when res_in is given: then the activations are
// RMSNorm(res_in + pending) * norm_w computed in the kernel, and res_out (if not null) receives res_in + pending.
// epilogue: 0 = bfloat16 out[M, N]; 1 = float32 out[M, N]; 2 = rows [0, up_offset) are gates and rows
// [up_offset, N) the matching ups: out[M, up_offset] = silu(gate) * up in bfloat16.
// warm / warm_bytes: memory that the kernel after this one reads first (its weights), or null: fetched into the L2 meanwhile.
extern "C" int cib_gemm_skinny(const void* w, int ldw, int N, int K, const void* act, int lda, const float* res_in,
                               const void* pending, int pending_dtype, const void* norm_w, int norm_w_dtype, float eps,
                               float* res_out, void* out, int ldo, int M, int epilogue, int up_offset, int use_pdl,
                               const void* warm, long long warm_bytes, cudaStream_t stream) {
    CIB_REQUIRE(cib_gemm_skinny_supports(M, N, K, res_in != nullptr), "gemm_skinny: M=%d N=%d K=%d is not taken by this kernel (M <= 16, K a multiple of 8)", M, N, K);
    CIB_REQUIRE(ldw >= K && ldw % 8 == 0 && ((uintptr_t)w % 16) == 0, "gemm_skinny: weight rows must be 16-byte aligned");
    CIB_REQUIRE((act != nullptr) != (res_in != nullptr), "gemm_skinny: give plain activations or a residual to normalise");
    CIB_REQUIRE(act == nullptr || (lda >= K && lda % 8 == 0 && ((uintptr_t)act % 16) == 0), "gemm_skinny: activation rows must be 16-byte aligned");
    CIB_REQUIRE(res_in == nullptr || (norm_w != nullptr && K % 4 == 0 && res_out != res_in), "gemm_skinny: the norm needs its weight and a second residual buffer");
    CIB_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_skinny: unknown epilogue %d", epilogue);
    CIB_REQUIRE(epilogue != kSiluPair || (up_offset > 0 && 2 * up_offset == N && ldo >= up_offset), "gemm_skinny: a gate/up pair needs N = 2 * up_offset");
    CIB_REQUIRE(epilogue == kSiluPair || ldo >= N, "gemm_skinny: ldo too small");
    SkinnyArgs a;
    a.w = (const __nv_bfloat16*)w; a.ldw = ldw; a.N = N; a.K = K;
    a.act = (const __nv_bfloat16*)act; a.lda = lda;
    a.res_in = res_in; a.pending = pending; a.pending_bf16 = pending_dtype == kBF16;
    a.norm_w = AnyVec{norm_w, norm_w_dtype == kBF16}; a.eps = eps; a.res_out = res_out;
    a.out = out; a.ldo = ldo; a.M = M; a.up_offset = up_offset; a.act_stride = 0;
    a.warm = ((uintptr_t)warm % 16) == 0 && warm_bytes > 0 ? warm : nullptr;
    a.warm_bytes = a.warm ? (unsigned long long)warm_bytes : 0;
    if (M <= 8) return dispatch_skinny<1>(a, epilogue, use_pdl, stream);
    return dispatch_skinny<2>(a, epilogue, use_pdl, stream);
}
