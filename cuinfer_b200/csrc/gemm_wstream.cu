// out[M, N] = act[M, K] · W[N, K]^T in bfloat16 for up to 128 rows: the weight matrix is the streamed operand.
//
// The reference sends every projection to cuBLAS (csrc/ops/projection.cu:32-44).  With few rows a projection is one
// pass over its weights, and what matters is how many bytes an SM keeps in flight.  The few-rows kernel of this
// package (gemm_skinny.cu) reads weights through registers and keeps the activations of all of K in shared memory; at
// hidden sizes of 4096 and more that leaves one CTA per SM with a few KB in flight.  Here the roles of the operands
// are swapped on the 5th-generation tensor cores instead:
//
//   * a CTA owns 128 output features: its weight rows are the 128-row A operand of `tcgen05.mma.kind::f16`, fetched by
//     TMA in 16 KB boxes (128 features x 64 k, 128-byte swizzle) through a ring of 6-8 stages (over 100 KB in flight
//     per SM); the rows of the batch are the B operand (N = 16, 32, 64 or 128, rows beyond M read as zeros); the
//     accumulator, out^T, lives in tensor memory (features = lanes, batch rows = columns);
//   * where 128-feature tiles are fewer than the SMs, K is split over the 2 or 4 CTAs of a cluster; the partial
//     tiles meet in the shared memory of the cluster's first CTA (distributed shared memory, in the ring that the
//     main loop no longer needs) and are added in a fixed order, so results do not depend on timing;
//   * epilogues: bfloat16 or float32 rows, or silu(gate) * up for a weight of gate rows followed by up rows (a tile then
//     holds 64 gate features and the 64 matching up features);
//   * the weight copies of the first stages are issued before `griddepcontrol.wait`: under programmatic dependent
//     launch a projection streams its weights while the kernel before it still runs.
//
// Every mbarrier wait is bounded; on a time-out the kernel raises the error flag, skips its stores, frees its tensor
// memory and returns.
#include "tcgen05_utils.cuh"

#include "mma_utils.cuh"

namespace cib {
namespace ws {

enum Epilogue : int { kBf16 = 0, kF32 = 1, kSilu = 2 };

constexpr int kWBytes = kTcBM * kTcBK * 2;          // a weight box: 128 features x 64 k

template <int BX, int STAGES>
struct Smem {
    static constexpr int kXBytes = BX * kTcBK * 2;
    static constexpr int kStageBytes = kWBytes + kXBytes;
    static constexpr int kRing = STAGES * kStageBytes;
    static constexpr int kTotal = kRing + 1024 /* alignment slack */ + 256 /* barriers */;
};

__device__ __forceinline__ uint32_t cluster_size() {
    uint32_t n;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n));
    return n;
}
__device__ __forceinline__ void st_cluster_f32x4(uint32_t cluster_addr, float4 v) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}

// Grid: (128-feature tiles) x (cluster of S CTAs that split K).  192 threads: warp 0 TMA producer, warp 1 MMA issuer
// and tensor-memory owner, warps 2-5 epilogue (TMEM lanes 32 * (warp % 4) .. + 31 = features of the tile).
template <int BX, int STAGES, int EPI>
__global__ void __launch_bounds__(192)
gemm_wstream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    void* __restrict__ out, int ldo, int M, int N, int K, int up_offset, int* __restrict__ error_flag) {
    using S = Smem<BX, STAGES>;
    constexpr int kTmemCols = BX < 32 ? 32 : BX;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring + S::kRing);
    uint64_t* full = bars;                   // [STAGES] bytes of a stage have landed
    uint64_t* empty = bars + STAGES;         // [STAGES] the MMAs that read a stage are done
    uint64_t* acc_full = bars + 2 * STAGES;  // the accumulator holds this CTA's share
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t splits = cluster_size();
    const uint32_t rank = splits > 1 ? cluster_ctarank() : 0u;
    const int tile = (int)(blockIdx.x / splits);
    constexpr int kTileCols = EPI == kSilu ? 64 : 128;       // output features of a tile
    const int n0 = tile * kTileCols;
    const int steps_total = (K + kTcBK - 1) / kTcBK;
    const int steps_per = (steps_total + (int)splits - 1) / (int)splits;
    const int kb0 = (int)rank * steps_per;
    const int nsteps = max(0, min(steps_total, kb0 + steps_per) - kb0);

    griddep_launch();
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    float acc[BX];
#pragma unroll
    for (int i = 0; i < BX; ++i) acc[i] = 0.f;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer ----
            auto load_w = [&](int i) {
                unsigned char* w_dst = ring + (size_t)(i % STAGES) * S::kStageBytes;
                const int k = (kb0 + i) * kTcBK;
                if (EPI == kSilu) {
                    tma_load_2d(w_dst, &map_w, &full[i % STAGES], k, n0);                            // 64 gate rows
                    tma_load_2d(w_dst + 64 * 128, &map_w, &full[i % STAGES], k, up_offset + n0);     // the 64 matching up rows
                } else {
                    tma_load_2d(w_dst, &map_w, &full[i % STAGES], k, n0);
                }
            };
            auto load_x = [&](int i) {
                tma_load_2d(ring + (size_t)(i % STAGES) * S::kStageBytes + kWBytes, &map_x, &full[i % STAGES], (kb0 + i) * kTcBK, 0);
            };
            // the weights of the first stages do not depend on the kernel before this one
            const int pre = min(STAGES, nsteps);
            for (int i = 0; i < pre; ++i) {
                mbar_expect_tx(&full[i], S::kStageBytes);
                load_w(i);
            }
            griddep_wait();
            for (int i = 0; i < pre; ++i) load_x(i);
            for (int i = pre; i < nsteps; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(&empty[s], (uint32_t)((i / STAGES - 1) & 1))) { atomicExch(error_flag, 31); s_abort = 1; break; }
                if (*(volatile int*)&s_abort) break;
                mbar_expect_tx(&full[s], S::kStageBytes);
                load_w(i);
                load_x(i);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer: D[128 features, BX rows] += W[128, 16 k] · X[BX, 16 k]^T ----
            constexpr uint32_t idesc = umma_idesc_bf16(kTcBM, BX);
            bool ok = true;
            for (int i = 0; i < nsteps; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(&full[s], (uint32_t)((i / STAGES) & 1))) { atomicExch(error_flag, 32); s_abort = 1; ok = false; break; }
                tcgen05_fence_after();
                const unsigned char* w_src = ring + (size_t)s * S::kStageBytes;
                const uint64_t adesc = umma_desc_k_major_sw128(w_src);
                const uint64_t bdesc = umma_desc_k_major_sw128(w_src + kWBytes);
#pragma unroll
                for (int k = 0; k < kTcBK / 16; ++k)
                    umma_bf16(tmem_base, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (i | k) != 0 ? 1u : 0u);
                umma_commit(&empty[s]);
            }
            if (ok && nsteps > 0) umma_commit(acc_full);
            else mbar_arrive(acc_full);            // nothing to wait for: this CTA's share of K is empty (or it gave up)
        }
    } else {
        // ---- epilogue threads: this CTA's share of the tile, one feature per thread ----
        const int quarter = warp & 3;
        bool ok = mbar_wait(acc_full, 0);
        if (!ok && lane == 0) { atomicExch(error_flag, 33); s_abort = 1; }
        tcgen05_fence_after();
        if (nsteps > 0 && ok && !(*(volatile int*)&s_abort)) {
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
            if constexpr (BX == 16) {
                uint32_t v[16];
                tmem_ld_32x32b_x16(taddr, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[i] = __uint_as_float(v[i]);
            } else {
#pragma unroll
                for (int c = 0; c < BX / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + (uint32_t)(c * 32), v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) acc[c * 32 + i] = __uint_as_float(v[i]);
                }
            }
        }
    }

    // ---- the K splits meet in the first CTA's ring (its main loop is over: its epilogue threads waited for its MMAs) ----
    const bool epilogue_thread = warp >= 2;
    const int feature = (warp & 3) * 32 + lane;               // of the tile, for epilogue threads
    float* parts = reinterpret_cast<float*>(ring);            // [splits - 1][128][BX] in the first CTA
    if (splits > 1) {
        tcgen05_fence_before();
        __syncthreads();
        cluster_sync_all();
        if (epilogue_thread && rank != 0) {
            const uint32_t dst = map_to_cta(parts + ((size_t)(rank - 1) * kTcBM + feature) * BX, 0);
#pragma unroll
            for (int i = 0; i < BX; i += 4) st_cluster_f32x4(dst + (uint32_t)(i * 4), make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]));
        }
        cluster_sync_all();
        if (epilogue_thread && rank == 0) {
            for (uint32_t r = 1; r < splits; ++r) {            // fixed order
                const float4* src = reinterpret_cast<const float4*>(parts + ((size_t)(r - 1) * kTcBM + feature) * BX);
#pragma unroll
                for (int i = 0; i < BX / 4; ++i) {
                    const float4 v = src[i];
                    acc[4 * i] += v.x; acc[4 * i + 1] += v.y; acc[4 * i + 2] += v.z; acc[4 * i + 3] += v.w;
                }
            }
        }
    }

    // ---- stores (first CTA of the cluster) ----
    const bool healthy = !(*(volatile int*)&s_abort);
    if (EPI == kSilu) {
        // gates are features 0-63 of the tile, ups 64-127: exchange through shared memory behind the partial tiles
        float* ex = parts + (size_t)(splits - 1) * kTcBM * BX;        // [128][BX]
        if (splits > 1) __syncthreads();                               // every partial has been read
        if (epilogue_thread && rank == 0) {
#pragma unroll
            for (int i = 0; i < BX; ++i) ex[(size_t)feature * BX + i] = acc[i];
        }
        __syncthreads();
        if (epilogue_thread && rank == 0 && healthy && feature < 64 && n0 + feature < up_offset) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + n0 + feature;
            for (int m = 0; m < M && m < BX; ++m) {
                const float g = ex[(size_t)feature * BX + m], u = ex[(size_t)(feature + 64) * BX + m];
                dst[(size_t)m * ldo] = __float2bfloat16_rn(g / (1.f + expf(-g)) * u);
            }
        }
    } else if (epilogue_thread && rank == 0 && healthy && n0 + feature < N) {
        if (EPI == kF32) {
            float* dst = reinterpret_cast<float*>(out) + n0 + feature;
#pragma unroll
            for (int m = 0; m < BX; ++m)
                if (m < M) dst[(size_t)m * ldo] = acc[m];
        } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + n0 + feature;
#pragma unroll
            for (int m = 0; m < BX; ++m)
                if (m < M) dst[(size_t)m * ldo] = __float2bfloat16_rn(acc[m]);
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
}

template <int BX, int STAGES, int EPI>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, void* out, int ldo, int M, int N, int K, int up_offset,
                  int tiles, int splits, int* error_flag, bool use_pdl, cudaStream_t stream) {
    auto kernel = gemm_wstream_kernel<BX, STAGES, EPI>;
    constexpr int smem = Smem<BX, STAGES>::kTotal;
    static_assert(smem <= 227 * 1024, "a CTA has 227 KB of shared memory");
    static SmemLimit limit;
    if (int rc = raise_smem_limit(limit, kernel, smem, "gemm_wstream")) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * splits);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (splits > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = splits;
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
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, mw, mx, out, ldo, M, N, K, up_offset, error_flag);
    if (e != cudaSuccess) {
        set_error("gemm_wstream: launch failed: %s", cudaGetErrorString(e));
        return -2;
    }
    return 0;
}

template <int BX, int STAGES>
static int dispatch(const CUtensorMap& mw, const CUtensorMap& mx, void* out, int ldo, int M, int N, int K, int epilogue,
                    int up_offset, int* error_flag, bool use_pdl, cudaStream_t stream) {
    const int tile_cols = epilogue == kSilu ? 64 : 128;
    const int n_out = epilogue == kSilu ? up_offset : N;
    const int tiles = (n_out + tile_cols - 1) / tile_cols;
    // K is split over the CTAs of a cluster until there is a CTA for every SM, as long as every split keeps a few
    // steps and the partial tiles (and the gate/up exchange tile) fit into the first CTA's ring
    const int steps = (K + kTcBK - 1) / kTcBK;
    constexpr int kMaxSplits = 4;        // clusters of 8 measured three times slower (they wait for 8 free SMs of one GPC)
    int splits = 1;
    while (tiles * splits < 148 && splits < kMaxSplits && steps / (2 * splits) >= 2 &&
           (size_t)(2 * splits) * kTcBM * BX * 4 <= (size_t)Smem<BX, STAGES>::kRing)
        splits *= 2;
    if (epilogue == kSilu) return launch<BX, STAGES, kSilu>(mw, mx, out, ldo, M, N, K, up_offset, tiles, splits, error_flag, use_pdl, stream);
    if (epilogue == kF32) return launch<BX, STAGES, kF32>(mw, mx, out, ldo, M, N, K, up_offset, tiles, splits, error_flag, use_pdl, stream);
    return launch<BX, STAGES, kBf16>(mw, mx, out, ldo, M, N, K, up_offset, tiles, splits, error_flag, use_pdl, stream);
}

}  // namespace ws
}  // namespace cib

using namespace cib;

extern "C" int cib_gemm_wstream_supports(int M, int N, int K) {
    return M >= 1 && M <= 128 && N >= 8 && K >= 8 && K % 8 == 0;
}

// act: [M, K] bfloat16 rows (lda), w: [N, K] bfloat16 rows (ldw).  epilogue: 0 = bfloat16 out[M, N]; 1 = float32
// out[M, N]; 2 = rows [0, N / 2) of w are gates and rows [N / 2, N) the matching ups: out[M, N / 2] = silu(gate) * up in
// bfloat16.  error_flag: one zero int in device memory.
extern "C" int cib_gemm_wstream(const void* act, int lda, const void* w, int ldw, void* out, int ldo, int epilogue, int M,
                                int N, int K, int use_pdl, int* error_flag, cudaStream_t stream) {
    CIB_REQUIRE(cib_gemm_wstream_supports(M, N, K), "gemm_wstream: M=%d N=%d K=%d is not taken (at most 128 rows, K a multiple of 8)", M, N, K);
    CIB_REQUIRE(lda >= K && ldw >= K && lda % 8 == 0 && ldw % 8 == 0 && ((uintptr_t)act % 16) == 0 && ((uintptr_t)w % 16) == 0,
                "gemm_wstream: rows must be 16-byte aligned");
    CIB_REQUIRE(epilogue >= 0 && epilogue <= 2 && error_flag != nullptr, "gemm_wstream: bad arguments");
    CIB_REQUIRE(epilogue != ws::kSilu || N % 2 == 0, "gemm_wstream: a gate/up weight has an even number of rows");
    CIB_REQUIRE(ldo >= (epilogue == ws::kSilu ? N / 2 : N), "gemm_wstream: ldo too small");
    CUtensorMap mw, mx;
    if (tc_make_map(&mw, w, N, K, ldw, epilogue == ws::kSilu ? 64 : 128, "gemm_wstream") != 0) return -1;
    const int bx = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
    if (tc_make_map(&mx, act, M, K, lda, bx, "gemm_wstream") != 0) return -1;
    const int up_offset = N / 2;
    switch (bx) {
        case 16: return ws::dispatch<16, 8>(mw, mx, out, ldo, M, N, K, epilogue, up_offset, error_flag, use_pdl != 0, stream);
        case 32: return ws::dispatch<32, 8>(mw, mx, out, ldo, M, N, K, epilogue, up_offset, error_flag, use_pdl != 0, stream);
        case 64: return ws::dispatch<64, 7>(mw, mx, out, ldo, M, N, K, epilogue, up_offset, error_flag, use_pdl != 0, stream);
        default: return ws::dispatch<128, 6>(mw, mx, out, ldo, M, N, K, epilogue, up_offset, error_flag, use_pdl != 0, stream);
    }
}
