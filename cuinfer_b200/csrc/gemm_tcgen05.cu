// out[M, N] = a[M, K] · w[N, K]^T in bfloat16 on the 5th-generation tensor cores: TMA-fed, TMEM-accumulated.
//
// The reference calls cuBLAS for every projection (csrc/ops/projection.cu:32-44).  This is the prompt-sized
// replacement (many rows).  The kernel is persistent: one CTA per SM walks over 128 x BN output tiles, K in
// 64-element steps, and two accumulators in tensor memory let the epilogue of one tile run under the MMAs of the next.
//
//   warp 0, one thread : TMA producer.  Per step two `cp.async.bulk.tensor.2d` loads (an activation tile 128 x 64 and
//                        a weight tile BN x 64, both K-major, 128-byte swizzle) into a ring of shared-memory stages,
//                        completion counted in bytes on the stage's "full" mbarrier.  No multicast.
//   warp 1, one thread : MMA issuer.  Waits for "full", issues four `tcgen05.mma.cta_group::1.kind::f16`
//                        (128 x BN x 16 each) whose accumulator lives in tensor memory, then `tcgen05.commit` to the
//                        stage's "empty" mbarrier; after the last step a commit to the "accumulator ready" mbarrier.
//   warps 2-5          : epilogue.  Each warp owns the 32 TMEM lanes (= output rows) its rank allows, reads them with
//                        `tcgen05.ld.32x32b`, converts and stores rows to global memory (bfloat16 or float32).
//
// Rows beyond M, features beyond N and the tail of K read as zeros (TMA out-of-bounds fill) and are not stored.
// Every mbarrier wait is bounded: if a limit is hit the kernel raises a flag in global memory, stops issuing,
// drains what it started, frees its tensor memory and returns, so a fault in this kernel cannot hang the device.
#include "mma_utils.cuh"
#include "tcgen05_utils.cuh"

#include <stdlib.h>

namespace cib {

template <int BN, int STAGES, bool PAIR = false>
struct TcSmem {
    static constexpr int kABytes = kTcBM * kTcBK * 2;
    static constexpr int kBBytes = (PAIR ? BN / 2 : BN) * kTcBK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStagingBytes = kTcBM * 128 * 2;        // 128 rows x 128 bfloat16 columns for the TMA store
    static constexpr int kTotal = STAGES * kStageBytes + kStagingBytes + 1024 /* alignment slack */ + 512 /* barriers */;
};

// TMA_STORE: bfloat16 results leave through a 128-byte-swizzled staging buffer and `cp.async.bulk.tensor` stores
// (whole 128-byte lines per row; tails clipped by the tensor map).  Otherwise every thread stores its row itself.
// SILU: the weight rows are (gate, up) halves, rows [0, up_offset) and [up_offset, 2 up_offset); a tile multiplies BN / 2
// gate rows and the matching BN / 2 up rows (two weight boxes per stage) and stores silu(gate) * up, BN / 2 columns wide,
// straight from the 32-bit accumulators: the activation kernel and the round trip of the gate/up matrix are gone.
// PAIR: launched as clusters of two CTAs that share each 256 x BN tile (see the helpers above).  Per 64-k step a CTA
// then fetches 16 KB of activations and BN / 2 weight rows instead of BN: the kernel is bound by what an SM can fetch
// from the L2, so fewer bytes per flop is what makes it faster.
template <int BN, int STAGES, bool F32OUT, bool TMA_STORE, bool SILU = false, bool PAIR = false>
__global__ void __launch_bounds__(192)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_out, void* __restrict__ out, int ldo, int M, int N, int K,
                    int up_offset, int* __restrict__ error_flag) {
    static_assert(!SILU || (BN == 256 && TMA_STORE && !F32OUT), "the gated epilogue is built for 256-wide tiles stored by TMA");
    constexpr int kOutCols = SILU ? BN / 2 : BN;      // output columns of a tile
    extern __shared__ unsigned char smem_raw[];
    // stages must start on a 1024-byte boundary (one swizzle atom)
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* staging = tiles + STAGES * TcSmem<BN, STAGES, PAIR>::kStageBytes;      // 1024-byte aligned as well
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + TcSmem<BN, STAGES, PAIR>::kStagingBytes);
    uint64_t* full = bars;                     // [STAGES]  bytes of a stage have landed
    uint64_t* empty = bars + STAGES;           // [STAGES]  the MMAs that read a stage are done
    uint64_t* acc_full = bars + 2 * STAGES;    // [2]       an accumulator holds a finished tile
    uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2]    the epilogue has read an accumulator
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_steps = (K + kTcBK - 1) / kTcBK;
    constexpr int kTileRows = PAIR ? 2 * kTcBM : kTcBM;       // rows of a tile (of the pair's tile)
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;       // 0: the CTA that issues the MMAs
    const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int n_out = SILU ? up_offset : N;
    const int n_blocks = (n_out + kOutCols - 1) / kOutCols, m_blocks = (M + kTileRows - 1) / kTileRows;
    const int num_tiles = n_blocks * m_blocks;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], PAIR ? 8 : 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(tmem_slot)), "r"((uint32_t)(2 * BN)) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(tmem_slot)), "r"((uint32_t)(2 * BN)) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();          // the other CTA's barriers exist before anything arrives on them
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // set-up (barriers, tensor memory) may run under the tail of the kernel before this one; its results may not be read
    // nor this kernel's written before it has ended
    griddep_launch();
    griddep_wait();

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer: one running step counter over all tiles of this CTA ----
            int step = 0;
            bool ok = true;
            for (int tile = worker; tile < num_tiles && ok; tile += workers) {
                const int m0 = (tile / n_blocks) * kTileRows + (int)rank * kTcBM, n0 = (tile % n_blocks) * kOutCols;
                for (int kb = 0; kb < k_steps; ++kb, ++step) {
                    const int s = step % STAGES;
                    const uint32_t phase = (step / STAGES) & 1;
                    if (!mbar_wait(&empty[s], phase ^ 1)) { atomicExch(error_flag, 1); s_abort = 1; ok = false; break; }
                    if (*(volatile int*)&s_abort) { ok = false; break; }
                    unsigned char* a_dst = tiles + (size_t)s * TcSmem<BN, STAGES, PAIR>::kStageBytes;
                    unsigned char* b_dst = a_dst + TcSmem<BN, STAGES, PAIR>::kABytes;
                    if constexpr (PAIR) {
                        // both CTAs' bytes are counted on the first CTA's barrier; it expects them all
                        const uint32_t bar = map_to_cta(&full[s], 0);
                        if (rank == 0) mbar_expect_tx(&full[s], 2 * TcSmem<BN, STAGES, PAIR>::kStageBytes);
                        tma_load_2d_pair(a_dst, &map_a, bar, kb * kTcBK, m0);
                        // this CTA's half of the tile's weight rows (gated: the first CTA the gates, the second the ups)
                        const int w_row = SILU ? (rank == 0 ? n0 : up_offset + n0) : n0 + (int)rank * (BN / 2);
                        tma_load_2d_pair(b_dst, &map_w, bar, kb * kTcBK, w_row);
                        continue;
                    }
                    mbar_expect_tx(&full[s], TcSmem<BN, STAGES, PAIR>::kStageBytes);
                    tma_load_2d(a_dst, &map_a, &full[s], kb * kTcBK, m0);
                    if (SILU) {
                        // gate rows, then the matching up rows: accumulator columns [0, BN/2) and [BN/2, BN)
                        tma_load_2d(b_dst, &map_w, &full[s], kb * kTcBK, n0);
                        tma_load_2d(b_dst + (BN / 2) * 128, &map_w, &full[s], kb * kTcBK, up_offset + n0);
                    } else {
                        tma_load_2d(b_dst, &map_w, &full[s], kb * kTcBK, n0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- MMA issuer (of the pair) ----
            constexpr uint32_t idesc = umma_idesc_bf16(kTileRows, BN);
            int step = 0, local = 0;
            bool ok = true;
            for (int tile = worker; tile < num_tiles && ok; tile += workers, ++local) {
                const int buf = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1;
                if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1)) { atomicExch(error_flag, 4); s_abort = 1; ok = false; break; }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < k_steps; ++kb, ++step) {
                    const int s = step % STAGES;
                    const uint32_t phase = (step / STAGES) & 1;
                    if (!mbar_wait(&full[s], phase)) { atomicExch(error_flag, 2); s_abort = 1; ok = false; break; }
                    tcgen05_fence_after();
                    const unsigned char* a_src = tiles + (size_t)s * TcSmem<BN, STAGES, PAIR>::kStageBytes;
                    const unsigned char* b_src = a_src + TcSmem<BN, STAGES, PAIR>::kABytes;
                    const uint64_t adesc = umma_desc_k_major_sw128(a_src);
                    const uint64_t bdesc = umma_desc_k_major_sw128(b_src);
#pragma unroll
                    for (int k = 0; k < kTcBK / 16; ++k) {
                        // 16 elements of K = 32 bytes further inside the swizzle atom: +2 in 16-byte units
                        if (PAIR) umma_bf16_pair(tmem_d, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
                        else umma_bf16(tmem_d, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    if (PAIR) umma_commit_pair(&empty[s]);
                    else umma_commit(&empty[s]);   // frees the stage when these MMAs have read it
                }
                if (PAIR) umma_commit_pair(&acc_full[buf]);
                else umma_commit(&acc_full[buf]);  // arrives when every MMA issued so far has finished
            }
        }
    } else {
        // ---- epilogue: warps 2..5 own TMEM lanes 32 * (warp % 4) .. +31 ----
        const int quarter = warp & 3;
        int local = 0;
        bool ok = true;
        // the accumulator goes back to the CTA that issues the MMAs
        auto release_accumulator = [&](int buf) {
            if (PAIR) mbar_arrive_cluster(map_to_cta(&acc_empty[buf], 0));
            else mbar_arrive(&acc_empty[buf]);
        };
        for (int tile = worker; tile < num_tiles && ok; tile += workers, ++local) {
            const int buf = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            const int m0 = (tile / n_blocks) * kTileRows + (int)rank * kTcBM, n0 = (tile % n_blocks) * kOutCols;
            const int row = m0 + quarter * 32 + lane;
            ok = mbar_wait(&acc_full[buf], acc_phase);
            if (!ok && lane == 0) { atomicExch(error_flag, 3); s_abort = 1; }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0 && !(*(volatile int*)&s_abort);
            if (!ok) break;
            tcgen05_fence_after();
            if constexpr (SILU) {
                const int r_local = quarter * 32 + lane;
                const bool store_thread = threadIdx.x == 64;
                if (store_thread) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // staging is free again
                epilogue_barrier();
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t gv[32], uv[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c * 32);
                    tmem_ld_32x32b_x32(taddr, gv);
                    tmem_ld_32x32b_x32(taddr + (uint32_t)(BN / 2), uv);
                    tmem_ld_wait();
                    if (c == 3) {
                        tcgen05_fence_before();
                        if (lane == 0) release_accumulator(buf);     // the accumulator has been read completely
                    }
                    unsigned char* panel = staging + (size_t)(c >> 1) * (kTcBM * 128) + (size_t)r_local * 128;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float y[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float g = __uint_as_float(gv[8 * j + e]), u = __uint_as_float(uv[8 * j + e]);
                            // silu(g) = g / (1 + 2^(-g log2 e)) with the hardware's ex2 and reciprocal: the exact expf
                            // and division, with four epilogue warps, took longer than the tile's MMAs (a 2048 x 6144 x
                            // 1024 product went from 26 to 40 us).  The two approximations are good to about 2^-21
                            // relative, far inside the 2^-9 of the bfloat16 rounding that follows; exp overflowing to
                            // infinity for g < -88 gives g / inf = -0, the limit
                            float ex;
                            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"(-g * 1.4426950408889634f));
                            y[e] = __fdividef(g, 1.f + ex) * u;
                        }
                        uint4 pk;
                        __nv_bfloat162 t0 = __floats2bfloat162_rn(y[0], y[1]), t1 = __floats2bfloat162_rn(y[2], y[3]);
                        __nv_bfloat162 t2 = __floats2bfloat162_rn(y[4], y[5]), t3 = __floats2bfloat162_rn(y[6], y[7]);
                        pk.x = *reinterpret_cast<uint32_t*>(&t0); pk.y = *reinterpret_cast<uint32_t*>(&t1);
                        pk.z = *reinterpret_cast<uint32_t*>(&t2); pk.w = *reinterpret_cast<uint32_t*>(&t3);
                        const int chunk = ((c & 1) * 4 + j) ^ (r_local & 7);       // 128-byte swizzle
                        *reinterpret_cast<uint4*>(panel + chunk * 16) = pk;
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                epilogue_barrier();
                if (store_thread) {
#pragma unroll
                    for (int p = 0; p < 2; ++p) {
                        const int col = n0 + p * 64;
                        if (col < n_out) tma_store_2d(&map_out, staging + (size_t)p * (kTcBM * 128), col, m0);
                    }
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            } else if constexpr (TMA_STORE) {
                const int r_local = quarter * 32 + lane;                 // row of the tile = TMEM lane
                const bool store_thread = threadIdx.x == 64;
#pragma unroll 1
                for (int half = 0; half < BN / 128; ++half) {
                    if (store_thread) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // staging is free again
                    epilogue_barrier();
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t v[32];
                        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + half * 128 + c * 32), v);
                        tmem_ld_wait();
                        if (half == BN / 128 - 1 && c == 3) {
                            tcgen05_fence_before();
                            if (lane == 0) release_accumulator(buf);     // the accumulator has been read completely
                        }
                        // 32 columns = 64 bytes = four 16-byte chunks of this row, in panel c / 2, chunks (c % 2) * 4 ..
                        unsigned char* panel = staging + (size_t)(c >> 1) * (kTcBM * 128) + (size_t)r_local * 128;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint4 pk;
                            __nv_bfloat162 t0 = __floats2bfloat162_rn(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1]));
                            __nv_bfloat162 t1 = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
                            __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
                            __nv_bfloat162 t3 = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
                            pk.x = *reinterpret_cast<uint32_t*>(&t0); pk.y = *reinterpret_cast<uint32_t*>(&t1);
                            pk.z = *reinterpret_cast<uint32_t*>(&t2); pk.w = *reinterpret_cast<uint32_t*>(&t3);
                            const int chunk = ((c & 1) * 4 + j) ^ (r_local & 7);       // 128-byte swizzle
                            *reinterpret_cast<uint4*>(panel + chunk * 16) = pk;
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    epilogue_barrier();
                    if (store_thread) {
#pragma unroll
                        for (int p = 0; p < 2; ++p) {
                            const int col = n0 + half * 128 + p * 64;
                            if (col < N) tma_store_2d(&map_out, staging + (size_t)p * (kTcBM * 128), col, m0);
                        }
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
            } else {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c0), v);
                tmem_ld_wait();
                if (c0 + 32 >= BN) {
                    // the accumulator has been read completely: hand it back before the stores
                    tcgen05_fence_before();
                    if (lane == 0) release_accumulator(buf);
                }
                if (row < M) {
                    const int n = n0 + c0;
                    if (F32OUT) {
                        float* dst = reinterpret_cast<float*>(out) + (size_t)row * ldo + n;
                        if (n + 32 <= N && (ldo % 4) == 0) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                                  __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (n + j < N) dst[j] = __uint_as_float(v[j]);
                        }
                    } else {
                        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * ldo + n;
                        if (n + 32 <= N && (ldo % 8) == 0) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint4 pk;
                                __nv_bfloat162 t0 = __floats2bfloat162_rn(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                                __nv_bfloat162 t1 = __floats2bfloat162_rn(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                                __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
                                __nv_bfloat162 t3 = __floats2bfloat162_rn(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
                                pk.x = *reinterpret_cast<uint32_t*>(&t0); pk.y = *reinterpret_cast<uint32_t*>(&t1);
                                pk.z = *reinterpret_cast<uint32_t*>(&t2); pk.w = *reinterpret_cast<uint32_t*>(&t3);
                                *reinterpret_cast<uint4*>(dst + j) = pk;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (n + j < N) dst[j] = __float2bfloat16_rn(__uint_as_float(v[j]));
                        }
                    }
                }
            }
            }
        }
    }
    // ---- teardown: everything issued has been waited for on the normal path; free the tensor memory ----
    if (TMA_STORE && threadIdx.x == 64) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();          // neither CTA leaves while the other may still arrive on its barriers
    if (warp == 1) {
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * BN)) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * BN)) : "memory");
    }
}

static int make_map(CUtensorMap* map, const void* base, int rows, int K, int ld, int box_rows) {
    return tc_make_map(map, base, rows, K, ld, box_rows, "gemm_tcgen05");
}

template <int BN, int STAGES, bool F32OUT, bool TMA_STORE, bool SILU = false, bool PAIR = false>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, void* out, int ldo, int M, int N,
                     int K, int* error_flag, cudaStream_t stream, int up_offset = 0) {
    auto kernel = gemm_tcgen05_kernel<BN, STAGES, F32OUT, TMA_STORE, SILU, PAIR>;
    constexpr int smem = TcSmem<BN, STAGES, PAIR>::kTotal;
    static_assert(smem <= 227 * 1024, "a CTA has 227 KB of shared memory");
    static SmemLimit limit;
    if (int rc = raise_smem_limit(limit, kernel, smem, "gemm_tcgen05")) return rc;
    static int num_sms = 0;
    if (num_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0) num_sms = 148;
    }
    const int out_cols = SILU ? BN / 2 : BN, n_out = SILU ? up_offset : N;
    const int tile_rows = PAIR ? 2 * kTcBM : kTcBM;
    const int tiles = ((n_out + out_cols - 1) / out_cols) * ((M + tile_rows - 1) / tile_rows);
    if (!PAIR) {
        dim3 grid(tiles < num_sms ? tiles : num_sms);
        cudaError_t e = launch_pdl(kernel, grid, dim3(192), (size_t)smem, stream, prompt_pdl(), ma, mw, mo, out, ldo, M, N, K, up_offset, error_flag);
        if (e != cudaSuccess) {
            set_error("gemm_tcgen05: launch failed: %s", cudaGetErrorString(e));
            return -2;
        }
        return 0;
    }
    // clusters of two CTAs, one pair per tile at a time
    const int pairs = tiles < num_sms / 2 ? tiles : num_sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = prompt_pdl() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ma, mw, mo, out, ldo, M, N, K, up_offset, error_flag);
    if (e != cudaSuccess) {
        set_error("gemm_tcgen05: launch of CTA pairs failed: %s", cudaGetErrorString(e));
        return -2;
    }
    return 0;
}

}  // namespace cib

using namespace cib;

extern "C" int cib_gemm_tcgen05_supports(int M, int N, int K) {
    return M >= 1 && N >= 8 && K >= 8 && K % 8 == 0;
}

// a: [M, K] bfloat16 rows (lda), w: [N, K] bfloat16 rows (ldw), out: [M, N] bfloat16 (out_f32 = 0) or float32.
// error_flag: one int in device memory, zero before the call; non-zero afterwards means a bounded wait gave up.
// silu_pair: w holds N / 2 gate rows followed by N / 2 up rows and out is [M, N / 2] bfloat16 = silu(a gate^T) * (a up^T).
extern "C" int cib_gemm_tcgen05(const void* a, int lda, const void* w, int ldw, void* out, int ldo, int out_f32, int silu_pair,
                                int M, int N, int K, int* error_flag, cudaStream_t stream) {
    CIB_REQUIRE(cib_gemm_tcgen05_supports(M, N, K), "gemm_tcgen05: M=%d N=%d K=%d is not taken (K must be a multiple of 8)", M, N, K);
    CIB_REQUIRE(lda >= K && ldw >= K && lda % 8 == 0 && ldw % 8 == 0, "gemm_tcgen05: row strides must be multiples of 8 elements");
    CIB_REQUIRE(((uintptr_t)a % 16) == 0 && ((uintptr_t)w % 16) == 0, "gemm_tcgen05: operands must be 16-byte aligned");
    CIB_REQUIRE(ldo >= (silu_pair ? N / 2 : N) && error_flag != nullptr, "gemm_tcgen05: bad output arguments");
    CUtensorMap ma, mw;
    // From 256 rows on, pairs of CTAs share 256-row tiles (CUINFER_B200_GEMM_PAIR=0 keeps one CTA per tile, for comparisons).
    static const bool pair_allowed = [] { const char* e = getenv("CUINFER_B200_GEMM_PAIR"); return !(e && e[0] == '0'); }();
    // (only when there are enough 256-row tiles for every pair of SMs: with fewer, one CTA per 128-row tile measured faster)
    const int pair_tiles = ((M + 255) / 256) * (((silu_pair ? N / 2 : N) + 127) / 128);
    const bool pair = pair_allowed && M >= 256 && pair_tiles >= 74;
    if (silu_pair) {
        const int half = N / 2;
        CIB_REQUIRE(N % 2 == 0 && !out_f32 && ldo % 8 == 0 && ((uintptr_t)out % 16) == 0,
                    "gemm_tcgen05: the gated epilogue stores bfloat16 rows that are 16-byte aligned, N even");
        CUtensorMap mo;
        if (make_map(&ma, a, M, K, lda, kTcBM) != 0 || make_map(&mw, w, N, K, ldw, 128) != 0 ||
            make_map(&mo, out, M, half, ldo, kTcBM) != 0)
            return -1;
        if (pair) return launch_tc<256, 6, false, true, true, true>(ma, mw, mo, out, ldo, M, N, K, error_flag, stream, half);
        return launch_tc<256, 4, false, true, true>(ma, mw, mo, out, ldo, M, N, K, error_flag, stream, half);
    }
    if (pair) {
        // 256 x 256 tiles when those still give most pairs a tile, else 256 x 128; a CTA loads half of a tile's weight rows
        const int m_pairs = (M + 255) / 256;
        const int bn2 = (N % 256 == 0 && (N / 256) * m_pairs >= 60) ? 256 : 128;
        const bool tma_out2 = !out_f32 && ldo % 8 == 0 && ((uintptr_t)out % 16) == 0;
        CUtensorMap mo2;
        if (make_map(&ma, a, M, K, lda, kTcBM) != 0 || make_map(&mw, w, N, K, ldw, bn2 / 2) != 0) return -1;
        mo2 = ma;
        if (tma_out2 && make_map(&mo2, out, M, N, ldo, kTcBM) != 0) return -1;
        if (bn2 == 256) {
            if (out_f32) return launch_tc<256, 6, true, false, false, true>(ma, mw, mo2, out, ldo, M, N, K, error_flag, stream);
            if (tma_out2) return launch_tc<256, 6, false, true, false, true>(ma, mw, mo2, out, ldo, M, N, K, error_flag, stream);
            return launch_tc<256, 6, false, false, false, true>(ma, mw, mo2, out, ldo, M, N, K, error_flag, stream);
        }
        if (out_f32) return launch_tc<128, 8, true, false, false, true>(ma, mw, mo2, out, ldo, M, N, K, error_flag, stream);
        if (tma_out2) return launch_tc<128, 8, false, true, false, true>(ma, mw, mo2, out, ldo, M, N, K, error_flag, stream);
        return launch_tc<128, 8, false, false, false, true>(ma, mw, mo2, out, ldo, M, N, K, error_flag, stream);
    }
    // Tile width: 256 when that still gives most SMs a tile, else 128.
    const int m_blocks = (M + 127) / 128;
    int bn = 128;
    if (N % 256 == 0 && (N / 256) * m_blocks >= 120) bn = 256;
    if (make_map(&ma, a, M, K, lda, kTcBM) != 0) return -1;
    if (make_map(&mw, w, N, K, ldw, bn) != 0) return -1;
    // bfloat16 results with 16-byte aligned rows leave by TMA store; anything else is stored by the threads
    const bool tma_out = !out_f32 && ldo % 8 == 0 && ((uintptr_t)out % 16) == 0;
    CUtensorMap mo = ma;
    if (tma_out && make_map(&mo, out, M, N, ldo, kTcBM) != 0) return -1;
    if (bn == 256) {
        if (out_f32) return launch_tc<256, 4, true, false>(ma, mw, mo, out, ldo, M, N, K, error_flag, stream);
        if (tma_out) return launch_tc<256, 4, false, true>(ma, mw, mo, out, ldo, M, N, K, error_flag, stream);
        return launch_tc<256, 4, false, false>(ma, mw, mo, out, ldo, M, N, K, error_flag, stream);
    }
    if (out_f32) return launch_tc<128, 5, true, false>(ma, mw, mo, out, ldo, M, N, K, error_flag, stream);
    if (tma_out) return launch_tc<128, 5, false, true>(ma, mw, mo, out, ldo, M, N, K, error_flag, stream);
    return launch_tc<128, 5, false, false>(ma, mw, mo, out, ldo, M, N, K, error_flag, stream);
}
