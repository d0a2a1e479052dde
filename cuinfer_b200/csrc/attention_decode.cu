// Paged attention for decode steps (one query token per request), bfloat16, split over the keys.
//
// The reference runs decode tokens through its one attention kernel with 64-row tiles, of which a decoded
// token fills nq/nkv rows, and one CTA walks all keys of a request (csrc/ops/paged_attention.cu:133-383).
// Decode is a stream of the cache through the SMs, so here the keys of a (request, kv head) are split over
// `splits` CTAs, and inside a CTA over 4 warps; each warp copies its 16-key blocks into a private
// shared-memory ring with cp.async (no block-wide barrier in the loop), multiplies the group's query heads
// (rows of one m16 tile) with them on the tensor cores, and keeps a running softmax in base 2.  Warps are
// merged in shared memory, CTAs through a scratch buffer: every CTA writes its partial (max, sum, weighted
// values) and bumps a counter; the last CTA of a (request, kv head) combines all partials and writes the
// output, then resets the counter so that the kernel can be replayed from a CUDA graph.  Where the splits are few and
// their partials small (`cluster_combine_fits`), the CTAs of a (request, kv head) are one thread-block cluster instead
// and meet in the shared memory of its first CTA: the others write their partials there (distributed shared memory),
// signal with a release on the cluster's barrier and leave; no scratch, fence, counter or second trip to the L2.
//
// Scratch layout (float32): part_o[(request * nkv + kvh) * splits + split][g][D], part_ml[...][g][2].
// Cache layout of one layer: [page][0 = keys, 1 = values][kv head][slot in page][D].
//
// Where pages hold a multiple of 16 slots and the head size is a multiple of 64 (and there is no window), the
// blocks come through TMA instead of cp.async: one `cp.async.bulk.tensor.2d` per 64-column panel of a block's keys
// and of its values (128-byte swizzle), counted in bytes on an mbarrier per ring stage.  An SM keeps more bytes in
// flight this way than its load/store unit allows for cp.async, which is what bounds a kernel that only streams.
#include "mma_utils.cuh"
#include "tcgen05_utils.cuh"

#include <cooperative_groups.h>
#include <cuda.h>
#include <string.h>

#include <mutex>

namespace cib {

constexpr int kDecWarps = 4;
constexpr int kDecStages = 3;
constexpr int kDecKeys = 16;   // keys per warp block

template <int D>
struct DecodeSmem {
    // per warp: kDecStages x (K block + V block), each [16][D] bf16, XOR-swizzled in 16-byte chunks
    static constexpr int kBlockBytes = kDecKeys * D * 2;
    static constexpr int kWarpBytes = kDecStages * 2 * kBlockBytes;
    static constexpr int kTotal = kDecWarps * kWarpBytes;
};

// Element offset of 16-byte chunk `chunk` of row `row` inside a 16-row block.  cp.async path: rows of D elements,
// chunks XOR-swizzled by the row.  TMA path: 64-column panels of 16 rows x 128 bytes, chunks swizzled inside a panel.
template <int D, bool TMA>
__device__ __forceinline__ int block_off(int row, int chunk) {
    if (TMA) return (chunk >> 3) * (kDecKeys * 64) + row * 64 + (((chunk & 7) ^ (row & 7)) * 8);
    return row * D + ((chunk ^ (row & 7)) * 8);
}

template <int D>
__device__ __forceinline__ void load_block(__nv_bfloat16* sK, __nv_bfloat16* sV, const __nv_bfloat16* cache,
                                           const int* table, int key0, int key_end, int page_size, int num_pages,
                                           int nkv, int kvh, int lane) {
    // Neighbouring lanes copy neighbouring 16-byte chunks of a row, so one instruction of the warp reads
    // whole 128-byte lines: with D = 128 lanes 0-15 take one key row, lanes 16-31 the next.
    constexpr int kChunks = D / 8;                               // 16-byte chunks per row
    constexpr int kLanesPerRow = kChunks < 32 ? kChunks : 32;
    constexpr int kRowsPerPass = 32 / kLanesPerRow;
    constexpr int kPasses = kDecKeys / kRowsPerPass;
    constexpr int kChunkPasses = kChunks / kLanesPerRow;         // > 1 only for D > 256
    const size_t head_stride = (size_t)page_size * D;
    const int sub_row = lane / kLanesPerRow;
    const int chunk0 = lane % kLanesPerRow;
    // fast path: the whole block lies in one page
    const int off0 = key0 % page_size;
    const bool one_page = off0 + kDecKeys <= page_size;
    int page0 = -1;
    if (one_page && key0 < key_end) {
        page0 = table[key0 / page_size];
        if (page0 >= num_pages) page0 = -1;
    }
#pragma unroll
    for (int pass = 0; pass < kPasses; ++pass) {
        const int row = pass * kRowsPerPass + sub_row;
        const int j = key0 + row;
        bool valid = j < key_end;
        int page = page0, off = off0 + row;
        if (!one_page && valid) {
            page = table[j / page_size];
            off = j % page_size;
            if (page >= num_pages) page = -1;
        }
        valid = valid && page >= 0;
        const __nv_bfloat16* kp = cache + (((size_t)(valid ? page : 0) * 2 + 0) * nkv + kvh) * head_stride +
                                  (size_t)(valid ? off : 0) * D;
        const __nv_bfloat16* vp = kp + (size_t)nkv * head_stride;
#pragma unroll
        for (int cp = 0; cp < kChunkPasses; ++cp) {
            const int chunk = chunk0 + cp * kLanesPerRow;
            const int sw = (chunk ^ (row & 7)) * 8;
            cp_async16(sK + row * D + sw, kp + chunk * 8, valid);
            cp_async16(sV + row * D + sw, vp + chunk * 8, valid);
        }
    }
}

// Shared memory the first CTA of a cluster keeps for the partials of all its CTAs: [splits][g][D + 2] floats, in a
// region of its own behind everything else (the other CTAs may write while the first still streams keys).
__host__ __device__ inline size_t cluster_inbox_bytes(int splits, int g, int d) { return (size_t)splits * g * (d + 2) * sizeof(float); }
// The cluster path is taken for up to 4 CTAs per (request, kv head) whose partials fit 9 KB: two CTAs of head size 128
// then still share an SM.  (Clusters of 8 measured slower than the combine through memory once they fill the GPU: 4
// requests x 8 heads x 8 splits ran a decode step in 1.42 ms against 1.17.)
inline bool cluster_combine_fits(int splits, int g, int d) { return splits > 1 && splits <= 4 && cluster_inbox_bytes(splits, g, d) <= 9 * 1024; }

template <int D, bool TMA, bool CL>
__global__ void __launch_bounds__(kDecWarps * 32)
paged_attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                              int out_stride, const __nv_bfloat16* __restrict__ cache, int num_pages, int page_size,
                              const int* __restrict__ block_table, int table_stride,
                              const int* __restrict__ seq_lens, int nq, int nkv, float scale_log2, int window,
                              int splits, float* __restrict__ part_o, float* __restrict__ part_ml,
                              int* __restrict__ counters, const __grid_constant__ CUtensorMap kv_map,
                              int* __restrict__ error_flag, const void* __restrict__ warm, unsigned long long warm_bytes,
                              int inbox_offset) {
    // "this CTA runs": the others of its cluster may write to its shared memory once all have said so
    if (CL) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    extern __shared__ __align__(128) unsigned char smem_unaligned[];
    // TMA writes whole 1024-byte swizzle atoms: the rings then start on such a boundary
    unsigned char* smem_raw = TMA ? reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023))
                                  : smem_unaligned;
    __shared__ uint64_t s_full[kDecWarps * kDecStages];          // TMA: bytes of a ring stage have landed
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z;
    const int g = nq / nkv;
    const int quad = lane & 3, qrow = lane >> 2;

    const int seq_len = seq_lens[r];
    const int pos = seq_len - 1;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int span = max(0, seq_len - lo);
    int chunk = (span + splits - 1) / splits;
    chunk = (chunk + kDecKeys - 1) / kDecKeys * kDecKeys;
    const int k_begin = lo + split * chunk;
    const int k_end = min(seq_len, k_begin + chunk);
    const int* table = block_table + (size_t)r * table_stride;

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};

    __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(smem_raw + (size_t)warp * DecodeSmem<D>::kWarpBytes);
    auto stage_k = [&](int s) { return ring + (size_t)s * 2 * kDecKeys * D; };
    auto stage_v = [&](int s) { return ring + (size_t)s * 2 * kDecKeys * D + kDecKeys * D; };

    const int total_blocks = k_end > k_begin ? (k_end - k_begin + kDecKeys - 1) / kDecKeys : 0;
    const int my_blocks = total_blocks > warp ? (total_blocks - warp + kDecWarps - 1) / kDecWarps : 0;
    auto block_key = [&](int i) { return k_begin + (i * kDecWarps + warp) * kDecKeys; };

    if (TMA) {
        if (threadIdx.x == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&kv_map) : "memory");
            for (int i = 0; i < kDecWarps * kDecStages; ++i) mbar_init(&s_full[i], 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncthreads();
    }
    // TMA path: lane 0 asks for the four boxes of a block (keys and values, two 64-column panels each for D = 128);
    // a block is 16 slots of one page (pages hold a multiple of 16 slots, blocks start at multiples of 16).  A page
    // number outside the pool becomes a row outside the tensor map: zeros, with the bytes still counted.
    auto tma_block = [&](int s, int key0) {
        if (lane != 0) return;
        const int pidx = key0 / page_size, off = key0 - pidx * page_size;
        const int page = table[pidx];
        const long long total_rows = (long long)num_pages * 2 * nkv * page_size;
        const bool okp = page >= 0 && page < num_pages;
        const long long row_k = okp ? (((long long)page * 2) * nkv + kvh) * page_size + off : total_rows;
        const long long row_v = okp ? row_k + (long long)nkv * page_size : total_rows;
        uint64_t* bar = &s_full[warp * kDecStages + s];
        mbar_expect_tx(bar, 2 * DecodeSmem<D>::kBlockBytes);
#pragma unroll
        for (int pn = 0; pn < D / 64; ++pn) {
            tma_load_2d(stage_k(s) + pn * kDecKeys * 64, &kv_map, bar, pn * 64, (int)row_k);
            tma_load_2d(stage_v(s) + pn * kDecKeys * 64, &kv_map, bar, pn * 64, (int)row_v);
        }
    };

    // Keys and values of earlier steps do not depend on the kernel before this one: their first blocks are
    // requested before `griddepcontrol.wait`.  Only the block that holds this step's own token (position
    // seq_len - 1, written by the kernel before) has to wait; so do the queries.
    griddep_launch();
    int deferred = -1;
#pragma unroll
    for (int s = 0; s < kDecStages - 1; ++s) {
        if (s < my_blocks) {
            if (block_key(s) + kDecKeys > pos) deferred = s;
            else if (TMA) tma_block(s, block_key(s));
            else load_block<D>(stage_k(s), stage_v(s), cache, table, block_key(s), k_end, page_size, num_pages, nkv, kvh, lane);
        }
        if (!TMA) cp_async_commit();
    }
    griddep_wait();
    if (deferred >= 0) {
        if (TMA) {
            tma_block(deferred, block_key(deferred));
        } else {
            // one warp per (request, kv head): its late block is its own commit group, so let everything land first
            // and the loop's group counting starts clean
            load_block<D>(stage_k(deferred), stage_v(deferred), cache, table, block_key(deferred), k_end, page_size, num_pages, nkv, kvh, lane);
            cp_async_commit();
            cp_async_wait<0>();
        }
    }
    // ---- query fragments: rows 0..g-1 are the heads of this kv head, the rest are zero ----
    uint32_t qf[D / 16][4];
    {
        const __nv_bfloat16* qp = q + (size_t)r * q_stride + (size_t)kvh * g * D;
#pragma unroll
        for (int kt = 0; kt < D / 16; ++kt) {
            const int c0 = kt * 16 + quad * 2;
            qf[kt][0] = qrow < g ? *reinterpret_cast<const uint32_t*>(qp + (size_t)qrow * D + c0) : 0u;
            qf[kt][1] = qrow + 8 < g ? *reinterpret_cast<const uint32_t*>(qp + (size_t)(qrow + 8) * D + c0) : 0u;
            qf[kt][2] = qrow < g ? *reinterpret_cast<const uint32_t*>(qp + (size_t)qrow * D + c0 + 8) : 0u;
            qf[kt][3] = qrow + 8 < g ? *reinterpret_cast<const uint32_t*>(qp + (size_t)(qrow + 8) * D + c0 + 8) : 0u;
        }
    }

    bool landed = true;
    for (int i = 0; i < my_blocks; ++i) {
        if (TMA) {
            landed = mbar_wait(&s_full[warp * kDecStages + i % kDecStages], (uint32_t)((i / kDecStages) & 1));
            landed = __all_sync(0xffffffffu, landed);
            if (!landed) {
                if (lane == 0) atomicExch(error_flag, 21);
                break;
            }
            // the stage that block i - 1 was read from is refilled: every lane has finished reading it
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            const int nxt = i + kDecStages - 1;
            if (nxt < my_blocks) tma_block(nxt % kDecStages, block_key(nxt));
        } else {
            cp_async_wait<kDecStages - 2>();
            __syncwarp();
            const int nxt = i + kDecStages - 1;
            if (nxt < my_blocks)
                load_block<D>(stage_k(nxt % kDecStages), stage_v(nxt % kDecStages), cache, table, block_key(nxt), k_end,
                              page_size, num_pages, nkv, kvh, lane);
            cp_async_commit();
        }
        const __nv_bfloat16* sK = stage_k(i % kDecStages);
        const __nv_bfloat16* sV = stage_v(i % kDecStages);
        const int key0 = block_key(i);
        if (TMA && key0 + kDecKeys > seq_len) {
            // the page came whole: value rows past the request's last token may hold anything, and 0 x NaN is NaN
            const int valid = seq_len - key0;
            for (int idx = valid * (D / 8) + lane; idx < kDecKeys * (D / 8); idx += 32)
                *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(sV) + block_off<D, true>(idx / (D / 8), idx % (D / 8))) = make_uint4(0, 0, 0, 0);
            __syncwarp();
        }
        // ---- S = Q K^T for 16 keys ----
        float s[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
        {
            const int mat = lane >> 3, rr = lane & 7;
            const int krow = (mat >> 1) * 8 + rr;
#pragma unroll
            for (int kt = 0; kt < D / 16; ++kt) {
                const int chunkc = 2 * kt + (mat & 1);
                uint32_t b[4];
                ldmatrix_x4(b, smem_u32(sK + block_off<D, TMA>(krow, chunkc)));
                mma_bf16_16816(s[0], qf[kt], b[0], b[1]);
                mma_bf16_16816(s[1], qf[kt], b[2], b[3]);
            }
        }
        // ---- mask, running softmax (base 2) ----
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + n * 8 + quad * 2 + (e & 1);
                const float v = key < k_end ? s[n][e] * scale_log2 : -INFINITY;
                s[n][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        }
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            corr[h] = m_run[h] == -INFINITY ? 0.f : exp2f(m_run[h] - m_new);
            m_run[h] = m_new;
            l_run[h] *= corr[h];
        }
        uint32_t pf[4];
        {
            float p[2][4];
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float mref = m_run[e >> 1];
                    p[n][e] = (s[n][e] == -INFINITY || mref == -INFINITY) ? 0.f : exp2f(s[n][e] - mref);
                    l_run[e >> 1] += p[n][e];
                }
            pf[0] = pack_bf16(p[0][0], p[0][1]);
            pf[1] = pack_bf16(p[0][2], p[0][3]);
            pf[2] = pack_bf16(p[1][0], p[1][1]);
            pf[3] = pack_bf16(p[1][2], p[1][3]);
        }
        // ---- O = O * corr + P V ----
        {
            const int mat = lane >> 3, rr = lane & 7;
            const int vrow = (mat & 1) * 8 + rr;
#pragma unroll
            for (int nt = 0; nt < D / 16; ++nt) {
                const int chunkc = 2 * nt + (mat >> 1);
                uint32_t b[4];
                ldmatrix_x4_trans(b, smem_u32(sV + block_off<D, TMA>(vrow, chunkc)));
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    float* acc = o[2 * nt + t];
                    acc[0] *= corr[0]; acc[1] *= corr[0]; acc[2] *= corr[1]; acc[3] *= corr[1];
                }
                mma_bf16_16816(o[2 * nt], pf, b[0], b[1]);
                mma_bf16_16816(o[2 * nt + 1], pf, b[2], b[3]);
            }
        }
    }
    // the stream of keys and values is over: what the kernel after this one reads first (the output projection's weights)
    // can come into the L2 while the partial results are merged
    if (threadIdx.x == 0)
        warm_l2_share(warm, warm_bytes, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x, gridDim.x * gridDim.y * gridDim.z);
    if (!TMA) cp_async_wait<0>();
    __syncthreads();     // all rings are free: reuse shared memory for the merge of the warps

    // ---- merge the warps (only the g real rows) ----
    float* sm_m = reinterpret_cast<float*>(smem_raw);             // [warps][16]
    float* sm_l = sm_m + kDecWarps * 16;                          // [warps][16]
    float* sm_o = sm_l + kDecWarps * 16;                          // [warps][g][D]
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float l = l_run[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int row = qrow + 8 * h;
        if (quad == 0) { sm_m[warp * 16 + row] = m_run[h]; sm_l[warp * 16 + row] = l; }
        if (row < g) {
#pragma unroll
            for (int nt = 0; nt < D / 8; ++nt) {
                float* dst = sm_o + ((size_t)(warp * g + row)) * D + nt * 8 + quad * 2;
                dst[0] = o[nt][2 * h];
                dst[1] = o[nt][2 * h + 1];
            }
        }
    }
    __syncthreads();
    const size_t part_base = ((size_t)r * nkv + kvh) * splits + split;
    // cluster path: the partials go to the first CTA's shared memory, [split][g][D] values then [split][g][2] maxima and sums
    float* inbox_o = nullptr;
    float* inbox_ml = nullptr;
    if (CL) {
        namespace cg = cooperative_groups;
        float* inbox = reinterpret_cast<float*>(smem_raw + inbox_offset);
        if (split != 0) inbox = cg::this_cluster().map_shared_rank(inbox, 0);
        inbox_o = inbox + (size_t)split * g * D;
        inbox_ml = inbox + (size_t)splits * g * D + (size_t)split * g * 2;
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");       // every CTA of the cluster runs
    }
    for (int idx = threadIdx.x; idx < g * D; idx += blockDim.x) {
        const int row = idx / D, dim = idx - row * D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, sm_m[w * 16 + row]);
        float L = 0.f, O = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < kDecWarps; ++w) {
                const float mw = sm_m[w * 16 + row];
                const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
                L += sm_l[w * 16 + row] * f;
                O += sm_o[((size_t)(w * g + row)) * D + dim] * f;
            }
        }
        if (splits == 1) {
            out[(size_t)r * out_stride + (size_t)(kvh * g + row) * D + dim] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        } else if (CL) {
            inbox_o[row * D + dim] = O;
            if (dim == 0) {
                inbox_ml[row * 2 + 0] = M;
                inbox_ml[row * 2 + 1] = L;
            }
        } else {
            part_o[(part_base * g + row) * D + dim] = O;
            if (dim == 0) {
                part_ml[(part_base * g + row) * 2 + 0] = M;
                part_ml[(part_base * g + row) * 2 + 1] = L;
            }
        }
    }
    if (splits == 1) return;
    if (CL) {
        // ---- the first CTA of the cluster combines what the others have written into its shared memory ----
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        if (split != 0) return;
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        __syncthreads();                                              // this CTA's own partial too
        const float* all_o = reinterpret_cast<const float*>(smem_raw + inbox_offset);
        const float* all_ml = all_o + (size_t)splits * g * D;
        for (int idx = threadIdx.x; idx < g * D; idx += blockDim.x) {
            const int row = idx / D, dim = idx - row * D;
            float M = -INFINITY;
            for (int sp = 0; sp < splits; ++sp) M = fmaxf(M, all_ml[(sp * g + row) * 2]);
            float L = 0.f, O = 0.f;
            for (int sp = 0; sp < splits; ++sp) {
                const float ms = all_ml[(sp * g + row) * 2];
                const float f = (ms == -INFINITY || M == -INFINITY) ? 0.f : exp2f(ms - M);
                L = fmaf(all_ml[(sp * g + row) * 2 + 1], f, L);
                O = fmaf(all_o[((size_t)sp * g + row) * D + dim], f, O);
            }
            out[(size_t)r * out_stride + (size_t)(kvh * g + row) * D + dim] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        }
        return;
    }

    // ---- the last CTA of this (request, kv head) combines the splits ----
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int done = atomicAdd(&counters[r * nkv + kvh], 1);
        s_last = done == splits - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // maxima and sums of all splits in one parallel round of loads; a warp per row turns them into weights (lanes over
    // the splits); then the weighted sums with up to sixteen loads in flight per thread.  (Read one by one in a loop
    // over the splits, the sums cost a round trip to the L2 each: some 5 us with 32 splits.)
    const size_t base = ((size_t)r * nkv + kvh) * splits;
    float* sm_w = reinterpret_cast<float*>(smem_raw);            // [g][splits] maximum, then weight of each split
    float* sm_ls = sm_w + (size_t)g * splits;                     // [g][splits] sum of each split
    float* sm_inv = sm_ls + (size_t)g * splits;                   // [g] 1 / total
    for (int idx = threadIdx.x; idx < g * splits; idx += blockDim.x) {
        const int row = idx / splits, sp = idx - row * splits;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(&part_ml[((base + sp) * g + row) * 2]));
        sm_w[idx] = ml.x;
        sm_ls[idx] = ml.y;
    }
    __syncthreads();
    for (int row = warp; row < g; row += kDecWarps) {
        float M = -INFINITY;
        for (int sp = lane; sp < splits; sp += 32) M = fmaxf(M, sm_w[row * splits + sp]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
        float L = 0.f;
        for (int sp = lane; sp < splits; sp += 32) {
            const float ms = sm_w[row * splits + sp];
            const float f = (ms == -INFINITY || M == -INFINITY) ? 0.f : exp2f(ms - M);
            sm_w[row * splits + sp] = f;
            L += sm_ls[row * splits + sp] * f;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
        if (lane == 0) sm_inv[row] = L > 0.f ? 1.f / L : 0.f;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < g * D; idx += blockDim.x) {
        const int row = idx / D, dim = idx - row * D;
        float O = 0.f;
        int sp = 0;
        for (; sp + 16 <= splits; sp += 16) {
            float v[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) v[u] = __ldcg(&part_o[((base + sp + u) * g + row) * D + dim]);
#pragma unroll
            for (int u = 0; u < 16; ++u) O = fmaf(v[u], sm_w[row * splits + sp + u], O);
        }
        for (; sp + 4 <= splits; sp += 4) {
            float v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = __ldcg(&part_o[((base + sp + u) * g + row) * D + dim]);
#pragma unroll
            for (int u = 0; u < 4; ++u) O = fmaf(v[u], sm_w[row * splits + sp + u], O);
        }
        for (; sp < splits; ++sp) O = fmaf(__ldcg(&part_o[((base + sp) * g + row) * D + dim]), sm_w[row * splits + sp], O);
        out[(size_t)r * out_stride + (size_t)(kvh * g + row) * D + dim] = __float2bfloat16_rn(O * sm_inv[row]);
    }
    if (threadIdx.x == 0) counters[r * nkv + kvh] = 0;
}

// How many clusters of `cluster_x` CTAs of this kernel the device runs at one time (0 if that cannot be told); asked
// once per cluster size and kernel, then remembered.
template <typename Kernel>
static int max_resident_clusters(Kernel kernel, int cluster_x, size_t smem) {
    static std::mutex mutex;
    static int known[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};     // by cluster size; 0: not asked yet, -1: the query failed
    if (cluster_x < 2 || cluster_x > 8) return 0;
    std::lock_guard<std::mutex> lock(mutex);
    if (known[cluster_x] == 0) {
        known[cluster_x] = -1;
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(cluster_x * 64, 1, 1);
            cfg.blockDim = dim3(kDecWarps * 32);
            cfg.dynamicSmemBytes = smem;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = (unsigned)cluster_x;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) == cudaSuccess && n > 0) known[cluster_x] = n;
            else (void)cudaGetLastError();
        }
    }
    return known[cluster_x] > 0 ? known[cluster_x] : 0;
}

template <int D>
static int launch_decode(const void* q, int q_stride, void* out, int out_stride, const void* cache, int num_pages,
                         int page_size, const int* block_table, int table_stride, const int* seq_lens,
                         int num_requests, int nq, int nkv, float scale, int window, int splits, float* part_o,
                         float* part_ml, int* counters, cudaStream_t stream, bool use_pdl = false,
                         int* error_flag = nullptr, const void* warm = nullptr, unsigned long long warm_bytes = 0) {
    const int g = nq / nkv;
    // TMA needs whole 16-slot blocks inside a page, blocks that start at multiples of 16 (no window), 64-column
    // panels, a place to report a wait that ran out, and row coordinates that fit 32 bits
    const long long total_rows = (long long)num_pages * 2 * nkv * page_size;
    const bool tma = error_flag != nullptr && page_size % kDecKeys == 0 && window <= 0 && D % 64 == 0 &&
                     total_rows < (1ll << 31) && ((uintptr_t)cache % 16) == 0;
    CUtensorMap kv_map;
    memset(&kv_map, 0, sizeof(kv_map));
    if (tma && encode_tensor_map_bf16_2d(&kv_map, cache, (unsigned long long)total_rows, D, D, 64, kDecKeys,
                                         "paged_attention_decode") != 0)
        return -1;
    size_t smem = DecodeSmem<D>::kTotal + (tma ? 1024 : 0);
    size_t merge = (size_t)(2 * kDecWarps * 16 + kDecWarps * g * D) * sizeof(float) + (tma ? 1024 : 0);
    const size_t combine = (size_t)(2 * g * splits + g) * sizeof(float) + (tma ? 1024 : 0);
    if (combine > merge) merge = combine;
    if (merge > smem) smem = merge;
    smem = (smem + 15) & ~size_t(15);
    // counted from the aligned start of the rings: the slack for that alignment lies in front of it, not behind
    const int inbox_offset = (int)(smem - (tma ? 1024 : 0));
    // The cluster path only where all clusters of the launch run at once: a cluster needs its CTAs on SMs of one GPC, so
    // fewer fit than single CTAs would, and a second round of clusters costs far more than the combine through memory
    // (12 requests x 8 heads x 3 splits: 51 us against 37).
    bool cluster = tma && cluster_combine_fits(splits, g, D);
    if (cluster) {
        const size_t with_inbox = smem + cluster_inbox_bytes(splits, g, D);
        const int resident = max_resident_clusters(paged_attention_decode_kernel<D, true, true>, splits, with_inbox);
        cluster = resident >= nkv * num_requests;
        if (cluster) smem = with_inbox;
    }
    CIB_REQUIRE(smem <= 225 * 1024, "paged_attention_decode: needs %zu bytes of shared memory", smem);
    dim3 grid(splits, nkv, num_requests);
    const float scale_log2 = scale * 1.4426950408889634f;
    auto launch = [&](auto kernel, SmemLimit& limit) -> cudaError_t {
        if (raise_smem_limit(limit, kernel, 225 * 1024, "paged_attention_decode") != 0) return cudaErrorUnknown;
        return launch_pdl_cluster(kernel, grid, dim3(kDecWarps * 32), smem, stream, use_pdl, cluster ? splits : 1,
                                  (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride,
                                  (const __nv_bfloat16*)cache, num_pages, page_size, block_table, table_stride, seq_lens, nq,
                                  nkv, scale_log2, window, splits, part_o, part_ml, counters, kv_map, error_flag, warm,
                                  warm_bytes, inbox_offset);
    };
    static SmemLimit limits[3];          // one per instantiation of this head size
    cudaError_t e = cudaSuccess;
    if (cluster) {
        // should the cluster launch be refused after all (the occupancy query is a forecast), the step is not lost:
        // the same work runs without clusters, combined through the scratch
        e = launch(paged_attention_decode_kernel<D, true, true>, limits[0]);
        if (e != cudaSuccess && e != cudaErrorUnknown) {
            (void)cudaGetLastError();
            cluster = false;
            smem -= cluster_inbox_bytes(splits, g, D);
        }
    }
    if (!cluster) {
        e = tma ? launch(paged_attention_decode_kernel<D, true, false>, limits[1])
                : launch(paged_attention_decode_kernel<D, false, false>, limits[2]);
    }
    if (e == cudaErrorUnknown) return -2;          // the message is set
    if (e != cudaSuccess) {
        set_error("paged_attention_decode: launch failed: %s", cudaGetErrorString(e));
        return -2;
    }
    return 0;
}

}  // namespace cib

using namespace cib;

// Head sizes this kernel takes; others are refused (the caller falls back to the all-sizes kernel).
extern "C" int cib_paged_attention_decode_supports(int head_dim, int nq, int nkv) {
    return (head_dim == 64 || head_dim == 128 || head_dim == 256) && nkv > 0 && nq % nkv == 0 && nq / nkv <= 16;
}

// Floats of scratch that `splits` splits need: part_o then part_ml, laid out one after the other.
extern "C" long long cib_paged_attention_decode_scratch_floats(int num_requests, int nq, int head_dim, int splits) {
    return (long long)num_requests * nq * splits * (head_dim + 2);
}

// One query token per request.  `scratch` holds cib_paged_attention_decode_scratch_floats floats (unused when
// splits == 1); `counters` holds num_requests * nkv ints that are zero before the first call (the kernel leaves
// them zero).  `error_flag` (one zero int in device memory, or null) lets the kernel fetch the cache through TMA
// where the geometry allows it: a copy that does not land in time sets the flag instead of hanging the kernel.
// warm / warm_bytes: memory that the kernel after this one reads first, or null: fetched into the L2 at the kernel's end.
extern "C" int cib_paged_attention_decode(const void* q, int q_stride, void* out, int out_stride, const void* cache,
                                          int num_pages, int page_size, const int* block_table, int table_stride,
                                          const int* seq_lens, int num_requests, int nq, int nkv, int head_dim,
                                          float scale, int window, int splits, float* scratch, int* counters,
                                          int use_pdl, int* error_flag, const void* warm, long long warm_bytes,
                                          cudaStream_t stream) {
    CIB_REQUIRE(cib_paged_attention_decode_supports(head_dim, nq, nkv),
                "paged_attention_decode: head_dim %d with %d/%d heads is not taken by this kernel (64, 128 or 256; at most 16 query heads per kv head)",
                head_dim, nq, nkv);
    CIB_REQUIRE(num_requests >= 0 && splits >= 1 && splits <= 128, "paged_attention_decode: bad sizes R=%d splits=%d", num_requests, splits);
    CIB_REQUIRE(page_size > 0 && num_pages > 0 && table_stride > 0, "paged_attention_decode: bad cache geometry");
    CIB_REQUIRE(q_stride % 2 == 0 && ((uintptr_t)q % 4) == 0, "paged_attention_decode: q rows must be 4-byte aligned");
    CIB_REQUIRE(splits == 1 || (scratch && counters), "paged_attention_decode: splits need scratch and counters");
    CIB_REQUIRE(((uintptr_t)scratch % 8) == 0, "paged_attention_decode: the scratch must be 8-byte aligned");
    CIB_REQUIRE(num_requests <= 65535 && nkv <= 65535, "paged_attention_decode: grid too large");
    if (num_requests == 0) return 0;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)num_requests * nq * splits * head_dim : nullptr;
    if (((uintptr_t)warm % 16) != 0 || warm_bytes <= 0) { warm = nullptr; warm_bytes = 0; }
    const unsigned long long wb = (unsigned long long)warm_bytes;
    switch (head_dim) {
        case 64: return launch_decode<64>(q, q_stride, out, out_stride, cache, num_pages, page_size, block_table, table_stride, seq_lens, num_requests, nq, nkv, scale, window, splits, part_o, part_ml, counters, stream, use_pdl != 0, error_flag, warm, wb);
        case 128: return launch_decode<128>(q, q_stride, out, out_stride, cache, num_pages, page_size, block_table, table_stride, seq_lens, num_requests, nq, nkv, scale, window, splits, part_o, part_ml, counters, stream, use_pdl != 0, error_flag, warm, wb);
        case 256: return launch_decode<256>(q, q_stride, out, out_stride, cache, num_pages, page_size, block_table, table_stride, seq_lens, num_requests, nq, nkv, scale, window, splits, part_o, part_ml, counters, stream, use_pdl != 0, error_flag, warm, wb);
    }
    return -1;
}

// ---- the variant that allocates nothing (see attention_decode_static.h) --------------------------------------
#include "attention_decode_static.h"

namespace cib {

// Partial results of the splits, then the counters (as ints) behind them.  In host code this name is only a
// stand-in for the symbol; the device address is looked up once per device below.
static __device__ __align__(256) float g_static_decode_scratch[kStaticScratchFloats + kStaticCounters];

static float* g_static_scratch_ptr[kMaxDevices] = {nullptr};
static std::mutex g_static_scratch_mutex;

// Device address of the array on the current device; looked up on the first call on that device.
static int static_scratch_address(float** ptr) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_error("paged_attention_decode_static: cannot tell the current device (%s)", cudaGetErrorString(e));
        return -2;
    }
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_ptr[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_static_decode_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_error("paged_attention_decode_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
            return -2;
        }
        g_static_scratch_ptr[dev] = p;
    }
    *ptr = g_static_scratch_ptr[dev];
    return 0;
}

}  // namespace cib

extern "C" int cib_paged_attention_decode_static(const void* q, int q_stride, void* out, int out_stride, const void* cache,
                                                 int num_pages, int page_size, const int* block_table, int table_stride,
                                                 const int* seq_lens, int num_requests, int nq, int nkv, int head_dim,
                                                 float scale, int window, int splits, cudaStream_t stream) {
    CIB_REQUIRE(cib_paged_attention_decode_supports(head_dim, nq, nkv),
                "paged_attention_decode_static: head_dim %d with %d/%d heads is not taken by this kernel (64, 128 or 256; at most 16 query heads per kv head)",
                head_dim, nq, nkv);
    CIB_REQUIRE(num_requests >= 0 && splits >= 1 && splits <= 128, "paged_attention_decode_static: bad sizes R=%d splits=%d", num_requests, splits);
    CIB_REQUIRE(page_size > 0 && num_pages > 0 && table_stride > 0, "paged_attention_decode_static: bad cache geometry");
    CIB_REQUIRE(q_stride % 2 == 0 && ((uintptr_t)q % 4) == 0, "paged_attention_decode_static: q rows must be 4-byte aligned");
    CIB_REQUIRE(num_requests <= 65535 && nkv <= 65535, "paged_attention_decode_static: grid too large");
    const long long need = (long long)num_requests * nq * splits * (head_dim + 2);
    CIB_REQUIRE(need <= (long long)kStaticScratchFloats,
                "paged_attention_decode_static: %d requests x %d heads x %d splits x head_dim %d need %lld floats of scratch, the built-in array holds %d; use fewer splits or cib_paged_attention_decode with a buffer of your own",
                num_requests, nq, splits, head_dim, need, (int)kStaticScratchFloats);
    CIB_REQUIRE((long long)num_requests * nkv <= (long long)kStaticCounters,
                "paged_attention_decode_static: %d requests x %d kv heads exceed the %d built-in counters",
                num_requests, nkv, (int)kStaticCounters);
    if (num_requests == 0) return 0;
    float* base = nullptr;
    if (static_scratch_address(&base) != 0) return -2;
    float* part_o = base;
    float* part_ml = base + (size_t)num_requests * nq * splits * head_dim;
    int* counters = reinterpret_cast<int*>(base + kStaticScratchFloats);
    if (splits > 1) {
        // the array keeps the last call's contents: the counters must start at zero
        cudaError_t e = cudaMemsetAsync(counters, 0, sizeof(int) * (size_t)num_requests * nkv, stream);
        if (e != cudaSuccess) {
            set_error("paged_attention_decode_static: clearing the counters failed: %s", cudaGetErrorString(e));
            return -2;
        }
    }
    switch (head_dim) {
        case 64: return launch_decode<64>(q, q_stride, out, out_stride, cache, num_pages, page_size, block_table, table_stride, seq_lens, num_requests, nq, nkv, scale, window, splits, part_o, part_ml, counters, stream);
        case 128: return launch_decode<128>(q, q_stride, out, out_stride, cache, num_pages, page_size, block_table, table_stride, seq_lens, num_requests, nq, nkv, scale, window, splits, part_o, part_ml, counters, stream);
        case 256: return launch_decode<256>(q, q_stride, out, out_stride, cache, num_pages, page_size, block_table, table_stride, seq_lens, num_requests, nq, nkv, scale, window, splits, part_o, part_ml, counters, stream);
    }
    return -1;
}
