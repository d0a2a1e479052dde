// Per-head RMSNorm of queries and keys, rotary position encoding, and the write of keys and values
// into their cache pages, in one pass over the packed qkv rows.
//
// Reference counterparts: csrc/ops/qk_norm_rope_fused.cu:47-142 (norm + rotate-half RoPE over the
// whole head, one warp per head) and csrc/ops/unified_kv_cache_update.cu:20-49 (copy of K and V to
// cache[slot]).  Differences: every size is a run-time parameter (any head_dim, any head counts, a
// rotary width up to the head), the norm and the encoding are optional, the normed value is not
// rounded before it is rotated, and keys/values go straight to their page without passing through
// the qkv row again.
//
// Row layout: [num_q_heads * d | num_kv_heads * d (keys) | num_kv_heads * d (values)].
// Cache layout of one layer: [page][0 = keys, 1 = values][kv head][slot in page][d].
#include "mma_utils.cuh"

namespace cib {

constexpr int kRopeWarps = 4;

template <typename T>
__global__ void qk_norm_rope_kv_write_kernel(T* __restrict__ qkv, int row_stride,
                                             const int* __restrict__ positions,
                                             const int* __restrict__ slot_mapping, AnyVec q_weight,
                                             AnyVec k_weight, int has_norm, float eps,
                                             const float* __restrict__ rope_table, int rotary_dim,
                                             int max_positions, T* __restrict__ cache, int num_pages,
                                             int page_size, int nq, int nkv, int d, int write_cache) {
    extern __shared__ float smem[];
    griddep_launch();
    griddep_wait();          // the rows come from the projection before this kernel
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int head = blockIdx.y * kRopeWarps + warp;
    const int total_heads = write_cache ? nq + 2 * nkv : nq;
    if (head >= total_heads) return;
    float* sv = smem + warp * d;
    T* src = qkv + (size_t)t * row_stride + (size_t)head * d;

    const bool is_q = head < nq;
    const bool is_k = !is_q && head < nq + nkv;
    const int kvh = is_q ? 0 : (is_k ? head - nq : head - nq - nkv);

    T* dst = nullptr;   // where the finished head goes
    if (is_q) {
        dst = src;
    } else {
        const int slot = slot_mapping[t];
        if (slot < 0) return;
        const int page = slot / page_size, off = slot - page * page_size;
        if (page >= num_pages) return;
        dst = cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * nkv + kvh) * page_size + off) * d;
    }

    if (!is_q && !is_k) {   // values: plain copy
        for (int i = lane; i < d; i += 32) dst[i] = src[i];
        return;
    }

    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
        const float x = to_f32(src[i]);
        sv[i] = x;
        ss += x * x;
    }
    if (has_norm) {
        ss = warp_sum(ss);
        const float factor = rsqrtf(ss / (float)d + eps);
        const AnyVec& w = is_q ? q_weight : k_weight;
        for (int i = lane; i < d; i += 32) sv[i] = sv[i] * factor * w[i];
    }
    __syncwarp();
    const int half = rotary_dim >> 1;
    if (half > 0) {
        int pos = positions[t];
        pos = pos < 0 ? 0 : (pos >= max_positions ? max_positions - 1 : pos);
        const float* tab = rope_table + (size_t)pos * half * 2;
        for (int i = lane; i < half; i += 32) {
            const float c = tab[2 * i], s = tab[2 * i + 1];
            const float a = sv[i], b = sv[i + half];
            dst[i] = from_f32<T>(a * c - b * s);
            dst[i + half] = from_f32<T>(b * c + a * s);
        }
    }
    for (int i = rotary_dim + lane; i < d; i += 32) dst[i] = from_f32<T>(sv[i]);
}

// The common case — the encoding spans the whole head (or is absent) and the head size is a multiple of 32 —
// without loops: a lane owns E = d / 32 neighbouring values, every load is issued before anything is used (one
// memory latency per head instead of one per pass), the partner of a rotation pair sits 16 lanes away.
template <typename T, int E>
struct alignas(sizeof(T) * E > 16 ? 16 : sizeof(T) * E) LaneValues {
    T v[E];
};

template <typename T, int E>
__global__ void qk_norm_rope_kv_write_fast_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                                                  const int* __restrict__ slot_mapping, AnyVec q_weight, AnyVec k_weight,
                                                  int has_norm, float eps, const float* __restrict__ rope_table,
                                                  int has_rope, int max_positions, T* __restrict__ cache, int num_pages,
                                                  int page_size, int nq, int nkv, int write_cache) {
    constexpr int D = E * 32;
    griddep_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int head = blockIdx.y * kRopeWarps + warp;
    const int total_heads = write_cache ? nq + 2 * nkv : nq;
    if (head >= total_heads) return;
    T* src = qkv + (size_t)t * row_stride + (size_t)head * D + lane * E;
    const bool is_q = head < nq;
    const bool is_k = !is_q && head < nq + nkv;
    const int kvh = is_q ? 0 : (is_k ? head - nq : head - nq - nkv);
    // What does not come from the kernel before this one (the slot, the position and its table row, the gains) is
    // fetched before `griddepcontrol.wait`: after it only the head's own values are a round trip away.
    T* dst = src;
    if (!is_q) {
        const int slot = slot_mapping[t];
        if (slot < 0) return;
        const int page = slot / page_size, off = slot - page * page_size;
        if (page >= num_pages) return;
        dst = cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * nkv + kvh) * page_size + off) * D + lane * E;
    }
    using Vec = LaneValues<T, E>;
    float x[E], wv[E], cs[2 * E];
    const bool is_v = !is_q && !is_k;
    const AnyVec& w = is_q ? q_weight : k_weight;
    if (has_norm && !is_v) {
#pragma unroll
        for (int e = 0; e < E; ++e) wv[e] = w[lane * E + e];
    }
    if (has_rope && !is_v) {
        int pos = positions[t];
        pos = pos < 0 ? 0 : (pos >= max_positions ? max_positions - 1 : pos);
        const float* tp = rope_table + (size_t)pos * D + 2 * ((lane & 15) * E);
        if constexpr (E % 2 == 0) {
#pragma unroll
            for (int e = 0; e < E / 2; ++e) {
                const float4 v = reinterpret_cast<const float4*>(tp)[e];
                cs[4 * e] = v.x, cs[4 * e + 1] = v.y, cs[4 * e + 2] = v.z, cs[4 * e + 3] = v.w;
            }
        } else {
            const float2 v = *reinterpret_cast<const float2*>(tp);
            cs[0] = v.x, cs[1] = v.y;
        }
    }
    griddep_wait();
    const Vec rawv = *reinterpret_cast<const Vec*>(src);
    const T* raw = rawv.v;
    if (is_v) {
        *reinterpret_cast<Vec*>(dst) = rawv;
        return;
    }
#pragma unroll
    for (int e = 0; e < E; ++e) x[e] = to_f32(raw[e]);
    if (has_norm) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) ss += x[e] * x[e];
        ss = warp_sum(ss);
        const float factor = rsqrtf(ss / (float)D + eps);
#pragma unroll
        for (int e = 0; e < E; ++e) x[e] = x[e] * factor * wv[e];
    }
    if (has_rope) {
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, x[e], 16);
            const float c = cs[2 * e], sn = cs[2 * e + 1];
            x[e] = lane < 16 ? x[e] * c - other * sn : x[e] * c + other * sn;
        }
    }
    Vec outv;
#pragma unroll
    for (int e = 0; e < E; ++e) outv.v[e] = from_f32<T>(x[e]);
    *reinterpret_cast<Vec*>(dst) = outv;
}

// The same for many tokens (prompt portions), where the kernel above is bound by its instruction count (a lane
// handles four values of a head).  Here a head is spread over L = d / 8 lanes; a lane holds four values of the
// first half of the head and their four rotation partners of the second half, so that the rotation needs no
// exchange; a warp takes up to 4 x (32 / L) heads of one token, issues all their loads first, and computes what
// depends on the token only (cache slot, table row, weights) once.
template <typename T>
struct alignas(sizeof(T) * 4) Four {
    T v[4];
};

constexpr int kBulkWarps = 8;
constexpr int kBulkPasses = 4;

template <typename T, int L>
__global__ void __launch_bounds__(kBulkWarps * 32, 4)
qk_norm_rope_kv_write_bulk_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                                  const int* __restrict__ slot_mapping, AnyVec q_weight, AnyVec k_weight, int has_norm,
                                  float eps, const float* __restrict__ rope_table, int has_rope, int max_positions,
                                  T* __restrict__ cache, int num_pages, int page_size, int nq, int nkv, int write_cache,
                                  int num_tokens) {
    constexpr int D = 8 * L, HPP = 32 / L;                    // heads per pass
    using Vec = Four<T>;
    __shared__ __align__(16) float s_w[2][D];                 // the norms' gains (weights: not written by the kernel before)
    if (has_norm)
        for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) s_w[i / D][i % D] = i < D ? q_weight[i] : k_weight[i - D];
    griddep_launch();
    griddep_wait();
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_heads = write_cache ? nq + 2 * nkv : nq;
    const int groups = (total_heads + HPP * kBulkPasses - 1) / (HPP * kBulkPasses);
    const int wg = blockIdx.x * kBulkWarps + warp;
    const int t = wg / groups;
    if (t >= num_tokens) return;
    const int head_base = (wg - t * groups) * HPP * kBulkPasses;
    const int sub = lane / L, li = lane % L;
    T* row = qkv + (size_t)t * row_stride;
    // this lane's eight values of each head: [4 li, 4 li + 4) and the same range of the second half
    Vec lo[kBulkPasses], hi[kBulkPasses];
#pragma unroll
    for (int p = 0; p < kBulkPasses; ++p) {
        const int head = head_base + p * HPP + sub;
        if (head < total_heads) {
            const T* src = row + (size_t)head * D + 4 * li;
            lo[p] = *reinterpret_cast<const Vec*>(src);
            hi[p] = *reinterpret_cast<const Vec*>(src + D / 2);
        }
    }
    // what depends on the token only
    T* cache_row = nullptr;                                   // slot `off` of kv head 0 of the key half of the page
    if (write_cache) {
        const int slot = slot_mapping[t];
        if (slot >= 0) {
            const int page = slot / page_size, off = slot - page * page_size;
            if (page < num_pages) cache_row = cache + ((size_t)page * 2 * nkv * page_size + off) * D;
        }
    }
    float cs[8];
    if (has_rope) {
        int pos = positions[t];
        pos = pos < 0 ? 0 : (pos >= max_positions ? max_positions - 1 : pos);
        const float4* tp = reinterpret_cast<const float4*>(rope_table + (size_t)pos * D + 8 * li);
        const float4 a = tp[0], b = tp[1];
        cs[0] = a.x, cs[1] = a.y, cs[2] = a.z, cs[3] = a.w, cs[4] = b.x, cs[5] = b.y, cs[6] = b.z, cs[7] = b.w;
    }
#pragma unroll
    for (int p = 0; p < kBulkPasses; ++p) {
        const int head = head_base + p * HPP + sub;
        const bool live = head < total_heads;
        const int kind = head < nq ? 0 : (head < nq + nkv ? 1 : 2);          // query, key, value
        T* dst = row + (size_t)head * D + 4 * li;
        if (kind != 0) {
            const int kvh = kind == 1 ? head - nq : head - nq - nkv;
            dst = cache_row == nullptr ? nullptr : cache_row + ((size_t)(kind - 1) * nkv + kvh) * page_size * D + 4 * li;
        }
        float x[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) x[e] = live ? to_f32(lo[p].v[e]) : 0.f, x[4 + e] = live ? to_f32(hi[p].v[e]) : 0.f;
        if (kind != 2) {
            if (has_norm) {                                   // every lane takes part in the shuffles
                float ss = 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
#pragma unroll
                for (int o = L / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                const float factor = rsqrtf(ss / (float)D + eps);
                const float4 wa = *reinterpret_cast<const float4*>(&s_w[kind][4 * li]);
                const float4 wb = *reinterpret_cast<const float4*>(&s_w[kind][D / 2 + 4 * li]);
                const float w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = x[e] * factor * w[e];
            }
            if (has_rope) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float c = cs[2 * e], sn = cs[2 * e + 1], x1 = x[e], x2 = x[4 + e];
                    x[e] = x1 * c - x2 * sn;
                    x[4 + e] = x2 * c + x1 * sn;
                }
            }
        }
        if (live && dst != nullptr) {
            Vec a, b;
            if (kind == 2) {
                a = lo[p], b = hi[p];
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) a.v[e] = from_f32<T>(x[e]), b.v[e] = from_f32<T>(x[4 + e]);
            }
            *reinterpret_cast<Vec*>(dst) = a;
            *reinterpret_cast<Vec*>(dst + D / 2) = b;
        }
    }
}

// bfloat16 rows of many tokens, staged.  The kernel above keeps a warp's rows in registers: 2 KB in flight per warp,
// 48-64 KB per SM, which at the latency seen moves a third of the memory bandwidth (14.7 us for the 34 MB of 2 048
// tokens x 32 heads; wider loads and an earlier table fetch changed nothing).  Here a warp asks for kStageHeads
// consecutive heads of one token (4 KB at d = 128) with `cp.async` into shared memory, all at once, and holds in
// registers only the pass it works on: 32 KB in flight per block, four blocks to an SM (10.7 us; 30 against 45 us at
// 8 192 tokens).  L = d / 16 lanes per head, eight values of the first half and their eight rotation partners per
// lane; what depends on the token only is fetched before the dependency wait.
constexpr int kStageHeads = 16;

template <int L>
__global__ void __launch_bounds__(kBulkWarps * 32, 4)
qk_norm_rope_kv_write_staged_kernel(__nv_bfloat16* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                                    const int* __restrict__ slot_mapping, AnyVec q_weight, AnyVec k_weight, int has_norm,
                                    float eps, const float* __restrict__ rope_table, int has_rope, int max_positions,
                                    __nv_bfloat16* __restrict__ cache, int num_pages, int page_size, int nq, int nkv,
                                    int write_cache, int num_tokens) {
    using T = __nv_bfloat16;
    constexpr int D = 16 * L, HPP = 32 / L, PASSES = kStageHeads / HPP, PER_HEAD = D / 8;      // 16-byte pieces per head
    extern __shared__ __align__(16) unsigned char staged_raw[];
    uint4* slab = reinterpret_cast<uint4*>(staged_raw) + (size_t)(threadIdx.x >> 5) * kStageHeads * PER_HEAD;
    __shared__ __align__(16) float s_w[2][D];                 // the norms' gains (weights: not written by the kernel before)
    if (has_norm)
        for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) s_w[i / D][i % D] = i < D ? q_weight[i] : k_weight[i - D];
    griddep_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_heads = write_cache ? nq + 2 * nkv : nq;
    const int groups = (total_heads + kStageHeads - 1) / kStageHeads;
    const int wg = blockIdx.x * kBulkWarps + warp;
    const bool mine = wg / groups < num_tokens;
    const int t = mine ? wg / groups : 0;
    const int head_base = (wg % groups) * kStageHeads;
    const int sub = lane / L, li = lane % L;
    const unsigned group_mask = L == 32 ? 0xffffffffu : ((1u << L) - 1u) << (sub * L);     // the lanes of this lane's head
    T* row = qkv + (size_t)t * row_stride;
    // what depends on the token only does not come from the kernel before this one: fetched before `griddepcontrol.wait`
    T* cache_row = nullptr;                                   // slot `off` of kv head 0 of the key half of the page
    if (write_cache) {
        const int slot = slot_mapping[t];
        if (slot >= 0) {
            const int page = slot / page_size, off = slot - page * page_size;
            if (page < num_pages) cache_row = cache + ((size_t)page * 2 * nkv * page_size + off) * D;
        }
    }
    float cs[16];
    if (has_rope) {
        int pos = positions[t];
        pos = pos < 0 ? 0 : (pos >= max_positions ? max_positions - 1 : pos);
        const float4* tp = reinterpret_cast<const float4*>(rope_table + (size_t)pos * D + 16 * li);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float4 a = tp[e];
            cs[4 * e] = a.x, cs[4 * e + 1] = a.y, cs[4 * e + 2] = a.z, cs[4 * e + 3] = a.w;
        }
    }
    griddep_wait();
    __syncthreads();
    if (!mine) return;
    // the warp's heads are consecutive in the row: kStageHeads * PER_HEAD pieces of 16 bytes, lane after lane
    const int pieces = min(kStageHeads, total_heads - head_base) * PER_HEAD;
    const T* src0 = row + (size_t)head_base * D;
#pragma unroll
    for (int i = 0; i < kStageHeads * PER_HEAD / 32; ++i) {
        const int idx = i * 32 + lane;
        if (idx < pieces) cp_async16(&slab[idx], src0 + idx * 8, true);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncwarp();
#pragma unroll
    for (int p = 0; p < PASSES; ++p) {
        const int local = p * HPP + sub;
        const int head = head_base + local;
        if (head >= total_heads) continue;                    // the L lanes of a head go together; the shuffles below name only them
        const int kind = head < nq ? 0 : (head < nq + nkv ? 1 : 2);          // query, key, value
        T* dst = row + (size_t)head * D + 8 * li;
        if (kind != 0) {
            const int kvh = kind == 1 ? head - nq : head - nq - nkv;
            dst = cache_row == nullptr ? nullptr : cache_row + ((size_t)(kind - 1) * nkv + kvh) * page_size * D + 8 * li;
        }
        uint4 lo = slab[local * PER_HEAD + li], hi = slab[local * PER_HEAD + PER_HEAD / 2 + li];
        if (kind != 2) {
            const __nv_bfloat162* l2 = reinterpret_cast<const __nv_bfloat162*>(&lo);
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&hi);
            float x[16];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 a = __bfloat1622float2(l2[e]), b = __bfloat1622float2(h2[e]);
                x[2 * e] = a.x, x[2 * e + 1] = a.y, x[8 + 2 * e] = b.x, x[8 + 2 * e + 1] = b.y;
            }
            if (has_norm) {
                float ss = 0.f;
#pragma unroll
                for (int e = 0; e < 16; ++e) ss += x[e] * x[e];
#pragma unroll
                for (int o = L / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(group_mask, ss, o);
                const float factor = rsqrtf(ss / (float)D + eps);
#pragma unroll
                for (int e = 0; e < 8; e += 4) {
                    const float4 wa = *reinterpret_cast<const float4*>(&s_w[kind][8 * li + e]);
                    const float4 wb = *reinterpret_cast<const float4*>(&s_w[kind][D / 2 + 8 * li + e]);
                    x[e] = x[e] * factor * wa.x, x[e + 1] = x[e + 1] * factor * wa.y;
                    x[e + 2] = x[e + 2] * factor * wa.z, x[e + 3] = x[e + 3] * factor * wa.w;
                    x[8 + e] = x[8 + e] * factor * wb.x, x[8 + e + 1] = x[8 + e + 1] * factor * wb.y;
                    x[8 + e + 2] = x[8 + e + 2] * factor * wb.z, x[8 + e + 3] = x[8 + e + 3] * factor * wb.w;
                }
            }
            if (has_rope) {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float c = cs[2 * e], sn = cs[2 * e + 1], x1 = x[e], x2 = x[8 + e];
                    x[e] = x1 * c - x2 * sn;
                    x[8 + e] = x2 * c + x1 * sn;
                }
            }
            __nv_bfloat162* lo2 = reinterpret_cast<__nv_bfloat162*>(&lo);
            __nv_bfloat162* hi2 = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                lo2[e] = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
                hi2[e] = __floats2bfloat162_rn(x[8 + 2 * e], x[8 + 2 * e + 1]);
            }
        }
        if (dst != nullptr) {
            *reinterpret_cast<uint4*>(dst) = lo;
            *reinterpret_cast<uint4*>(dst + D / 2) = hi;
        }
    }
}

constexpr int kBulkTokens = 256;       // the many-token kernel from this many tokens on

template <typename T>
static cudaError_t launch_fast(int E, dim3 grid, cudaStream_t stream, bool use_pdl, T* qkv, int row_stride, const int* positions,
                               const int* slot_mapping, AnyVec qw, AnyVec kw, int has_norm, float eps, const float* rope_table,
                               int has_rope, int max_positions, T* cache, int num_pages, int page_size, int nq, int nkv,
                               int write_cache, int num_tokens) {
    if constexpr (sizeof(T) == 2) {
        const int d = E * 32;
        if (num_tokens >= kBulkTokens && d >= 64) {
            const int total_heads = write_cache ? nq + 2 * nkv : nq;
            const long long warps = (long long)num_tokens * ((total_heads + kStageHeads - 1) / kStageHeads);
            dim3 staged((unsigned)((warps + kBulkWarps - 1) / kBulkWarps));
            const size_t smem = (size_t)kBulkWarps * kStageHeads * d * 2;
#define CIB_ROPE_STAGED(LV)                                                                                                    \
    if (d == 16 * LV) {                                                                                                        \
        static SmemLimit limit;                                                                                                \
        if (raise_smem_limit(limit, qk_norm_rope_kv_write_staged_kernel<LV>, (int)smem, "qk_norm_rope") != 0)                  \
            return cudaErrorInvalidValue;                                                                                      \
        return launch_pdl(qk_norm_rope_kv_write_staged_kernel<LV>, staged, dim3(kBulkWarps * 32), smem, stream, use_pdl, qkv,  \
                          row_stride, positions, slot_mapping, qw, kw, has_norm, eps, rope_table, has_rope, max_positions,    \
                          cache, num_pages, page_size, nq, nkv, write_cache, num_tokens);                                      \
    }
            CIB_ROPE_STAGED(4)
            CIB_ROPE_STAGED(8)
            CIB_ROPE_STAGED(16)
#undef CIB_ROPE_STAGED
        }
    }
    if (num_tokens >= kBulkTokens && E * 32 >= 64) {
        const int L = E * 4;                                  // lanes per head: d / 8
        const int total_heads = write_cache ? nq + 2 * nkv : nq;
        const int per_warp = (32 / L) * kBulkPasses;
        const long long warps = (long long)num_tokens * ((total_heads + per_warp - 1) / per_warp);
        dim3 bulk((unsigned)((warps + kBulkWarps - 1) / kBulkWarps));
#define CIB_ROPE_BULK(LV)                                                                                                      \
    if (L == LV)                                                                                                               \
        return launch_pdl(qk_norm_rope_kv_write_bulk_kernel<T, LV>, bulk, dim3(kBulkWarps * 32), 0, stream, use_pdl, qkv,     \
                          row_stride, positions, slot_mapping, qw, kw, has_norm, eps, rope_table, has_rope, max_positions,    \
                          cache, num_pages, page_size, nq, nkv, write_cache, num_tokens);
        CIB_ROPE_BULK(8)
        CIB_ROPE_BULK(16)
        CIB_ROPE_BULK(32)
#undef CIB_ROPE_BULK
    }
#define CIB_ROPE_FAST(EV)                                                                                                   \
    if (E == EV)                                                                                                            \
        return launch_pdl(qk_norm_rope_kv_write_fast_kernel<T, EV>, grid, dim3(kRopeWarps * 32), 0, stream, use_pdl, qkv,   \
                          row_stride, positions, slot_mapping, qw, kw, has_norm, eps, rope_table, has_rope, max_positions, \
                          cache, num_pages, page_size, nq, nkv, write_cache);
    CIB_ROPE_FAST(1)
    CIB_ROPE_FAST(2)
    CIB_ROPE_FAST(4)
    CIB_ROPE_FAST(8)
#undef CIB_ROPE_FAST
    return cudaErrorInvalidValue;
}

}  // namespace cib

using namespace cib;

extern "C" int cib_qk_norm_rope_kv_write(void* qkv, int dtype, int row_stride, const int* positions,
                                         const int* slot_mapping, const void* q_weight,
                                         const void* k_weight, int weight_dtype, int has_norm, float eps,
                                         const float* rope_table, int rotary_dim, int max_positions,
                                         void* cache, int num_pages, int page_size, int num_tokens, int nq,
                                         int nkv, int d, int write_cache, int use_pdl, cudaStream_t stream) {
    CIB_REQUIRE(num_tokens >= 0 && nq > 0 && nkv > 0 && d > 0, "qk_norm_rope: bad sizes T=%d nq=%d nkv=%d d=%d",
                num_tokens, nq, nkv, d);
    CIB_REQUIRE(rotary_dim >= 0 && rotary_dim <= d && rotary_dim % 2 == 0,
                "qk_norm_rope: rotary_dim %d must be even and at most head_dim %d", rotary_dim, d);
    CIB_REQUIRE(rotary_dim == 0 || (rope_table != nullptr && max_positions > 0), "qk_norm_rope: rotary table missing");
    CIB_REQUIRE(!has_norm || (q_weight && k_weight), "qk_norm_rope: norm weights missing");
    CIB_REQUIRE(row_stride >= (nq + 2 * nkv) * d || (!write_cache && row_stride >= nq * d),
                "qk_norm_rope: row stride %d too small", row_stride);
    CIB_REQUIRE(!write_cache || (cache && page_size > 0 && num_pages > 0), "qk_norm_rope: cache missing");
    CIB_REQUIRE(d * kRopeWarps * 4 <= 48 * 1024, "qk_norm_rope: head_dim %d too large", d);
    if (num_tokens == 0) return 0;
    const int heads = write_cache ? nq + 2 * nkv : nq;
    dim3 grid(num_tokens, (heads + kRopeWarps - 1) / kRopeWarps);
    const size_t smem = (size_t)kRopeWarps * d * sizeof(float);
    AnyVec qw{q_weight, weight_dtype == kBF16}, kw{k_weight, weight_dtype == kBF16};
    cudaError_t e;
    const int per_lane = d / 32;
    const bool fast = d % 32 == 0 && (per_lane == 1 || per_lane == 2 || per_lane == 4 || per_lane == 8) &&
                      (rotary_dim == 0 || rotary_dim == d) && (size_t)qkv % 16 == 0 && (size_t)cache % 16 == 0 && (size_t)rope_table % 16 == 0 &&
                      ((size_t)row_stride * (dtype == kF32 ? 4 : 2)) % 16 == 0;
    if (fast && dtype == kF32) {
        e = launch_fast<float>(per_lane, grid, stream, use_pdl != 0, (float*)qkv, row_stride, positions, slot_mapping, qw, kw,
                               has_norm, eps, rope_table, rotary_dim > 0, max_positions, (float*)cache, num_pages, page_size, nq,
                               nkv, write_cache, num_tokens);
    } else if (fast && dtype == kBF16) {
        e = launch_fast<__nv_bfloat16>(per_lane, grid, stream, use_pdl != 0, (__nv_bfloat16*)qkv, row_stride, positions,
                                       slot_mapping, qw, kw, has_norm, eps, rope_table, rotary_dim > 0, max_positions,
                                       (__nv_bfloat16*)cache, num_pages, page_size, nq, nkv, write_cache, num_tokens);
    } else if (dtype == kF32) {
        e = launch_pdl(qk_norm_rope_kv_write_kernel<float>, grid, dim3(kRopeWarps * 32), smem, stream, use_pdl != 0,
                       (float*)qkv, row_stride, positions, slot_mapping, qw, kw, has_norm, eps, rope_table, rotary_dim,
                       max_positions, (float*)cache, num_pages, page_size, nq, nkv, d, write_cache);
    } else if (dtype == kBF16) {
        e = launch_pdl(qk_norm_rope_kv_write_kernel<__nv_bfloat16>, grid, dim3(kRopeWarps * 32), smem, stream, use_pdl != 0,
                       (__nv_bfloat16*)qkv, row_stride, positions, slot_mapping, qw, kw, has_norm, eps, rope_table,
                       rotary_dim, max_positions, (__nv_bfloat16*)cache, num_pages, page_size, nq, nkv, d, write_cache);
    } else {
        CIB_REQUIRE(false, "qk_norm_rope: unsupported dtype %d", dtype);
    }
    if (e != cudaSuccess) {
        set_error("qk_norm_rope_kv_write: launch failed: %s", cudaGetErrorString(e));
        return -2;
    }
    return 0;
}
