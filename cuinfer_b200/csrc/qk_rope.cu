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
    if (dtype == kF32) {
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
