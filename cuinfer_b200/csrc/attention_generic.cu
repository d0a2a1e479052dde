// Paged causal attention, the plain all-sizes kernel: one warp per (query token, query head), keys
// and values read from cache pages through the request's block table.
//
// Reference counterpart: csrc/ops/paged_attention.cu:133-383 (one kernel for prompt portions and
// decoded tokens; queries are the last n positions of seq_len, keys 0..seq_len-1 come from pages;
// scale 1/sqrt(d); causal mask; online softmax in 32 bits).  This kernel is the 32-bit path and the
// fallback for head sizes the tensor-core kernels do not take: any head_dim up to 256, any head
// counts, any page size, an optional window.  Scores, softmax and the weighted sum are 32-bit with
// the exact exponential; the weights are not rounded before they multiply the values.
//
// Cache layout of one layer: [page][0 = keys, 1 = values][kv head][slot in page][d].
#include "common.cuh"

namespace cib {

constexpr int kAttnWarps = 4;
constexpr int kMaxHeadDim = 256;

template <typename T>
__global__ void paged_attention_generic_kernel(
    const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride, const T* __restrict__ cache,
    int num_pages, int page_size, const int* __restrict__ block_table, int table_stride,
    const int* __restrict__ query_start_loc, const int* __restrict__ seq_lens,
    const int* __restrict__ token_request, int nq, int nkv, int d, float scale, int window) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int head = blockIdx.y * kAttnWarps + warp;
    if (head >= nq) return;
    const int kvh = head / (nq / nkv);
    float* qs = smem + warp * d;

    const int r = token_request[t];
    const int q0 = query_start_loc[r];
    const int n = query_start_loc[r + 1] - q0;
    const int pos = seq_lens[r] - n + (t - q0);          // absolute position of this query
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* table = block_table + (size_t)r * table_stride;

    const T* qp = q + (size_t)t * q_stride + (size_t)head * d;
    for (int i = lane; i < d; i += 32) qs[i] = to_f32(qp[i]) * scale;
    __syncwarp();

    constexpr int kAcc = kMaxHeadDim / 32;
    float acc[kAcc];
#pragma unroll
    for (int k = 0; k < kAcc; ++k) acc[k] = 0.f;
    float m = -INFINITY, l = 0.f;
    const size_t head_stride = (size_t)page_size * d;

    for (int c = lo; c <= pos; c += 32) {
        const int j = c + lane;
        const bool valid = j <= pos;
        int page = -1, off = 0;
        float s = -INFINITY;
        if (valid) {
            page = table[j / page_size];
            off = j % page_size;
            if (page >= 0 && page < num_pages) {
                const T* kp = cache + (((size_t)page * 2 + 0) * nkv + kvh) * head_stride + (size_t)off * d;
                float dot = 0.f;
                for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_f32(kp[i]), dot);
                s = dot;
            } else {
                page = -1;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;              // no readable key in this chunk
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int k = 0; k < kAcc; ++k) acc[k] *= corr;
        const int count = min(32, pos - c + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int pg = __shfl_sync(0xffffffffu, page, jj);
            const int of = __shfl_sync(0xffffffffu, off, jj);
            if (pg < 0) continue;
            const T* vp = cache + (((size_t)pg * 2 + 1) * nkv + kvh) * head_stride + (size_t)of * d;
#pragma unroll
            for (int k = 0; k < kAcc; ++k) {
                const int i = lane + 32 * k;
                if (i < d) acc[k] = fmaf(pj, to_f32(vp[i]), acc[k]);
            }
        }
    }
    T* op = out + (size_t)t * out_stride + (size_t)head * d;
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int k = 0; k < kAcc; ++k) {
        const int i = lane + 32 * k;
        if (i < d) op[i] = from_f32<T>(acc[k] * inv);
    }
}

}  // namespace cib

using namespace cib;

extern "C" int cib_paged_attention_generic(const void* q, int dtype, int q_stride, void* out, int out_stride,
                                           const void* cache, int num_pages, int page_size,
                                           const int* block_table, int table_stride,
                                           const int* query_start_loc, const int* seq_lens,
                                           const int* token_request, int num_tokens, int nq, int nkv, int d,
                                           float scale, int window, cudaStream_t stream) {
    CIB_REQUIRE(num_tokens >= 0 && nq > 0 && nkv > 0 && d > 0 && nq % nkv == 0,
                "paged_attention: bad sizes T=%d nq=%d nkv=%d d=%d", num_tokens, nq, nkv, d);
    CIB_REQUIRE(d <= kMaxHeadDim, "paged_attention: head_dim %d exceeds %d", d, kMaxHeadDim);
    CIB_REQUIRE(page_size > 0 && num_pages > 0 && table_stride > 0, "paged_attention: bad cache geometry");
    CIB_REQUIRE(window >= 0, "paged_attention: window must be >= 0 (0 = all keys)");
    if (num_tokens == 0) return 0;
    dim3 grid(num_tokens, (nq + kAttnWarps - 1) / kAttnWarps);
    const size_t smem = (size_t)kAttnWarps * d * sizeof(float);
    if (dtype == kF32) {
        paged_attention_generic_kernel<float><<<grid, kAttnWarps * 32, smem, stream>>>(
            (const float*)q, q_stride, (float*)out, out_stride, (const float*)cache, num_pages, page_size,
            block_table, table_stride, query_start_loc, seq_lens, token_request, nq, nkv, d, scale, window);
    } else if (dtype == kBF16) {
        paged_attention_generic_kernel<__nv_bfloat16><<<grid, kAttnWarps * 32, smem, stream>>>(
            (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)cache,
            num_pages, page_size, block_table, table_stride, query_start_loc, seq_lens, token_request, nq, nkv,
            d, scale, window);
    } else {
        CIB_REQUIRE(false, "paged_attention: unsupported dtype %d", dtype);
    }
    CIB_LAUNCH_CHECK("paged_attention_generic");
    return 0;
}
