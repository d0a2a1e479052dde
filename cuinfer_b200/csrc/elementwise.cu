// Row-wise kernels around the matrix products: embedding gather, residual-add + RMSNorm,
// gather of the rows whose logits are wanted, and the SiLU-gated product.
//
// Reference counterparts: csrc/ops/embedding.cu:18-36, csrc/ops/rms_norm.cu:18-73,
// csrc/ops/residual_rms_norm_fused.cu:26-110, csrc/ops/residual_add.cu:23-82, csrc/ops/swiglu.cu:34-60.
// Unlike those, every size is a run-time parameter, the residual stream is kept in 32 bits, and the
// add, the norm and the store of the new residual are one pass over the row.
#include "common.cuh"
#include "mma_utils.cuh"

namespace cib {

template <typename T, int V> struct Vec;
template <> struct Vec<float, 4> {
    static __device__ __forceinline__ void load(const float* p, float* v) {
        float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* v) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec<__nv_bfloat16, 4> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
        uint2 t = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
        __nv_bfloat162 b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 t;
        t.x = *reinterpret_cast<uint32_t*>(&a);
        t.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = t;
    }
};
template <typename T> struct Vec<T, 1> {
    static __device__ __forceinline__ void load(const T* p, float* v) { v[0] = to_f32(*p); }
    static __device__ __forceinline__ void store(T* p, const float* v) { *p = from_f32<T>(v[0]); }
};

// ---- embedding ---------------------------------------------------------------------------------
// out[t, :] = table[ids[t], :] as 32-bit residual rows; an id outside the table gives a zero row
// and raises the flag (the host rejects such ids before they get here).
template <typename T, int V>
__global__ void embedding_gather_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                        float* __restrict__ out, int hidden, int vocab,
                                        int* __restrict__ bad_flag) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0 && bad_flag) atomicExch(bad_flag, 1);
    const T* src = table + (size_t)(ok ? id : 0) * hidden;
    float* dst = out + (size_t)t * hidden;
    for (int i = threadIdx.x * V; i < hidden; i += blockDim.x * V) {
        float v[V];
        Vec<T, V>::load(src + i, v);
        if (!ok) {
#pragma unroll
            for (int k = 0; k < V; ++k) v[k] = 0.f;
        }
        Vec<float, V>::store(dst + i, v);
    }
}

// ---- residual add + RMSNorm ---------------------------------------------------------------------
// x = residual (+ delta); residual = x (when a delta is given); out = x * rsqrt(mean(x^2) + eps) * w.
// Squares, mean, rsqrt and the product are 32-bit; the output is rounded once.
template <typename TD, typename TO, int V>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                   AnyVec weight, float eps, TO* __restrict__ out, int hidden) {
    __shared__ float scratch[33];
    const size_t row = (size_t)blockIdx.x * hidden;
    float* res = residual + row;
    float ss = 0.f;
    for (int i = threadIdx.x * V; i < hidden; i += blockDim.x * V) {
        float x[V];
        Vec<float, V>::load(res + i, x);
        if (delta) {
            float d[V];
            Vec<TD, V>::load(delta + row + i, d);
#pragma unroll
            for (int k = 0; k < V; ++k) x[k] += d[k];
            Vec<float, V>::store(res + i, x);
        }
#pragma unroll
        for (int k = 0; k < V; ++k) ss += x[k] * x[k];
    }
    ss = block_sum(ss, scratch);
    const float factor = rsqrtf(ss / (float)hidden + eps);
    if (!out) return;
    for (int i = threadIdx.x * V; i < hidden; i += blockDim.x * V) {
        float x[V];
        Vec<float, V>::load(res + i, x);   // this thread wrote exactly these elements above
#pragma unroll
        for (int k = 0; k < V; ++k) x[k] = x[k] * factor * weight[i + k];
        Vec<TO, V>::store(out + row + i, x);
    }
}

// Many rows (prompt portions): a warp per row, the whole row in registers (CH chunks of four values per lane), every
// load issued before the first use, one shuffle reduction, no second read of the residual.  Same arithmetic and the
// same order of operations per element as the kernel above; only the order of the sum of squares differs.
template <typename TD, typename TO, int CH>
__global__ void __launch_bounds__(256)
add_rmsnorm_rows_kernel(float* __restrict__ residual, const TD* __restrict__ delta, AnyVec weight, float eps,
                        TO* __restrict__ out, int hidden, int rows) {
    // the gains do not come from the kernel before this one: they are in shared memory before the dependency wait,
    // instead of a trip to the L2 after the reduction
    __shared__ __align__(16) float s_gain[CH * 128];
    griddep_launch();
    if (out)
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) s_gain[i] = weight[i];
    griddep_wait();          // residual and delta come from the kernels before this one
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const size_t row = (size_t)r * hidden;
    float x[CH][4], d[CH][4];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int i = (c * 32 + lane) * 4;
        if (i < hidden) Vec<float, 4>::load(residual + row + i, x[c]);
    }
    if (delta) {
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const int i = (c * 32 + lane) * 4;
            if (i < hidden) Vec<TD, 4>::load(delta + row + i, d[c]);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int i = (c * 32 + lane) * 4;
        if (i < hidden) {
            if (delta) {
#pragma unroll
                for (int k = 0; k < 4; ++k) x[c][k] += d[c][k];
                Vec<float, 4>::store(residual + row + i, x[c]);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) ss += x[c][k] * x[c][k];
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!out) return;
    const float factor = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int i = (c * 32 + lane) * 4;
        if (i < hidden) {
            float y[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) y[k] = x[c][k] * factor * s_gain[i + k];
            Vec<TO, 4>::store(out + row + i, y);
        }
    }
}

// ---- gather of wanted rows ------------------------------------------------------------------------
// out[s, :] = residual[idx[s], :] (+ delta[idx[s], :]) in 32 bits.
template <typename TD>
__global__ void gather_rows_kernel(const float* __restrict__ residual, const TD* __restrict__ delta,
                                   const int* __restrict__ idx, float* __restrict__ out, int hidden,
                                   int num_rows) {
    const int s = blockIdx.x;
    int r = idx[s];
    if (r < 0 || r >= num_rows) r = 0;
    const size_t src = (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = residual[src + i];
        if (delta) v += to_f32(delta[src + i]);
        out[(size_t)s * hidden + i] = v;
    }
}

// ---- SiLU-gated product ---------------------------------------------------------------------------
// act[t, j] = silu(gate_up[t, j]) * gate_up[t, I + j], silu(g) = g / (1 + exp(-g)), in 32 bits with the
// exact exponential.
template <typename T, int V>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ act, int inter, int rows) {
    const int per_row = inter / V;
    const size_t total = (size_t)rows * per_row;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / per_row;
        const int j = (int)(e % per_row) * V;
        float g[V], u[V];
        Vec<T, V>::load(gate_up + t * 2 * inter + j, g);
        Vec<T, V>::load(gate_up + t * 2 * inter + inter + j, u);
#pragma unroll
        for (int k = 0; k < V; ++k) g[k] = g[k] / (1.f + expf(-g[k])) * u[k];
        Vec<T, V>::store(act + t * inter + j, g);
    }
}

}  // namespace cib

using namespace cib;

static inline int norm_threads(int hidden, int vec) {
    int per = (hidden + vec - 1) / vec;
    int t = 32;
    while (t < per && t < 1024) t <<= 1;
    return t;
}

extern "C" int cib_embedding_gather(const int* ids, const void* table, int table_dtype, float* out,
                                    int num_tokens, int hidden, int vocab, int* bad_flag,
                                    cudaStream_t stream) {
    CIB_REQUIRE(num_tokens >= 0 && hidden > 0 && vocab > 0, "embedding_gather: bad sizes T=%d H=%d V=%d",
                num_tokens, hidden, vocab);
    if (num_tokens == 0) return 0;
    const bool v4 = hidden % 4 == 0;
    const int threads = norm_threads(hidden, v4 ? 4 : 1) > 256 ? 256 : norm_threads(hidden, v4 ? 4 : 1);
    if (table_dtype == kF32) {
        if (v4) embedding_gather_kernel<float, 4><<<num_tokens, threads, 0, stream>>>(ids, (const float*)table, out, hidden, vocab, bad_flag);
        else embedding_gather_kernel<float, 1><<<num_tokens, threads, 0, stream>>>(ids, (const float*)table, out, hidden, vocab, bad_flag);
    } else if (table_dtype == kBF16) {
        if (v4) embedding_gather_kernel<__nv_bfloat16, 4><<<num_tokens, threads, 0, stream>>>(ids, (const __nv_bfloat16*)table, out, hidden, vocab, bad_flag);
        else embedding_gather_kernel<__nv_bfloat16, 1><<<num_tokens, threads, 0, stream>>>(ids, (const __nv_bfloat16*)table, out, hidden, vocab, bad_flag);
    } else {
        CIB_REQUIRE(false, "embedding_gather: unsupported table dtype %d", table_dtype);
    }
    CIB_LAUNCH_CHECK("embedding_gather");
    return 0;
}

template <typename TD, typename TO>
static void launch_add_rmsnorm(float* residual, const void* delta, AnyVec w, float eps, void* out, int rows,
                               int hidden, cudaStream_t stream) {
    // from 256 rows on and up to 2048 values a row: a warp per row
    if (hidden % 4 == 0 && rows >= 256 && hidden <= 2048) {
        const int ch = (hidden + 127) / 128;
        const dim3 grid((rows + 7) / 8);
        const bool pdl = prompt_pdl();
        if (ch <= 4) launch_pdl(add_rmsnorm_rows_kernel<TD, TO, 4>, dim3(grid), dim3(256), 0, stream, pdl, residual, (const TD*)delta, w, eps, (TO*)out, hidden, rows);
        else if (ch <= 8) launch_pdl(add_rmsnorm_rows_kernel<TD, TO, 8>, dim3(grid), dim3(256), 0, stream, pdl, residual, (const TD*)delta, w, eps, (TO*)out, hidden, rows);
        else launch_pdl(add_rmsnorm_rows_kernel<TD, TO, 16>, dim3(grid), dim3(256), 0, stream, pdl, residual, (const TD*)delta, w, eps, (TO*)out, hidden, rows);
    } else if (hidden % 4 == 0) {
        add_rmsnorm_kernel<TD, TO, 4><<<rows, norm_threads(hidden, 4), 0, stream>>>(residual, (const TD*)delta, w, eps, (TO*)out, hidden);
    } else {
        add_rmsnorm_kernel<TD, TO, 1><<<rows, norm_threads(hidden, 1), 0, stream>>>(residual, (const TD*)delta, w, eps, (TO*)out, hidden);
    }
}

// delta may be null (plain norm of the residual rows); out may be null (add only).
extern "C" int cib_add_rmsnorm(float* residual, const void* delta, int delta_dtype, const void* weight,
                               int weight_dtype, float eps, void* out, int out_dtype, int rows, int hidden,
                               cudaStream_t stream) {
    CIB_REQUIRE(rows >= 0 && hidden > 0, "add_rmsnorm: bad sizes rows=%d hidden=%d", rows, hidden);
    CIB_REQUIRE(out == nullptr || weight != nullptr, "add_rmsnorm: a norm needs its weight");
    if (rows == 0) return 0;
    AnyVec w{weight, weight_dtype == kBF16};
    const int dd = delta ? delta_dtype : kF32;
    if (dd == kF32 && out_dtype == kF32) launch_add_rmsnorm<float, float>(residual, delta, w, eps, out, rows, hidden, stream);
    else if (dd == kF32 && out_dtype == kBF16) launch_add_rmsnorm<float, __nv_bfloat16>(residual, delta, w, eps, out, rows, hidden, stream);
    else if (dd == kBF16 && out_dtype == kF32) launch_add_rmsnorm<__nv_bfloat16, float>(residual, delta, w, eps, out, rows, hidden, stream);
    else if (dd == kBF16 && out_dtype == kBF16) launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(residual, delta, w, eps, out, rows, hidden, stream);
    else CIB_REQUIRE(false, "add_rmsnorm: unsupported dtypes delta=%d out=%d", delta_dtype, out_dtype);
    CIB_LAUNCH_CHECK("add_rmsnorm");
    return 0;
}

extern "C" int cib_gather_rows(const float* residual, const void* delta, int delta_dtype, const int* idx,
                               float* out, int num_out, int hidden, int num_rows, cudaStream_t stream) {
    CIB_REQUIRE(num_out >= 0 && hidden > 0, "gather_rows: bad sizes");
    if (num_out == 0) return 0;
    const int threads = hidden >= 256 ? 256 : 64;
    if (!delta || delta_dtype == kF32) gather_rows_kernel<float><<<num_out, threads, 0, stream>>>(residual, (const float*)delta, idx, out, hidden, num_rows);
    else if (delta_dtype == kBF16) gather_rows_kernel<__nv_bfloat16><<<num_out, threads, 0, stream>>>(residual, (const __nv_bfloat16*)delta, idx, out, hidden, num_rows);
    else CIB_REQUIRE(false, "gather_rows: unsupported delta dtype %d", delta_dtype);
    CIB_LAUNCH_CHECK("gather_rows");
    return 0;
}

extern "C" int cib_silu_mul(const void* gate_up, void* act, int dtype, int rows, int inter, cudaStream_t stream) {
    CIB_REQUIRE(rows >= 0 && inter > 0, "silu_mul: bad sizes rows=%d I=%d", rows, inter);
    if (rows == 0) return 0;
    const bool v4 = inter % 4 == 0;
    const size_t total = (size_t)rows * (inter / (v4 ? 4 : 1));
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == kF32) {
        if (v4) silu_mul_kernel<float, 4><<<blocks, 256, 0, stream>>>((const float*)gate_up, (float*)act, inter, rows);
        else silu_mul_kernel<float, 1><<<blocks, 256, 0, stream>>>((const float*)gate_up, (float*)act, inter, rows);
    } else if (dtype == kBF16) {
        if (v4) silu_mul_kernel<__nv_bfloat16, 4><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)act, inter, rows);
        else silu_mul_kernel<__nv_bfloat16, 1><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)act, inter, rows);
    } else {
        CIB_REQUIRE(false, "silu_mul: unsupported dtype %d", dtype);
    }
    CIB_LAUNCH_CHECK("silu_mul");
    return 0;
}
