// out[M, N] = a[M, K] · w[N, K]^T on the ordinary 32-bit FMA pipe, for any M, N, K.
//
// The reference sends every projection to cuBLAS with 32-bit accumulation
// (csrc/ops/projection.cu:13-45).  This kernel is the true 32-bit path (no tensor cores, no reduced
// precision mode) and the fallback for shapes the tensor-core kernels refuse.  Every output element
// is one fused-multiply-add chain over k = 0..K-1 in that order, so a row's result does not depend on
// how many other rows are in the batch.
#include "common.cuh"

namespace cib {

constexpr int kBM = 64, kBN = 64, kBK = 16;

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gemm_generic_kernel(const TI* __restrict__ a, int lda, const TI* __restrict__ w, int ldw,
                    TO* __restrict__ out, int ldo, int M, int N, int K) {
    __shared__ float As[kBK][kBM + 4];
    __shared__ float Ws[kBK][kBN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * kBM, n0 = blockIdx.x * kBN;
    const int tx = tid & 15, ty = tid >> 4;       // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    // each thread loads 4 elements of each tile per step: row = tid / 4, k = (tid % 4) * 4 ..
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += kBK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            const int am = m0 + lrow, wn = n0 + lrow;
            As[lk + e][lrow] = (am < M && k < K) ? to_f32(a[(size_t)am * lda + k]) : 0.f;
            Ws[lk + e][lrow] = (wn < N && k < K) ? to_f32(w[(size_t)wn * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kBK; ++kk) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) out[(size_t)m * ldo + n] = from_f32<TO>(acc[i][j]);
        }
    }
}

}  // namespace cib

using namespace cib;

extern "C" int cib_gemm_generic(const void* a, int lda, const void* w, int ldw, int in_dtype, void* out, int ldo,
                                int out_dtype, int M, int N, int K, cudaStream_t stream) {
    CIB_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    CIB_REQUIRE(lda >= K && ldw >= K && ldo >= N, "gemm: leading dimensions too small (lda=%d ldw=%d ldo=%d)", lda, ldw, ldo);
    if (M == 0) return 0;
    dim3 grid((N + kBN - 1) / kBN, (M + kBM - 1) / kBM);
    CIB_REQUIRE(grid.y <= 65535, "gemm: M=%d too large for this kernel", M);
    if (in_dtype == kF32 && out_dtype == kF32)
        gemm_generic_kernel<float, float><<<grid, 256, 0, stream>>>((const float*)a, lda, (const float*)w, ldw, (float*)out, ldo, M, N, K);
    else if (in_dtype == kBF16 && out_dtype == kBF16)
        gemm_generic_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)w, ldw, (__nv_bfloat16*)out, ldo, M, N, K);
    else if (in_dtype == kBF16 && out_dtype == kF32)
        gemm_generic_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)w, ldw, (float*)out, ldo, M, N, K);
    else
        CIB_REQUIRE(false, "gemm: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
    CIB_LAUNCH_CHECK("gemm_generic");
    return 0;
}
