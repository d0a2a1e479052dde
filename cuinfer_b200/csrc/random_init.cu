// Seeded random weights written straight into device memory, without a file or a host copy.
//
// The reference has no random-weights mode (it only loads checkpoints, csrc/model/checkpoint.cpp:39-178); the
// benchmark's larger shapes (65 GB of weights) need one that does not pass through the host.  Element i of a tensor
// with key k is a function of (k, i) alone — a counter-based generator — so that any number of threads fills a
// tensor in any order, and the host can compute the very same values (cuinfer_b200/weights/random_init.py does, in
// numpy; a test compares them bit by bit).  Only integer sums and IEEE basic operations are used, no library
// function whose last bit could differ between the two sides:
//     four splitmix64 hashes of k + 4 i + j give twelve 21-bit integers u; their sum is approximately normal
//     (Irwin-Hall, variance exactly 12 * (2^42 - 1) / 12 / 2^42 of one after scaling);
//     z = (sum - (6 * 2^21 - 6)) / 2^21 in double, x = float(mean + std * z), then x * factor in float,
//     rounded to bfloat16 first if the tensor is stored in bfloat16.
#include "common.cuh"

namespace cib {

__host__ __device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__device__ __forceinline__ float counter_normal(unsigned long long key, unsigned long long i, double mean, double std,
                                                float factor, int via_bf16) {
    unsigned long long sum = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const unsigned long long h = splitmix64(key + 4ull * i + (unsigned long long)j);
        sum += (h & 0x1FFFFFull) + ((h >> 21) & 0x1FFFFFull) + ((h >> 42) & 0x1FFFFFull);
    }
    const double z = ((double)(long long)sum - 12582906.0) / 2097152.0;       // 6 * 2^21 - 6, 2^21
    float x = (float)__dadd_rn(mean, __dmul_rn(std, z));       // two roundings, as the host does: no fused multiply-add
    x = x * factor;
    if (via_bf16) x = __bfloat162float(__float2bfloat16_rn(x));
    return x;
}

template <typename T>
__global__ void fill_random_kernel(T* __restrict__ out, unsigned long long n, unsigned long long key, double mean,
                                   double std, float factor, int via_bf16) {
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = from_f32<T>(counter_normal(key, i, mean, std, factor, via_bf16));
}

}  // namespace cib

using namespace cib;

// out[i] = factor * (mean + std * z(key, i)) for i < n, as float32 or bfloat16; via_bf16: the value is rounded to
// bfloat16 before it is converted to the output type (a tensor that a checkpoint would store in bfloat16).
extern "C" int cib_fill_random(void* out, int dtype, long long n, unsigned long long key, double mean, double std,
                               float factor, int via_bf16, cudaStream_t stream) {
    CIB_REQUIRE(out != nullptr && n >= 0, "fill_random: bad arguments");
    CIB_REQUIRE(dtype == kF32 || dtype == kBF16, "fill_random: dtype must be float32 or bfloat16");
    if (n == 0) return 0;
    const int threads = 256;
    long long blocks = (n + threads - 1) / threads;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (dtype == kF32)
        fill_random_kernel<float><<<(int)blocks, threads, 0, stream>>>((float*)out, (unsigned long long)n, key, mean, std, factor, via_bf16);
    else
        fill_random_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>((__nv_bfloat16*)out, (unsigned long long)n, key, mean, std, factor, via_bf16);
    CIB_LAUNCH_CHECK("fill_random");
    return 0;
}
