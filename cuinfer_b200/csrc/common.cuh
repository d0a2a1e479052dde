// Shared helpers for the sm_100a kernels: element types, 32-bit loads of either storage type,
// warp/block reductions and the error convention of the exported entry points.
//
// Every exported function is `extern "C"`, takes raw device pointers, sizes and a stream, checks
// what it cannot handle and returns 0 on success or a negative code after recording a message
// that `cuinfer_last_error()` hands to the caller.  Nothing here allocates.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

namespace cib {

enum DType : int { kF32 = 0, kBF16 = 1 };

constexpr int kWarp = 32;

// ---- error reporting -------------------------------------------------------------------
void set_error(const char* fmt, ...);

// Whether the kernels of prompt-sized steps (tcgen05 GEMM and attention, row-wise norm) are launched with the
// programmatic-dependent-launch attribute, so that a kernel's set-up runs under the tail of the kernel before it
// (`cib_set_prompt_pdl`; off until the host switches it on).  Each of them waits for that kernel before it reads or
// writes anything a kernel produces.
bool prompt_pdl();

// A 2-D tensor map over bfloat16 rows (`cols` elements, `ld` elements apart) with boxes of box_cols x box_rows,
// 128-byte swizzle, zero fill outside.  `map` points at a CUtensorMap (kept opaque here so that only the files that
// issue TMA copies include the driver header).  0, or -1 with the error text set.
int encode_tensor_map_bf16_2d(void* map, const void* base, unsigned long long rows, int cols, int ld, int box_cols,
                              int box_rows, const char* who);

// The larger limit on dynamic shared memory is a property of a kernel on ONE device: it is set the first time the kernel
// is launched on each device, under a mutex (the entry points may be called from several threads).  A launcher keeps one
// `SmemLimit` per kernel instantiation as a function-local static.
constexpr int kMaxDevices = 64;
struct SmemLimit {
    std::mutex mutex;
    bool raised[kMaxDevices] = {false};
};
template <typename Kernel>
inline int raise_smem_limit(SmemLimit& state, Kernel kernel, size_t bytes, const char* who) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_error("%s: cannot tell the current device (%s)", who, cudaGetErrorString(e));
        return -2;
    }
    std::lock_guard<std::mutex> lock(state.mutex);
    if (state.raised[dev]) return 0;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) {
        set_error("%s: cannot raise shared memory to %zu bytes: %s", who, bytes, cudaGetErrorString(e));
        return -2;
    }
    state.raised[dev] = true;
    return 0;
}

#define CIB_REQUIRE(cond, ...)            \
    do {                                  \
        if (!(cond)) {                    \
            ::cib::set_error(__VA_ARGS__); \
            return -1;                    \
        }                                 \
    } while (0)

#define CIB_LAUNCH_CHECK(name)                                                     \
    do {                                                                           \
        cudaError_t e__ = cudaGetLastError();                                      \
        if (e__ != cudaSuccess) {                                                  \
            ::cib::set_error("%s: launch failed: %s", name, cudaGetErrorString(e__)); \
            return -2;                                                             \
        }                                                                          \
    } while (0)

// ---- typed access ------------------------------------------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// A vector that is stored either in 32 bits or in bfloat16, chosen at run time (norm gains keep
// the precision they were stored in, whatever the engine's dtype).
struct AnyVec {
    const void* ptr;
    int is_bf16;
    __device__ __forceinline__ float operator[](int i) const {
        return is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(ptr)[i])
                       : reinterpret_cast<const float*>(ptr)[i];
    }
};

// ---- reductions ----------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

}  // namespace cib
