// Next-token sampling from 32-bit logits: greedy, temperature, top-k, top-p.  One block per row.
//
// Meaning of the options follows the reference's sampler (csrc/ops/sampler.cu:134-387):
//   temperature == 0   -> argmax, ties to the lowest id (:207-212)
//   top_k  in (0, V)   -> keep the values >= the exact k-th largest, ties at the edge kept (:216-250)
//   top_p  in (0, 1)   -> the smallest set of most probable kept tokens whose mass reaches top_p
//   weight_i = exp((x_i - max) / temperature) (:252-281)
// The reference draws with Philox inside the kernel and accepts or rejects candidates; here the
// uniform number u in [0, 1) of every row is an input (the host derives it from seed, request and
// output index), and the kept set is found exactly by a radix descent, so the kernel is a pure
// function of (logits, options, u) and needs no scratch memory.
//
// Masses are summed as 32.32 fixed-point integers: q_i = floor(weight_i * 2^32) (at most 2^32 - 1), so
// that every sum is exact and independent of the order in which threads add.
#include "common.cuh"

#include <cooperative_groups.h>

namespace cib {

constexpr int kSampleThreads = 1024;

struct SampleParams {
    float temperature;
    int top_k;
    float top_p;
    float u;
};

__device__ __forceinline__ uint32_t order_key(float x) {
    const uint32_t b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ uint32_t mass_of(float x, float mx, float temperature, uint32_t key_min) {
    if (order_key(x) < key_min) return 0u;
    const float w = expf((x - mx) / temperature);
    const float scaled = w * 4294967296.f;
    return scaled >= 4294967040.f ? 0xffffffffu : (uint32_t)scaled;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, int ld, int vocab, const SampleParams* __restrict__ params,
              int* __restrict__ out_ids) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ unsigned long long s_hist[256];
    __shared__ unsigned long long s_scan[kSampleThreads];
    __shared__ unsigned int s_prefix, s_mask;
    __shared__ unsigned long long s_above, s_need;
    __shared__ float s_max;
    __shared__ int s_argmax;

    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)row * ld;
    const SampleParams p = params[row];

    // ---- max and argmax (lowest index wins ties) ----
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = tid; i < vocab; i += kSampleThreads) {
        const float v = x[i];
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        best = s_val[lane]; best_i = s_idx[lane];
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0) { s_max = best; s_argmax = best_i == 0x7fffffff ? 0 : best_i; }
    }
    __syncthreads();
    const float mx = s_max;
    if (!(p.temperature > 0.f) || p.top_k == 1) {
        if (tid == 0) out_ids[row] = s_argmax;
        return;
    }

    // ---- top-k: exact k-th largest key by radix descent over the order-preserving bits ----
    uint32_t key_min = 0u;
    if (p.top_k > 0 && p.top_k < vocab) {
        if (tid == 0) { s_prefix = 0u; s_mask = 0u; s_need = (unsigned long long)p.top_k; }
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) s_hist[tid] = 0ull;
            __syncthreads();
            const uint32_t prefix = s_prefix, mask = s_mask;
            for (int i = tid; i < vocab; i += kSampleThreads) {
                const uint32_t k = order_key(x[i]);
                if ((k & mask) == prefix) atomicAdd(&s_hist[(k >> shift) & 0xffu], 1ull);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long cum = 0ull;
                int b = 255;
                for (; b > 0; --b) {
                    if (cum + s_hist[b] >= s_need) break;
                    cum += s_hist[b];
                }
                s_need -= cum;
                s_prefix = prefix | ((uint32_t)b << shift);
                s_mask = mask | (0xffu << shift);
            }
            __syncthreads();
        }
        key_min = s_prefix;
    }

    // ---- total mass of the kept tokens ----
    unsigned long long part = 0ull;
    for (int i = tid; i < vocab; i += kSampleThreads) part += mass_of(x[i], mx, p.temperature, key_min);
    s_scan[tid] = part;
    __syncthreads();
    for (int o = kSampleThreads / 2; o > 0; o >>= 1) {
        if (tid < o) s_scan[tid] += s_scan[tid + o];
        __syncthreads();
    }
    const unsigned long long total = s_scan[0];
    __syncthreads();

    // ---- top-p: largest mass threshold whose kept set still reaches top_p of the total ----
    uint32_t q_min = 0u;
    if (p.top_p > 0.f && p.top_p < 1.f) {
        if (tid == 0) {
            s_prefix = 0u; s_mask = 0u; s_above = 0ull;
            const double want = (double)p.top_p * (double)total;
            unsigned long long need = (unsigned long long)want;
            if ((double)need < want) ++need;
            s_need = need > total ? total : (need == 0ull ? 1ull : need);
        }
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) s_hist[tid] = 0ull;
            __syncthreads();
            const uint32_t prefix = s_prefix, mask = s_mask;
            for (int i = tid; i < vocab; i += kSampleThreads) {
                const uint32_t q = mass_of(x[i], mx, p.temperature, key_min);
                if ((q & mask) == prefix && q != 0u) atomicAdd(&s_hist[(q >> shift) & 0xffu], (unsigned long long)q);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long above = s_above;
                int b = 255;
                for (; b > 0; --b) {
                    if (above + s_hist[b] >= s_need) break;
                    above += s_hist[b];
                }
                s_above = above;
                s_prefix = prefix | ((uint32_t)b << shift);
                s_mask = mask | (0xffu << shift);
            }
            __syncthreads();
        }
        q_min = s_prefix;
    }

    // ---- draw: the first index whose running kept mass exceeds u * kept mass ----
    const int chunk = (vocab + kSampleThreads - 1) / kSampleThreads;
    const int begin = min(tid * chunk, vocab), end = min(begin + chunk, vocab);
    part = 0ull;
    for (int i = begin; i < end; ++i) {
        const uint32_t q = mass_of(x[i], mx, p.temperature, key_min);
        if (q >= q_min) part += q;
    }
    s_scan[tid] = part;
    __syncthreads();
    // inclusive scan (Hillis-Steele) over the 1024 chunk masses
    for (int o = 1; o < kSampleThreads; o <<= 1) {
        const unsigned long long add = tid >= o ? s_scan[tid - o] : 0ull;
        __syncthreads();
        s_scan[tid] += add;
        __syncthreads();
    }
    const unsigned long long kept = s_scan[kSampleThreads - 1];
    if (kept == 0ull) {
        if (tid == 0) out_ids[row] = s_argmax;
        return;
    }
    float u = p.u;
    u = u < 0.f ? 0.f : (u >= 1.f ? 0.99999994f : u);
    unsigned long long target = (unsigned long long)((double)u * (double)kept);
    if (target >= kept) target = kept - 1ull;
    const unsigned long long incl = s_scan[tid], excl = incl - part;
    if (target >= excl && target < incl) {
        unsigned long long run = excl;
        int chosen = end - 1;
        for (int i = begin; i < end; ++i) {
            const uint32_t q = mass_of(x[i], mx, p.temperature, key_min);
            if (q >= q_min && q != 0u) {
                run += q;
                if (run > target) { chosen = i; break; }
            }
        }
        out_ids[row] = chosen;
    }
}

// ---- every row greedy: a cluster of eight CTAs per row, each over an eighth of the vocabulary ----
// One CTA walking a row of 150 k logits is bound by what one SM fetches from the L2 (about 15 us); eight of them take
// an eighth each and meet in the first CTA's shared memory.  The largest value wins, ties go to the lowest id, values
// that are not numbers never win: the same answer as the kernel above, whatever the order of the comparisons.
constexpr int kArgmaxCtas = 8;
constexpr int kArgmaxThreads = 512;

__device__ __forceinline__ void take_better(float& best, int& best_i, float v, int i) {
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
}

__global__ void __launch_bounds__(kArgmaxThreads)
argmax_cluster_kernel(const float* __restrict__ logits, int ld, int vocab, int* __restrict__ out_ids) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float s_val[kArgmaxThreads / 32];
    __shared__ int s_idx[kArgmaxThreads / 32];
    __shared__ float s_part_val[kArgmaxCtas];
    __shared__ int s_part_idx[kArgmaxCtas];
    const int row = blockIdx.x / kArgmaxCtas, rank = (int)cluster.block_rank();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)row * ld;
    // Distributed shared memory may only be touched once every CTA of the cluster runs: arrive here, wait before the
    // remote store, so that the scan hides the barrier.
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    const int chunk = ((vocab + kArgmaxCtas - 1) / kArgmaxCtas + 3) & ~3;
    const int begin = min(vocab, rank * chunk), end = min(vocab, begin + chunk);
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        // begin is a multiple of four: whole float4 groups, then the tail
        const int groups = (end - begin) / 4;
        const float4* x4 = reinterpret_cast<const float4*>(x + begin);
        for (int g = tid; g < groups; g += kArgmaxThreads) {
            const float4 v = x4[g];
            const int i = begin + 4 * g;
            take_better(best, best_i, v.x, i); take_better(best, best_i, v.y, i + 1);
            take_better(best, best_i, v.z, i + 2); take_better(best, best_i, v.w, i + 3);
        }
        for (int i = begin + 4 * groups + tid; i < end; i += kArgmaxThreads) take_better(best, best_i, x[i], i);
    } else {
        for (int i = begin + tid; i < end; i += kArgmaxThreads) take_better(best, best_i, x[i], i);
    }
    for (int o = 16; o > 0; o >>= 1)
        take_better(best, best_i, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, best_i, o));
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        best = lane < kArgmaxThreads / 32 ? s_val[lane] : -INFINITY;
        best_i = lane < kArgmaxThreads / 32 ? s_idx[lane] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1)
            take_better(best, best_i, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, best_i, o));
        if (lane == 0) {
            // every CTA of the cluster has started (the barrier above the scan): its shared memory may be written
            *cluster.map_shared_rank(&s_part_val[rank], 0) = best;
            *cluster.map_shared_rank(&s_part_idx[rank], 0) = best_i;
        }
    }
    cluster.sync();
    if (rank == 0 && tid == 0) {
        best = -INFINITY; best_i = 0x7fffffff;
        for (int r = 0; r < kArgmaxCtas; ++r) take_better(best, best_i, s_part_val[r], s_part_idx[r]);
        out_ids[row] = best_i == 0x7fffffff ? 0 : best_i;
    }
}

}  // namespace cib

using namespace cib;

// Every row greedy (temperature 0): out_ids[r] = argmax of logits[r], ties to the lowest id.
extern "C" int cib_argmax_rows(const float* logits, int ld, int rows, int vocab, int* out_ids, cudaStream_t stream) {
    CIB_REQUIRE(rows >= 0 && vocab > 0 && ld >= vocab, "argmax_rows: bad sizes rows=%d V=%d ld=%d", rows, vocab, ld);
    if (rows == 0) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows * kArgmaxCtas);
    cfg.blockDim = dim3(kArgmaxThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kArgmaxCtas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, argmax_cluster_kernel, logits, ld, vocab, out_ids);
    if (e != cudaSuccess) {
        set_error("argmax_rows: launch failed: %s", cudaGetErrorString(e));
        return -2;
    }
    return 0;
}

// params: [rows] of {float temperature, int top_k, float top_p, float u}.
extern "C" int cib_sample(const float* logits, int ld, int rows, int vocab, const void* params, int* out_ids,
                          cudaStream_t stream) {
    CIB_REQUIRE(rows >= 0 && vocab > 0 && ld >= vocab, "sample: bad sizes rows=%d V=%d ld=%d", rows, vocab, ld);
    if (rows == 0) return 0;
    sample_kernel<<<rows, kSampleThreads, 0, stream>>>(logits, ld, vocab, (const SampleParams*)params, out_ids);
    CIB_LAUNCH_CHECK("sample");
    return 0;
}
