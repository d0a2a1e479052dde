// Self-test of the failure path that every TMA / tcgen05 kernel of this library shares: a wait on an mbarrier is
// bounded, and a wait that runs out raises the device error word instead of hanging the GPU.  A healthy run never
// takes that path, so this entry point takes it on purpose, harmlessly: one thread waits, with the kernels' own
// `mbar_wait` loop and a limit given by the caller, on a barrier that nothing ever arrives on; when the limit is
// reached it writes a code into the error word and returns.  The kernel gives up; it does not hang or fault.
#include "tcgen05_utils.cuh"

namespace cib {

constexpr int kSelftestCode = 91;
constexpr long long kSelftestMaxCycles = 200000000ll;     // a tenth of a second at most, whatever the caller asks

__global__ void bounded_wait_selftest_kernel(long long limit_cycles, int* error_flag, int* gave_up) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const bool landed = mbar_wait(&bar, 0, limit_cycles);        // phase 0 never completes: no one arrives
        if (!landed) {
            atomicExch(error_flag, kSelftestCode);
            if (gave_up) *gave_up = 1;
        }
    }
}

}  // namespace cib

using namespace cib;

// error_flag: the device's error word (one int).  gave_up: optional int that is set to 1 when the wait ran out.
extern "C" int cib_selftest_bounded_wait(long long limit_cycles, int* error_flag, int* gave_up, cudaStream_t stream) {
    CIB_REQUIRE(error_flag != nullptr, "selftest_bounded_wait: needs the error word");
    CIB_REQUIRE(limit_cycles > 0 && limit_cycles <= kSelftestMaxCycles,
                "selftest_bounded_wait: the limit must be between 1 and %lld cycles", kSelftestMaxCycles);
    bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(limit_cycles, error_flag, gave_up);
    CIB_LAUNCH_CHECK("selftest_bounded_wait");
    return 0;
}
