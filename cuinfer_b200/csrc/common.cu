// Error text of the last failed entry point (per thread) and a version probe for the loader.
#include "common.cuh"

#include <cuda.h>
#include <stdarg.h>

namespace cib {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_tensor_map_bf16_2d(void* map, const void* base, unsigned long long rows, int cols, int ld, int box_cols,
                              int box_rows, const char* who) {
    // the driver's encoder, looked up through the runtime so that nothing links against the driver library
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    CIB_REQUIRE(fn != nullptr, "%s: the driver does not give cuTensorMapEncodeTiled", who);
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(reinterpret_cast<CUtensorMap*>(map), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    CIB_REQUIRE(r == CUDA_SUCCESS, "%s: cuTensorMapEncodeTiled failed with code %d (rows=%llu cols=%d ld=%d box=%dx%d)", who, (int)r,
                rows, cols, ld, box_cols, box_rows);
    return 0;
}

}  // namespace cib

extern "C" const char* cib_last_error() { return cib::g_error; }

namespace cib {
static int g_prompt_pdl = 0;
bool prompt_pdl() { return g_prompt_pdl != 0; }
}  // namespace cib
extern "C" void cib_set_prompt_pdl(int on) { cib::g_prompt_pdl = on; }

// Bumped whenever an exported signature changes, so that a stale library is rebuilt, not misused.
extern "C" int cib_abi_version() { return 2; }
