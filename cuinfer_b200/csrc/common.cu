// Error text of the last failed entry point (per thread) and a version probe for the loader.
#include "common.cuh"

#include <stdarg.h>

namespace cib {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

}  // namespace cib

extern "C" const char* cib_last_error() { return cib::g_error; }

// Bumped whenever an exported signature changes, so that a stale library is rebuilt, not misused.
extern "C" int cib_abi_version() { return 1; }
