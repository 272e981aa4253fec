// Error reporting and build identification for libqsrt_b200.
#include <cstdio>
#include <cstring>

#include "qsrtb_internal.h"

namespace {
thread_local char g_last_error[256] = "";
}

int qsrtb_fail(int code, const char* message)
{
    std::snprintf(g_last_error, sizeof(g_last_error), "%s", message ? message : "");
    return code;
}

int qsrtb_fail_cuda(cudaError_t err, const char* where)
{
    std::snprintf(g_last_error, sizeof(g_last_error), "%s: %s", where ? where : "cuda",
                  cudaGetErrorString(err));
    return QSRTB_ECUDA;
}

extern "C" int qsrtb_abi_version(void) { return 1; }

extern "C" const char* qsrtb_last_error(void) { return g_last_error; }
