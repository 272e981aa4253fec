// Shared by the translation units of libqsrt_b200: status codes and error reporting.
#pragma once

#include <cuda_runtime.h>

#include "../../include/qsrt_b200.h"

// Record a message for qsrtb_last_error() (thread local) and return `code`.
int qsrtb_fail(int code, const char* message);
int qsrtb_fail_cuda(cudaError_t err, const char* where);
