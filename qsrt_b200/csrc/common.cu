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

// ---- measurement aid -------------------------------------------------------------------
// Issues `iters` x 8 independent half2 fused multiply-adds per thread on a grid that fills
// every SM.  The benchmark times it to obtain this device's half2 FMA rate, the denominator of
// the Viterbi kernel's ALU roofline.  `*fma_lanes` (host) receives the number of half lanes.
#include <cuda_fp16.h>

namespace {
__global__ void __launch_bounds__(512) probe_half2_fma_kernel(int iters, float* sink)
{
    __half2 a[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = __floats2half2_rn(0.001f * (threadIdx.x + i), 0.002f * (i + 1));
    const __half2 m = __floats2half2_rn(0.999f, 1.001f);
    const __half2 c = __floats2half2_rn(0.0001f, -0.0001f);
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = __hfma2(a[i], m, c);
    }
    __half2 s = a[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) s = __hadd2(s, a[i]);
    if (__low2float(s) == 12345.678f) sink[0] = __high2float(s);
}
}  // namespace

extern "C" int qsrtb_probe_half2_fma(int iters, float* sink, double* fma_lanes, void* stream)
{
    if (iters <= 0 || !sink || !fma_lanes) return qsrtb_fail(QSRTB_EINVAL, "bad probe arguments");
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
        return qsrtb_fail(QSRTB_ECUDA, "cannot query the device");
    const int grid = sms * 4;
    probe_half2_fma_kernel<<<grid, 512, 0, static_cast<cudaStream_t>(stream)>>>(iters, sink);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "probe launch");
    *fma_lanes = double(grid) * 512.0 * double(iters) * 8.0 * 2.0;
    return QSRTB_OK;
}
