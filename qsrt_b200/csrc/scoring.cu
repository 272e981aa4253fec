// Routed-error scoring helpers around the tensor-core products.
//
//   gated_activation_kernel : [R, 2I] pre-activations (gate | up, one product against the stacked
//                             gate and up matrices) -> middle activation act(gate) * up, written as
//                             the TF32 head / tail planes the down product consumes and, optionally,
//                             as float32 rows (the covariance of the middle activations needs them).
//                             The [R, I] middle is therefore never stored twice nor re-read to split.
//   row_sse_kernel          : per routed row  sum (candidate - reference)^2  and  sum reference^2
//                             in float64, the reductions of functional_sse_by_request
//                             (qsrt/qsrt_candidates.py:621-654) and _defer_functional_row_sse
//                             (qsrt/pack/qsrt_candidates.py:318-349).  HBM-bound: 8 bytes per element.
#include <cuda_runtime.h>
#include <stdint.h>

#include "qsrtb_internal.h"

namespace {

__device__ __forceinline__ float tf32_head(float x)
{
    uint32_t u = __float_as_uint(x);
    u += 0x00000fffu + ((u >> 13) & 1u);
    return __uint_as_float(u & 0xffffe000u);
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// activation 0: SiLU(gate) * up;  1: the bounded gated activation of qsrt/tp_simulator.py:82-93,
// beta * tanh(gate / beta) * sigmoid(gate) times linear_beta * tanh(up / linear_beta).
__device__ __forceinline__ float gated(float gate, float up, int activation)
{
    if (activation == 0) return gate * sigmoidf_(gate) * up;
    const float beta = 4.0f, linear_beta = 25.0f;
    return (beta * tanhf(gate / beta) * sigmoidf_(gate)) * (linear_beta * tanhf(up / linear_beta));
}

__global__ void __launch_bounds__(256)
gated_activation_kernel(const float* __restrict__ gate_up, int64_t rows, int inter, int ld, int activation,
                        float* __restrict__ hi, float* __restrict__ lo, int ld_planes,
                        float* __restrict__ middle, int ld_middle)
{
    const int64_t quads = int64_t(inter / 4);
    const int64_t total = rows * quads;
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
        const int64_t r = i / quads;
        const int c = int(i - r * quads) * 4;
        const float4 g = *reinterpret_cast<const float4*>(gate_up + r * ld + c);
        const float4 u = *reinterpret_cast<const float4*>(gate_up + r * ld + inter + c);
        float4 m;
        m.x = gated(g.x, u.x, activation);
        m.y = gated(g.y, u.y, activation);
        m.z = gated(g.z, u.z, activation);
        m.w = gated(g.w, u.w, activation);
        if (middle) *reinterpret_cast<float4*>(middle + r * ld_middle + c) = m;
        if (hi) {
            const float4 h = make_float4(tf32_head(m.x), tf32_head(m.y), tf32_head(m.z), tf32_head(m.w));
            *reinterpret_cast<float4*>(hi + r * ld_planes + c) = h;
            *reinterpret_cast<float4*>(lo + r * ld_planes + c) =
                make_float4(tf32_head(m.x - h.x), tf32_head(m.y - h.y), tf32_head(m.z - h.z), tf32_head(m.w - h.w));
        }
    }
}

// One warp per row.
__global__ void __launch_bounds__(256)
row_sse_kernel(const float* __restrict__ reference, const float* __restrict__ candidate, int64_t rows, int d,
               int ld_ref, int ld_cand, double* __restrict__ row_sse, double* __restrict__ row_energy)
{
    const int lane = threadIdx.x & 31;
    const int64_t row = blockIdx.x * int64_t(blockDim.x / 32) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* a = reference + row * ld_ref;
    const float* b = candidate + row * ld_cand;
    double sse = 0.0, energy = 0.0;
    const int quads = d / 4;
    for (int q = lane; q < quads; q += 32) {
        const float4 r = *reinterpret_cast<const float4*>(a + 4 * q);
        const float4 c = *reinterpret_cast<const float4*>(b + 4 * q);
        const double d0 = double(c.x) - double(r.x), d1 = double(c.y) - double(r.y);
        const double d2 = double(c.z) - double(r.z), d3 = double(c.w) - double(r.w);
        sse += d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3;
        energy += double(r.x) * r.x + double(r.y) * r.y + double(r.z) * r.z + double(r.w) * r.w;
    }
    for (int i = 4 * quads + lane; i < d; i += 32) {
        const double dv = double(b[i]) - double(a[i]);
        sse += dv * dv;
        energy += double(a[i]) * a[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sse += __shfl_down_sync(0xffffffffu, sse, o);
        energy += __shfl_down_sync(0xffffffffu, energy, o);
    }
    if (lane == 0) {
        row_sse[row] = sse;
        if (row_energy) row_energy[row] = energy;
    }
}

}  // namespace

extern "C" int qsrtb_gated_activation(const float* gate_up, int64_t rows, int inter, int ld, int activation,
                                      float* hi, float* lo, int ld_planes, float* middle, int ld_middle,
                                      void* stream)
{
    if (!gate_up || rows < 0 || inter <= 0 || (inter % 4) != 0 || ld < 2 * inter || (ld % 4) != 0)
        return qsrtb_fail(QSRTB_EINVAL, "pre-activations must be [rows, 2 * intermediate] with intermediate % 4 == 0");
    if (activation != 0 && activation != 1) return qsrtb_fail(QSRTB_EINVAL, "activation must be 0 (SiLU) or 1 (SiTU)");
    if ((hi == nullptr) != (lo == nullptr)) return qsrtb_fail(QSRTB_EINVAL, "head and tail planes come together");
    if (!hi && !middle) return qsrtb_fail(QSRTB_EINVAL, "no output requested");
    if ((hi && (ld_planes < inter || (ld_planes % 4) != 0)) || (middle && (ld_middle < inter || (ld_middle % 4) != 0)))
        return qsrtb_fail(QSRTB_EINVAL, "output pitch must be a multiple of 4 and at least the intermediate width");
    const uintptr_t bits = reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(hi) |
                           reinterpret_cast<uintptr_t>(lo) | reinterpret_cast<uintptr_t>(middle);
    if (bits & 15) return qsrtb_fail(QSRTB_EINVAL, "activation buffers must be 16-byte aligned");
    if (rows == 0) return QSRTB_OK;
    const int64_t work = rows * (inter / 4);
    const int64_t blocks = (work + 255) / 256;
    gated_activation_kernel<<<unsigned(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        gate_up, rows, inter, ld, activation, hi, lo, ld_planes, middle, ld_middle);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "gated_activation launch");
    return QSRTB_OK;
}

extern "C" int qsrtb_routed_row_sse(const float* reference, const float* candidate, int64_t rows, int d,
                                    int ld_reference, int ld_candidate, double* row_sse, double* row_energy,
                                    void* stream)
{
    if (!reference || !candidate || !row_sse || rows < 0 || d <= 0 || ld_reference < d || ld_candidate < d)
        return qsrtb_fail(QSRTB_EINVAL, "bad routed-error arguments");
    if ((ld_reference % 4) != 0 || (ld_candidate % 4) != 0 ||
        ((reinterpret_cast<uintptr_t>(reference) | reinterpret_cast<uintptr_t>(candidate)) & 15))
        return qsrtb_fail(QSRTB_EINVAL, "output rows must be 16-byte aligned");
    if (rows == 0) return QSRTB_OK;
    row_sse_kernel<<<unsigned((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reference, candidate, rows, d, ld_reference, ld_candidate, row_sse, row_energy);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "row_sse launch");
    return QSRTB_OK;
}
