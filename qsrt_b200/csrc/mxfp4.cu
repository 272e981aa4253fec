// MXFP4 source ingest (HBM-bound byte work): packed E2M1 codes + E8M0 block scales -> float32.
//
// Storage of a source expert matrix (qsrt/io/mxfp4.py:1-63): weight_packed uint8 [out, in/2], two
// codes per byte with the low nibble at the even input index; weight_scale uint8 [out, in/32],
// value 2^(byte-127) for 32 consecutive inputs.  Every product code_value * scale is exact in
// float32, so the result equals the reference's torch arithmetic bit for bit, including its
// corner cases (scale byte 0 -> 2^-127, a subnormal; byte 255 -> +inf, so code 0 gives NaN - whose
// payload bits are the GPU's, not the host's).
//
// Two output orientations from the same 0.53 bytes/weight of input:
//   plain      : [out, in] row-major, as the reference's dequant() returns;
//   transposed : [in, out] row-major - the orientation the encoder consumes - through a
//                shared-memory tile so that both sides stay coalesced.  The reference
//                materialises [out, in] and transposes it in a second pass.
#include <cuda_runtime.h>
#include <stdint.h>

#include "qsrtb_internal.h"

namespace {

__device__ __forceinline__ float e2m1_value(uint32_t code)
{
    // 0, 0.5, 1, 1.5, 2, 3, 4, 6 and their negatives (qsrt/constants.py:71-74)
    const uint32_t m = code & 7u;
    const float mag = m < 2u ? 0.5f * float(m) : __uint_as_float(((126u + (m >> 1)) << 23) | ((m & 1u) << 22));
    return (code & 8u) ? -mag : mag;
}

__device__ __forceinline__ float e8m0_scale(uint32_t byte)
{
    return __uint_as_float(byte == 0u ? 0x00400000u : byte << 23);   // 2^(byte-127); 255 -> +inf
}

// One thread per 4 packed bytes (8 weights): one 32-bit load, two 16-byte stores.
__global__ void __launch_bounds__(256)
mxfp4_plain_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scale, int64_t groups,
                   int in_cols, float* __restrict__ dst, int ld)
{
    const int groups_per_row = in_cols / 8;
    for (int64_t g = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; g < groups;
         g += int64_t(gridDim.x) * blockDim.x) {
        const int64_t row = g / groups_per_row;
        const int col = int(g - row * groups_per_row) * 8;
        const uint32_t bytes = *reinterpret_cast<const uint32_t*>(packed + row * (in_cols / 2) + col / 2);
        const float s = e8m0_scale(scale[row * (in_cols / 32) + col / 32]);
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = e2m1_value((bytes >> (4 * i)) & 15u) * s;
        float4* out = reinterpret_cast<float4*>(dst + row * ld + col);
        out[0] = make_float4(v[0], v[1], v[2], v[3]);
        out[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}

// Block = 32 source rows x 128 inputs -> a [128, 32] patch of the transposed output.
__global__ void __launch_bounds__(256)
mxfp4_transposed_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scale, int out_rows,
                        int in_cols, float* __restrict__ dst, int ld)
{
    __shared__ float tile[128][33];
    const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 128;
    // 32 rows x 16 groups of 8 weights = 512 groups, two per thread
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int g = threadIdx.x + 256 * i;
        const int r = g >> 4, gc = (g & 15) * 8;
        const int row = r0 + r, col = c0 + gc;
        if (row < out_rows && col < in_cols) {
            const uint32_t bytes = *reinterpret_cast<const uint32_t*>(packed + int64_t(row) * (in_cols / 2) + col / 2);
            const float s = e8m0_scale(scale[int64_t(row) * (in_cols / 32) + col / 32]);
#pragma unroll
            for (int k = 0; k < 8; ++k) tile[gc + k][r] = e2m1_value((bytes >> (4 * k)) & 15u) * s;
        }
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int c = warp * 16 + i;
        if (c0 + c < in_cols && r0 + lane < out_rows) dst[int64_t(c0 + c) * ld + r0 + lane] = tile[c][lane];
    }
}

}  // namespace

extern "C" int qsrtb_mxfp4_dequant(const uint8_t* packed, const uint8_t* scale, int out_rows, int in_cols,
                                   float* dst, int ld, int transposed, void* stream)
{
    if (out_rows < 0 || in_cols < 0 || (in_cols % 32) != 0)
        return qsrtb_fail(QSRTB_EINVAL, "input dimension must be a multiple of the 32-element scale block");
    if (ld < (transposed ? out_rows : in_cols)) return qsrtb_fail(QSRTB_EINVAL, "row pitch smaller than the row");
    if (out_rows == 0 || in_cols == 0) return QSRTB_OK;
    if (!packed || !scale || !dst) return qsrtb_fail(QSRTB_EINVAL, "null pointer");
    if ((reinterpret_cast<uintptr_t>(packed) & 3) || (reinterpret_cast<uintptr_t>(dst) & 15) || (!transposed && (ld % 4)))
        return qsrtb_fail(QSRTB_EINVAL, "packed codes need 4-byte and the output 16-byte alignment");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (transposed) {
        const dim3 grid(unsigned((in_cols + 127) / 128), unsigned((out_rows + 31) / 32));
        mxfp4_transposed_kernel<<<grid, 256, 0, s>>>(packed, scale, out_rows, in_cols, dst, ld);
    } else {
        const int64_t groups = int64_t(out_rows) * (in_cols / 8);
        int device = 0, sms = 148;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        const int64_t wanted = (groups + 255) / 256, cap = int64_t(sms) * 16;
        mxfp4_plain_kernel<<<unsigned(wanted < cap ? wanted : cap), 256, 0, s>>>(packed, scale, groups, in_cols, dst, ld);
    }
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "mxfp4_dequant launch");
    return QSRTB_OK;
}
