// Signed block Walsh-Hadamard transforms of the coupled gate/up/down reparameterisation
// (qsrt/qsrt_coupled.py:49-132): x := H_block(x * signs) / sqrt(block)  ("D H"), or its inverse
// x := H_block(x) / sqrt(block) * signs ("H D"), along either axis of a row-major matrix, for
// blocks of 128, 256 or 512.  HBM-bound: one read and one write per pass, no temporaries (the
// reference makes log2(block) strided passes with two clones each).
//
// The butterflies run in the reference's order (pair width 1, 2, 4, ... block/2, lower index
// holds the sum) and the normalisation is a true division, so results equal the reference's
// float32 CPU path bit for bit.
//
//   axis 1: one warp per (row, block); a lane holds block/128 float4s: widths 1,2 in registers,
//           4..64 through warp shuffles, 128 and 256 across the lane's float4s.
//   axis 0: one thread per column holds a 128-row strip in registers (widths 1..64); blocks
//           of 256 / 512 rows add a second pass that combines the strips (widths 128, 256).
#include <cuda_runtime.h>
#include <stdint.h>

#include "qsrtb_internal.h"

namespace {

// Unnormalised Walsh-Hadamard of one block of 128 * SEGS values held by a warp: lane l owns
// values 4l .. 4l+3 of every 128-value segment.
template <int SEGS>
__device__ __forceinline__ void butterflies(float (&v)[SEGS][4], const int lane)
{
#pragma unroll
    for (int s = 0; s < SEGS; ++s) {
        // widths 1 and 2: inside the lane's four consecutive values
        const float a = v[s][0] + v[s][1], d = v[s][0] - v[s][1];
        const float e = v[s][2] + v[s][3], f = v[s][2] - v[s][3];
        v[s][0] = a + e; v[s][1] = d + f; v[s][2] = a - e; v[s][3] = d - f;
        // widths 4 .. 64: across lanes
#pragma unroll
        for (int bit = 1; bit < 32; bit <<= 1) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float other = __shfl_xor_sync(0xffffffffu, v[s][i], bit);
                v[s][i] = (lane & bit) ? other - v[s][i] : v[s][i] + other;
            }
        }
    }
    // widths 128 and 256: across the lane's segments
#pragma unroll
    for (int w = 1; w < SEGS; w <<= 1) {
#pragma unroll
        for (int s = 0; s < SEGS; ++s) {
            if ((s & w) == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float a = v[s][i], b = v[s | w][i];
                    v[s][i] = a + b;
                    v[s | w][i] = a - b;
                }
            }
        }
    }
}

template <int SEGS>
__global__ void __launch_bounds__(256)
signed_hadamard_rows_kernel(float* __restrict__ x, int64_t rows, int cols, int ld,
                            const float* __restrict__ signs, int sign_after, float norm)
{
    constexpr int BLOCK = 128 * SEGS;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int blocks_per_row = cols / BLOCK;
    if (warp >= rows * blocks_per_row) return;
    const int64_t r = warp / blocks_per_row;
    const int c0 = int(warp - r * blocks_per_row) * BLOCK;
    float* base = x + r * ld + c0;
    float v[SEGS][4];
#pragma unroll
    for (int s = 0; s < SEGS; ++s) {
        const float4 t = *reinterpret_cast<const float4*>(base + s * 128 + lane * 4);
        v[s][0] = t.x; v[s][1] = t.y; v[s][2] = t.z; v[s][3] = t.w;
        if (signs && !sign_after) {
            const float4 g = *reinterpret_cast<const float4*>(signs + c0 + s * 128 + lane * 4);
            v[s][0] *= g.x; v[s][1] *= g.y; v[s][2] *= g.z; v[s][3] *= g.w;
        }
    }
    butterflies<SEGS>(v, lane);
#pragma unroll
    for (int s = 0; s < SEGS; ++s) {
#pragma unroll
        for (int i = 0; i < 4; ++i) v[s][i] = __fdiv_rn(v[s][i], norm);
        if (signs && sign_after) {
            const float4 g = *reinterpret_cast<const float4*>(signs + c0 + s * 128 + lane * 4);
            v[s][0] *= g.x; v[s][1] *= g.y; v[s][2] *= g.z; v[s][3] *= g.w;
        }
        *reinterpret_cast<float4*>(base + s * 128 + lane * 4) = make_float4(v[s][0], v[s][1], v[s][2], v[s][3]);
    }
}


// The same transform along the input axis, reading the source matrix in its packed MXFP4 storage
// (E2M1 codes, two per byte, low nibble first; one E8M0 scale byte per 32 inputs;
// qsrt/io/mxfp4.py:1-63) instead of a float32 copy of it: 0.53 bytes per weight come in, the
// transformed float32 row goes out, and the dequantised matrix never exists in memory.
// Source row r lands in output row r * row_step + row_offset, which interleaves the gate and up
// matrices as the coupled coordinates want them (qsrt/qsrt_coupled.py:145-196).
__device__ __forceinline__ float e2m1_times_scale(uint32_t code, float scale, int round_bf16)
{
    const uint32_t m = code & 7u;
    const float mag = m < 2u ? 0.5f * float(m) : __uint_as_float(((126u + (m >> 1)) << 23) | ((m & 1u) << 22));
    float v = ((code & 8u) ? -mag : mag) * scale;
    if (round_bf16) {   // round to nearest even on 8 significand bits, as a bfloat16 checkpoint stores it
        uint32_t u = __float_as_uint(v);
        if ((u & 0x7f800000u) != 0x7f800000u) u += 0x00007fffu + ((u >> 16) & 1u);
        v = __uint_as_float(u & 0xffff0000u);
    }
    return v;
}

// Lane l of a warp owns VALS = 4 * SEGS consecutive values of the block (one 2 * SEGS-byte load of
// codes); the butterflies keep the reference's order of widths (1, 2, 4, ... block / 2): the widths
// below VALS run inside the lane's registers, the others across lanes by shuffles.  Which lane
// holds which element does not change any sum, so the result equals the float32 kernel's.
template <int SEGS>
__global__ void __launch_bounds__(256)
mxfp4_signed_hadamard_rows_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scale,
                                  int64_t rows, int cols, float* __restrict__ out, int ld, int row_step,
                                  int row_offset, const float* __restrict__ signs, int round_bf16, float norm)
{
    constexpr int BLOCK = 128 * SEGS;
    constexpr int VALS = 4 * SEGS;      // 4, 8 or 16 consecutive values per lane
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int blocks_per_row = cols / BLOCK;
    if (warp >= rows * blocks_per_row) return;
    const int64_t r = warp / blocks_per_row;
    const int c = int(warp - r * blocks_per_row) * BLOCK + lane * VALS;
    uint32_t codes[(VALS + 7) / 8];
    const uint8_t* src = packed + r * (cols / 2) + c / 2;
    if constexpr (VALS == 4) codes[0] = *reinterpret_cast<const uint16_t*>(src);
    else if constexpr (VALS == 8) codes[0] = *reinterpret_cast<const uint32_t*>(src);
    else {
        const uint2 two = *reinterpret_cast<const uint2*>(src);
        codes[0] = two.x;
        codes[1] = two.y;
    }
    const uint32_t byte = scale[r * (cols / 32) + c / 32];   // VALS <= 16 values never straddle a scale block
    const float sc = __uint_as_float(byte == 0u ? 0x00400000u : byte << 23);
    float v[VALS];
#pragma unroll
    for (int i = 0; i < VALS; ++i) v[i] = e2m1_times_scale((codes[i >> 3] >> (4 * (i & 7))) & 15u, sc, round_bf16);
    if (signs) {
#pragma unroll
        for (int q = 0; q < VALS / 4; ++q) {
            const float4 g = *reinterpret_cast<const float4*>(signs + c + 4 * q);
            v[4 * q] *= g.x; v[4 * q + 1] *= g.y; v[4 * q + 2] *= g.z; v[4 * q + 3] *= g.w;
        }
    }
    // widths 1 .. VALS / 2: inside the lane
#pragma unroll
    for (int w = 1; w < VALS; w <<= 1) {
#pragma unroll
        for (int i = 0; i < VALS; ++i) {
            if ((i & w) == 0) {
                const float a = v[i], b = v[i | w];
                v[i] = a + b;
                v[i | w] = a - b;
            }
        }
    }
    // widths VALS .. block / 2: across lanes
#pragma unroll
    for (int bit = 1; bit < 32; bit <<= 1) {
#pragma unroll
        for (int i = 0; i < VALS; ++i) {
            const float other = __shfl_xor_sync(0xffffffffu, v[i], bit);
            v[i] = (lane & bit) ? other - v[i] : v[i] + other;
        }
    }
    float* base = out + (r * row_step + row_offset) * ld + c;
#pragma unroll
    for (int q = 0; q < VALS / 4; ++q)
        *reinterpret_cast<float4*>(base + 4 * q) =
            make_float4(__fdiv_rn(v[4 * q], norm), __fdiv_rn(v[4 * q + 1], norm), __fdiv_rn(v[4 * q + 2], norm),
                        __fdiv_rn(v[4 * q + 3], norm));
}

// 128-row strips; `finish` applies the division and the trailing signs (single-pass blocks).
__global__ void __launch_bounds__(128)
signed_hadamard_strip_kernel(float* __restrict__ x, int cols, int ld, const float* __restrict__ signs,
                             int sign_after, int finish, float norm)
{
    const int c = blockIdx.x * 128 + threadIdx.x;
    if (c >= cols) return;
    const int r0 = blockIdx.y * 128;
    float* base = x + int64_t(r0) * ld + c;
    float v[128];
#pragma unroll
    for (int r = 0; r < 128; ++r) v[r] = base[int64_t(r) * ld];
    if (signs && !sign_after) {
#pragma unroll
        for (int r = 0; r < 128; ++r) v[r] *= signs[r0 + r];
    }
#pragma unroll
    for (int bit = 1; bit < 128; bit <<= 1) {
#pragma unroll
        for (int r = 0; r < 128; ++r) {
            if ((r & bit) == 0) {
                const float a = v[r], b = v[r | bit];
                v[r] = a + b;
                v[r | bit] = a - b;
            }
        }
    }
    if (finish) {
#pragma unroll
        for (int r = 0; r < 128; ++r) v[r] = __fdiv_rn(v[r], norm);
        if (signs && sign_after) {
#pragma unroll
            for (int r = 0; r < 128; ++r) v[r] *= signs[r0 + r];
        }
    }
#pragma unroll
    for (int r = 0; r < 128; ++r) base[int64_t(r) * ld] = v[r];
}

// Second pass for blocks of S * 128 rows: widths 128 (and 256) across the strips.
template <int S>
__global__ void __launch_bounds__(256)
signed_hadamard_cross_kernel(float* __restrict__ x, int rows, int cols, int ld,
                             const float* __restrict__ signs, int sign_after, float norm)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    const int group = blockIdx.y / 128;      // which S*128-row block
    const int r_in = blockIdx.y % 128;       // row inside a strip
    const int r0 = group * S * 128 + r_in;
    float v[S];
#pragma unroll
    for (int s = 0; s < S; ++s) v[s] = x[int64_t(r0 + s * 128) * ld + c];
#pragma unroll
    for (int w = 1; w < S; w <<= 1) {
#pragma unroll
        for (int s = 0; s < S; ++s) {
            if ((s & w) == 0) {
                const float a = v[s], b = v[s | w];
                v[s] = a + b;
                v[s | w] = a - b;
            }
        }
    }
#pragma unroll
    for (int s = 0; s < S; ++s) {
        float out = __fdiv_rn(v[s], norm);
        if (signs && sign_after) out *= signs[r0 + s * 128];
        x[int64_t(r0 + s * 128) * ld + c] = out;
    }
}

}  // namespace

extern "C" int qsrtb_signed_block_hadamard(float* x, int64_t rows, int cols, int ld, int axis,
                                           int block_size, const float* signs, int sign_after,
                                           void* stream)
{
    if (!x || rows < 0 || cols < 0 || ld < cols) return qsrtb_fail(QSRTB_EINVAL, "bad matrix arguments");
    if (axis != 0 && axis != 1) return qsrtb_fail(QSRTB_EINVAL, "axis must be 0 or 1");
    if (block_size != 128 && block_size != 256 && block_size != 512)
        return qsrtb_fail(QSRTB_EINVAL, "block_size must be 128, 256 or 512");
    const int64_t extent = axis == 1 ? cols : rows;
    if (extent % block_size) return qsrtb_fail(QSRTB_EINVAL, "Hadamard axis must be divisible by block_size");
    if (axis == 1 && (ld % 4)) return qsrtb_fail(QSRTB_EINVAL, "row pitch must be a multiple of 4 floats");
    if (rows == 0 || cols == 0) return QSRTB_OK;
    if (axis == 0 && rows > 262144) return qsrtb_fail(QSRTB_EINVAL, "too many rows for a column transform");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const float norm = sqrtf(float(block_size));
    if (axis == 1) {
        const int64_t warps = rows * (cols / block_size);
        const unsigned blocks = unsigned((warps + 7) / 8);
        if (block_size == 128)
            signed_hadamard_rows_kernel<1><<<blocks, 256, 0, s>>>(x, rows, cols, ld, signs, sign_after, norm);
        else if (block_size == 256)
            signed_hadamard_rows_kernel<2><<<blocks, 256, 0, s>>>(x, rows, cols, ld, signs, sign_after, norm);
        else
            signed_hadamard_rows_kernel<4><<<blocks, 256, 0, s>>>(x, rows, cols, ld, signs, sign_after, norm);
    } else {
        const int strips = int(rows / 128);
        const int single = block_size == 128;
        signed_hadamard_strip_kernel<<<dim3((cols + 127) / 128, strips), 128, 0, s>>>(
            x, cols, ld, signs, sign_after, single, norm);
        if (!single) {
            const dim3 grid((cols + 255) / 256, unsigned(rows / block_size) * 128);
            if (block_size == 256)
                signed_hadamard_cross_kernel<2><<<grid, 256, 0, s>>>(x, int(rows), cols, ld, signs, sign_after, norm);
            else
                signed_hadamard_cross_kernel<4><<<grid, 256, 0, s>>>(x, int(rows), cols, ld, signs, sign_after, norm);
        }
    }
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "signed_block_hadamard launch");
    return QSRTB_OK;
}

extern "C" int qsrtb_mxfp4_signed_block_hadamard(const uint8_t* packed, const uint8_t* scale, int64_t rows, int cols,
                                                 float* out, int ld, int row_step, int row_offset, int block_size,
                                                 const float* signs, int round_bf16, void* stream)
{
    if (rows < 0 || cols < 0 || ld < cols || (ld % 4) != 0 || row_step < 1 || row_offset < 0 || row_offset >= row_step)
        return qsrtb_fail(QSRTB_EINVAL, "bad matrix arguments");
    if (block_size != 128 && block_size != 256 && block_size != 512)
        return qsrtb_fail(QSRTB_EINVAL, "block_size must be 128, 256 or 512");
    if (cols % block_size) return qsrtb_fail(QSRTB_EINVAL, "Hadamard axis must be divisible by block_size");
    if (rows == 0 || cols == 0) return QSRTB_OK;
    if (!packed || !scale || !out) return qsrtb_fail(QSRTB_EINVAL, "null pointer");
    if ((reinterpret_cast<uintptr_t>(packed) & 7) || (reinterpret_cast<uintptr_t>(out) & 15) ||
        (signs && (reinterpret_cast<uintptr_t>(signs) & 15)))
        return qsrtb_fail(QSRTB_EINVAL, "packed codes need 8-byte, output and signs 16-byte alignment");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const float norm = sqrtf(float(block_size));
    const int64_t warps = rows * (cols / block_size);
    const unsigned blocks = unsigned((warps + 7) / 8);
    if (block_size == 128)
        mxfp4_signed_hadamard_rows_kernel<1><<<blocks, 256, 0, s>>>(packed, scale, rows, cols, out, ld, row_step, row_offset, signs, round_bf16, norm);
    else if (block_size == 256)
        mxfp4_signed_hadamard_rows_kernel<2><<<blocks, 256, 0, s>>>(packed, scale, rows, cols, out, ld, row_step, row_offset, signs, round_bf16, norm);
    else
        mxfp4_signed_hadamard_rows_kernel<4><<<blocks, 256, 0, s>>>(packed, scale, rows, cols, out, ld, row_step, row_offset, signs, round_bf16, norm);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "mxfp4_signed_block_hadamard launch");
    return QSRTB_OK;
}
