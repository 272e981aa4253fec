// Blockwise 128-point Hadamard transforms fused with the sign/scale vectors around them, and
// the reductions the regulariser needs.  All HBM-bound float32 work: one read and one write of
// the matrix per call, no materialised Hadamard matrix and no per-block matmul launches
// (the reference multiplies every 128-row / 128-column block by a dense 128x128 matrix from a
// Python loop, qsrt/exl3_encoder_backend.py:275-320).
//
//   axis 1 (along a row):   one warp per matrix row walks its 128-column segments; a lane holds
//                           4 consecutive values (one 16-byte load), 2 butterfly stages run in
//                           registers and 5 through warp shuffles.  The warp also owns the
//                           row's sum of squares, accumulated in a fixed order, so the
//                           input-channel scales are deterministic.
//   axis 0 (along a column): one thread per column holds a 128-row strip in registers (128
//                           coalesced row loads in flight), 7 butterfly stages in registers.
#include <cuda_runtime.h>
#include <stdint.h>

#include "qsrtb_internal.h"

namespace {

constexpr float kInvSqrt128 = 0.08838834764831845f;

struct ScaleSpec {
    const float* vec;      // NULL: no scaling
    int64_t stride;        // elements between consecutive matrices
    int per_col;           // 1: vec[col], 0: vec[row]
    int divide;            // 1: x / s, 0: x * s
    int after;             // 1: applied to the transformed value, 0: before the transform
};

__device__ __forceinline__ float apply_scale(float x, float s, int divide)
{
    return divide ? __fdiv_rn(x, s) : __fmul_rn(x, s);
}

// grid.x * warps_per_block warps cover batch * rows rows.
__global__ void __launch_bounds__(256)
hadamard_rows_kernel(float* __restrict__ x, int batch, int rows, int cols, int ld, int64_t x_stride,
                     ScaleSpec sc, float* __restrict__ sumsq, int64_t sumsq_stride)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t total = int64_t(batch) * rows;
    if (warp >= total) return;
    const int b = int(warp / rows);
    const int r = int(warp - int64_t(b) * rows);
    float* row = x + b * x_stride + int64_t(r) * ld;
    const float* vec = sc.vec ? sc.vec + b * sc.stride : nullptr;
    const float row_s = (vec && !sc.per_col) ? vec[r] : 1.0f;
    float acc = 0.0f;
    for (int c0 = 0; c0 < cols; c0 += 128) {
        float4 v4 = *reinterpret_cast<const float4*>(row + c0 + lane * 4);
        float v[4] = {v4.x, v4.y, v4.z, v4.w};
        if (vec && !sc.after) {
            if (sc.per_col) {
                const float4 s4 = *reinterpret_cast<const float4*>(vec + c0 + lane * 4);
                v[0] = apply_scale(v[0], s4.x, sc.divide); v[1] = apply_scale(v[1], s4.y, sc.divide);
                v[2] = apply_scale(v[2], s4.z, sc.divide); v[3] = apply_scale(v[3], s4.w, sc.divide);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] = apply_scale(v[i], row_s, sc.divide);
            }
        }
        // element index = lane * 4 + i: bits 0-1 in registers, bits 2-6 across lanes
        float a = v[0] + v[1], d = v[0] - v[1], e = v[2] + v[3], f = v[2] - v[3];
        v[0] = a + e; v[1] = d + f; v[2] = a - e; v[3] = d - f;
#pragma unroll
        for (int bit = 1; bit < 32; bit <<= 1) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float other = __shfl_xor_sync(0xffffffffu, v[i], bit);
                v[i] = (lane & bit) ? other - v[i] : v[i] + other;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] *= kInvSqrt128;
        if (vec && sc.after) {
            if (sc.per_col) {
                const float4 s4 = *reinterpret_cast<const float4*>(vec + c0 + lane * 4);
                v[0] = apply_scale(v[0], s4.x, sc.divide); v[1] = apply_scale(v[1], s4.y, sc.divide);
                v[2] = apply_scale(v[2], s4.z, sc.divide); v[3] = apply_scale(v[3], s4.w, sc.divide);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] = apply_scale(v[i], row_s, sc.divide);
            }
        }
        acc += (v[0] * v[0] + v[1] * v[1]) + (v[2] * v[2] + v[3] * v[3]);
        *reinterpret_cast<float4*>(row + c0 + lane * 4) = make_float4(v[0], v[1], v[2], v[3]);
    }
    if (sumsq) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) sumsq[b * sumsq_stride + r] = acc;
    }
}

// Column transform (axis 0).  block = 256 threads = 128 columns; blockIdx.y = 128-row strip;
// blockIdx.z = matrix.  A warp takes 16 columns: lanes 0..15 hold rows 0..63 of their column in
// registers, lanes 16..31 rows 64..127 of the same columns, so a thread carries 64 values (no
// local-memory spills) and every load or store instruction moves two full 64-byte row segments.
// Butterflies of width 1..32 stay inside the thread, width 64 is one shuffle per value with the
// same operands and rounding as a single 128-value strip would use.
// MODE: 0 no scaling, 1 scale inputs, 2 scale results; the scaling flavour is compiled in so
// the unrolled strip carries no per-element branches.
template <int MODE, bool PER_COL, bool DIVIDE>
__global__ void __launch_bounds__(256, 2)
hadamard_cols_kernel(float* __restrict__ x, int rows, int cols, int ld, int64_t x_stride,
                     const float* __restrict__ scale, int64_t scale_stride)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int half = lane >> 4;
    const int c_want = blockIdx.x * 128 + warp * 16 + (lane & 15);
    const bool active = c_want < cols;
    const int c = active ? c_want : cols - 1;   // inactive lanes shadow a valid column for the shuffles
    const int r0 = blockIdx.y * 128 + half * 64;
    float* base = x + blockIdx.z * x_stride + int64_t(r0) * ld + c;
    // per-row scales of the strip go through shared memory (one value serves the whole row)
    __shared__ float row_scale[128];
    float col_s = 1.0f;
    if constexpr (MODE != 0) {
        const float* vec = scale + blockIdx.z * scale_stride;
        if constexpr (PER_COL) {
            col_s = vec[c];
        } else {
            if (threadIdx.x < 128) row_scale[threadIdx.x] = vec[blockIdx.y * 128 + threadIdx.x];
            __syncthreads();
        }
    }
    auto scaled = [&](float value, int r) {
        const float s = PER_COL ? col_s : row_scale[half * 64 + r];
        return DIVIDE ? __fdiv_rn(value, s) : value * s;
    };
    float v[64];
#pragma unroll
    for (int r = 0; r < 64; ++r) v[r] = base[int64_t(r) * ld];
    if constexpr (MODE == 1) {
#pragma unroll
        for (int r = 0; r < 64; ++r) {
            v[r] = scaled(v[r], r);
            // keep the scalings in order: interleaving 64 of them (IEEE divisions above all) with
            // their row addresses costs more registers than the strip leaves free
            asm volatile("" : "+f"(v[r]));
        }
    }
#pragma unroll
    for (int bit = 1; bit < 64; bit <<= 1) {
#pragma unroll
        for (int r = 0; r < 64; ++r) {
            if ((r & bit) == 0) {
                const float a = v[r], b = v[r | bit];
                v[r] = a + b;
                v[r | bit] = a - b;
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 64; ++r) {
        const float other = __shfl_xor_sync(0xffffffffu, v[r], 16);
        v[r] = half ? other - v[r] : v[r] + other;
    }
#pragma unroll
    for (int r = 0; r < 64; ++r) {
        v[r] *= kInvSqrt128;
        asm volatile("" : "+f"(v[r]));
    }
    if constexpr (MODE == 2) {
#pragma unroll
        for (int r = 0; r < 64; ++r) {
            v[r] = scaled(v[r], r);
            asm volatile("" : "+f"(v[r]));
        }
    }
    if (active) {
        // a pointer the compiler cannot equate with the load addresses: otherwise it keeps all 64
        // row addresses alive across the butterflies for the stores and spills
        float* out = base;
        asm volatile("" : "+l"(out));
#pragma unroll
        for (int r = 0; r < 64; ++r) out[int64_t(r) * ld] = v[r];
    }
}

template <int MODE>
void launch_hadamard_cols(dim3 grid, cudaStream_t s, float* x, int rows, int cols, int ld, int64_t x_stride,
                          const ScaleSpec& sc)
{
    if (sc.per_col) {
        if (sc.divide) hadamard_cols_kernel<MODE, true, true><<<grid, 256, 0, s>>>(x, rows, cols, ld, x_stride, sc.vec, sc.stride);
        else hadamard_cols_kernel<MODE, true, false><<<grid, 256, 0, s>>>(x, rows, cols, ld, x_stride, sc.vec, sc.stride);
    } else {
        if (sc.divide) hadamard_cols_kernel<MODE, false, true><<<grid, 256, 0, s>>>(x, rows, cols, ld, x_stride, sc.vec, sc.stride);
        else hadamard_cols_kernel<MODE, false, false><<<grid, 256, 0, s>>>(x, rows, cols, ld, x_stride, sc.vec, sc.stride);
    }
}

// Column sums of squares: partial[chunk][col] over 256-row chunks, then a fixed-order fold.
__global__ void __launch_bounds__(128)
col_sumsq_partial_kernel(const float* __restrict__ x, int rows, int cols, int ld, int64_t x_stride,
                         float* __restrict__ partial, int chunks)
{
    const int c = blockIdx.x * 128 + threadIdx.x;
    if (c >= cols) return;
    const int chunk = blockIdx.y;
    const int r0 = chunk * 256, r1 = min(rows, r0 + 256);
    const float* base = x + blockIdx.z * x_stride + c;
    float acc = 0.0f;
    for (int r = r0; r < r1; ++r) {
        const float v = base[int64_t(r) * ld];
        acc += v * v;
    }
    partial[(int64_t(blockIdx.z) * chunks + chunk) * cols + c] = acc;
}

__global__ void col_sumsq_fold_kernel(const float* __restrict__ partial, int cols, int chunks,
                                      float* __restrict__ out, int64_t out_stride)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    const float* p = partial + int64_t(blockIdx.z) * chunks * cols + c;
    float acc = 0.0f;
    for (int k = 0; k < chunks; ++k) acc += p[int64_t(k) * cols];
    out[blockIdx.z * out_stride + c] = acc;
}

// Turn a lower Cholesky factor C into the unit block-lower LDL factor used by the feedback
// loop (qsrt/exl3_encoder_backend.py:372-393, 2152-2153): every 16-column block is multiplied
// on the right by the inverse of its diagonal block, diagonal blocks and everything above
// them become zero (identity blocks whose main diagonal is then cleared).  Three launches:
//   inverse : one warp per diagonal block inverts it by forward substitution and parks the
//             result in the tile to its right (above the diagonal: free until the last launch);
//   apply   : grid.x = group of 8 block columns, grid.y = 128-row chunk; every 16-value row piece
//             below its diagonal block is multiplied by that block's parked inverse;
//   zero    : diagonal blocks and everything above them, the parked inverses included.
// The last block column has no rows below it and needs no inverse.
__global__ void __launch_bounds__(32)
block_ldl_inverse_kernel(float* __restrict__ c, int ld)
{
    __shared__ float dl[16][17];
    const int d0 = blockIdx.x * 16;
    const int t = threadIdx.x;
#pragma unroll
    for (int i = t; i < 256; i += 32) dl[i >> 4][i & 15] = c[int64_t(d0 + (i >> 4)) * ld + d0 + (i & 15)];
    __syncwarp();
    if (t < 16) {
        // column t of inv(DL): forward substitution on the lower-triangular diagonal block
        float col[16];
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            float s = (r == t) ? 1.0f : 0.0f;
#pragma unroll
            for (int k = 0; k < 16; ++k)
                if (k < r) s -= dl[r][k] * col[k];
            col[r] = (r < t) ? 0.0f : s / dl[r][r];
        }
#pragma unroll
        for (int r = 0; r < 16; ++r) c[int64_t(d0 + r) * ld + d0 + 16 + t] = col[r];
    }
}

// 128 rows x 8 block columns (128 columns) per CTA.  A lane owns one float4 of a row: block column
// lane/4, columns 4*(lane%4)..+3 of it, so a warp reads and writes 512 contiguous bytes of one row.
// Its 64 inverse entries inv[k][4q..4q+3] stay in registers for all 16 rows the warp visits; the 16
// inputs of a row piece come from the 4 lanes of the group by shuffle.  Sums run over k = 0..15 in
// order, as a single thread per row piece would add them.
__global__ void __launch_bounds__(256)
block_ldl_apply_kernel(float* __restrict__ c, int n, int ld)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b = blockIdx.x * 8 + (lane >> 2), q = lane & 3;
    const int row_begin = blockIdx.y * 128;
    if (row_begin + 127 < blockIdx.x * 128 + 16) return;   // nothing of this chunk lies below the group
    const int d0 = b * 16;
    const bool has_rows = d0 + 16 < n;                      // also excludes block columns past the end
    float4 inv[16];
#pragma unroll
    for (int k = 0; k < 16; ++k)
        inv[k] = has_rows ? *reinterpret_cast<const float4*>(c + int64_t(d0 + k) * ld + d0 + 16 + 4 * q)
                          : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const int group = lane & ~3;
    // eight rows per batch: all loads are issued before the first store of the batch, which the
    // compiler cannot do by itself for loads and stores through the same array
    for (int i0 = 0; i0 < 16; i0 += 8) {
        float4 v[8];
        bool active[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int r = row_begin + warp + 8 * (i0 + u);
            active[u] = has_rows && r < n && r >= d0 + 16;
            v[u] = active[u] ? *reinterpret_cast<const float4*>(c + int64_t(r) * ld + d0 + 4 * q)
                             : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            float4 out = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                const float mine = (k & 3) == 0 ? v[u].x : (k & 3) == 1 ? v[u].y : (k & 3) == 2 ? v[u].z : v[u].w;
                const float in = __shfl_sync(0xffffffffu, mine, group + (k >> 2));
                out.x = fmaf(in, inv[k].x, out.x);
                out.y = fmaf(in, inv[k].y, out.y);
                out.z = fmaf(in, inv[k].z, out.z);
                out.w = fmaf(in, inv[k].w, out.w);
            }
            const int r = row_begin + warp + 8 * (i0 + u);
            if (active[u]) *reinterpret_cast<float4*>(c + int64_t(r) * ld + d0 + 4 * q) = out;
        }
    }
}

// Zero the diagonal blocks and everything above them (row r, columns >= 16*floor(r/16)).
// One block per row, 16-byte stores from the row's diagonal block to its end.
__global__ void __launch_bounds__(256)
block_ldl_zero_upper_kernel(float* __restrict__ c, int n, int ld)
{
    const int r = blockIdx.x;
    float4* row = reinterpret_cast<float4*>(c + int64_t(r) * ld);
    for (int q = (r & ~15) / 4 + threadIdx.x; q < n / 4; q += blockDim.x) row[q] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
}

}  // namespace

extern "C" int qsrtb_hadamard128(float* x, int batch, int rows, int cols, int ld, int64_t x_stride,
                                 int axis, const float* scale, int64_t scale_stride,
                                 int scale_per_col, int scale_divide, int scale_after,
                                 float* row_sumsq, int64_t sumsq_stride, void* stream)
{
    if (!x || batch < 0 || rows < 0 || cols < 0 || ld < cols)
        return qsrtb_fail(QSRTB_EINVAL, "bad matrix arguments");
    if (axis != 0 && axis != 1) return qsrtb_fail(QSRTB_EINVAL, "axis must be 0 or 1");
    if (axis == 1 && ((cols % 128) != 0 || (ld % 4) != 0))
        return qsrtb_fail(QSRTB_EINVAL, "columns must be a multiple of 128");
    if (axis == 0 && (rows % 128) != 0) return qsrtb_fail(QSRTB_EINVAL, "rows must be a multiple of 128");
    if (axis == 0 && row_sumsq) return qsrtb_fail(QSRTB_EINVAL, "row sums are produced by axis 1 only");
    if (batch == 0 || rows == 0 || cols == 0) return QSRTB_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    ScaleSpec sc{scale, scale_stride, scale_per_col, scale_divide, scale_after};
    if (axis == 1) {
        const int64_t warps = int64_t(batch) * rows;
        const int64_t blocks = (warps + 7) / 8;
        hadamard_rows_kernel<<<unsigned(blocks), 256, 0, s>>>(x, batch, rows, cols, ld, x_stride, sc,
                                                             row_sumsq, sumsq_stride);
    } else {
        dim3 grid((cols + 127) / 128, rows / 128, batch);
        if (!sc.vec) hadamard_cols_kernel<0, false, false><<<grid, 256, 0, s>>>(x, rows, cols, ld, x_stride, nullptr, 0);
        else if (sc.after) launch_hadamard_cols<2>(grid, s, x, rows, cols, ld, x_stride, sc);
        else launch_hadamard_cols<1>(grid, s, x, rows, cols, ld, x_stride, sc);
    }
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "hadamard launch");
    return QSRTB_OK;
}

extern "C" int qsrtb_col_sumsq(const float* x, int batch, int rows, int cols, int ld,
                               int64_t x_stride, float* out, int64_t out_stride, float* workspace,
                               size_t workspace_bytes, void* stream)
{
    if (!x || !out || batch < 0 || rows < 0 || cols < 0 || ld < cols)
        return qsrtb_fail(QSRTB_EINVAL, "bad matrix arguments");
    if (batch == 0 || cols == 0) return QSRTB_OK;
    const int chunks = rows > 0 ? (rows + 255) / 256 : 1;
    if (!workspace || workspace_bytes < sizeof(float) * size_t(batch) * chunks * cols)
        return qsrtb_fail(QSRTB_ESCRATCH, "column-sum workspace too small");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    dim3 grid((cols + 127) / 128, chunks, batch);
    col_sumsq_partial_kernel<<<grid, 128, 0, s>>>(x, rows, cols, ld, x_stride, workspace, chunks);
    dim3 grid2((cols + 127) / 128, 1, batch);
    col_sumsq_fold_kernel<<<grid2, 128, 0, s>>>(workspace, cols, chunks, out, out_stride);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "col_sumsq launch");
    return QSRTB_OK;
}

extern "C" int qsrtb_block_ldl_normalize(float* chol, int n, int ld, void* stream)
{
    if (!chol || n < 0 || (n % 16) != 0 || ld < n)
        return qsrtb_fail(QSRTB_EINVAL, "factor must be square with n a multiple of 16");
    if ((ld % 4) != 0 || (reinterpret_cast<uintptr_t>(chol) & 15))
        return qsrtb_fail(QSRTB_EINVAL, "factor rows must be 16-byte aligned");
    if (n == 0) return QSRTB_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int columns = n / 16 - 1;   // block columns with rows below them
    if (columns > 0) {
        block_ldl_inverse_kernel<<<columns, 32, 0, s>>>(chol, ld);
        block_ldl_apply_kernel<<<dim3((n + 127) / 128, (n + 127) / 128), 256, 0, s>>>(chol, n, ld);
    }
    block_ldl_zero_upper_kernel<<<n, 256, 0, s>>>(chol, n, ld);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "block_ldl_normalize launch");
    return QSRTB_OK;
}
