// Per-tile error surfaces for rate allocation (HBM-bound): one float64 value per 16x16 encoder
// tile of two aligned row-major float32 matrices a, b [K, N]:
//   mode 0 : sum (b - a)^2   - tile_squared_error (qsrt/high_rate_allocation.py:55-73);
//   mode 1 : sum  a * b      - the last step of dense_h_tile_error_contributions (:136-148), the
//            elementwise product of the regularised error and its gradient.
// As in the reference the difference / product is rounded to float32 and the 256 terms are
// added in float64.  One warp per tile: a lane reads half a tile row (two 16-byte loads per
// matrix), folds its eight terms and the warp reduces with shuffles in a fixed order; eight
// tiles of one tile row per block, so every load instruction covers whole 64-byte row pieces of
// neighbouring tiles.
#include <cuda_runtime.h>
#include <stdint.h>

#include "qsrtb_internal.h"

namespace {

template <int MODE>
__global__ void __launch_bounds__(256)
tile_reduce_kernel(const float* __restrict__ a, const float* __restrict__ b, int tiles_k, int tiles_n,
                   int lda, int ldb, double* __restrict__ out)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tn = blockIdx.x * 8 + warp, tk = blockIdx.y;
    if (tn >= tiles_n) return;
    const int row = tk * 16 + (lane >> 1), col = tn * 16 + (lane & 1) * 8;
    const float4* pa = reinterpret_cast<const float4*>(a + int64_t(row) * lda + col);
    const float4* pb = reinterpret_cast<const float4*>(b + int64_t(row) * ldb + col);
    const float4 a0 = pa[0], a1 = pa[1], b0 = pb[0], b1 = pb[1];
    const float x[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const float y[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    double acc = 0.0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float term;
        if constexpr (MODE == 0) {
            const float e = __fsub_rn(y[i], x[i]);
            term = __fmul_rn(e, e);
        } else {
            term = __fmul_rn(x[i], y[i]);
        }
        acc += double(term);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
    if (lane == 0) out[int64_t(tk) * tiles_n + tn] = acc;
}

}  // namespace

extern "C" int qsrtb_tile_reduce(const float* a, const float* b, int rows, int cols, int lda, int ldb, int mode,
                                 double* out, void* stream)
{
    if (rows < 0 || cols < 0 || (rows % 16) != 0 || (cols % 16) != 0)
        return qsrtb_fail(QSRTB_EINVAL, "tile error inputs must be 16-by-16 aligned");
    if (mode != 0 && mode != 1) return qsrtb_fail(QSRTB_EINVAL, "mode must be 0 (squared difference) or 1 (product)");
    if (rows == 0 || cols == 0) return QSRTB_OK;
    if (!a || !b || !out) return qsrtb_fail(QSRTB_EINVAL, "null pointer");
    if (lda < cols || ldb < cols || (lda % 4) != 0 || (ldb % 4) != 0 || (reinterpret_cast<uintptr_t>(a) & 15) ||
        (reinterpret_cast<uintptr_t>(b) & 15))
        return qsrtb_fail(QSRTB_EINVAL, "matrices need 16-byte aligned rows");
    const int tiles_k = rows / 16, tiles_n = cols / 16;
    if (tiles_k > 65535) return qsrtb_fail(QSRTB_EINVAL, "too many tile rows");
    const dim3 grid(unsigned((tiles_n + 7) / 8), unsigned(tiles_k));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (mode == 0) tile_reduce_kernel<0><<<grid, 256, 0, s>>>(a, b, tiles_k, tiles_n, lda, ldb, out);
    else tile_reduce_kernel<1><<<grid, 256, 0, s>>>(a, b, tiles_k, tiles_n, lda, ldb, out);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "tile_reduce launch");
    return QSRTB_OK;
}
