// Calibration Hessian accumulation:  C (+)= sum_r w_r * x_r x_r^T  over routed activation rows.
//
// Restates the chunked `addmm_(x.T, x * w)` of the reference (qsrt/candidate_hessian.py:70-112,
// qsrt/capture.py:714-731) as a weighted SYRK that only computes the lower-triangular tiles
// (half the flops of the reference's full square) with float32 accumulation, followed by one
// pass that divides by the weight sum and mirrors the triangle, which yields the exactly
// symmetric matrix the reference obtains from (C + C^T) / 2.
//
// Register-tiled SIMT kernel: a CTA owns a BM x BM output tile, streams 16-row slabs of X
// (row-major, so both operand slabs are contiguous 512-byte runs) through shared memory with
// the row weight folded into one operand, and each thread keeps a TM x TM accumulator block.
#include <cuda_runtime.h>
#include <stdint.h>

#include "qsrtb_internal.h"

namespace {

constexpr int kSlab = 16;

template <int BM, int TM>
__global__ void __launch_bounds__((BM / TM) * (BM / TM))
weighted_syrk_lower_kernel(const float* __restrict__ x, const float* __restrict__ w, int64_t rows,
                           int d, int ldx, float* __restrict__ c, int ldc, int accumulate)
{
    constexpr int T = BM / TM;          // threads per tile edge
    constexpr int NT = T * T;
    __shared__ __align__(16) float sa[kSlab][BM];
    __shared__ __align__(16) float sb[kSlab][BM];
    // blockIdx.x enumerates tile pairs (bi >= bj) row by row
    int bi = int((sqrtf(8.0f * float(blockIdx.x) + 1.0f) - 1.0f) * 0.5f);
    while ((bi + 1) * (bi + 2) / 2 <= int(blockIdx.x)) ++bi;
    while (bi * (bi + 1) / 2 > int(blockIdx.x)) --bi;
    const int bj = int(blockIdx.x) - bi * (bi + 1) / 2;
    const int i0 = bi * BM, j0 = bj * BM;
    const int tid = threadIdx.x;
    const int ty = tid / T, tx = tid % T;

    float acc[TM][TM];
#pragma unroll
    for (int a = 0; a < TM; ++a)
#pragma unroll
        for (int b = 0; b < TM; ++b) acc[a][b] = 0.0f;

    for (int64_t r0 = 0; r0 < rows; r0 += kSlab) {
        // load a slab of kSlab rows x BM columns for each operand (guarded)
        for (int e = tid; e < kSlab * BM; e += NT) {
            const int rr = e / BM, cc = e % BM;
            const int64_t r = r0 + rr;
            float va = 0.0f, vb = 0.0f;
            if (r < rows) {
                const float wr = w ? w[r] : 1.0f;
                if (i0 + cc < d) va = x[r * ldx + i0 + cc];
                if (j0 + cc < d) vb = x[r * ldx + j0 + cc] * wr;
            }
            sa[rr][cc] = va;
            sb[rr][cc] = vb;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kSlab; ++k) {
            float ra[TM], rb[TM];
#pragma unroll
            for (int a = 0; a < TM; a += 4) {
                const float4 v = *reinterpret_cast<const float4*>(&sa[k][ty * TM + a]);
                ra[a] = v.x; ra[a + 1] = v.y; ra[a + 2] = v.z; ra[a + 3] = v.w;
            }
#pragma unroll
            for (int b = 0; b < TM; b += 4) {
                const float4 v = *reinterpret_cast<const float4*>(&sb[k][tx * TM + b]);
                rb[b] = v.x; rb[b + 1] = v.y; rb[b + 2] = v.z; rb[b + 3] = v.w;
            }
#pragma unroll
            for (int a = 0; a < TM; ++a)
#pragma unroll
                for (int b = 0; b < TM; ++b) acc[a][b] = fmaf(ra[a], rb[b], acc[a][b]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int a = 0; a < TM; ++a) {
        const int i = i0 + ty * TM + a;
        if (i >= d) continue;
#pragma unroll
        for (int b = 0; b < TM; ++b) {
            const int j = j0 + tx * TM + b;
            if (j >= d || j > i) continue;
            float* dst = c + int64_t(i) * ldc + j;
            *dst = accumulate ? (*dst + acc[a][b]) : acc[a][b];
        }
    }
}

// lower triangle / denom -> full symmetric matrix.  One block (32 x 8 threads) per 32 x 32 tile
// of the lower triangle (tile pairs enumerated in one dimension, so no block is idle); a thread
// moves four elements of the tile and four of its mirror image.
__global__ void __launch_bounds__(256)
finish_symmetric_kernel(float* __restrict__ c, int d, int ldc, float denom)
{
    __shared__ float tile[32][33];
    int bi = int((sqrtf(8.0f * float(blockIdx.x) + 1.0f) - 1.0f) * 0.5f);
    while ((bi + 1) * (bi + 2) / 2 <= int(blockIdx.x)) ++bi;
    while (bi * (bi + 1) / 2 > int(blockIdx.x)) --bi;
    const int bj = int(blockIdx.x) - bi * (bi + 1) / 2;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = bi * 32 + ty + 8 * k, j = bj * 32 + tx;
        v[k] = (i < d && j < d && j <= i) ? c[int64_t(i) * ldc + j] : 0.0f;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = bi * 32 + ty + 8 * k, j = bj * 32 + tx;
        v[k] = __fdiv_rn(v[k], denom);
        if (i < d && j < d && j <= i) c[int64_t(i) * ldc + j] = v[k];
        tile[ty + 8 * k][tx] = v[k];
    }
    __syncthreads();
    // transposed store: element (row = bj*32 + r, col = bi*32 + tx) strictly above the diagonal
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int ti = bj * 32 + ty + 8 * k, tj = bi * 32 + tx;
        if (ti < d && tj < d && tj > ti) c[int64_t(ti) * ldc + tj] = tile[tx][ty + 8 * k];
    }
}

}  // namespace

extern "C" int qsrtb_hessian_accumulate(const float* rows, const float* weights, int64_t n_rows,
                                        int d, int ld_rows, float* lower, int ld_h, int accumulate,
                                        void* stream)
{
    if (!lower || d <= 0 || ld_h < d || n_rows < 0) return qsrtb_fail(QSRTB_EINVAL, "bad Hessian arguments");
    if (n_rows > 0 && (!rows || ld_rows < d)) return qsrtb_fail(QSRTB_EINVAL, "bad activation rows");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (d >= 1024) {
        const int nb = (d + 127) / 128;
        weighted_syrk_lower_kernel<128, 8><<<nb * (nb + 1) / 2, 256, 0, s>>>(
            rows, weights, n_rows, d, ld_rows, lower, ld_h, accumulate);
    } else {
        const int nb = (d + 63) / 64;
        weighted_syrk_lower_kernel<64, 4><<<nb * (nb + 1) / 2, 256, 0, s>>>(
            rows, weights, n_rows, d, ld_rows, lower, ld_h, accumulate);
    }
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "hessian_accumulate launch");
    return QSRTB_OK;
}

extern "C" int qsrtb_hessian_finish(float* h, int d, int ld_h, double weight_sum, void* stream)
{
    if (!h || d <= 0 || ld_h < d) return qsrtb_fail(QSRTB_EINVAL, "bad Hessian arguments");
    if (!(weight_sum > 0.0)) return qsrtb_fail(QSRTB_EINVAL, "covariance weights must have a positive finite sum");
    const int nb = (d + 31) / 32;
    finish_symmetric_kernel<<<nb * (nb + 1) / 2, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        h, d, ld_h, float(weight_sum));
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "hessian_finish launch");
    return QSRTB_OK;
}
