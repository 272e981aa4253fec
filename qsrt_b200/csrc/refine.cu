// Dense-H path refinement: scoring and acceptance of replacement paths for one 16-row block
// (the per-block tail of refine_h2_viterbi_paths, qsrt/h2_viterbi_refine.py:451-505, with
// _conditional_scores :261-279 inside).
//
// One CTA per 16x16 tile, one thread per tile element (i = row, c = column).  For the stored
// reconstruction (candidate 0) and each proposed one the CTA forms D = target - candidate in
// float32, converts it to the score type T, computes (H_bb D)[i, c] from shared memory and reduces
// D * (H_bb D) * a_c over the tile in a fixed order.  The first candidate with the smallest score
// replaces the stored tile when  best + abs_tol + rel_tol * |current| < current;  the CTA then
// rewrites the reconstruction rows, the tile's 256 states, the error rows (T(weight - new)) and
// the error change every later row block needs (delta = new error - old error, zero for a tile
// that keeps its path).  Traffic per tile is (3 + V) float rows + 2 T rows + (1 + V) * 512 B of
// states, touched once: the kernel is a single streaming pass over the block.
#include <cuda_runtime.h>
#include <stdint.h>

#include "qsrtb_internal.h"

namespace {

template <typename T>
__device__ __forceinline__ T block_sum(T value, T* partial)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) value += __shfl_xor_sync(0xffffffffu, value, o);
    __syncthreads();  // the previous reduction's readers are done with `partial`
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = value;
    __syncthreads();
    T total = partial[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) total += partial[w];
    return total;
}

template <typename T>
__global__ void __launch_bounds__(256)
refine_select_kernel(const float* __restrict__ weight, int ldw, const float* __restrict__ target, int ldt,
                     float* __restrict__ recon, int ldq, const float* __restrict__ cand, int ldc,
                     int64_t cand_stride, int variants, const int16_t* __restrict__ cand_states,
                     int64_t cand_state_stride, int16_t* __restrict__ states, const T* __restrict__ h_block,
                     int ldh, const T* __restrict__ col_weights, T* __restrict__ err, int lde,
                     T* __restrict__ delta, int ldd, T abs_tol, T rel_tol,
                     unsigned long long* __restrict__ counters)
{
    __shared__ T sh_h[16][17];
    __shared__ T sh_d[16][17];
    __shared__ T sh_partial[8];
    const int t = threadIdx.x, i = t >> 4, c = t & 15;
    const int tile = blockIdx.x;
    const int64_t col = int64_t(tile) * 16 + c;
    sh_h[i][c] = h_block[int64_t(i) * ldh + c];
    const float tgt = target[int64_t(i) * ldt + col];
    const float current = recon[int64_t(i) * ldq + col];
    const T a_c = col_weights[col];

    T current_score = T(0), best_score = T(0);
    int best = 0;
    float best_value = current;
    for (int m = 0; m <= variants; ++m) {
        const float value = m == 0 ? current : cand[int64_t(m - 1) * cand_stride + int64_t(i) * ldc + col];
        const T d = T(__fsub_rn(tgt, value));
        __syncthreads();  // sh_d of the previous candidate has been read; sh_h is written
        sh_d[i][c] = d;
        __syncthreads();
        T hd = T(0);
#pragma unroll
        for (int j = 0; j < 16; ++j) hd += sh_h[i][j] * sh_d[j][c];
        const T score = block_sum<T>(d * hd * a_c, sh_partial);
        if (m == 0) {
            current_score = best_score = score;
        } else if (score < best_score) {
            best_score = score;
            best = m;
            best_value = value;
        }
    }
    const T tolerance = abs_tol + rel_tol * (current_score < T(0) ? -current_score : current_score);
    const bool accept = best_score + tolerance < current_score;

    // distinct payloads among the stored path and the proposals (a statistic of the sweep)
    const int16_t own = states[int64_t(tile) * 256 + t];
    int unique = 1;
    for (int m = 0; m < variants; ++m) {
        const int16_t mine = cand_states[int64_t(m) * cand_state_stride + int64_t(tile) * 256 + t];
        int duplicate = __syncthreads_and(mine == own);
        for (int e = 0; e < m && !duplicate; ++e) {
            const int16_t other = cand_states[int64_t(e) * cand_state_stride + int64_t(tile) * 256 + t];
            duplicate = __syncthreads_and(mine == other);
        }
        unique += duplicate ? 0 : 1;
    }

    const int64_t e_at = int64_t(i) * lde + col;
    if (accept) {
        recon[int64_t(i) * ldq + col] = best_value;
        states[int64_t(tile) * 256 + t] = cand_states[int64_t(best - 1) * cand_state_stride + int64_t(tile) * 256 + t];
        const T fresh = T(__fsub_rn(weight[int64_t(i) * ldw + col], best_value));
        delta[int64_t(i) * ldd + col] = fresh - err[e_at];
        err[e_at] = fresh;
    } else {
        delta[int64_t(i) * ldd + col] = T(0);
    }
    if (t == 0) {
        if (accept) atomicAdd(&counters[0], 1ull);
        atomicAdd(&counters[1], static_cast<unsigned long long>(unique));
    }
}

}  // namespace

extern "C" int qsrtb_refine_select(const float* weight, int ldw, const float* target, int ldt, float* recon, int ldq,
                                   int n, const float* cand, int ldc, int64_t cand_stride, int variants,
                                   const int16_t* cand_states, int64_t cand_state_stride, int16_t* states,
                                   const void* h_block, int ldh, const void* col_weights, void* err, int lde,
                                   void* delta, int ldd, double abs_tol, double rel_tol, int score_is_double,
                                   unsigned long long* counters, void* stream)
{
    if (n < 0 || (n % 16) != 0) return qsrtb_fail(QSRTB_EINVAL, "n must be a multiple of 16");
    if (variants < 0) return qsrtb_fail(QSRTB_EINVAL, "variants must be nonnegative");
    if (n == 0) return QSRTB_OK;
    if (!weight || !target || !recon || !states || !h_block || !col_weights || !err || !delta || !counters ||
        (variants > 0 && (!cand || !cand_states)))
        return qsrtb_fail(QSRTB_EINVAL, "null pointer");
    if (ldw < n || ldt < n || ldq < n || lde < n || ldd < n || (variants > 0 && ldc < n) || ldh < 16)
        return qsrtb_fail(QSRTB_EINVAL, "row pitch smaller than the block");
    const int tiles = n / 16;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (score_is_double)
        refine_select_kernel<double><<<tiles, 256, 0, s>>>(
            weight, ldw, target, ldt, recon, ldq, cand, ldc, cand_stride, variants, cand_states, cand_state_stride,
            states, static_cast<const double*>(h_block), ldh, static_cast<const double*>(col_weights),
            static_cast<double*>(err), lde, static_cast<double*>(delta), ldd, abs_tol, rel_tol, counters);
    else
        refine_select_kernel<float><<<tiles, 256, 0, s>>>(
            weight, ldw, target, ldt, recon, ldq, cand, ldc, cand_stride, variants, cand_states, cand_state_stride,
            states, static_cast<const float*>(h_block), ldh, static_cast<const float*>(col_weights),
            static_cast<float*>(err), lde, static_cast<float*>(delta), ldd, float(abs_tol), float(rel_tol), counters);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return qsrtb_fail_cuda(e, "refine_select launch");
    return QSRTB_OK;
}
