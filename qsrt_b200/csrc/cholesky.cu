// Blocked Cholesky factorisation of a damped Hessian, entirely on the device.
//
// Right-looking over panels of 128 columns.  Per panel j:
//   chol_diag_kernel : one CTA factors the 128 x 128 diagonal block in shared memory (unblocked,
//                      float32).  A pivot that is not positive is reported through a device status
//                      word (its 1-based column, as LAPACK's `info`) and every later kernel of the
//                      call turns into a no-op: nothing traps, nothing throws, the host reads the
//                      word once after the call and runs the retry-with-damping loop of the reference
//                      (qsrt/exl3_encoder_backend.py:331-370).
//   chol_panel_kernel: the rows below solve  X * L_jj^T = A  by forward substitution, one row per
//                      thread with eight columns register-blocked; X goes back into the matrix and,
//                      split into its TF32 head and tail, into the two operand planes of the update.
//   trailing update  : A_22 -= X X^T on the tensor cores (qsrtb_gemm3x_tc: tcgen05 / TMEM, three
//                      TF32 products per float32 product), lower tiles only.
// The strict upper triangle is scratch: the diagonal blocks keep a transposed copy of their factor
// there and the rest is left as it was.  Callers that want the zeros of torch's `cholesky` clear it
// (qsrtb_block_ldl_normalize overwrites it anyway).
#include <cuda_runtime.h>
#include <stdint.h>

#include "qsrtb_internal.h"

namespace {

constexpr int kPanel = 128;
constexpr int kRowsPerCta = 64;

__device__ __forceinline__ float tf32_head(float x)
{
    uint32_t u = __float_as_uint(x);
    u += 0x00000fffu + ((u >> 13) & 1u);
    return __uint_as_float(u & 0xffffe000u);
}

// Factor the w x w block at a[0 .. w)[0 .. w) (pitch ld) in place (lower triangle).
// status[0]: 0 or the 1-based global column of the first non-positive pivot.
__global__ void __launch_bounds__(256)
chol_diag_kernel(float* __restrict__ a, int w, int ld, int first_column, int* __restrict__ status)
{
    if (status[0] != 0) return;
    extern __shared__ float block[];   // [w][kPanel + 1]
    constexpr int pitch = kPanel + 1;
    __shared__ int bad;
    const int t = threadIdx.x;
    if (t == 0) bad = 0;
    for (int i = t; i < w * w; i += blockDim.x) {
        const int r = i / w, c = i - r * w;
        block[r * pitch + c] = (c <= r) ? a[int64_t(r) * ld + c] : 0.0f;
    }
    __syncthreads();
    for (int c = 0; c < w; ++c) {
        if (t == 0) {
            const float pivot = block[c * pitch + c];
            if (!(pivot > 0.0f) || !(pivot <= 3.0e38f)) {   // also catches NaN and infinity
                bad = first_column + c + 1;
                block[c * pitch + c] = 1.0f;
            } else {
                block[c * pitch + c] = sqrtf(pivot);
            }
        }
        __syncthreads();
        if (bad != 0) break;
        const float diag = block[c * pitch + c];
        for (int r = c + 1 + t; r < w; r += blockDim.x) block[r * pitch + c] = block[r * pitch + c] / diag;
        __syncthreads();
        // rank-1 update of the trailing lower triangle: element (r, k), c < k <= r < w
        for (int r = c + 1 + (t >> 4); r < w; r += 16) {
            const float lr = block[r * pitch + c];
            for (int k = c + 1 + (t & 15); k <= r; k += 16)
                block[r * pitch + k] = fmaf(-lr, block[k * pitch + c], block[r * pitch + k]);
        }
        __syncthreads();
    }
    if (bad != 0) {
        if (t == 0) atomicCAS(status, 0, bad);
        return;
    }
    // lower triangle: the factor; strict upper triangle: its transpose, which is how the panel
    // kernel wants to read it (row k holds L[k..w)[k], contiguous)
    for (int i = t; i < w * w; i += blockDim.x) {
        const int r = i / w, c = i - r * w;
        a[int64_t(r) * ld + c] = (c <= r) ? block[r * pitch + c] : block[c * pitch + r];
    }
}

// X = A * L^-T for kRowsPerCta rows below a factored kPanel x kPanel diagonal block.
//   diag  : the factored diagonal block (lower triangle and its transpose above it, pitch ld)
//   below : first row below it (same columns, pitch ld), `rows` rows
//   hi/lo : [rows, kPanel] planes receiving the TF32 head and tail of X
__global__ void __launch_bounds__(kRowsPerCta)
chol_panel_kernel(const float* __restrict__ diag, float* __restrict__ below, int rows, int ld,
                  float* __restrict__ hi, float* __restrict__ lo, const int* __restrict__ status)
{
    if (status[0] != 0) return;
    extern __shared__ float smem[];
    float* lt = smem;                          // lt[t * kPanel + c] = L[c][t]  (t <= c)
    float* x = smem + kPanel * kPanel;         // x[r * (kPanel + 1) + c]
    constexpr int xp = kPanel + 1;
    const int t = threadIdx.x;
    const int row0 = blockIdx.x * kRowsPerCta;
    const int count = min(kRowsPerCta, rows - row0);
    for (int i = t; i < kPanel * kPanel; i += kRowsPerCta) {
        const int k = i / kPanel, c = i - k * kPanel;   // entries with c < k are never read
        lt[i] = diag[int64_t(k) * ld + c];
    }
    for (int i = t; i < count * kPanel; i += kRowsPerCta) {
        const int r = i / kPanel, c = i - r * kPanel;
        x[r * xp + c] = below[int64_t(row0 + r) * ld + c];
    }
    __syncthreads();
    if (t < count) {
        float* mine = x + t * xp;
        for (int c0 = 0; c0 < kPanel; c0 += 8) {
            float acc[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = mine[c0 + i];
            for (int k = 0; k < c0; ++k) {
                const float xv = mine[k];
                const float4 l0 = *reinterpret_cast<const float4*>(lt + k * kPanel + c0);
                const float4 l1 = *reinterpret_cast<const float4*>(lt + k * kPanel + c0 + 4);
                acc[0] = fmaf(-xv, l0.x, acc[0]); acc[1] = fmaf(-xv, l0.y, acc[1]);
                acc[2] = fmaf(-xv, l0.z, acc[2]); acc[3] = fmaf(-xv, l0.w, acc[3]);
                acc[4] = fmaf(-xv, l1.x, acc[4]); acc[5] = fmaf(-xv, l1.y, acc[5]);
                acc[6] = fmaf(-xv, l1.z, acc[6]); acc[7] = fmaf(-xv, l1.w, acc[7]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float s = acc[i];
#pragma unroll
                for (int k = 0; k < i; ++k) s = fmaf(-acc[k], lt[(c0 + k) * kPanel + c0 + i], s);
                acc[i] = s / lt[(c0 + i) * kPanel + c0 + i];
                mine[c0 + i] = acc[i];
            }
        }
    }
    __syncthreads();
    for (int i = t; i < count * kPanel; i += kRowsPerCta) {
        const int r = i / kPanel, c = i - r * kPanel;
        const float v = x[r * xp + c];
        const float head = tf32_head(v);
        below[int64_t(row0 + r) * ld + c] = v;
        hi[int64_t(row0 + r) * kPanel + c] = head;
        lo[int64_t(row0 + r) * kPanel + c] = tf32_head(v - head);
    }
}

}  // namespace

extern "C" int qsrtb_cholesky_workspace_bytes(int n, size_t* bytes)
{
    if (!bytes || n < 0) return qsrtb_fail(QSRTB_EINVAL, "bad workspace query");
    const size_t rows = n > kPanel ? size_t(n - kPanel) : 0;
    *bytes = 2 * rows * kPanel * sizeof(float) + 256;
    return QSRTB_OK;
}

extern "C" int qsrtb_cholesky_blocked(float* a, int n, int ld, void* workspace, size_t workspace_bytes,
                                      int* status, void* stream)
{
    if (!a || n < 0 || ld < n) return qsrtb_fail(QSRTB_EINVAL, "bad matrix arguments");
    if ((ld % 4) != 0 || (reinterpret_cast<uintptr_t>(a) & 15))
        return qsrtb_fail(QSRTB_EINVAL, "matrix rows must be 16-byte aligned");
    if (!status) return qsrtb_fail(QSRTB_EINVAL, "status pointer required");
    if (n == 0) return QSRTB_OK;
    size_t need = 0;
    qsrtb_cholesky_workspace_bytes(n, &need);
    if (n > kPanel && (!workspace || workspace_bytes < need))
        return qsrtb_fail(QSRTB_ESCRATCH, "Cholesky workspace too small");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* hi = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
    float* lo = hi + (n > kPanel ? size_t(n - kPanel) * kPanel : 0);

    const int diag_smem = kPanel * (kPanel + 1) * int(sizeof(float));
    const int panel_smem = (kPanel * kPanel + kRowsPerCta * (kPanel + 1)) * int(sizeof(float));
    cudaError_t err = cudaFuncSetAttribute(chol_diag_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, diag_smem);
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "cudaFuncSetAttribute(chol_diag)");
    err = cudaFuncSetAttribute(chol_panel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, panel_smem);
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "cudaFuncSetAttribute(chol_panel)");

    for (int j = 0; j < n; j += kPanel) {
        const int w = n - j < kPanel ? n - j : kPanel;
        float* block = a + int64_t(j) * ld + j;
        chol_diag_kernel<<<1, 256, diag_smem, s>>>(block, w, ld, j, status);
        const int rows = n - j - w;
        if (rows <= 0) break;
        // w == kPanel here: only the last panel can be narrower, and it has no rows below
        float* below = a + int64_t(j + w) * ld + j;
        chol_panel_kernel<<<(rows + kRowsPerCta - 1) / kRowsPerCta, kRowsPerCta, panel_smem, s>>>(
            block, below, rows, ld, hi, lo, status);
        err = cudaGetLastError();
        if (err != cudaSuccess) return qsrtb_fail_cuda(err, "Cholesky panel launch");
        const int rc = qsrtb_gemm3x_tc(hi, lo, kPanel, 0, hi, lo, kPanel, 0, 1, rows, rows, kPanel,
                                       a + int64_t(j + w) * ld + (j + w), ld, 0, -1.0f, 1.0f,
                                       /*lower_only=*/1, /*transposed_out=*/0, status, status + 1, stream);
        if (rc != QSRTB_OK) return rc;
    }
    err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "Cholesky launch");
    return QSRTB_OK;
}
