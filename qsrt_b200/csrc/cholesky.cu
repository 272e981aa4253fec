// Blocked Cholesky factorisation of a damped Hessian, entirely on the device.
//
// Right-looking over panels of 128 columns.  Per panel j:
//   chol_diag_kernel : one CTA factors the 128 x 128 diagonal block in shared memory, blocked by 16
//                      columns (float32).  A pivot that is not positive is reported through a device status
//                      word (its 1-based column, as LAPACK's `info`) and every later kernel of the
//                      call turns into a no-op: nothing traps, nothing throws, the host reads the
//                      word once after the call and runs the retry-with-damping loop of the reference
//                      (qsrt/exl3_encoder_backend.py:331-370).
//   chol_panel_kernel: the rows below solve  X * L_jj^T = A  by forward substitution, one row per
//                      thread, 16 columns at a time in registers; X goes back into the matrix and,
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

__device__ __forceinline__ float tf32_head(float x)
{
    uint32_t u = __float_as_uint(x);
    u += 0x00000fffu + ((u >> 13) & 1u);
    return __uint_as_float(u & 0xffffe000u);
}

constexpr int kPitch = kPanel + 1;   // shared-memory tile pitch: conflict-free row and column access
constexpr int kSub = 16;             // inner block of the diagonal factorisation
constexpr int kThreads = 256;

// Factor the w x w block at a[0 .. w)[0 .. w) (pitch ld) in place; w is a multiple of 16.
// Blocked right-looking inside shared memory, 16 columns at a time:
//   (a) warp 0 factors the 16 x 16 diagonal sub-block, a lane per row, the row in registers, the
//       column exchanged by shuffles (no block barrier inside);
//   (b) a thread per remaining row solves its 16 panel entries against that sub-block;
//   (c) two threads per remaining row subtract the panel's outer product from the row's entries
//       left of the diagonal (each reads the other rows' panel entries as 16-byte broadcasts).
// On return the lower triangle holds the factor and the strict upper triangle its transpose
// (which is how the panel kernel wants to read it).
// status[0]: 0 or the 1-based global column of the first non-positive pivot.
__global__ void __launch_bounds__(kThreads)
chol_diag_kernel(float* __restrict__ a, int w, int ld, int first_column, int* __restrict__ status)
{
    if (status[0] != 0) return;
    extern __shared__ __align__(16) float smem[];
    float* tile = smem;                           // [kPanel][kPitch]
    float* pan = smem + kPanel * kPitch;          // [kPanel][kSub]: current panel, rows below the sub-block
    float* fac = pan + kPanel * kSub;             // [kSub][kSub + 1]: current factored sub-block
    __shared__ float fac_inv[kSub];               // reciprocals of its diagonal
    __shared__ int bad;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    if (t == 0) bad = 0;
    if (w == kPanel) {
        // a warp per row and iteration (512 contiguous bytes); all loads are issued before the
        // first shared-memory store, so that their latencies overlap
        constexpr int kRowsPerWarp = kPanel / (kThreads / 32);
        float4 v[kRowsPerWarp];
#pragma unroll
        for (int i = 0; i < kRowsPerWarp; ++i)
            v[i] = *reinterpret_cast<const float4*>(a + int64_t(warp + i * (kThreads / 32)) * ld + 4 * lane);
#pragma unroll
        for (int i = 0; i < kRowsPerWarp; ++i) {
            float* dst = tile + (warp + i * (kThreads / 32)) * kPitch + 4 * lane;
            dst[0] = v[i].x; dst[1] = v[i].y; dst[2] = v[i].z; dst[3] = v[i].w;
        }
    } else {
        for (int i = t; i < w * w; i += kThreads) {
            const int r = i / w, c = i - r * w;
            tile[r * kPitch + c] = a[int64_t(r) * ld + c];
        }
    }
    __syncthreads();
    for (int j0 = 0; j0 < w; j0 += kSub) {
        if (warp == 0) {
            float row[kSub];
            float row_inv = 1.0f;   // lane c: reciprocal of the c-th diagonal entry of the factor
            const int src = lane < kSub ? lane : 0;
#pragma unroll
            for (int k = 0; k < kSub; ++k) row[k] = tile[(j0 + src) * kPitch + j0 + k];
#pragma unroll
            for (int c = 0; c < kSub; ++c) {
                const float p = __shfl_sync(0xffffffffu, row[c], c);
                const bool ok = p > 0.0f && p <= 3.0e38f;   // also rejects NaN and infinity
                if (!ok && lane == 0 && bad == 0) bad = first_column + j0 + c + 1;
                // 1 / sqrt(p) once per column, then products: the serial part of the whole
                // factorisation runs through these few instructions.  Hardware estimate plus one
                // Newton step (relative error about 1e-7, that of a rounded division).
                float inv = 1.0f;
                if (ok) {
                    const float y = rsqrtf(p);
                    inv = y * fmaf(-0.5f * p * y, y, 1.5f);
                }
                const float l = lane > c ? row[c] * inv : (lane == c ? p * inv : 0.0f);
                if (lane == c) row_inv = inv;
                row[c] = l;
#pragma unroll
                for (int k = c + 1; k < kSub; ++k) {
                    const float lk = __shfl_sync(0xffffffffu, l, k);
                    // (entries right of the diagonal, lane < k, are left as they are; written as
                    // arithmetic, since a predicated store makes the compiler keep the row in
                    // local memory)
                    row[k] = fmaf(lane >= k ? -l : 0.0f, lk, row[k]);
                }
            }
            if (lane < kSub) {
#pragma unroll
                for (int k = 0; k < kSub; ++k) {
                    fac[lane * (kSub + 1) + k] = row[k];
                    if (k <= lane) tile[(j0 + lane) * kPitch + j0 + k] = row[k];
                }
                fac_inv[lane] = row_inv;
            }
        }
        __syncthreads();
        if (bad != 0) break;
        const int below = w - j0 - kSub;   // rows under the sub-block
        if (t < below) {
            const int r = j0 + kSub + t;
            float x[kSub];
#pragma unroll
            for (int k = 0; k < kSub; ++k) x[k] = tile[r * kPitch + j0 + k];
            // column by column, so that the updates of one column are independent of each other
#pragma unroll
            for (int c = 0; c < kSub; ++c) {
                x[c] *= fac_inv[c];
#pragma unroll
                for (int k = c + 1; k < kSub; ++k) x[k] = fmaf(-x[c], fac[k * (kSub + 1) + c], x[k]);
            }
#pragma unroll
            for (int k = 0; k < kSub; ++k) {
                tile[r * kPitch + j0 + k] = x[k];
                pan[t * kSub + k] = x[k];
            }
        }
        __syncthreads();
        {
            const int rr = t >> 1, half = t & 1;
            if (rr < below) {
                float mine[kSub];
#pragma unroll
                for (int q = 0; q < kSub / 4; ++q) {
                    const float4 v = *reinterpret_cast<const float4*>(pan + rr * kSub + 4 * q);
                    mine[4 * q] = v.x; mine[4 * q + 1] = v.y; mine[4 * q + 2] = v.z; mine[4 * q + 3] = v.w;
                }
                float* row = tile + (j0 + kSub + rr) * kPitch + j0 + kSub;
                for (int k = half; k <= rr; k += 2) {
                    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
                    for (int q = 0; q < kSub / 4; ++q) {
                        const float4 v = *reinterpret_cast<const float4*>(pan + k * kSub + 4 * q);
                        s0 = fmaf(mine[4 * q], v.x, s0);
                        s1 = fmaf(mine[4 * q + 1], v.y, s1);
                        s2 = fmaf(mine[4 * q + 2], v.z, s2);
                        s3 = fmaf(mine[4 * q + 3], v.w, s3);
                    }
                    row[k] -= (s0 + s1) + (s2 + s3);
                }
            }
        }
        __syncthreads();
    }
    if (bad != 0) {
        if (t == 0) atomicCAS(status, 0, bad);
        return;
    }
    if (w == kPanel) {
#pragma unroll 4
        for (int r = warp; r < kPanel; r += kThreads / 32) {
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = 4 * lane + j;
                v[j] = (c <= r) ? tile[r * kPitch + c] : tile[c * kPitch + r];
            }
            *reinterpret_cast<float4*>(a + int64_t(r) * ld + 4 * lane) = make_float4(v[0], v[1], v[2], v[3]);
        }
    } else {
        for (int i = t; i < w * w; i += kThreads) {
            const int r = i / w, c = i - r * w;
            a[int64_t(r) * ld + c] = (c <= r) ? tile[r * kPitch + c] : tile[c * kPitch + r];
        }
    }
}

// X = A * L^-T for the rows below a factored kPanel x kPanel diagonal block: one row per thread
// (threads 0 .. 127; all 256 threads stage the operands), forward substitution in chunks of 16
// columns held in registers against the transposed factor in shared memory (every thread reads the
// same factor addresses: broadcasts).
//   diag  : the factored diagonal block (lower triangle and its transpose above it, pitch ld)
//   below : first row below it (same columns, pitch ld), `rows` rows
//   hi/lo : [rows, kPanel] planes receiving the TF32 head and tail of X
__global__ void __launch_bounds__(kThreads)
chol_panel_kernel(const float* __restrict__ diag, float* __restrict__ below, int rows, int ld,
                  float* __restrict__ hi, float* __restrict__ lo, const int* __restrict__ status)
{
    if (status[0] != 0) return;
    extern __shared__ __align__(16) float smem[];
    float* lt = smem;                          // lt[k * kPanel + c] = L[c][k]  (k <= c)
    float* tile = smem + kPanel * kPanel;      // [kPanel][kPitch]
    const int t = threadIdx.x;
    const int row0 = blockIdx.x * kPanel;
    const int count = min(kPanel, rows - row0);
    for (int i = t; i < kPanel * kPanel / 4; i += kThreads) {
        const int k = i / (kPanel / 4), c4 = i - k * (kPanel / 4);   // entries left of the diagonal are never read
        reinterpret_cast<float4*>(lt)[i] = *reinterpret_cast<const float4*>(diag + int64_t(k) * ld + 4 * c4);
    }
    for (int i = t; i < count * (kPanel / 4); i += kThreads) {
        const int r = i / (kPanel / 4), c = (i - r * (kPanel / 4)) * 4;
        const float4 v = *reinterpret_cast<const float4*>(below + int64_t(row0 + r) * ld + c);
        float* dst = tile + r * kPitch + c;
        dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
    }
    __syncthreads();
    if (t < count) {
        float* mine = tile + t * kPitch;
        for (int c0 = 0; c0 < kPanel; c0 += kSub) {
            float acc[kSub];
#pragma unroll
            for (int i = 0; i < kSub; ++i) acc[i] = mine[c0 + i];
#pragma unroll 8
            for (int k = 0; k < c0; ++k) {
                const float xv = mine[k];
#pragma unroll
                for (int q = 0; q < kSub / 4; ++q) {
                    const float4 l = *reinterpret_cast<const float4*>(lt + k * kPanel + c0 + 4 * q);
                    acc[4 * q] = fmaf(-xv, l.x, acc[4 * q]);
                    acc[4 * q + 1] = fmaf(-xv, l.y, acc[4 * q + 1]);
                    acc[4 * q + 2] = fmaf(-xv, l.z, acc[4 * q + 2]);
                    acc[4 * q + 3] = fmaf(-xv, l.w, acc[4 * q + 3]);
                }
            }
#pragma unroll
            for (int i = 0; i < kSub; ++i) {
                acc[i] = acc[i] / lt[(c0 + i) * kPanel + c0 + i];
#pragma unroll
                for (int k = i + 1; k < kSub; ++k) acc[k] = fmaf(-acc[i], lt[(c0 + i) * kPanel + c0 + k], acc[k]);
                mine[c0 + i] = acc[i];
            }
        }
    }
    __syncthreads();
    for (int i = t; i < count * (kPanel / 4); i += kThreads) {
        const int r = i / (kPanel / 4), c = (i - r * (kPanel / 4)) * 4;
        const float* src = tile + r * kPitch + c;
        const float4 v = make_float4(src[0], src[1], src[2], src[3]);
        const float4 head = make_float4(tf32_head(v.x), tf32_head(v.y), tf32_head(v.z), tf32_head(v.w));
        *reinterpret_cast<float4*>(below + int64_t(row0 + r) * ld + c) = v;
        *reinterpret_cast<float4*>(hi + int64_t(row0 + r) * kPanel + c) = head;
        *reinterpret_cast<float4*>(lo + int64_t(row0 + r) * kPanel + c) =
            make_float4(tf32_head(v.x - head.x), tf32_head(v.y - head.y), tf32_head(v.z - head.z), tf32_head(v.w - head.w));
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
    if (!a || n < 0 || ld < n || (n % 16) != 0)
        return qsrtb_fail(QSRTB_EINVAL, "the matrix size must be a multiple of 16 (the block size of the block-LDL factor)");
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

    const int diag_smem = (kPanel * kPitch + kPanel * kSub + kSub * (kSub + 1)) * int(sizeof(float));
    const int panel_smem = (kPanel * kPanel + kPanel * kPitch) * int(sizeof(float));
    cudaError_t err = cudaFuncSetAttribute(chol_diag_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, diag_smem);
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "cudaFuncSetAttribute(chol_diag)");
    err = cudaFuncSetAttribute(chol_panel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, panel_smem);
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "cudaFuncSetAttribute(chol_panel)");

    for (int j = 0; j < n; j += kPanel) {
        const int w = n - j < kPanel ? n - j : kPanel;
        float* block = a + int64_t(j) * ld + j;
        chol_diag_kernel<<<1, kThreads, diag_smem, s>>>(block, w, ld, j, status);
        const int rows = n - j - w;
        if (rows <= 0) break;
        // w == kPanel here: only the last panel can be narrower, and it has no rows below
        float* below = a + int64_t(j + w) * ld + j;
        chol_panel_kernel<<<(rows + kPanel - 1) / kPanel, kThreads, panel_smem, s>>>(
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
