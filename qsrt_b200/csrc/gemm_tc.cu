// Float32-accurate matrix product on the 5th-generation tensor cores:
//
//     D[z] = alpha * A[z] * B[z]^T + beta * D[z]        A: [M, K],  B: [N, K]  (both K-major)
//
// as a TMA-fed, warp-specialised tcgen05 (UMMA) TF32 contraction with the accumulators in tensor
// memory.  It serves the three dense contractions of the encoder that are not the Hessian itself:
// the trailing update of the blocked Cholesky (A = B = the panel, lower tiles only, alpha = -1),
// the BlockLDLQ feedback products (A = transposed factor, B = transposed error rows) and the routed
// scoring products (A = rows, B = decoded weights).
//
// Precision: the operands arrive already split into a TF32 head and a TF32 tail (x = hi + lo, both
// exactly representable in TF32; qsrtb_split_tf32 makes them) and the kernel accumulates the three
// significant products hi*hi + lo*hi + hi*lo in float32.  The tensor core adds each 8-deep product
// group to its accumulator with truncation, so long contractions are cut into segments of 60
// instruction groups whose partial sums leave tensor memory and are added in round-to-nearest
// float32 registers (the scheme of the Hessian kernel in hessian_tc.cu).
//
// One CTA (6 warps) per 128 x 128 tile of D:
//   warp 0     : TMA producer; per step of 32 contraction elements four 128 x 32 operand tiles
//                (16 KiB each, 128-byte swizzle) into one of three stages, "full" mbarrier;
//   warp 1     : MMA issuer; twelve 128x128x8 tcgen05.mma.kind::tf32 per stage, tcgen05.commit to
//                the stage's "empty" mbarrier and per segment to the accumulator's "ready" mbarrier;
//   warps 2..5 : epilogue; each owns the 32 tensor-memory lanes (= rows of the tile) of its warp
//                quadrant, adds the segments in registers and finally writes alpha * sum + beta * D,
//                either row-major (through a shared-memory transpose, so that global memory is read
//                and written in whole 512-byte row pieces) or transposed (D[n, m]), with row / column
//                limits so that M and N need not be multiples of 128 (the loads rely on TMA's zero
//                fill past the end).
// No clusters and no multicast: all operands are this GPU's own memory.  Every mbarrier wait is
// bounded; on expiry the kernel raises a status flag, lets its copies land, frees its tensor
// memory and returns.
#include <cuda_runtime.h>
#include <stdint.h>

#include "qsrtb_internal.h"

#if !defined(QSRTB_NO_CUTLASS)

#include "tc_common.cuh"

namespace qsrtb_tc {

using namespace cute;

namespace gemm3x {

constexpr int kTile = 128;
constexpr int kBlockK = 32;
constexpr int kStages = 3;
constexpr int kThreads = 192;
constexpr int kSegmentSteps = 5;
constexpr int kTileBytes = kTile * kBlockK * 4;
constexpr int kStagePitch = kTile + 4;   // floats per row of the epilogue's staging block (16-byte aligned rows)
static_assert(4 * 32 * kStagePitch * 4 <= 4 * kStages * kTileBytes, "the staging blocks must fit the operand stages");

using Element = cutlass::tfloat32_t;

struct Maps {
    CUtensorMap a_hi, a_lo, b_hi, b_lo;
};

struct Params {
    int m, n, k_steps;
    int tiles_m, tiles_n;
    int lower_only;        // square problems: only tiles with bi >= bj
    int transposed_out;    // 0: D[m * ldd + n], 1: D[n * ldd + m]
    int ldd;
    int64_t d_stride;      // elements between consecutive matrices of D
    float alpha, beta;
    float* d;
    const int* skip_flag;  // optional device flag: a nonzero value turns the launch into a no-op
    int* status;
};

template <class SmemLayout>
struct SharedStorage {
    // operand kinds: 0 = hi(A), 1 = lo(A) (rows of tile bi); 2 = hi(B), 3 = lo(B) (rows of tile bj)
    alignas(1024) cute::ArrayEngine<Element, cute::cosize_v<SmemLayout>> operand[4];
    alignas(16) uint64_t full[kStages];
    alignas(16) uint64_t empty[kStages];
    alignas(16) uint64_t ready[2];
    alignas(16) uint64_t free_[2];
    uint32_t tmem_base_ptr;
    volatile int failed;
    volatile uint32_t first_failure;
};

template <class TiledMMA, class SmemLayout>
__global__ void __launch_bounds__(kThreads, 1)
gemm3x_tcgen05_kernel(const __grid_constant__ Maps maps, const Params p, TiledMMA tiled_mma, SmemLayout)
{
    if (p.skip_flag != nullptr && *p.skip_flag != 0) return;   // uniform for the whole grid

    extern __shared__ __align__(1024) char smem_raw[];
    using Storage = SharedStorage<SmemLayout>;
    Storage& shared = *reinterpret_cast<Storage*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    int bi, bj;
    if (p.lower_only) {
        bi = int((sqrtf(8.0f * float(blockIdx.x) + 1.0f) - 1.0f) * 0.5f);
        while ((bi + 1) * (bi + 2) / 2 <= int(blockIdx.x)) ++bi;
        while (bi * (bi + 1) / 2 > int(blockIdx.x)) --bi;
        bj = int(blockIdx.x) - bi * (bi + 1) / 2;
    } else {
        bi = int(blockIdx.x) / p.tiles_n;
        bj = int(blockIdx.x) - bi * p.tiles_n;
    }
    const int z = blockIdx.y;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    ThrMMA cta_mma = tiled_mma.get_slice(0);
    Tensor sAhi = make_tensor(make_smem_ptr(shared.operand[0].begin()), SmemLayout{});
    Tensor sAlo = make_tensor(make_smem_ptr(shared.operand[1].begin()), SmemLayout{});
    Tensor sBhi = make_tensor(make_smem_ptr(shared.operand[2].begin()), SmemLayout{});
    Tensor sBlo = make_tensor(make_smem_ptr(shared.operand[3].begin()), SmemLayout{});
    Tensor dAhi = cta_mma.make_fragment_A(sAhi);
    Tensor dAlo = cta_mma.make_fragment_A(sAlo);
    Tensor dBhi = cta_mma.make_fragment_B(sBhi);
    Tensor dBlo = cta_mma.make_fragment_B(sBlo);

    // only the shape of this view matters: it sizes the tensor-memory accumulator fragments
    Tensor mC = make_tensor(make_gmem_ptr(p.d), make_shape(Int<kTile>{}, Int<kTile>{}), make_stride(Int<kTile>{}, _1{}));
    Tensor tCgC = cta_mma.partition_C(mC);
    Tensor tCtAcc0 = cta_mma.make_fragment_C(tCgC);
    Tensor tCtAcc1 = cta_mma.make_fragment_C(tCgC);

    using TmemAllocator = cute::TMEM::Allocator1Sm;
    TmemAllocator tmem_allocator{};
    if (warp == 0) tmem_allocator.allocate(2 * kTile, &shared.tmem_base_ptr);
    if (threadIdx.x == 32) {
        for (int s = 0; s < kStages; ++s) {
            cute::initialize_barrier(shared.full[s], 1);
            cute::initialize_barrier(shared.empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            cute::initialize_barrier(shared.ready[a], 1);
            cute::initialize_barrier(shared.free_[a], 4 * 32);
        }
        shared.failed = 0;
        shared.first_failure = 0;
        cutlass::arch::fence_barrier_init();
    }
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = shared.tmem_base_ptr;
    tCtAcc0.data() = tmem_base;
    tCtAcc1.data() = tmem_base + kTile;

    const int k_steps = p.k_steps;
    const int segments = (k_steps + kSegmentSteps - 1) / kSegmentSteps;

    if (warp == 0) {
        // ---- TMA producer ---------------------------------------------------------------------
        if (lane == 0) {
            bool ok = true;
            for (int kt = 0; kt < k_steps && ok; ++kt) {
                const int s = kt % kStages;
                if (kt >= kStages) ok = bounded_wait(shared, &shared.empty[s], uint32_t((kt / kStages - 1) & 1), 0x11000000u | uint32_t(kt));
                if (!ok) break;
                cute::set_barrier_transaction_bytes(shared.full[s], 4 * kTileBytes);
                const int x = kt * kBlockK;
                tma_load_tile_3d(&maps.a_hi, shared.operand[0].begin() + s * (kTile * kBlockK), &shared.full[s], x, bi * kTile, z);
                tma_load_tile_3d(&maps.a_lo, shared.operand[1].begin() + s * (kTile * kBlockK), &shared.full[s], x, bi * kTile, z);
                tma_load_tile_3d(&maps.b_hi, shared.operand[2].begin() + s * (kTile * kBlockK), &shared.full[s], x, bj * kTile, z);
                tma_load_tile_3d(&maps.b_lo, shared.operand[3].begin() + s * (kTile * kBlockK), &shared.full[s], x, bj * kTile, z);
            }
            // tail: the last commits still arrive on the "empty" barriers; do not leave before them
            for (int kt = max(0, k_steps - kStages); kt < k_steps && ok; ++kt)
                ok = bounded_wait(shared, &shared.empty[kt % kStages], uint32_t((kt / kStages) & 1), 0x12000000u | uint32_t(kt));
        }
    } else if (warp == 1) {
        // ---- MMA issuer (whole warp: the MMA atom and umma_arrive elect one lane themselves) -----
        bool ok = true;
        for (int seg = 0; seg < segments && ok; ++seg) {
            const int acc = seg & 1;
            if (seg >= 2)
                ok = __all_sync(0xffffffffu, bounded_wait(shared, &shared.free_[acc], uint32_t((seg / 2 - 1) & 1),
                                                          0x13000000u | uint32_t(seg)));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            tiled_mma.accumulate_ = UMMA::ScaleOut::Zero;
            const int kt_end = min(k_steps, (seg + 1) * kSegmentSteps);
            for (int kt = seg * kSegmentSteps; kt < kt_end; ++kt) {
                const int s = kt % kStages;
                ok = __all_sync(0xffffffffu, bounded_wait(shared, &shared.full[s], uint32_t((kt / kStages) & 1),
                                                          0x14000000u | uint32_t(kt)));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int kb = 0; kb < size<2>(dAhi); ++kb) {
                    if (acc == 0) {
                        gemm(tiled_mma, dAhi(_, _, kb, s), dBhi(_, _, kb, s), tCtAcc0);
                        tiled_mma.accumulate_ = UMMA::ScaleOut::One;
                        gemm(tiled_mma, dAlo(_, _, kb, s), dBhi(_, _, kb, s), tCtAcc0);
                        gemm(tiled_mma, dAhi(_, _, kb, s), dBlo(_, _, kb, s), tCtAcc0);
                    } else {
                        gemm(tiled_mma, dAhi(_, _, kb, s), dBhi(_, _, kb, s), tCtAcc1);
                        tiled_mma.accumulate_ = UMMA::ScaleOut::One;
                        gemm(tiled_mma, dAlo(_, _, kb, s), dBhi(_, _, kb, s), tCtAcc1);
                        gemm(tiled_mma, dAhi(_, _, kb, s), dBlo(_, _, kb, s), tCtAcc1);
                    }
                }
                cutlass::arch::umma_arrive(&shared.empty[s]);
            }
            if (ok) cutlass::arch::umma_arrive(&shared.ready[acc]);
        }
    } else {
        // ---- epilogue: rows 32q .. 32q+31 of the tile, q = warp % 4 (the warp's tensor-memory lanes)
        const int q = warp & 3;
        float total[kTile];
#pragma unroll
        for (int i = 0; i < kTile; ++i) total[i] = 0.0f;
        bool ok = true;
        for (int seg = 0; seg < segments && ok; ++seg) {
            const int acc = seg & 1;
            ok = bounded_wait(shared, &shared.ready[acc], uint32_t((seg / 2) & 1), 0x15000000u | uint32_t(seg));
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * kTile);
#pragma unroll
            for (int c = 0; c < kTile / 16; ++c) {
                float v[16];
                tmem_load16(taddr + c * 16, v);
#pragma unroll
                for (int i = 0; i < 16; ++i) total[c * 16 + i] += v[i];
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            arrive(&shared.free_[acc]);
        }
        if (ok) {
            const int m = bi * kTile + q * 32 + lane;
            const int n0 = bj * kTile;
            float* base = p.d + int64_t(z) * p.d_stride;
            const float alpha = p.alpha, beta = p.beta;
            if (!p.transposed_out) {
                // Through shared memory, so that global memory sees whole rows: a thread holds one
                // row of the tile, but a warp that wrote its 32 rows directly would touch 32 rows
                // with every 16-byte access.  Each epilogue warp parks its 32 x 128 block in its
                // own part of the operand stages (idle by now: the last segment's MMAs have read
                // them) and then moves it row by row, a lane per float4 = 512 contiguous bytes.
                float* stage = reinterpret_cast<float*>(shared.operand[0].begin()) + q * (32 * kStagePitch);
#pragma unroll
                for (int c = 0; c < kTile / 4; ++c)
                    *reinterpret_cast<float4*>(stage + lane * kStagePitch + 4 * c) =
                        make_float4(alpha * total[4 * c], alpha * total[4 * c + 1], alpha * total[4 * c + 2],
                                    alpha * total[4 * c + 3]);
                __syncwarp();
                const int row0 = bi * kTile + q * 32;
                const int col = n0 + 4 * lane;
                if (col + 3 < p.n) {
                    // all loads of the old values are issued before the first store (the rows are
                    // independent; a row-by-row loop would wait for memory 32 times)
                    const int rows_here = min(32, p.m - row0);
                    float4 old[32];
                    if (beta != 0.0f) {
#pragma unroll
                        for (int r = 0; r < 32; ++r)
                            if (r < rows_here)
                                old[r] = *reinterpret_cast<const float4*>(base + int64_t(row0 + r) * p.ldd + col);
                    }
#pragma unroll
                    for (int r = 0; r < 32; ++r) {
                        if (r < rows_here) {
                            float4 out = *reinterpret_cast<const float4*>(stage + r * kStagePitch + 4 * lane);
                            if (beta != 0.0f) {
                                out.x = fmaf(beta, old[r].x, out.x); out.y = fmaf(beta, old[r].y, out.y);
                                out.z = fmaf(beta, old[r].z, out.z); out.w = fmaf(beta, old[r].w, out.w);
                            }
                            *reinterpret_cast<float4*>(base + int64_t(row0 + r) * p.ldd + col) = out;
                        }
                    }
                } else if (col < p.n) {
                    for (int r = 0; r < 32 && row0 + r < p.m; ++r) {
                        for (int i = 0; i < 4 && col + i < p.n; ++i) {
                            float* dst = base + int64_t(row0 + r) * p.ldd + col + i;
                            float out = stage[r * kStagePitch + 4 * lane + i];
                            if (beta != 0.0f) out = fmaf(beta, *dst, out);
                            *dst = out;
                        }
                    }
                }
            } else {
                // D[n, m]: for a fixed n the 32 lanes of the warp write 32 consecutive floats
#pragma unroll
                for (int c = 0; c < kTile; ++c) {
                    if (n0 + c < p.n && m < p.m) {
                        float* dst = base + int64_t(n0 + c) * p.ldd + m;
                        float out = alpha * total[c];
                        if (beta != 0.0f) out = fmaf(beta, *dst, out);
                        *dst = out;
                    }
                }
            }
        }
    }

    __syncthreads();
    if (shared.failed) {
        if (threadIdx.x == 0) atomicCAS(p.status, 0, int(shared.first_failure));
        // let copies that are still in flight land before the shared memory is given back
        const long long start = clock64();
        while (clock64() - start < 4000000) {}
        __syncthreads();
    }
    if (warp == 0) {
        tmem_allocator.release_allocation_lock();
        tmem_allocator.free(tmem_base, 2 * kTile);
    }
}

// src [rows, cols] (row pitch ld, matrix stride) -> hi / lo planes.  transpose == 0: planes are
// [rows, cols_pad] with pitch ld_out; transpose == 1: planes are [cols, rows_pad] with pitch ld_out.
// Elements of the padded region are not written.
__global__ void __launch_bounds__(256)
split_tf32_kernel(const float* __restrict__ src, int rows, int cols, int ld, int64_t src_stride,
                  float* __restrict__ hi, float* __restrict__ lo, int ld_out, int64_t out_stride, int transpose)
{
    __shared__ float tile[32][33];
    const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    src += int64_t(blockIdx.z) * src_stride;
    hi += int64_t(blockIdx.z) * out_stride;
    lo += int64_t(blockIdx.z) * out_stride;
    if (!transpose) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = r0 + ty + 8 * i, c = c0 + tx;
            if (r < rows && c < cols) {
                const float x = src[int64_t(r) * ld + c];
                const float h = tf32_round(x);
                hi[int64_t(r) * ld_out + c] = h;
                lo[int64_t(r) * ld_out + c] = tf32_round(x - h);
            }
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + ty + 8 * i, c = c0 + tx;
        tile[ty + 8 * i][tx] = (r < rows && c < cols) ? src[int64_t(r) * ld + c] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = c0 + ty + 8 * i, r = r0 + tx;
        if (c < cols && r < rows) {
            const float x = tile[tx][ty + 8 * i];
            const float h = tf32_round(x);
            hi[int64_t(c) * ld_out + r] = h;
            lo[int64_t(c) * ld_out + r] = tf32_round(x - h);
        }
    }
}

}  // namespace gemm3x
}  // namespace qsrtb_tc

using namespace qsrtb_tc;
using namespace qsrtb_tc::gemm3x;

extern "C" int qsrtb_split_tf32(const float* src, int batch, int rows, int cols, int ld, int64_t src_stride,
                                float* hi, float* lo, int ld_out, int64_t out_stride, int transpose, void* stream)
{
    if (!src || !hi || !lo || batch < 0 || rows < 0 || cols < 0 || ld < cols)
        return qsrtb_fail(QSRTB_EINVAL, "bad split arguments");
    if (ld_out < (transpose ? rows : cols)) return qsrtb_fail(QSRTB_EINVAL, "plane pitch smaller than the plane's row");
    if (batch == 0 || rows == 0 || cols == 0) return QSRTB_OK;
    if (batch > 65535) return qsrtb_fail(QSRTB_EINVAL, "too many matrices in one split call");
    dim3 grid(unsigned((cols + 31) / 32), unsigned((rows + 31) / 32), unsigned(batch));
    if (grid.y > 65535) return qsrtb_fail(QSRTB_EINVAL, "too many rows in one split call");
    split_tf32_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(src, rows, cols, ld, src_stride, hi, lo,
                                                                          ld_out, out_stride, transpose);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "split_tf32 launch");
    return QSRTB_OK;
}

namespace {

int encode_operand(EncodeTiled encode, CUtensorMap* map, const float* plane, int rows, int k, int ld,
                   int64_t stride, int batch)
{
    // [batch][rows][k] float32, boxes of 128 rows x 32 columns of one matrix, 128-byte swizzle
    // (the layout the K-major UMMA descriptors expect); out-of-range rows and columns read zero.
    const cuuint64_t dims[3] = {cuuint64_t(k), cuuint64_t(rows), cuuint64_t(batch)};
    const cuuint64_t strides[2] = {cuuint64_t(ld) * sizeof(float),
                                   cuuint64_t(batch > 1 ? stride : int64_t(rows) * ld) * sizeof(float)};
    const cuuint32_t box[3] = {cuuint32_t(kBlockK), cuuint32_t(kTile), 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(plane), dims, strides,
                               box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS ? QSRTB_OK : QSRTB_ECUDA;
}

bool operand_ok(const float* hi, const float* lo, int ld, int64_t stride, int batch)
{
    if (!hi || !lo || (ld % 4) != 0) return false;
    if ((reinterpret_cast<uintptr_t>(hi) & 15) || (reinterpret_cast<uintptr_t>(lo) & 15)) return false;
    if (batch > 1 && (stride % 4) != 0) return false;
    return true;
}

}  // namespace

extern "C" int qsrtb_gemm3x_tc(const float* a_hi, const float* a_lo, int lda, int64_t a_stride,
                               const float* b_hi, const float* b_lo, int ldb, int64_t b_stride,
                               int batch, int m, int n, int k,
                               float* d, int ldd, int64_t d_stride, float alpha, float beta,
                               int lower_only, int transposed_out,
                               const int* skip_flag, int* status_flag, void* stream)
{
    if (batch < 0 || m < 0 || n < 0 || k <= 0) return qsrtb_fail(QSRTB_EINVAL, "bad product shape");
    if (batch == 0 || m == 0 || n == 0) return QSRTB_OK;
    if (batch > 65535) return qsrtb_fail(QSRTB_EINVAL, "too many matrices in one product call");
    if (!operand_ok(a_hi, a_lo, lda, a_stride, batch) || !operand_ok(b_hi, b_lo, ldb, b_stride, batch))
        return qsrtb_fail(QSRTB_EINVAL, "operand planes must be 16-byte aligned with pitches that are multiples of 4");
    if (lda < k || ldb < k) return qsrtb_fail(QSRTB_EINVAL, "operand pitch smaller than k");
    if (!d || (reinterpret_cast<uintptr_t>(d) & 15) || (ldd % 4) != 0 || ldd < (transposed_out ? m : n) ||
        (batch > 1 && (d_stride % 4) != 0))
        return qsrtb_fail(QSRTB_EINVAL, "output must be 16-byte aligned with a pitch that is a multiple of 4");
    if (lower_only && m != n) return qsrtb_fail(QSRTB_EINVAL, "lower-triangular mode needs a square product");
    if (!status_flag) return qsrtb_fail(QSRTB_EINVAL, "status flag pointer required");
    EncodeTiled encode = encode_tiled_entry();
    if (!encode) return qsrtb_fail(QSRTB_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");

    Maps maps;
    if (encode_operand(encode, &maps.a_hi, a_hi, m, k, lda, a_stride, batch) ||
        encode_operand(encode, &maps.a_lo, a_lo, m, k, lda, a_stride, batch) ||
        encode_operand(encode, &maps.b_hi, b_hi, n, k, ldb, b_stride, batch) ||
        encode_operand(encode, &maps.b_lo, b_lo, n, k, ldb, b_stride, batch))
        return qsrtb_fail(QSRTB_ECUDA, "cuTensorMapEncodeTiled failed");

    Params p;
    p.m = m;
    p.n = n;
    p.k_steps = (k + kBlockK - 1) / kBlockK;
    p.tiles_m = (m + kTile - 1) / kTile;
    p.tiles_n = (n + kTile - 1) / kTile;
    p.lower_only = lower_only ? 1 : 0;
    p.transposed_out = transposed_out ? 1 : 0;
    p.ldd = ldd;
    p.d_stride = d_stride;
    p.alpha = alpha;
    p.beta = beta;
    p.d = d;
    p.skip_flag = skip_flag;
    p.status = status_flag;

    TiledMMA tiled_mma = make_tiled_mma(
        SM100_MMA_TF32_SS<Element, Element, float, kTile, kTile, UMMA::Major::K, UMMA::Major::K>{});
    auto mma_shape = partition_shape_A(tiled_mma, make_shape(Int<kTile>{}, Int<kBlockK>{}));
    auto smem_layout = UMMA::tile_to_mma_shape(UMMA::Layout_K_SW128_Atom<Element>{},
                                               append(mma_shape, Int<kStages>{}));
    static_assert(cute::cosize_v<decltype(smem_layout)> == kStages * kTile * kBlockK, "stages must be 16 KiB apart");
    using Storage = SharedStorage<decltype(smem_layout)>;
    const int smem_bytes = int(sizeof(Storage)) + 1024;
    auto kernel = gemm3x_tcgen05_kernel<decltype(tiled_mma), decltype(smem_layout)>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "cudaFuncSetAttribute(gemm3x_tcgen05)");
    const int64_t tiles = lower_only ? int64_t(p.tiles_m) * (p.tiles_m + 1) / 2 : int64_t(p.tiles_m) * p.tiles_n;
    if (tiles > (int64_t(1) << 30)) return qsrtb_fail(QSRTB_EINVAL, "product too large for one launch");
    kernel<<<dim3(unsigned(tiles), unsigned(batch)), kThreads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(
        maps, p, tiled_mma, smem_layout);
    err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "gemm3x_tcgen05 launch");
    return QSRTB_OK;
}

#else  // QSRTB_NO_CUTLASS

extern "C" int qsrtb_split_tf32(const float*, int, int, int, int, int64_t, float*, float*, int, int64_t, int, void*)
{
    return qsrtb_fail(QSRTB_EINVAL, "built without the CUTLASS/CuTe headers: tensor-core products unavailable");
}

extern "C" int qsrtb_gemm3x_tc(const float*, const float*, int, int64_t, const float*, const float*, int, int64_t, int,
                               int, int, int, float*, int, int64_t, float, float, int, int, const int*, int*, void*)
{
    return qsrtb_fail(QSRTB_EINVAL, "built without the CUTLASS/CuTe headers: tensor-core products unavailable");
}

#endif
