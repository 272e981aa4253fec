// Calibration Hessian on the 5th-generation tensor cores:  C (+)= sum_r w_r x_r x_r^T  as a
// tcgen05 (UMMA) TF32 contraction with the accumulator in tensor memory.
//
// Precision: one TF32 pass would give ~1e-4 relative error; the float32 inputs are therefore
// split into a TF32 head and a TF32 tail (x = hi + lo, exactly) and the three significant
// products hi*hi + lo*hi + hi*lo are accumulated in float32.  The split is folded into the
// contraction dimension: with A' = [hi(x) | lo(x) | hi(x)] and B' = [hi(wx) | hi(wx) | lo(wx)]
// (both feature-major, K-major operands) a single GEMM over K' = 3R does all three products.
//
//   prepare kernel : transposes a chunk of rows into A' and B' (shared-memory tile transpose,
//                    coalesced on both sides), applies the row weight and the split.
//   gemm kernel    : one CTA per lower-triangular 128x128 tile of C.  Per 32-wide K block the
//                    CTA stages 2 x 16 KiB operand tiles in 128-byte-swizzled shared memory
//                    (double buffered), one elected thread issues four 128x128x8
//                    tcgen05.mma.kind::tf32 instructions and commits them to an mbarrier; the
//                    128 x 128 float accumulator lives in 128 TMEM columns and is read back
//                    once with tcgen05.ld for the epilogue.
// Every mbarrier wait is bounded; on expiry the kernel raises a status flag, releases its
// tensor memory and returns.
//
// Built on the CuTe sm100 atoms (cute/arch/mma_sm100_umma.hpp, tmem_allocator_sm100.hpp).
#include <cuda_runtime.h>
#include <stdint.h>

#include "qsrtb_internal.h"

#if !defined(QSRTB_NO_CUTLASS)

#include <cute/tensor.hpp>
#include <cute/arch/cluster_sm90.hpp>
#include <cute/arch/tmem_allocator_sm100.hpp>
#include <cute/algorithm/cooperative_copy.hpp>
#include <cutlass/arch/barrier.h>
#include <cutlass/numeric_types.h>

namespace qsrtb_tc {

using namespace cute;

constexpr int kTile = 128;   // output tile edge
constexpr int kBlockK = 32;  // contraction elements per staged block (one 128-byte swizzle row)
constexpr int kThreads = 128;
constexpr int kWaitLimit = 4000000;
constexpr int kSegmentTiles = 16;  // 512 contraction elements per tensor-memory accumulation

using Element = cutlass::tfloat32_t;

__device__ __forceinline__ float tf32_round(float x)
{
    uint32_t u = __float_as_uint(x);
    u += 0x00000fffu + ((u >> 13) & 1u);   // round to nearest even on 10 mantissa bits
    return __uint_as_float(u & 0xffffe000u);
}

// rows [R, d] (row pitch ld) -> a_split, b_split [d, 3 * r_pad] (K-major)
__global__ void __launch_bounds__(256)
split_transpose_kernel(const float* __restrict__ rows, const float* __restrict__ weights, int64_t n_rows,
                       int d, int ld, int r_pad, float* __restrict__ a_split, float* __restrict__ b_split)
{
    __shared__ float tile[32][33];
    __shared__ float wts[32];
    const int r0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    if (ty == 0) wts[tx] = (r0 + tx < n_rows) ? (weights ? weights[r0 + tx] : 1.0f) : 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + ty + 8 * i, c = c0 + tx;
        tile[ty + 8 * i][tx] = (r < n_rows && c < d) ? rows[int64_t(r) * ld + c] : 0.0f;
    }
    __syncthreads();
    const int64_t pitch = 3 * int64_t(r_pad);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = c0 + ty + 8 * i;   // feature
        const int r = r0 + tx;           // row inside the chunk (padded rows are zero)
        if (c >= d || r >= r_pad) continue;
        const float x = tile[tx][ty + 8 * i];
        const float wx = x * wts[tx];
        const float x_hi = tf32_round(x), x_lo = tf32_round(x - x_hi);
        const float w_hi = tf32_round(wx), w_lo = tf32_round(wx - w_hi);
        float* a = a_split + int64_t(c) * pitch + r;
        float* b = b_split + int64_t(c) * pitch + r;
        a[0] = x_hi;         b[0] = w_hi;
        a[r_pad] = x_lo;     b[r_pad] = w_hi;
        a[2 * r_pad] = x_hi; b[2 * r_pad] = w_lo;
    }
}

template <class ASmemLayout, class BSmemLayout>
struct SharedStorage {
    alignas(128) cute::ArrayEngine<Element, cute::cosize_v<ASmemLayout>> A[2];
    alignas(128) cute::ArrayEngine<Element, cute::cosize_v<BSmemLayout>> B[2];
    alignas(16) cute::uint64_t mma_barrier[2];
    alignas(16) cute::uint32_t tmem_base_ptr;
};

__device__ __forceinline__ bool bounded_wait(uint64_t* barrier, uint32_t phase)
{
    const uint32_t addr = cute::cast_smem_ptr_to_uint(barrier);
    for (int i = 0; i < kWaitLimit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(phase) : "memory");
        if (done) return true;
    }
    return false;
}

// Copy one 128 x 32 operand block (row pitch k_total) into its swizzled shared-memory tile with
// 16-byte accesses: the 128-byte swizzle permutes whole 16-byte chunks, so four consecutive
// contraction elements stay contiguous.  Tile coordinates are ((row, k % 8), 0, k / 8).
template <class SmemTensor>
__device__ __forceinline__ void stage_tile(const Element* __restrict__ base, int tile_row, int k_tile,
                                           int k_total, SmemTensor& smem)
{
    const Element* src = base + int64_t(tile_row) * kTile * k_total + int64_t(k_tile) * kBlockK;
#pragma unroll
    for (int i = 0; i < (kTile * kBlockK / 4) / kThreads; ++i) {
        const int chunk = threadIdx.x + i * kThreads;   // 8 chunks of 16 bytes per row
        const int row = chunk >> 3, k4 = (chunk & 7) * 4;
        const uint4 v = *reinterpret_cast<const uint4*>(src + int64_t(row) * k_total + k4);
        Element* dst = &smem(make_coord(make_coord(row, k4 & 7), 0, k4 >> 3));
        *reinterpret_cast<uint4*>(dst) = v;
    }
}

template <class TiledMMA, class ASmemLayout, class BSmemLayout>
__global__ void __launch_bounds__(128, 1)
syrk_tcgen05_kernel(const Element* __restrict__ a_ptr, const Element* __restrict__ b_ptr, int d, int k_total,
                    float* __restrict__ c_ptr, int ldc, int accumulate, int* __restrict__ status,
                    TiledMMA tiled_mma, ASmemLayout, BSmemLayout)
{
    extern __shared__ __align__(128) char smem_raw[];
    using Storage = SharedStorage<ASmemLayout, BSmemLayout>;
    Storage& shared = *reinterpret_cast<Storage*>(smem_raw);

    // lower-triangular tile pair of this CTA
    int bi = int((sqrtf(8.0f * float(blockIdx.x) + 1.0f) - 1.0f) * 0.5f);
    while ((bi + 1) * (bi + 2) / 2 <= int(blockIdx.x)) ++bi;
    while (bi * (bi + 1) / 2 > int(blockIdx.x)) --bi;
    const int bj = int(blockIdx.x) - bi * (bi + 1) / 2;

    Tensor mA = make_tensor(make_gmem_ptr(a_ptr), make_shape(d, k_total), make_stride(k_total, _1{}));
    Tensor mB = make_tensor(make_gmem_ptr(b_ptr), make_shape(d, k_total), make_stride(k_total, _1{}));
    Tensor mC = make_tensor(make_gmem_ptr(c_ptr), make_shape(d, d), make_stride(ldc, _1{}));
    Tensor gA = local_tile(mA, Shape<Int<kTile>, Int<kBlockK>>{}, make_coord(bi, _));  // (128, 32, k_tiles)
    Tensor gB = local_tile(mB, Shape<Int<kTile>, Int<kBlockK>>{}, make_coord(bj, _));
    Tensor gC = local_tile(mC, Shape<Int<kTile>, Int<kTile>>{}, make_coord(bi, bj));    // (128, 128)

    ThrMMA cta_mma = tiled_mma.get_slice(0);
    Tensor tCgA = cta_mma.partition_A(gA);   // (MmaA, NumMma_M, NumMma_K, k_tiles)
    Tensor tCgB = cta_mma.partition_B(gB);
    Tensor tCgC = cta_mma.partition_C(gC);   // (MmaC, NumMma_M, NumMma_N)

    Tensor tCsA0 = make_tensor(make_smem_ptr(shared.A[0].begin()), ASmemLayout{});
    Tensor tCsA1 = make_tensor(make_smem_ptr(shared.A[1].begin()), ASmemLayout{});
    Tensor tCsB0 = make_tensor(make_smem_ptr(shared.B[0].begin()), BSmemLayout{});
    Tensor tCsB1 = make_tensor(make_smem_ptr(shared.B[1].begin()), BSmemLayout{});
    Tensor tCrA0 = cta_mma.make_fragment_A(tCsA0);   // shared-memory matrix descriptors
    Tensor tCrA1 = cta_mma.make_fragment_A(tCsA1);
    Tensor tCrB0 = cta_mma.make_fragment_B(tCsB0);
    Tensor tCrB1 = cta_mma.make_fragment_B(tCsB1);
    Tensor tCtAcc = cta_mma.make_fragment_C(tCgC);   // tensor-memory accumulator

    const uint32_t elect_one_warp = (threadIdx.x / 32 == 0);
    using TmemAllocator = cute::TMEM::Allocator1Sm;
    TmemAllocator tmem_allocator{};
    if (elect_one_warp) tmem_allocator.allocate(kTile, &shared.tmem_base_ptr);
    if (threadIdx.x == 0) {
        cute::initialize_barrier(shared.mma_barrier[0], 1);
        cute::initialize_barrier(shared.mma_barrier[1], 1);
    }
    __syncthreads();
    tCtAcc.data() = shared.tmem_base_ptr;

    const int k_tiles = size<3>(tCgA);
    bool ok = true;
    uint32_t phase[2] = {0, 0};

    TiledCopy tiled_t2r = make_tmem_copy(SM100_TMEM_LOAD_32dp32b1x{}, tCtAcc);
    ThrCopy thr_t2r = tiled_t2r.get_slice(threadIdx.x);
    Tensor tDtAcc = thr_t2r.partition_S(tCtAcc);
    Tensor tDgC = thr_t2r.partition_D(tCgC);

    // The tensor core adds each 8-deep product group to the float32 accumulator with
    // truncation; over thousands of groups that bias exceeds 1e-5.  The contraction is therefore
    // cut into segments of kSegmentTiles blocks whose partial sums are added to C in ordinary
    // round-to-nearest float32.
    for (int seg_begin = 0; seg_begin < k_tiles && ok; seg_begin += kSegmentTiles) {
        const int seg_end = min(k_tiles, seg_begin + kSegmentTiles);
        tiled_mma.accumulate_ = UMMA::ScaleOut::Zero;
        for (int k_tile = seg_begin; k_tile < seg_end; ++k_tile) {
            const int buf = k_tile & 1;
            // the buffer was last read by the MMAs of k_tile - 2: wait for their commit
            if (k_tile - seg_begin >= 2) {
                // block-uniform verdict, so that no thread is left behind at a barrier
                ok = __syncthreads_and(bounded_wait(&shared.mma_barrier[buf], phase[buf]));
                phase[buf] ^= 1;
                if (!ok) break;
            }
            if (buf == 0) {
                stage_tile(a_ptr, bi, k_tile, k_total, tCsA0);
                stage_tile(b_ptr, bj, k_tile, k_total, tCsB0);
            } else {
                stage_tile(a_ptr, bi, k_tile, k_total, tCsA1);
                stage_tile(b_ptr, bj, k_tile, k_total, tCsB1);
            }
            // generic-proxy writes to shared memory must be visible to the tensor-core proxy
            cutlass::arch::fence_view_async_shared();
            __syncthreads();
            if (elect_one_warp) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int k_block = 0; k_block < size<2>(tCrA0); ++k_block) {
                    if (buf == 0) gemm(tiled_mma, tCrA0(_, _, k_block), tCrB0(_, _, k_block), tCtAcc);
                    else gemm(tiled_mma, tCrA1(_, _, k_block), tCrB1(_, _, k_block), tCtAcc);
                    tiled_mma.accumulate_ = UMMA::ScaleOut::One;
                }
                cutlass::arch::umma_arrive(&shared.mma_barrier[buf]);
            }
        }
        if (!ok) break;
        // drain: the last one or two commits of the segment have not been waited for yet
        {
            const int n = seg_end - seg_begin;
            const int last = (seg_end - 1) & 1;
            bool drained = true;
            if (n >= 2) {
                drained = bounded_wait(&shared.mma_barrier[last ^ 1], phase[last ^ 1]);
                phase[last ^ 1] ^= 1;
            }
            if (drained) {
                drained = bounded_wait(&shared.mma_barrier[last], phase[last]);
                phase[last] ^= 1;
            }
            ok = __syncthreads_and(drained);
            if (!ok) break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        Tensor tDrAcc = make_tensor<float>(shape(tDgC));
        copy(tiled_t2r, tDtAcc, tDrAcc);
        cutlass::arch::fence_view_async_tmem_load();
        if (accumulate || seg_begin > 0) {
            CUTE_UNROLL
            for (int i = 0; i < size(tDrAcc); ++i) tDgC(i) += tDrAcc(i);
        } else {
            CUTE_UNROLL
            for (int i = 0; i < size(tDrAcc); ++i) tDgC(i) = tDrAcc(i);
        }
        // the next segment's MMAs overwrite the accumulator: order them after these loads
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
    }
    if (!ok && threadIdx.x == 0) atomicExch(status, 1);
    __syncthreads();
    if (elect_one_warp) {
        tmem_allocator.release_allocation_lock();
        tmem_allocator.free(shared.tmem_base_ptr, kTile);
    }
}

}  // namespace qsrtb_tc

using namespace qsrtb_tc;

extern "C" int qsrtb_hessian_tc_workspace_bytes(int64_t chunk_rows, int d, size_t* bytes)
{
    if (!bytes || chunk_rows <= 0 || d <= 0) return qsrtb_fail(QSRTB_EINVAL, "bad workspace query");
    const int64_t r_pad = (chunk_rows + kBlockK - 1) / kBlockK * kBlockK;
    *bytes = size_t(2) * size_t(d) * size_t(3 * r_pad) * sizeof(float) + 256;
    return QSRTB_OK;
}

extern "C" int qsrtb_hessian_accumulate_tc(const float* rows, const float* weights, int64_t n_rows, int d,
                                           int ld_rows, float* lower, int ld_h, int accumulate,
                                           void* workspace, size_t workspace_bytes, int* status_flag,
                                           void* stream)
{
    if (!lower || d <= 0 || (d % kTile) != 0 || ld_h < d || n_rows <= 0 || !rows || ld_rows < d)
        return qsrtb_fail(QSRTB_EINVAL, "tensor-core Hessian needs d a multiple of 128 and at least one row");
    if (!status_flag) return qsrtb_fail(QSRTB_EINVAL, "status flag pointer required");
    const int64_t r_pad64 = (n_rows + kBlockK - 1) / kBlockK * kBlockK;
    if (3 * r_pad64 > (int64_t(1) << 30)) return qsrtb_fail(QSRTB_EINVAL, "row chunk too large");
    const int r_pad = int(r_pad64);
    size_t need = 0;
    qsrtb_hessian_tc_workspace_bytes(n_rows, d, &need);
    if (!workspace || workspace_bytes < need) return qsrtb_fail(QSRTB_ESCRATCH, "Hessian workspace too small");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // 256-byte aligned halves of the workspace
    uintptr_t base = (reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255);
    float* a_split = reinterpret_cast<float*>(base);
    float* b_split = a_split + size_t(d) * size_t(3 * r_pad);

    dim3 grid_t(unsigned(r_pad / 32), unsigned((d + 31) / 32));
    split_transpose_kernel<<<grid_t, 256, 0, s>>>(rows, weights, n_rows, d, ld_rows, r_pad, a_split, b_split);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "split_transpose launch");

    TiledMMA tiled_mma = make_tiled_mma(
        SM100_MMA_TF32_SS<Element, Element, float, kTile, kTile, UMMA::Major::K, UMMA::Major::K>{});
    auto mma_tiler = make_shape(Int<kTile>{}, Int<kTile>{}, Int<kBlockK>{});
    auto mma_shape_A = partition_shape_A(tiled_mma, make_shape(size<0>(mma_tiler), size<2>(mma_tiler)));
    auto mma_shape_B = partition_shape_B(tiled_mma, make_shape(size<1>(mma_tiler), size<2>(mma_tiler)));
    auto sA_layout = UMMA::tile_to_mma_shape(UMMA::Layout_K_SW128_Atom<Element>{}, mma_shape_A);
    auto sB_layout = UMMA::tile_to_mma_shape(UMMA::Layout_K_SW128_Atom<Element>{}, mma_shape_B);
    using Storage = SharedStorage<decltype(sA_layout), decltype(sB_layout)>;
    const int smem_bytes = int(sizeof(Storage)) + 128;
    auto kernel = syrk_tcgen05_kernel<decltype(tiled_mma), decltype(sA_layout), decltype(sB_layout)>;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "cudaFuncSetAttribute(syrk_tcgen05)");
    const int nb = d / kTile;
    kernel<<<nb * (nb + 1) / 2, kThreads, smem_bytes, s>>>(
        reinterpret_cast<const Element*>(a_split), reinterpret_cast<const Element*>(b_split), d, 3 * r_pad,
        lower, ld_h, accumulate, status_flag, tiled_mma, sA_layout, sB_layout);
    err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "syrk_tcgen05 launch");
    return QSRTB_OK;
}

#else  // QSRTB_NO_CUTLASS

extern "C" int qsrtb_hessian_tc_workspace_bytes(int64_t, int, size_t*)
{
    return qsrtb_fail(QSRTB_EINVAL, "built without the CUTLASS/CuTe headers: tensor-core Hessian unavailable");
}

extern "C" int qsrtb_hessian_accumulate_tc(const float*, const float*, int64_t, int, int, float*, int, int,
                                           void*, size_t, int*, void*)
{
    return qsrtb_fail(QSRTB_EINVAL, "built without the CUTLASS/CuTe headers: tensor-core Hessian unavailable");
}

#endif
