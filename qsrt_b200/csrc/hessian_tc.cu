// Calibration Hessian on the 5th-generation tensor cores:  C (+)= sum_r w_r x_r x_r^T  as a
// TMA-fed, warp-specialised tcgen05 (UMMA) TF32 contraction with the accumulators in tensor memory.
//
// Precision: one TF32 pass would give ~1e-4 relative error; the float32 inputs are therefore
// split exactly into a TF32 head and a TF32 tail (x = hi + lo) and the three significant
// products hi*hi + lo*hi + hi*lo are accumulated in float32.  The tensor core adds each 8-deep
// product group to its float32 accumulator with truncation; over thousands of groups that bias
// alone exceeds 1e-5, so the contraction is cut into segments of 60 instruction groups whose
// partial sums leave tensor memory and are added up in round-to-nearest float32 registers.
//
//   prepare kernel : transposes a chunk of rows into four K-major planes [d, r_pad]:
//                    hi(x), lo(x), hi(w x), lo(w x)  (shared-memory tile transpose).
//   gemm kernel    : one CTA (6 warps) per lower-triangular 128x128 tile of C.
//       warp 0     : TMA producer.  Per step of 32 rows it brings four 128x32 operand tiles
//                    (16 KiB each, 128-byte swizzle) into one of three shared-memory stages
//                    with cp.async.bulk.tensor and arms the stage's "full" mbarrier.
//       warp 1     : MMA issuer.  The warp waits for the stage, one elected lane issues twelve 128x128x8
//                    tcgen05.mma.kind::tf32 (hi*whi, lo*whi, hi*wlo for four 8-deep blocks) and
//                    commits them to the stage's "empty" mbarrier; after a segment it commits to
//                    the accumulator's "ready" mbarrier and moves to the other accumulator.
//       warps 2..5 : epilogue.  Each warp owns 32 rows of the tile: it waits for "ready", reads its
//                    lanes of the 128-column accumulator with tcgen05.ld, adds them to 128
//                    float32 registers and arrives on the accumulator's "free" mbarrier; at the
//                    end it writes (or adds) its rows of C.
// The two 128-column accumulators let segment s+1 run on the tensor core while segment s is read
// out.  No multicast and no clusters: every tile comes from this GPU's own memory.
// Every mbarrier wait is bounded; on expiry the kernel raises a status flag, lets its copies
// land, releases its tensor memory and returns.
//
// MMA atoms, shared-memory layouts and matrix descriptors come from the CuTe sm100 headers
// (cute/arch/mma_sm100_umma.hpp, tmem_allocator_sm100.hpp); TMA, mbarrier and tcgen05.ld are
// inline PTX.
#include <cuda_runtime.h>
#include <stdint.h>

#include "qsrtb_internal.h"

#if !defined(QSRTB_NO_CUTLASS)

#include "tc_common.cuh"

namespace qsrtb_tc {

using namespace cute;

constexpr int kTile = 128;      // output tile edge
constexpr int kBlockK = 32;     // contraction elements per stage (one 128-byte swizzle row)
constexpr int kStages = 3;
constexpr int kThreads = 192;   // producer warp, MMA warp, four epilogue warps
constexpr int kSegmentSteps = 5;   // 5 steps x 12 instructions = 60 accumulations per segment
constexpr int kTileBytes = kTile * kBlockK * 4;

using Element = cutlass::tfloat32_t;

// rows [R, d] (row pitch ld) -> planes[4][d][r_pad]: hi(x), lo(x), hi(wx), lo(wx)
__global__ void __launch_bounds__(256)
split_transpose_kernel(const float* __restrict__ rows, const float* __restrict__ weights, int64_t n_rows,
                       int d, int ld, int r_pad, float* __restrict__ planes)
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
    const int64_t plane = int64_t(d) * r_pad;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = c0 + ty + 8 * i;   // feature
        const int r = r0 + tx;           // row inside the chunk (padded rows are zero)
        if (c >= d || r >= r_pad) continue;
        const float x = tile[tx][ty + 8 * i];
        const float wx = x * wts[tx];
        const float x_hi = tf32_round(x), w_hi = tf32_round(wx);
        float* out = planes + int64_t(c) * r_pad + r;
        out[0] = x_hi;
        out[plane] = tf32_round(x - x_hi);
        out[2 * plane] = w_hi;
        out[3 * plane] = tf32_round(wx - w_hi);
    }
}

struct Maps {
    CUtensorMap plane[4];
};

template <class SmemLayout>
struct SharedStorage {
    // operand kinds: 0 = hi(x), 1 = lo(x) (rows of tile bi); 2 = hi(wx), 3 = lo(wx) (rows of bj)
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
syrk_tcgen05_kernel(const __grid_constant__ Maps maps, int d, int k_steps, float* __restrict__ c_ptr, int ldc,
                    int accumulate, int* __restrict__ status, TiledMMA tiled_mma, SmemLayout)
{
    extern __shared__ __align__(1024) char smem_raw[];
    using Storage = SharedStorage<SmemLayout>;
    Storage& shared = *reinterpret_cast<Storage*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    // lower-triangular tile pair of this CTA
    int bi = int((sqrtf(8.0f * float(blockIdx.x) + 1.0f) - 1.0f) * 0.5f);
    while ((bi + 1) * (bi + 2) / 2 <= int(blockIdx.x)) ++bi;
    while (bi * (bi + 1) / 2 > int(blockIdx.x)) --bi;
    const int bj = int(blockIdx.x) - bi * (bi + 1) / 2;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // shared-memory operand views (MmaAtom, NumMma_M, NumMma_K, stage) and their descriptors
    ThrMMA cta_mma = tiled_mma.get_slice(0);
    Tensor sXhi = make_tensor(make_smem_ptr(shared.operand[0].begin()), SmemLayout{});
    Tensor sXlo = make_tensor(make_smem_ptr(shared.operand[1].begin()), SmemLayout{});
    Tensor sWhi = make_tensor(make_smem_ptr(shared.operand[2].begin()), SmemLayout{});
    Tensor sWlo = make_tensor(make_smem_ptr(shared.operand[3].begin()), SmemLayout{});
    Tensor dXhi = cta_mma.make_fragment_A(sXhi);
    Tensor dXlo = cta_mma.make_fragment_A(sXlo);
    Tensor dWhi = cta_mma.make_fragment_B(sWhi);
    Tensor dWlo = cta_mma.make_fragment_B(sWlo);

    Tensor mC = make_tensor(make_gmem_ptr(c_ptr), make_shape(d, d), make_stride(ldc, _1{}));
    Tensor gC = local_tile(mC, Shape<Int<kTile>, Int<kTile>>{}, make_coord(bi, bj));
    Tensor tCgC = cta_mma.partition_C(gC);
    Tensor tCtAcc0 = cta_mma.make_fragment_C(tCgC);   // tensor-memory accumulators
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

    const int segments = (k_steps + kSegmentSteps - 1) / kSegmentSteps;

    if (warp == 0) {
        // ---- TMA producer ---------------------------------------------------------------------
        if (lane == 0) {
            bool ok = true;
            for (int kt = 0; kt < k_steps && ok; ++kt) {
                const int s = kt % kStages;
                if (kt >= kStages) ok = bounded_wait(shared, &shared.empty[s], uint32_t((kt / kStages - 1) & 1), 0x01000000u | uint32_t(kt));
                if (!ok) break;
                cute::set_barrier_transaction_bytes(shared.full[s], 4 * kTileBytes);
                const int x = kt * kBlockK;
                tma_load_tile(&maps.plane[0], shared.operand[0].begin() + s * (kTile * kBlockK), &shared.full[s], x, bi * kTile);
                tma_load_tile(&maps.plane[1], shared.operand[1].begin() + s * (kTile * kBlockK), &shared.full[s], x, bi * kTile);
                tma_load_tile(&maps.plane[2], shared.operand[2].begin() + s * (kTile * kBlockK), &shared.full[s], x, bj * kTile);
                tma_load_tile(&maps.plane[3], shared.operand[3].begin() + s * (kTile * kBlockK), &shared.full[s], x, bj * kTile);
            }
            // tail: the last commits still arrive on the "empty" barriers; do not leave before them
            for (int kt = max(0, k_steps - kStages); kt < k_steps && ok; ++kt)
                ok = bounded_wait(shared, &shared.empty[kt % kStages], uint32_t((kt / kStages) & 1), 0x02000000u | uint32_t(kt));
        }
    } else if (warp == 1) {
        // ---- MMA issuer -----------------------------------------------------------------------
        // The whole warp runs this loop: the CuTe MMA atom and umma_arrive elect one lane
        // themselves with elect.sync over the full warp.
        bool ok = true;
        for (int seg = 0; seg < segments && ok; ++seg) {
            const int acc = seg & 1;
            if (seg >= 2)
                ok = __all_sync(0xffffffffu, bounded_wait(shared, &shared.free_[acc], uint32_t((seg / 2 - 1) & 1),
                                                          0x03000000u | uint32_t(seg)));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            tiled_mma.accumulate_ = UMMA::ScaleOut::Zero;
            const int kt_end = min(k_steps, (seg + 1) * kSegmentSteps);
            for (int kt = seg * kSegmentSteps; kt < kt_end; ++kt) {
                const int s = kt % kStages;
                ok = __all_sync(0xffffffffu, bounded_wait(shared, &shared.full[s], uint32_t((kt / kStages) & 1),
                                                          0x04000000u | uint32_t(kt)));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int kb = 0; kb < size<2>(dXhi); ++kb) {
                    if (acc == 0) {
                        gemm(tiled_mma, dXhi(_, _, kb, s), dWhi(_, _, kb, s), tCtAcc0);
                        tiled_mma.accumulate_ = UMMA::ScaleOut::One;
                        gemm(tiled_mma, dXlo(_, _, kb, s), dWhi(_, _, kb, s), tCtAcc0);
                        gemm(tiled_mma, dXhi(_, _, kb, s), dWlo(_, _, kb, s), tCtAcc0);
                    } else {
                        gemm(tiled_mma, dXhi(_, _, kb, s), dWhi(_, _, kb, s), tCtAcc1);
                        tiled_mma.accumulate_ = UMMA::ScaleOut::One;
                        gemm(tiled_mma, dXlo(_, _, kb, s), dWhi(_, _, kb, s), tCtAcc1);
                        gemm(tiled_mma, dXhi(_, _, kb, s), dWlo(_, _, kb, s), tCtAcc1);
                    }
                }
                cutlass::arch::umma_arrive(&shared.empty[s]);   // stage reusable once these MMAs have read it
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
            ok = bounded_wait(shared, &shared.ready[acc], uint32_t((seg / 2) & 1), 0x05000000u | uint32_t(seg));
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
            float* row = c_ptr + int64_t(bi * kTile + q * 32 + lane) * ldc + bj * kTile;
#pragma unroll
            for (int c = 0; c < kTile / 4; ++c) {
                float4 out = make_float4(total[4 * c], total[4 * c + 1], total[4 * c + 2], total[4 * c + 3]);
                float4* dst = reinterpret_cast<float4*>(row) + c;
                if (accumulate) {
                    const float4 old = *dst;
                    out.x += old.x; out.y += old.y; out.z += old.z; out.w += old.w;
                }
                *dst = out;
            }
        }
    }

    __syncthreads();
    if (shared.failed) {
        if (threadIdx.x == 0) atomicCAS(status, 0, int(shared.first_failure));
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

// A wait that nothing ever satisfies: exercises the bounded-wait path (expiry after kWaitCycles,
// status word, orderly return) without touching tensor memory or any copy engine.
struct ProbeStorage {
    alignas(16) uint64_t barrier;
    volatile int failed;
    volatile uint32_t first_failure;
};

__global__ void __launch_bounds__(32)
wait_probe_kernel(int* __restrict__ status)
{
    __shared__ ProbeStorage shared;
    if (threadIdx.x == 0) {
        cute::initialize_barrier(shared.barrier, 1);
        shared.failed = 0;
        shared.first_failure = 0;
        cutlass::arch::fence_barrier_init();
    }
    __syncwarp();
    const bool ok = bounded_wait(shared, &shared.barrier, 0u, 0x06000000u | threadIdx.x);
    __syncwarp();
    if (threadIdx.x == 0) atomicCAS(status, 0, ok ? 0 : int(shared.first_failure));
}

}  // namespace qsrtb_tc

using namespace qsrtb_tc;

extern "C" int qsrtb_hessian_tc_workspace_bytes(int64_t chunk_rows, int d, size_t* bytes)
{
    if (!bytes || chunk_rows <= 0 || d <= 0) return qsrtb_fail(QSRTB_EINVAL, "bad workspace query");
    const int64_t r_pad = (chunk_rows + kBlockK - 1) / kBlockK * kBlockK;
    *bytes = size_t(4) * size_t(d) * size_t(r_pad) * sizeof(float) + 256;
    return QSRTB_OK;
}

extern "C" int qsrtb_hessian_accumulate_tc(const float* rows, const float* weights, int64_t n_rows, int d,
                                           int ld_rows, float* lower, int ld_h, int accumulate,
                                           void* workspace, size_t workspace_bytes, int* status_flag,
                                           void* stream)
{
    if (!lower || d <= 0 || (d % kTile) != 0 || ld_h < d || (ld_h % 4) != 0 || n_rows <= 0 || !rows || ld_rows < d)
        return qsrtb_fail(QSRTB_EINVAL, "tensor-core Hessian needs d a multiple of 128 and at least one row");
    if (reinterpret_cast<uintptr_t>(lower) & 15) return qsrtb_fail(QSRTB_EINVAL, "accumulator must be 16-byte aligned");
    if (!status_flag) return qsrtb_fail(QSRTB_EINVAL, "status flag pointer required");
    const int64_t r_pad64 = (n_rows + kBlockK - 1) / kBlockK * kBlockK;
    if (r_pad64 > (int64_t(1) << 28)) return qsrtb_fail(QSRTB_EINVAL, "row chunk too large");
    const int r_pad = int(r_pad64);
    size_t need = 0;
    qsrtb_hessian_tc_workspace_bytes(n_rows, d, &need);
    if (!workspace || workspace_bytes < need) return qsrtb_fail(QSRTB_ESCRATCH, "Hessian workspace too small");
    EncodeTiled encode = encode_tiled_entry();
    if (!encode) return qsrtb_fail(QSRTB_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* planes = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));

    dim3 grid_t(unsigned(r_pad / 32), unsigned((d + 31) / 32));
    split_transpose_kernel<<<grid_t, 256, 0, s>>>(rows, weights, n_rows, d, ld_rows, r_pad, planes);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "split_transpose launch");

    // one tensor map per plane: [d rows, r_pad columns] float32, boxes of 128 rows x 32 columns,
    // 128-byte swizzle (the layout the K-major UMMA descriptors expect)
    Maps maps;
    const cuuint64_t dims[2] = {cuuint64_t(r_pad), cuuint64_t(d)};
    const cuuint64_t strides[1] = {cuuint64_t(r_pad) * sizeof(float)};
    const cuuint32_t box[2] = {cuuint32_t(kBlockK), cuuint32_t(kTile)};
    const cuuint32_t elem[2] = {1, 1};
    for (int p = 0; p < 4; ++p) {
        const CUresult rc = encode(&maps.plane[p], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                                   planes + size_t(p) * size_t(d) * size_t(r_pad), dims, strides, box, elem,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rc != CUDA_SUCCESS) return qsrtb_fail(QSRTB_ECUDA, "cuTensorMapEncodeTiled failed");
    }

    TiledMMA tiled_mma = make_tiled_mma(
        SM100_MMA_TF32_SS<Element, Element, float, kTile, kTile, UMMA::Major::K, UMMA::Major::K>{});
    auto mma_shape = partition_shape_A(tiled_mma, make_shape(Int<kTile>{}, Int<kBlockK>{}));
    auto smem_layout = UMMA::tile_to_mma_shape(UMMA::Layout_K_SW128_Atom<Element>{},
                                               append(mma_shape, Int<kStages>{}));
    static_assert(cute::cosize_v<decltype(smem_layout)> == kStages * kTile * kBlockK,
                  "stages must be 16 KiB apart");
    using Storage = SharedStorage<decltype(smem_layout)>;
    const int smem_bytes = int(sizeof(Storage)) + 1024;
    auto kernel = syrk_tcgen05_kernel<decltype(tiled_mma), decltype(smem_layout)>;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "cudaFuncSetAttribute(syrk_tcgen05)");
    const int nb = d / kTile;
    kernel<<<nb * (nb + 1) / 2, kThreads, smem_bytes, s>>>(maps, d, r_pad / kBlockK, lower, ld_h, accumulate,
                                                           status_flag, tiled_mma, smem_layout);
    err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "syrk_tcgen05 launch");
    return QSRTB_OK;
}

extern "C" int qsrtb_hessian_tc_wait_probe(int* status_flag, void* stream)
{
    if (!status_flag) return qsrtb_fail(QSRTB_EINVAL, "status flag pointer required");
    wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status_flag);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "wait_probe launch");
    return QSRTB_OK;
}

#else  // QSRTB_NO_CUTLASS

extern "C" int qsrtb_hessian_tc_wait_probe(int*, void*)
{
    return qsrtb_fail(QSRTB_EINVAL, "built without the CUTLASS/CuTe headers: tensor-core Hessian unavailable");
}


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
