// Shared pieces of the tcgen05 (UMMA) kernels: bounded mbarrier waits, TMA tile loads, tensor-memory
// reads, exact TF32 head/tail rounding and the driver entry point that encodes tensor maps.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cute/tensor.hpp>
#include <cute/arch/cluster_sm90.hpp>
#include <cute/arch/tmem_allocator_sm100.hpp>
#include <cutlass/arch/barrier.h>
#include <cutlass/numeric_types.h>

namespace qsrtb_tc {

constexpr long long kWaitCycles = 40000000;   // about 20 ms: far beyond any healthy wait

__device__ __forceinline__ float tf32_round(float x)
{
    uint32_t u = __float_as_uint(x);
    u += 0x00000fffu + ((u >> 13) & 1u);   // round to nearest even on 10 mantissa bits
    return __uint_as_float(u & 0xffffe000u);
}

// Waits for a phase of an mbarrier for at most kWaitCycles; `where` identifies the wait in the
// status word the host reads (role in the top byte, barrier index below, sequence number low).
// `shared` needs the members `volatile int failed` and `volatile uint32_t first_failure`.
template <class Storage>
__device__ __forceinline__ bool bounded_wait(Storage& shared, uint64_t* barrier, uint32_t phase, uint32_t where)
{
    const uint32_t addr = cute::cast_smem_ptr_to_uint(barrier);
    const long long start = clock64();
    for (int i = 0;; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(phase) : "memory");
        if (done) return true;
        if (shared.failed) return false;   // another role already gave up
        if ((i & 15) == 15 && clock64() - start > kWaitCycles) break;
    }
    if (atomicCAS(const_cast<int*>(&shared.failed), 0, int(where)) == 0) shared.first_failure = where;
    return false;
}

__device__ __forceinline__ void arrive(uint64_t* barrier)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(cute::cast_smem_ptr_to_uint(barrier)) : "memory");
}

// One box of a 2-D tensor map: element column x (x * 4 bytes a multiple of 16), row y.
__device__ __forceinline__ void tma_load_tile(const CUtensorMap* map, void* smem_dst, uint64_t* barrier, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        :: "r"(cute::cast_smem_ptr_to_uint(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y),
           "r"(cute::cast_smem_ptr_to_uint(barrier))
        : "memory");
}

// One box of a 3-D tensor map (column x, row y, matrix z of a stack).
__device__ __forceinline__ void tma_load_tile_3d(const CUtensorMap* map, void* smem_dst, uint64_t* barrier, int x,
                                                 int y, int z)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        :: "r"(cute::cast_smem_ptr_to_uint(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z),
           "r"(cute::cast_smem_ptr_to_uint(barrier))
        : "memory");
}

// 16 consecutive accumulator columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_load16(uint32_t taddr, float (&v)[16])
{
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiled encode_tiled_entry()
{
    static EncodeTiled fn = nullptr;
    if (fn) return fn;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<EncodeTiled>(ptr);
    return fn;
}

}  // namespace qsrtb_tc
