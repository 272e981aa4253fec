// Device code shared by the tile-search kernels: trellis geometry, the add-compare-select
// step, the boundary argmin with the reference tie order, the batched traceback, and the
// description of where tiles are read and written.
#pragma once

#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

namespace qsrtb_vit {


constexpr int kUnits = 1024;  // work units per tile; a thread owns UNITS of them
constexpr uint32_t kInf2 = 0x7c007c00u;
constexpr uint32_t kMax2 = 0x7bff7bffu;
constexpr int kSafeSteps = 8;  // >= ceil((16-K)/K) for K in {2,3,4}: all states reachable after

enum Mode { MODE_FAST = 0, MODE_SAFE = 1, MODE_K2 = 2 };

template <int K>
struct Geo {
    static constexpr int Kr = 16 - K;
    static constexpr int edges = 1 << Kr;
    static constexpr int NK = 1 << K;                  // predecessors per out-edge
    static constexpr int E = edges / kUnits;           // out-edges per unit: 16 / 8 / 4
    static constexpr int P = E / 2;                    // out-edge pairs per unit
    static constexpr int Q = (E >> K) > 0 ? (E >> K) : 1;  // predecessor groups per unit
    static constexpr int pred_stride = 1 << (Kr - K);  // 4096 / 1024 / 256
    static constexpr int row_bytes = (K == 2) ? edges / 4 : edges / 2;  // 4096 / 4096 / 2048
    static constexpr int rows_per_batch = (2 * edges * 2) / row_bytes;  // 16 / 8 / 8
    static constexpr int JB = Kr - 10;                 // bits of the per-thread scan index
};

__device__ __forceinline__ __half2 u2h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }
__device__ __forceinline__ uint32_t h22u(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }

__device__ __forceinline__ __half2 fp8x2_to_half2(uint32_t pair)
{
    const __half2_raw raw =
        __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(pair), __NV_E4M3);
    return __half2(raw);
}

__device__ __forceinline__ float e4m3_to_float(uint8_t b)
{
    const __half_raw raw = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
    return __half2float(__half(raw));
}

constexpr int ilog2(int n) { return n <= 1 ? 0 : 1 + ilog2(n / 2); }

// Minimum of a group of candidates plus, per 16-bit lane, the bits of the winner's position
// as full-lane masks (0xffff / 0): bit[j] is bit j of the position inside the group.
template <int LOG>
struct MinBits {
    __half2 m;
    uint32_t bit[LOG > 0 ? LOG : 1];
};

// Tournament over c[LO .. LO+N).  On ties the lower predecessor wins, which is what a
// sequential scan with a strict less-than keeps.  A merge costs one min, one compare and one
// three-input select per index bit already known below it; the compare mask itself is the new
// top bit, so no constants are folded in until the position is assembled once at the end.
template <int LO, int N, bool RECORD, int NK>
__device__ __forceinline__ MinBits<ilog2(N)> tournament(const __half2 (&c)[NK])
{
    MinBits<ilog2(N)> r;
    if constexpr (N == 1) {
        r.m = c[LO];
        r.bit[0] = 0u;
    } else {
        constexpr int LOG = ilog2(N);
        const auto a = tournament<LO, N / 2, RECORD, NK>(c);
        const auto b = tournament<LO + N / 2, N / 2, RECORD, NK>(c);
        r.m = __hmin2(b.m, a.m);
        if constexpr (RECORD) {
            const uint32_t lt = __hlt2_mask(b.m, a.m);
#pragma unroll
            for (int j = 0; j < LOG - 1; ++j) r.bit[j] = (lt & b.bit[j]) | (~lt & a.bit[j]);
            r.bit[LOG - 1] = lt;
        } else {
#pragma unroll
            for (int j = 0; j < LOG; ++j) r.bit[j] = 0u;
        }
    }
    return r;
}

// Minimum of c[0 .. N) where no position is wanted: a ternary tree, so that each level maps to
// the three-input half2 minimum (4 candidates in 2 instructions instead of 3).  Minima of
// non-NaN values do not depend on the order they are taken in.  Measured faster only for the
// four candidates of K2; with eight or sixteen the two-input tree wins.
template <int N, int NK>
__device__ __forceinline__ __half2 min_reduce(const __half2 (&c)[NK])
{
    __half2 v[N];
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = c[i];
    int n = N;
#pragma unroll
    for (int level = 0; level < 4; ++level) {
        if (n > 1) {
            const int m = (n + 2) / 3;
#pragma unroll
            for (int i = 0; i < m; ++i) {
                const int a = 3 * i, b = 3 * i + 1, d = 3 * i + 2;
                if (d < n)
                    v[i] = __hmin2(__hmin2(v[a], v[b]), v[d]);
                else if (b < n)
                    v[i] = __hmin2(v[a], v[b]);
                else
                    v[i] = v[a];
            }
            n = m;
        }
    }
    return v[0];
}

// One add-compare-select step for the calling thread's out-edges.
//   L        : the thread's 64 label bytes, [pair][pred/2] words of two fp8x2
//   inc/cur  : previous / new path costs (shared memory)
//   track    : MODE_FAST running max of stored costs; MODE_K2 running min of this step
//   u        : the unit (0..1023) these labels belong to
// NL = 16: labels kept as packed fp8 pairs and converted every step; NL = 32: labels kept as
// half2 (one register per out-edge pair and predecessor), no conversion in the loop.
// RECORD with COSTS = false writes the survivor decisions of the step to dec_row (a nibble, or
// two bits at K = 2, per out-edge).  RECORD with COSTS = true writes the step's new path costs
// there instead (one half per out-edge) and tracks no positions: the decision of the one
// out-edge a traceback visits is then recomputed from the costs of the step before.
template <int K, int MODE, bool FIRST, bool CONSTRAINED, bool RECORD, int NL, bool COSTS = false>
__device__ __forceinline__ void acs_step(const uint32_t (&L)[NL], const int u, const __half* inc,
                                         __half* cur, __half w, int pre_state, __half2 shift2,
                                         uint8_t* dec_row, __half2& track)
{
    using G = Geo<K>;
    constexpr int NK = G::NK;
    const int qbase = (G::E * u) >> K;
    const __half2 w2 = __half2half2(w);
    const __half2 inf2 = u2h2(kInf2);
    const __half2 max2 = u2h2(kMax2);

    // Predecessor costs: Q consecutive halves for each of the NK predecessors.
    uint32_t pw[NK][(G::Q + 1) / 2];
    if constexpr (!FIRST) {
#pragma unroll
        for (int k = 0; k < NK; ++k) {
            if constexpr (G::Q == 4) {
                const uint2 v = *reinterpret_cast<const uint2*>(inc + qbase + k * G::pred_stride);
                pw[k][0] = v.x;
                pw[k][1] = v.y;
            } else {
                pw[k][0] = *reinterpret_cast<const uint16_t*>(inc + qbase + k * G::pred_stride);
            }
        }
    }

    uint32_t outw[G::P];
    uint32_t dec[G::P];
    // Branch metrics of out-edge pair j against all NK predecessors (FP16 FMA pipe).
    auto metrics = [&](const int j, __half2 (&c)[NK]) {
        const int qq = (2 * j) >> K;  // predecessor group of this pair within the thread
#pragma unroll
        for (int k = 0; k < NK; ++k) {
            __half2 d;
            if constexpr (NL == 32) {
                d = u2h2(L[j * NK + k]);
            } else {
                const uint32_t word = L[j * (NK / 2) + (k >> 1)];
                d = fp8x2_to_half2((k & 1) ? (word >> 16) : (word & 0xffffu));
            }
            const __half2 dh = __hsub2(d, w2);
            if constexpr (FIRST) {
                __half2 v = __hmul2(dh, dh);
                if constexpr (MODE != MODE_K2) v = __hmin2(v, max2);
                if constexpr (CONSTRAINED) {
                    if (qbase + qq + k * G::pred_stride != pre_state) v = inf2;
                }
                c[k] = v;
            } else {
                __half2 p2;
                uint32_t pbits;
                if constexpr (G::Q == 4) {
                    const uint32_t pwv = pw[k][qq >> 1];
                    p2 = (qq & 1) ? __high2half2(u2h2(pwv)) : __low2half2(u2h2(pwv));
                    pbits = (qq & 1) ? (pwv >> 16) : (pwv & 0xffffu);
                } else {
                    p2 = __low2half2(u2h2(pw[k][0]));
                    pbits = pw[k][0];
                }
                __half2 v = __hfma2(dh, dh, p2);
                if constexpr (MODE == MODE_SAFE) {
                    v = __hmin2(v, max2);
                    if (pbits == 0x7c00u) v = inf2;
                }
                c[k] = v;
            }
        }
    };
    // Survivor of pair j and its position (ALU pipe).
    auto select = [&](const int j, __half2 (&c)[NK]) {
        MinBits<ilog2(NK)> r;
        if constexpr (RECORD && !COSTS)
            r = tournament<0, NK, true, NK>(c);
        else if constexpr (NK == 4)
            r.m = min_reduce<NK, NK>(c);  // K2: 258 k against 252 k tiles/s
        else
            r = tournament<0, NK, false, NK>(c);  // K3, K4: the binary tree is faster (348 k against 340 k)
        if constexpr (MODE == MODE_K2) {
            r.m = __hsub2(r.m, shift2);
            track = __hmin2(track, r.m);
        } else if constexpr (MODE == MODE_FAST) {
            track = __hmax2(track, r.m);
        }
        outw[j] = h22u(r.m);
        uint32_t position = 0u;
        if constexpr (RECORD && !COSTS) {
#pragma unroll
            for (int b = 0; b < K; ++b) position |= r.bit[b] & (0x00010001u << b);
        }
        dec[j] = position;
    };
    // Software pipeline: the metrics of the next pair are issued ahead of this pair's selection,
    // so that the two math pipes have independent work side by side.
    {
        __half2 cbuf[2][NK];
        metrics(0, cbuf[0]);
#pragma unroll
        for (int j = 0; j < G::P; ++j) {
            if (j + 1 < G::P) metrics(j + 1, cbuf[(j + 1) & 1]);
            select(j, cbuf[j & 1]);
        }
    }

    // Store the new costs: E consecutive halves.
    if constexpr (G::P == 8) {
        uint4* dst = reinterpret_cast<uint4*>(cur + G::E * u);
        dst[0] = make_uint4(outw[0], outw[1], outw[2], outw[3]);
        dst[1] = make_uint4(outw[4], outw[5], outw[6], outw[7]);
    } else if constexpr (G::P == 4) {
        *reinterpret_cast<uint4*>(cur + G::E * u) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
    } else {
        *reinterpret_cast<uint2*>(cur + G::E * u) = make_uint2(outw[0], outw[1]);
    }

    if constexpr (RECORD && COSTS) {
        // the cost row of this step: the same E halves as above, to global memory
        uint8_t* row = dec_row + 2 * G::E * u;
        if constexpr (G::P == 8) {
            uint4* dst = reinterpret_cast<uint4*>(row);
            dst[0] = make_uint4(outw[0], outw[1], outw[2], outw[3]);
            dst[1] = make_uint4(outw[4], outw[5], outw[6], outw[7]);
        } else if constexpr (G::P == 4) {
            *reinterpret_cast<uint4*>(row) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
        } else {
            *reinterpret_cast<uint2*>(row) = make_uint2(outw[0], outw[1]);
        }
    } else if constexpr (RECORD) {
        if constexpr (K == 2) {
            // byte q: two bits for each of out-edges 4q..4q+3
            uint32_t word = 0;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const uint32_t v = dec[2 * g] | (dec[2 * g + 1] << 4);
                word |= ((v | (v >> 14)) & 0xffu) << (8 * g);
            }
            *reinterpret_cast<uint32_t*>(dec_row + 4 * u) = word;
        } else {
            // byte e/2: one nibble for each of out-edges e, e+1
            uint32_t word = 0;
#pragma unroll
            for (int j = 0; j < G::P; ++j)
                word |= ((dec[j] | (dec[j] >> 12)) & 0xffu) << (8 * j);
            if constexpr (G::P == 4)
                *reinterpret_cast<uint32_t*>(dec_row + 4 * u) = word;
            else
                *reinterpret_cast<uint16_t*>(dec_row + 2 * u) = static_cast<uint16_t>(word);
        }
    }
}

__device__ __forceinline__ uint32_t bitrev5(uint32_t v) { return __brev(v) >> 27; }

// Sortable 16-bit key of a half (signed order; no NaN reaches this).
__device__ __forceinline__ uint32_t half_key(uint32_t h)
{
    return (h & 0x8000u) ? (~h & 0xffffu) : (h | 0x8000u);
}

// Minimum of a half over the warp (no NaN among the inputs): one integer reduction on the
// sortable keys instead of five dependent shuffle rounds.
__device__ __forceinline__ __half warp_min_half(__half v)
{
    const uint32_t key = __reduce_min_sync(0xffffffffu, half_key(__half_as_ushort(v)));
    return __ushort_as_half(static_cast<unsigned short>((key & 0x8000u) ? (key & 0x7fffu) : (~key & 0xffffu)));
}

// Boundary argmin with the reference's tie order.
//   TREE512: the generic kernel for K != 2 reduces with 512 threads holding two interleaved
//   streams (cuh:388-423); otherwise 1024 threads hold one stream (cuh:365-387, k2 cuh:276-325).
// In both, shuffle trees that only replace on strict less-than prefer the partner whose
// lane / slot index is smaller after 5-bit reversal, and a thread keeps its earliest edge.
// The key of an edge depends only on the edge, so the reduction may be carried out by any
// number of threads in any order: each thread folds the edges of UNITS reference threads.
template <int K, bool TREE512, int UNITS>
__device__ __forceinline__ int boundary_argmin(const __half* costs, uint32_t* red)
{
    using G = Geo<K>;
    constexpr int THREADS = kUnits / UNITS;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t best = 0xffffffffu;
#pragma unroll
    for (int uu = 0; uu < UNITS; ++uu) {
        const int t = threadIdx.x + uu * THREADS;  // thread index in the reference's 1024-thread block
        uint32_t prio_hi;
        if constexpr (TREE512) {
            const uint32_t slot = ((t >> 9) & 1) * 16 + ((t >> 5) & 15);
            prio_hi = (bitrev5(slot) << 5) | bitrev5(t & 31);
        } else {
            prio_hi = (bitrev5(t >> 5) << 5) | bitrev5(t & 31);
        }
#pragma unroll
        for (int j = 0; j < (1 << G::JB); ++j) {
            const uint32_t h = *reinterpret_cast<const uint16_t*>(costs + t + 1024 * j);
            const uint32_t key = (half_key(h) << 16) | (prio_hi << G::JB) | uint32_t(j);
            best = min(best, key);
        }
    }
    best = __reduce_min_sync(0xffffffffu, best);
    if (lane == 0) red[warp] = best;
    __syncthreads();
    uint32_t v = lane < THREADS / 32 ? red[lane] : 0xffffffffu;
    v = __reduce_min_sync(0xffffffffu, v);
    __syncthreads();
    const uint32_t j = v & ((1u << G::JB) - 1);
    const uint32_t hi = (v & 0xffffu) >> G::JB;
    const uint32_t l = bitrev5(hi & 31), s = bitrev5(hi >> 5);
    if constexpr (TREE512)
        return int(j * 1024 + (s >> 4) * 512 + (s & 15) * 32 + l);
    else
        return int(j * 1024 + s * 32 + l);
}

// Walk survivor rows ri_hi .. 0 starting from `edge`; returns the state before row 0.
// Rows are streamed from the CTA's scratch slice through `rowbuf` (the idle cost buffers).
template <int K, int UNITS>
__device__ __forceinline__ int traceback(uint8_t* scratch, uint8_t* rowbuf, int ri_hi, int edge,
                                         bool write, uint16_t* sh_states, int* sh_edge)
{
    using G = Geo<K>;
    for (int hi = ri_hi; hi >= 0; hi -= G::rows_per_batch) {
        const int lo = max(0, hi - G::rows_per_batch + 1);
        const int nvec = (hi - lo + 1) * (G::row_bytes / 16);
        const uint4* src = reinterpret_cast<const uint4*>(scratch + size_t(lo) * G::row_bytes);
        uint4* dst = reinterpret_cast<uint4*>(rowbuf);
        for (int v = threadIdx.x; v < nvec; v += kUnits / UNITS) dst[v] = src[v];
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int ri = hi; ri >= lo; --ri) {
                const uint8_t* row = rowbuf + (ri - lo) * G::row_bytes;
                int decision;
                if constexpr (K == 2)
                    decision = (row[edge >> 2] >> ((edge & 3) * 2)) & 3;
                else
                    decision = (row[edge >> 1] >> ((edge & 1) * 4)) & 15;
                const int prev = (decision << (16 - 2 * K)) | (edge >> K);
                if (write) sh_states[ri] = uint16_t((prev << K) | edge);
                edge = prev;
            }
            *sh_edge = edge;
        }
        __syncthreads();
        edge = *sh_edge;
    }
    return edge;
}

// Where a CTA finds tile `t` and where its results go.
//   rows_mode == 0: tiles are contiguous [n, 256] in tensor-core element order.
//   rows_mode == 1: tile t is the 16x16 block (matrix b = t / tiles_n, column tile t % tiles_n)
//     of a 16-row slab of row-major matrices; the encoder input is w + multiplier * comp
//     (exl3_encoder_backend.py:408-417, 502-509) and the reconstruction goes back to the
//     same 16 rows of wq (and, optionally, w - wq to err), so the per-step gather, permute,
//     un-permute and scatter kernels of the reference's LDLQ loop disappear.
struct TileIO {
    const float* tiles;
    float* out_tiles;
    uint16_t* out_states;
    const float* w;
    const float* comp;
    float* wq;
    float* err;
    int64_t w_stride;     // elements between consecutive matrices of w / wq / err
    int64_t comp_stride;  // elements between consecutive matrices of comp
    int64_t state_stride; // elements between consecutive matrices of out_states
    int ld;               // row pitch of w / wq / err
    int comp_ld;          // row pitch of comp
    int tiles_n;          // column tiles visited per matrix
    const int* tile_map;  // optional: visited column tile i is tile_map[i] (mixed-rate maps)
    const int2* members;  // optional: visited matrix b reads source matrix members[b].x of w and
                          // owns matrix members[b].y of comp / wq / err / out_states
    float multiplier;
    int rows_mode;
};

// Row-major offset (row * 16 + col) of tensor-core element t (exl3_encoder_backend.py:35-57).
__device__ __forceinline__ int tensor_core_rc(int t, int& col)
{
    const int lane = t >> 3, j = t & 7;
    const int r0 = (lane & 3) * 2;
    const int row = r0 + (j & 1) + ((j & 2) ? 8 : 0);
    col = (lane >> 2) + ((j & 4) ? 8 : 0);
    return row;
}

}  // namespace qsrtb_vit

// The tile search with lazily resolved decisions (viterbi_lazy.cu).  `grid` persistent CTAs, each
// owning qsrtb_lazy_scratch_per_cta(bits, dedicated) bytes of `scratch`.
size_t qsrtb_lazy_scratch_per_cta(int bits, int dedicated);
int qsrtb_lazy_launch(const qsrtb_vit::TileIO& io, int64_t n_tiles, const uint8_t* lut_state,
                      const uint8_t* lut_pm, int bits, int context, int dedicated, void* scratch, int grid,
                      cudaStream_t stream);
