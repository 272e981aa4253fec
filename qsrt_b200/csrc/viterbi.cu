// Tail-biting Viterbi tile encoder for sm_100a.
//
// One persistent CTA (1024 threads, one per SM) encodes one 256-value tile at a time:
//   primer pass over 2*C symbols centred on symbol 0 -> boundary state,
//   constrained pass over all 256 symbols from/to that state -> 256 trellis states.
// Results are bit-identical to the reference kernels
//   qsrt/csrc/qsrt_quantize_tiles_kernel.cuh:26-500      (MODE_FAST / MODE_SAFE below)
//   qsrt/csrc/qsrt_quantize_tiles_k2_kernel.cuh:47-366   (MODE_K2)
// but the work is organised differently:
//   * a thread owns a fixed run of 16/8/4 consecutive out-edges (K = 2/3/4).  Its 64 label
//     bytes stay in 16 registers for the life of the CTA (all tiles), so the table is read
//     from memory once per CTA rather than once per trellis step;
//   * path costs live in shared memory (2 x 2^(16-K) halves, double buffered), read with one
//     vector load per predecessor group and written with one vector store per thread;
//   * the best predecessor is found by a branch-free tournament on half2 lanes whose index
//     bits are carried in LOP3 masks (ties keep the lower predecessor, as the reference's
//     sequential strict-less scan does);
//   * survivor decisions stream to an L2-resident scratch slice owned by the CTA (a row of
//     4 KiB or 2 KiB per step).  The traceback streams those rows back through the then idle
//     cost buffers with 16-byte coalesced loads, 16 or 8 rows at a time, and walks them out of
//     shared memory, instead of chasing 256 dependent global loads;
//   * the boundary argmin is a single integer min-reduction over (cost, priority) keys where
//     the priority encodes the reference's shuffle-tree tie order in closed form;
//   * the saturation clamp and unreachable-state tests of the generic kernel are only
//     executed where they can matter (MODE_SAFE); MODE_FAST tracks the running maximum and
//     the tile is re-encoded in MODE_SAFE if any stored cost reached the clamp.
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "qsrtb_internal.h"

namespace {

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

// One add-compare-select step for the calling thread's out-edges.
//   L        : the thread's 64 label bytes, [pair][pred/2] words of two fp8x2
//   inc/cur  : previous / new path costs (shared memory)
//   track    : MODE_FAST running max of stored costs; MODE_K2 running min of this step
//   u        : the unit (0..1023) these labels belong to
// NL = 16: labels kept as packed fp8 pairs and converted every step; NL = 32: labels kept as
// half2 (one register per out-edge pair and predecessor), no conversion in the loop.
template <int K, int MODE, bool FIRST, bool CONSTRAINED, bool RECORD, int NL>
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
        auto r = tournament<0, NK, RECORD, NK>(c);
        if constexpr (MODE == MODE_K2) {
            r.m = __hsub2(r.m, shift2);
            track = __hmin2(track, r.m);
        } else if constexpr (MODE == MODE_FAST) {
            track = __hmax2(track, r.m);
        }
        outw[j] = h22u(r.m);
        uint32_t position = 0u;
        if constexpr (RECORD) {
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

    if constexpr (RECORD) {
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

struct Smem {
    __half in_h[256];
    uint16_t states[256];
    uint32_t red[32];
    __half warp_mins[2][32];
    __half shift[2];
    int edge;
    int pad[3];
};

// Encode the tile whose rounded input is already in sm->in_h.  Returns (block-uniform) whether
// the result is valid; only MODE_FAST can return false.
template <int K, int MODE, int UNITS, int NL>
__device__ __forceinline__ bool encode_tile(const uint32_t (&L)[UNITS][NL], Smem* sm, __half* cost0,
                                            __half* cost1, uint8_t* scratch, int context)
{
    using G = Geo<K>;
    constexpr int THREADS = kUnits / UNITS;
    constexpr int WARPS = THREADS / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __half* cur = cost0;
    __half* inc = cost1;
    __half2 track_max = u2h2(0u);
    bool valid = true;

    // The lag-2 renormalisation of the dedicated K2 kernel (k2 cuh:117-137, 211-230):
    // the shift used by step s is the block minimum stored by step s-2 when that is >= 1024.
    auto k2_fold = [&](int s) {
        if (warp == 0) {
            __half m = lane < WARPS ? sm->warp_mins[(s - 1) & 1][lane] : __ushort_as_half(0x7c00);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = __hmin(m, __shfl_down_sync(0xffffffffu, m, o));
            if (lane == 0)
                sm->shift[(s + 1) & 1] = __hge(m, __float2half_rn(1024.0f)) ? m : __ushort_as_half(0);
        }
    };
    auto k2_publish = [&](int s, __half2 step_min2) {
        __half m = __hmin(__low2half(step_min2), __high2half(step_min2));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = __hmin(m, __shfl_down_sync(0xffffffffu, m, o));
        if (lane == 0) sm->warp_mins[s & 1][warp] = m;
    };

#define UNIT_LOOP(...)                                                        \
    do {                                                                      \
        _Pragma("unroll") for (int uu = 0; uu < UNITS; ++uu) { __VA_ARGS__; } \
    } while (0)

    auto run_pass = [&](int roll, int steps, int pre_state, int trace_start, auto constrained_tag) {
        constexpr bool CONSTRAINED = decltype(constrained_tag)::value;
        if constexpr (MODE == MODE_K2) {
            if (threadIdx.x == 0) {
                sm->shift[0] = __ushort_as_half(0);
                sm->shift[1] = __ushort_as_half(0);
            }
            __syncthreads();
        }
        for (int i = 0; i < steps; ++i) {
            const int ri = (i + roll) & 255;
            __half* t = cur; cur = inc; inc = t;
            const __half w = sm->in_h[ri];
            uint8_t* dec_row = scratch + size_t(ri) * G::row_bytes;
            __half2 shift2 = u2h2(0u);
            __half2 step_min2 = u2h2(kInf2);
            if constexpr (MODE == MODE_K2) {
                if (i > 0) k2_fold(i);
                shift2 = __half2half2(sm->shift[i & 1]);
            }
            if (i == 0) {
                if constexpr (MODE == MODE_K2)
                    UNIT_LOOP(acs_step<K, MODE, true, CONSTRAINED, CONSTRAINED, NL>(L[uu], int(threadIdx.x) + uu * THREADS, inc, cur, w, pre_state, shift2, dec_row, step_min2));
                else if constexpr (MODE == MODE_FAST && CONSTRAINED)
                    UNIT_LOOP(acs_step<K, MODE_SAFE, true, true, true, NL>(L[uu], int(threadIdx.x) + uu * THREADS, inc, cur, w, pre_state, shift2, dec_row, track_max));
                else
                    UNIT_LOOP(acs_step<K, MODE, true, CONSTRAINED, CONSTRAINED, NL>(L[uu], int(threadIdx.x) + uu * THREADS, inc, cur, w, pre_state, shift2, dec_row, track_max));
            } else if (i < trace_start) {
                if constexpr (MODE == MODE_K2)
                    UNIT_LOOP(acs_step<K, MODE, false, false, false, NL>(L[uu], int(threadIdx.x) + uu * THREADS, inc, cur, w, -1, shift2, dec_row, step_min2));
                else
                    UNIT_LOOP(acs_step<K, MODE, false, false, false, NL>(L[uu], int(threadIdx.x) + uu * THREADS, inc, cur, w, -1, shift2, dec_row, track_max));
            } else {
                if constexpr (MODE == MODE_K2) {
                    UNIT_LOOP(acs_step<K, MODE, false, false, true, NL>(L[uu], int(threadIdx.x) + uu * THREADS, inc, cur, w, -1, shift2, dec_row, step_min2));
                } else if constexpr (MODE == MODE_FAST && CONSTRAINED) {
                    // Unreachable states exist for the first few constrained steps.
                    if (i < kSafeSteps)
                        UNIT_LOOP(acs_step<K, MODE_SAFE, false, false, true, NL>(L[uu], int(threadIdx.x) + uu * THREADS, inc, cur, w, -1, shift2, dec_row, track_max));
                    else
                        UNIT_LOOP(acs_step<K, MODE, false, false, true, NL>(L[uu], int(threadIdx.x) + uu * THREADS, inc, cur, w, -1, shift2, dec_row, track_max));
                } else {
                    UNIT_LOOP(acs_step<K, MODE, false, false, true, NL>(L[uu], int(threadIdx.x) + uu * THREADS, inc, cur, w, -1, shift2, dec_row, track_max));
                }
            }
            if constexpr (MODE == MODE_K2) k2_publish(i, step_min2);
            __syncthreads();
        }
    };

    // Primer: 2*C symbols centred on symbol 0, decisions kept for the last C of them.
    run_pass(256 - context, 2 * context, -1, context, std::false_type{});
    if constexpr (MODE == MODE_FAST) {
        const bool over = !(__hlt(__low2half(track_max), u2h2(kMax2).x) &&
                            __hlt(__high2half(track_max), u2h2(kMax2).x));
        if (__syncthreads_or(over)) return false;
    }
    int boundary;
    if constexpr (MODE == MODE_K2)
        boundary = boundary_argmin<K, false, UNITS>(cur, sm->red);  // final primer step (k2 cuh:282)
    else
        boundary = boundary_argmin<K, K != 2, UNITS>(inc, sm->red);  // step before the last (cuh:375,401)
    const int end_state = traceback<K, UNITS>(scratch, reinterpret_cast<uint8_t*>(cost0), context - 1,
                                       boundary, false, sm->states, &sm->edge);

    // Constrained pass: starts from and must return to end_state.
    run_pass(0, 256, end_state, 0, std::true_type{});
    if constexpr (MODE == MODE_FAST) {
        const bool over = !(__hlt(__low2half(track_max), u2h2(kMax2).x) &&
                            __hlt(__high2half(track_max), u2h2(kMax2).x));
        if (__syncthreads_or(over)) valid = false;
    }
    if (valid)
        traceback<K, UNITS>(scratch, reinterpret_cast<uint8_t*>(cost0), 255, end_state, true, sm->states,
                     &sm->edge);
    return valid;
#undef UNIT_LOOP
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

template <int K, bool DEDICATED, int UNITS>
__global__ void __launch_bounds__(kUnits / UNITS, 1)
viterbi_kernel(const TileIO io, const uint8_t* __restrict__ lut_pm,
               const uint8_t* __restrict__ lut_state, uint8_t* scratch_base, int64_t n_tiles,
               int context)
{
    using G = Geo<K>;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __half* cost0 = reinterpret_cast<__half*>(smem_raw);
    __half* cost1 = cost0 + G::edges;
    Smem* sm = reinterpret_cast<Smem*>(smem_raw + 2 * G::edges * sizeof(__half));
    uint8_t* scratch = scratch_base + size_t(blockIdx.x) * 256 * G::row_bytes;

    // With two units per thread there is room to keep the labels as half2 (32 registers per
    // unit), which takes the fp8 -> half conversion out of the add-compare-select loop.
    constexpr int THREADS = kUnits / UNITS;
    constexpr int NL = UNITS >= 2 ? 32 : 16;
    uint32_t L[UNITS][NL];
#pragma unroll
    for (int uu = 0; uu < UNITS; ++uu) {
        const uint4* src = reinterpret_cast<const uint4*>(lut_pm) + 4 * (threadIdx.x + uu * THREADS);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 v = src[i];
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                if constexpr (NL == 32) {
                    L[uu][2 * (4 * i + q) + 0] = h22u(fp8x2_to_half2(words[q] & 0xffffu));
                    L[uu][2 * (4 * i + q) + 1] = h22u(fp8x2_to_half2(words[q] >> 16));
                } else {
                    L[uu][4 * i + q] = words[q];
                }
            }
        }
    }

    // Offsets are recomputed after the search rather than kept live across it (registers).
    auto locate = [&](int64_t tile, int64_t& src_off, int64_t& w_off, int64_t& comp_off, int64_t& state_off) {
        const int64_t b = tile / io.tiles_n;
        int tn = int(tile - b * io.tiles_n);
        if (io.tile_map != nullptr) tn = io.tile_map[tn];
        int64_t source = b, owner = b;
        if (io.members != nullptr) {
            const int2 m = io.members[b];
            source = m.x;
            owner = m.y;
        }
        int col;
        const int row = tensor_core_rc(threadIdx.x, col);
        const int64_t inside = int64_t(row) * io.ld + tn * 16 + col;
        src_off = source * io.w_stride + inside;
        w_off = owner * io.w_stride + inside;
        comp_off = owner * io.comp_stride + int64_t(row) * io.comp_ld + tn * 16 + col;
        state_off = owner * io.state_stride + int64_t(tn) * 256 + threadIdx.x;
    };

    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        if (threadIdx.x < 256) {
            float w;
            if (io.rows_mode) {
                int64_t src_off, w_off, comp_off, state_off;
                locate(tile, src_off, w_off, comp_off, state_off);
                w = io.w[src_off];
                if (io.comp != nullptr && io.multiplier != 0.0f) {
                    const float c = io.comp[comp_off];
                    w = (io.multiplier == 1.0f) ? __fadd_rn(w, c) : __fadd_rn(w, __fmul_rn(io.multiplier, c));
                }
            } else {
                w = io.tiles[tile * 256 + threadIdx.x];
            }
            if constexpr (DEDICATED) w = fmaxf(-64.0f, fminf(w, 64.0f));  // k2 cuh:82-91
            sm->in_h[threadIdx.x] = __float2half_rn(w);
        }
        __syncthreads();
        if constexpr (DEDICATED) {
            encode_tile<K, MODE_K2, UNITS, NL>(L, sm, cost0, cost1, scratch, context);
        } else {
            if (!encode_tile<K, MODE_FAST, UNITS, NL>(L, sm, cost0, cost1, scratch, context))
                encode_tile<K, MODE_SAFE, UNITS, NL>(L, sm, cost0, cost1, scratch, context);
        }
        if (threadIdx.x < 256) {
            const uint16_t s = sm->states[threadIdx.x];
            const float q = e4m3_to_float(lut_state[s]);
            if (io.rows_mode) {
                int64_t src_off, w_off, comp_off, state_off;
                locate(tile, src_off, w_off, comp_off, state_off);
                io.out_states[state_off] = s;
                io.wq[w_off] = q;
                if (io.err != nullptr) io.err[w_off] = __fsub_rn(io.w[src_off], q);
            } else {
                io.out_states[tile * 256 + threadIdx.x] = s;
                io.out_tiles[tile * 256 + threadIdx.x] = q;
            }
        }
        __syncthreads();
    }
}

template <int K>
constexpr size_t smem_bytes() { return 2 * Geo<K>::edges * sizeof(__half) + sizeof(Smem); }

int resident_ctas()
{
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    return sms;
}

template <int K, bool DEDICATED, int UNITS>
int launch(const TileIO& io, int64_t n_tiles, const uint8_t* lut_state, const uint8_t* lut_pm,
           int context, void* scratch, size_t scratch_bytes, cudaStream_t stream)
{
    using G = Geo<K>;
    const int sms = resident_ctas();
    if (sms <= 0) return qsrtb_fail(QSRTB_ECUDA, "cannot query the device");
    int64_t grid = n_tiles < sms ? n_tiles : sms;
    const size_t slice = size_t(256) * G::row_bytes;
    if (scratch_bytes < slice) return qsrtb_fail(QSRTB_ESCRATCH, "traceback scratch smaller than one slice");
    if (int64_t(scratch_bytes / slice) < grid) grid = int64_t(scratch_bytes / slice);
    auto kernel = viterbi_kernel<K, DEDICATED, UNITS>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           int(smem_bytes<K>()));
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "cudaFuncSetAttribute(viterbi)");
    kernel<<<dim3(unsigned(grid)), dim3(kUnits / UNITS), smem_bytes<K>(), stream>>>(
        io, lut_pm, lut_state, static_cast<uint8_t*>(scratch), n_tiles, context);
    err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "viterbi kernel launch");
    return QSRTB_OK;
}

// [state] -> [out-edge pair][predecessor][2] and max |label|.
__global__ void lut_prepare_kernel(const uint8_t* __restrict__ lut_state, int bits,
                                   uint8_t* __restrict__ lut_pm, float* __restrict__ abs_max)
{
    const int Kr = 16 - bits;
    const int nk = 1 << bits;
    float local = 0.0f;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < 65536; i += gridDim.x * blockDim.x) {
        const int byte = i & 1;
        const int k = (i >> 1) & (nk - 1);
        const int pair = i >> (1 + bits);
        const uint8_t label = lut_state[(k << Kr) | (2 * pair + byte)];
        lut_pm[i] = label;
        const float v = fabsf(e4m3_to_float(label));
        local = (v > local || v != v) ? v : local;
    }
    // abs_max was zeroed by the caller; non-negative floats order like their bit patterns
    // and a NaN (0x7fc00000) orders above every finite value, which is what amax would report.
    atomicMax(reinterpret_cast<unsigned int*>(abs_max), __float_as_uint(local));
}

}  // namespace

extern "C" int qsrtb_lut_prepare(const uint8_t* lut_state, int bits, uint8_t* lut_pm,
                                 float* abs_max, void* stream)
{
    if (bits < 2 || bits > 4) return qsrtb_fail(QSRTB_EINVAL, "bits must be 2, 3 or 4");
    if (!lut_state || !lut_pm || !abs_max) return qsrtb_fail(QSRTB_EINVAL, "null table pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t err = cudaMemsetAsync(abs_max, 0, sizeof(float), s);
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "cudaMemsetAsync(abs_max)");
    lut_prepare_kernel<<<64, 256, 0, s>>>(lut_state, bits, lut_pm, abs_max);
    err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "lut_prepare launch");
    return QSRTB_OK;
}

extern "C" int qsrtb_viterbi_scratch_bytes(int bits, int64_t n_tiles, size_t* bytes)
{
    if (bits < 2 || bits > 4 || !bytes || n_tiles < 0) return qsrtb_fail(QSRTB_EINVAL, "bad scratch query");
    const int sms = resident_ctas();
    if (sms <= 0) return qsrtb_fail(QSRTB_ECUDA, "cannot query the device");
    const int64_t grid = n_tiles < sms ? n_tiles : sms;
    const size_t row_bytes = bits == 4 ? 2048 : 4096;
    *bytes = size_t(grid > 0 ? grid : 1) * 256 * row_bytes;
    return QSRTB_OK;
}

namespace {

int check_common(int bits, int tailbite_context, int variant, int64_t n_tiles)
{
    if (bits < 2 || bits > 4) return qsrtb_fail(QSRTB_EINVAL, "bits must be 2, 3 or 4");
    if (tailbite_context < 1 || tailbite_context > 128)
        return qsrtb_fail(QSRTB_EINVAL, "tailbite_context must be in 1..128");
    if ((variant & ~0x31) != 0 || (variant >> 4) == 3)
        return qsrtb_fail(QSRTB_EINVAL, "variant: bit 0 selects the dedicated K2 arithmetic, bits 4-5 the thread layout (0, 1 or 2)");
    if ((variant & 1) && bits != 2)
        return qsrtb_fail(QSRTB_EINVAL, "variant bit 0 (dedicated K2 arithmetic) needs bits == 2");
    if (n_tiles < 0) return qsrtb_fail(QSRTB_EINVAL, "negative tile count");
    return QSRTB_OK;
}

// Units per thread of the add-compare-select loop (bits 4-5 of `variant`): 2 = 512 threads with
// half2 labels in registers, 1 = 1024 threads with packed fp8 labels, 0 = the faster of the two
// as measured on B200 (K2 and K4: 2, K3: 1).  Same results either way.

template <int UNITS>
int dispatch_units(const TileIO& io, int64_t n_tiles, const uint8_t* lut_state, const uint8_t* lut_pm,
                   int bits, int context, int variant, void* scratch, size_t scratch_bytes, cudaStream_t s)
{
    switch (bits) {
        case 2:
            if (variant == 1)
                return launch<2, true, UNITS>(io, n_tiles, lut_state, lut_pm, context, scratch, scratch_bytes, s);
            return launch<2, false, UNITS>(io, n_tiles, lut_state, lut_pm, context, scratch, scratch_bytes, s);
        case 3:
            return launch<3, false, UNITS>(io, n_tiles, lut_state, lut_pm, context, scratch, scratch_bytes, s);
        default:
            return launch<4, false, UNITS>(io, n_tiles, lut_state, lut_pm, context, scratch, scratch_bytes, s);
    }
}

int dispatch(const TileIO& io, int64_t n_tiles, const uint8_t* lut_state, const uint8_t* lut_pm,
             int bits, int context, int variant, void* scratch, size_t scratch_bytes, cudaStream_t s)
{
    const int layout = (variant >> 4) & 3;
    const int units = layout != 0 ? layout : (bits == 3 ? 1 : 2);
    variant &= 1;
    if (units == 1)
        return dispatch_units<1>(io, n_tiles, lut_state, lut_pm, bits, context, variant, scratch, scratch_bytes, s);
    return dispatch_units<2>(io, n_tiles, lut_state, lut_pm, bits, context, variant, scratch, scratch_bytes, s);
}

}  // namespace

extern "C" int qsrtb_quantize_tiles(const float* tiles, int64_t n_tiles, const uint8_t* lut_state,
                                    const uint8_t* lut_pm, int bits, int tailbite_context,
                                    int variant, float* out_tiles, int16_t* out_states,
                                    void* scratch, size_t scratch_bytes, void* stream)
{
    const int bad = check_common(bits, tailbite_context, variant, n_tiles);
    if (bad) return bad;
    if (n_tiles == 0) return QSRTB_OK;
    if (!tiles || !lut_state || !lut_pm || !out_tiles || !out_states || !scratch)
        return qsrtb_fail(QSRTB_EINVAL, "null pointer");
    TileIO io{};
    io.tiles = tiles;
    io.out_tiles = out_tiles;
    io.out_states = reinterpret_cast<uint16_t*>(out_states);
    io.rows_mode = 0;
    io.tiles_n = 1;
    return dispatch(io, n_tiles, lut_state, lut_pm, bits, tailbite_context, variant, scratch,
                    scratch_bytes, static_cast<cudaStream_t>(stream));
}

namespace {
int quantize_rows_impl(const float* w, const float* comp, float multiplier, int batch, int n, int ld,
                       int comp_ld, int64_t w_stride, int64_t comp_stride, const uint8_t* lut_state,
                       const uint8_t* lut_pm, int bits, int tailbite_context, int variant, float* wq,
                       float* err, int16_t* out_states, int64_t state_stride, const int32_t* tile_map,
                       int tile_map_count, const int32_t* members, void* scratch, size_t scratch_bytes,
                       void* stream)
{
    if (batch < 0 || n < 0 || (n % 16) != 0) return qsrtb_fail(QSRTB_EINVAL, "n must be a multiple of 16");
    if (tile_map && (tile_map_count < 0 || tile_map_count > n / 16))
        return qsrtb_fail(QSRTB_EINVAL, "tile map longer than the row of tiles");
    const int visited = tile_map ? tile_map_count : n / 16;
    const int64_t n_tiles = int64_t(batch) * visited;
    const int bad = check_common(bits, tailbite_context, variant, n_tiles);
    if (bad) return bad;
    if (n_tiles == 0) return QSRTB_OK;
    if (!w || !wq || !out_states || !lut_state || !lut_pm || !scratch)
        return qsrtb_fail(QSRTB_EINVAL, "null pointer");
    if (ld < n || (comp && comp_ld < n)) return qsrtb_fail(QSRTB_EINVAL, "row pitch smaller than n");
    if (!(multiplier >= 0.0f && multiplier <= 1.0f))
        return qsrtb_fail(QSRTB_EINVAL, "ldlq feedback multiplier must be in [0, 1]");
    if (members && (reinterpret_cast<uintptr_t>(members) & 7))
        return qsrtb_fail(QSRTB_EINVAL, "member table must be 8-byte aligned");
    TileIO io{};
    io.w = w;
    io.comp = comp;
    io.wq = wq;
    io.err = err;
    io.out_states = reinterpret_cast<uint16_t*>(out_states);
    io.w_stride = w_stride;
    io.comp_stride = comp_stride;
    io.state_stride = state_stride;
    io.ld = ld;
    io.comp_ld = comp_ld;
    io.tiles_n = visited;
    io.tile_map = tile_map;
    io.members = reinterpret_cast<const int2*>(members);
    io.multiplier = multiplier;
    io.rows_mode = 1;
    return dispatch(io, n_tiles, lut_state, lut_pm, bits, tailbite_context, variant, scratch,
                    scratch_bytes, static_cast<cudaStream_t>(stream));
}
}  // namespace

extern "C" int qsrtb_ldlq_quantize_rows(const float* w, const float* comp, float multiplier,
                                        int batch, int n, int ld, int comp_ld, int64_t w_stride,
                                        int64_t comp_stride, const uint8_t* lut_state,
                                        const uint8_t* lut_pm, int bits, int tailbite_context,
                                        int variant, float* wq, float* err, int16_t* out_states,
                                        int64_t state_stride, const int32_t* tile_map,
                                        int tile_map_count, void* scratch, size_t scratch_bytes,
                                        void* stream)
{
    return quantize_rows_impl(w, comp, multiplier, batch, n, ld, comp_ld, w_stride, comp_stride, lut_state,
                              lut_pm, bits, tailbite_context, variant, wq, err, out_states, state_stride,
                              tile_map, tile_map_count, nullptr, scratch, scratch_bytes, stream);
}

extern "C" int qsrtb_ldlq_quantize_members(const float* w, const float* comp, float multiplier,
                                           const int32_t* members, int member_count, int n, int ld,
                                           int comp_ld, int64_t w_stride, int64_t comp_stride,
                                           const uint8_t* lut_state, const uint8_t* lut_pm, int bits,
                                           int tailbite_context, int variant, float* wq, float* err,
                                           int16_t* out_states, int64_t state_stride,
                                           const int32_t* tile_map, int tile_map_count, void* scratch,
                                           size_t scratch_bytes, void* stream)
{
    if (!members) return qsrtb_fail(QSRTB_EINVAL, "member table required");
    return quantize_rows_impl(w, comp, multiplier, member_count, n, ld, comp_ld, w_stride, comp_stride,
                              lut_state, lut_pm, bits, tailbite_context, variant, wq, err, out_states,
                              state_stride, tile_map, tile_map_count, members, scratch, scratch_bytes, stream);
}

// ---- tile search without any allocation ---------------------------------------------------
//
// Some hosts of this library may not allocate device memory once they are running: a serving
// process whose memory pool has already claimed the whole GPU, or a plugin that is handed its
// buffers by an embedding application and has no allocation rights of its own.  They cannot
// provide the traceback scratch the regular entry point asks for.  For them the survivor rows
// live in the fixed array below, which is part of the loaded module on every GPU that uses the
// library (16 MiB per device, held until the process exits).
//
// The array gives a grid of at most 16 (K2, K3) or 32 (K4) persistent CTAs, so this entry
// point is meant for modest batches and refuses more than QSRTB_STATIC_MAX_TILES per call.
// All calls share the array.  The search writes every survivor row before it reads it, so
// nothing has to be cleared between calls; but two calls that overlap on the GPU (different
// streams, or different host threads) would overwrite each other's rows - serialise them.
#define QSRTB_STATIC_SCRATCH_BYTES (16u << 20)
#define QSRTB_STATIC_MAX_TILES 4096

static __device__ __align__(256) uint8_t g_static_scratch[QSRTB_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
uint8_t* g_static_scratch_ptr[kMaxDevices] = {};

// Device address of the array on the current device.  In host code `g_static_scratch` is only
// a handle for the runtime, not an address a kernel could use; the address is looked up once
// per device, with that device current, and cached.  Host threads that race on the cache all
// store the same value for a device, so no lock is taken.
int static_scratch_for_current_device(uint8_t** out)
{
    int device = -1;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "cudaGetDevice");
    if (device < 0 || device >= kMaxDevices) return qsrtb_fail(QSRTB_EINVAL, "device ordinal out of range");
    if (g_static_scratch_ptr[device] == nullptr) {
        void* address = nullptr;
        err = cudaGetSymbolAddress(&address, g_static_scratch);
        if (err != cudaSuccess) return qsrtb_fail_cuda(err, "cudaGetSymbolAddress(static scratch)");
        g_static_scratch_ptr[device] = static_cast<uint8_t*>(address);
    }
    *out = g_static_scratch_ptr[device];
    return QSRTB_OK;
}
}  // namespace

extern "C" int qsrtb_quantize_tiles_static(const float* tiles, int64_t n_tiles,
                                           const uint8_t* lut_state, const uint8_t* lut_pm,
                                           int bits, int tailbite_context, int variant,
                                           float* out_tiles, int16_t* out_states, void* stream)
{
    const int bad = check_common(bits, tailbite_context, variant, n_tiles);
    if (bad) return bad;
    if (n_tiles > QSRTB_STATIC_MAX_TILES)
        return qsrtb_fail(QSRTB_EINVAL,
                          "qsrtb_quantize_tiles_static handles at most 4096 tiles per call; "
                          "split the batch or use qsrtb_quantize_tiles with caller scratch");
    if (n_tiles == 0) return QSRTB_OK;
    if (!tiles || !lut_state || !lut_pm || !out_tiles || !out_states)
        return qsrtb_fail(QSRTB_EINVAL, "null pointer");
    uint8_t* scratch = nullptr;
    const int status = static_scratch_for_current_device(&scratch);
    if (status != QSRTB_OK) return status;
    TileIO io{};
    io.tiles = tiles;
    io.out_tiles = out_tiles;
    io.out_states = reinterpret_cast<uint16_t*>(out_states);
    io.rows_mode = 0;
    io.tiles_n = 1;
    return dispatch(io, n_tiles, lut_state, lut_pm, bits, tailbite_context, variant, scratch,
                    size_t(QSRTB_STATIC_SCRATCH_BYTES), static_cast<cudaStream_t>(stream));
}
