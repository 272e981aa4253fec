// Tail-biting Viterbi tile encoder with lazily resolved survivor decisions (sm_100a).
//
// Same search, same results as viterbi.cu (and therefore as the reference kernels
//   qsrt/csrc/qsrt_quantize_tiles_kernel.cuh:26-500 and qsrt_quantize_tiles_k2_kernel.cuh:47-366),
// organised so that the constrained pass - half of all trellis steps - carries no
// compare / select / position bookkeeping at all:
//   * the constrained pass only takes minima and streams the step's path costs (one half per
//     state) to a scratch slice in global memory;
//   * the traceback needs the decision of ONE out-edge per step.  It recomputes that decision
//     from the costs of the step before with exactly the arithmetic of the forward pass (same
//     fp16 subtract / fused multiply-add / clamp, lowest predecessor on ties), so a traceback
//     is a chain of 256 dependent links, each a handful of 2-byte reads;
//   * a chain is latency-bound, so it is not run on its own: warp 0 advances the chain of the
//     PREVIOUS tile by one link every second trellis step of the CURRENT tile (cp.async into
//     shared memory, consumed two steps later), which hides the memory latency completely.
//     Two scratch slots per CTA alternate between consecutive tiles;
//   * the primer pass (its recorded half is a quarter of all steps) keeps the survivor
//     decisions and the batched traceback of viterbi.cu, because its result - the boundary
//     state - is needed before the constrained pass of the same tile can start;
//   * the last tile of a CTA records decisions in both passes, so no chain is left to be
//     walked at the end of the launch with nothing to hide its latency behind.
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "qsrtb_internal.h"
#include "viterbi_core.cuh"

namespace {

using namespace qsrtb_vit;

constexpr int kChainCadence = 2;  // trellis steps between two links of a chain (even: see run_pass)
constexpr int kChainWarp = 0;      // the warp that walks the chain (any does equally well)

// The traceback in flight: the constrained pass of tile `tile`, whose cost rows are in `slot`.
// `head` is what a link needs and changes with every link; warp 0 reads and writes it with one
// 16-byte access.
struct ChainHead {
    int ri;      // row whose decision is resolved next, 255 down to 0; -1 when no link is pending
    int edge;    // trellis state after row ri
    int slot;
    int w_bits;  // the tile's rounded input at row ri (half bits)
};
struct Chain {
    ChainHead head;
    int state;      // 0 none, 1 walking, 2 walked (states complete, outputs not yet written)
    int pre_state;  // start (= end) state of the constrained pass
    long long tile;
    uint32_t cost_word[16];   // per predecessor: the 4-byte word holding its cost
};

struct LazySmem {
    __half in_h[2][256];
    uint16_t states[2][256];
    uint32_t red[32];
    __half warp_mins[2][32];
    __half shift[2];
    int edge;
    int pad;
    __align__(16) Chain chain;
};

constexpr int kNever = 0x7fffffff;

__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src)
{
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ __half e4m3_to_half(uint32_t b)
{
    const __half_raw raw = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
    return __half(raw);
}

// Issue the reads the link at (ri, e) needs: the cost of every predecessor k of out-edge e after
// row ri - 1 (row 0 has no predecessors' costs).  The branch labels come from the copy of the
// state table in shared memory.  Warp 0 only.
template <int K>
__device__ __forceinline__ void chain_issue(Chain* ch, int ri, int e, const uint8_t* cost_rows, int lane)
{
    using G = Geo<K>;
    if (lane < G::NK) {
        if (ri > 0) {
            const int pred = (e >> K) + lane * G::pred_stride;
            cp_async4(&ch->cost_word[lane], cost_rows + (size_t(ri - 1) * G::edges + (pred & ~1)) * 2);
        }
    }
    cp_async_commit();
}

// Resolve the pending link and issue the reads of the next.  The decision is recomputed exactly
// as acs_step computes the branch metrics of that row (same fp16 operations, same clamp), and
// the lowest predecessor among the minima wins, as in the forward tournament.  Everything the
// link needs sits at fixed shared-memory addresses, so its loads go out together.  Warp 0
// only, after the link's reads have landed.  Returns false when no link was pending.
template <int K, int MODE>
__device__ __forceinline__ bool chain_link(Chain* ch, LazySmem* sm, const uint8_t* slot_base,
                                           size_t slot_bytes, const uint8_t* labels, int lane)
{
    using G = Geo<K>;
    cp_async_wait_all();
    const int4 h = *reinterpret_cast<const int4*>(&ch->head);
    const uint32_t label = labels[((lane & (G::NK - 1)) << G::Kr) | h.y];
    const uint32_t cw = ch->cost_word[lane & 15];
    const int pre_state = ch->pre_state;
    const int ri = h.x, e = h.y, slot = h.z;
    if (ri < 0) return false;
    uint32_t key = 0xffffffffu;
    if (lane < G::NK) {
        const __half dh = __hsub(e4m3_to_half(label), __ushort_as_half(static_cast<unsigned short>(h.w)));
        const int pred = (e >> K) + lane * G::pred_stride;
        const __half inf = __ushort_as_half(0x7c00), top = __ushort_as_half(0x7bff);
        __half v;
        if (ri == 0) {
            v = __hmul(dh, dh);
            if constexpr (MODE != MODE_K2) v = __hmin(v, top);
            if (pred != pre_state) v = inf;
        } else {
            const uint32_t pbits = (pred & 1) ? (cw >> 16) : (cw & 0xffffu);
            v = __hfma(dh, dh, __ushort_as_half(static_cast<unsigned short>(pbits)));
            if constexpr (MODE == MODE_FAST) {
                if (ri < kSafeSteps) {  // these rows ran the clamped arithmetic
                    v = __hmin(v, top);
                    if (pbits == 0x7c00u) v = inf;
                }
            }
        }
        key = (half_key(__half_as_ushort(v)) << 5) | uint32_t(lane);
    }
    key = __reduce_min_sync(0xffffffffu, key);
    const int decision = int(key & 31u);
    const int prev = (decision << (16 - 2 * K)) | (e >> K);
    const int next = ri - 1;
    if (next >= 0) chain_issue<K>(ch, next, prev, slot_base + size_t(slot) * slot_bytes, lane);
    if (lane == 0) {
        sm->states[slot][ri] = uint16_t((prev << K) | e);
        const int w_bits = next >= 0 ? int(__half_as_ushort(sm->in_h[slot][next])) : 0;
        *reinterpret_cast<int4*>(&ch->head) = make_int4(next, prev, slot, w_bits);
        if (next < 0) ch->state = 2;
    }
    __syncwarp();
    return true;
}

// Walk what is left of the chain without anything to hide the latency behind (at most 256
// links; normally none are left).  Warp 0 only.
template <int K, int MODE>
__device__ __forceinline__ void chain_drain(Chain* ch, LazySmem* sm, const uint8_t* slot_base,
                                            size_t slot_bytes, const uint8_t* labels, int lane)
{
    for (int guard = 0; guard < 257; ++guard)
        if (!chain_link<K, MODE>(ch, sm, slot_base, slot_bytes, labels, lane)) break;
}

// Where thread t (< 256) finds its value of `tile` and where the results go (see TileIO).
struct TileSpot {
    int64_t src, dst, comp, state;
};

__device__ __forceinline__ TileSpot locate(const TileIO& io, int64_t tile, int t)
{
    TileSpot spot;
    if (!io.rows_mode) {
        spot.src = spot.dst = spot.state = tile * 256 + t;
        spot.comp = 0;
        return spot;
    }
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
    const int row = tensor_core_rc(t, col);
    const int64_t inside = int64_t(row) * io.ld + tn * 16 + col;
    spot.src = source * io.w_stride + inside;
    spot.dst = owner * io.w_stride + inside;
    spot.comp = owner * io.comp_stride + int64_t(row) * io.comp_ld + tn * 16 + col;
    spot.state = owner * io.state_stride + int64_t(tn) * 256 + t;
    return spot;
}

template <bool DEDICATED>
__device__ __forceinline__ void load_tile(const TileIO& io, int64_t tile, __half* in_h)
{
    if (threadIdx.x < 256) {
        const TileSpot spot = locate(io, tile, threadIdx.x);
        float w;
        if (io.rows_mode) {
            w = io.w[spot.src];
            if (io.comp != nullptr && io.multiplier != 0.0f) {
                const float c = io.comp[spot.comp];
                w = (io.multiplier == 1.0f) ? __fadd_rn(w, c) : __fadd_rn(w, __fmul_rn(io.multiplier, c));
            }
        } else {
            w = io.tiles[spot.src];
        }
        if constexpr (DEDICATED) w = fmaxf(-64.0f, fminf(w, 64.0f));  // k2 cuh:82-91
        in_h[threadIdx.x] = __float2half_rn(w);
    }
}

__device__ __forceinline__ void store_tile(const TileIO& io, int64_t tile, const uint16_t* states,
                                           const uint8_t* __restrict__ lut_state)
{
    if (threadIdx.x < 256) {
        const TileSpot spot = locate(io, tile, threadIdx.x);
        const uint16_t s = states[threadIdx.x];
        const float q = e4m3_to_float(lut_state[s]);
        io.out_states[spot.state] = s;
        if (io.rows_mode) {
            io.wq[spot.dst] = q;
            if (io.err != nullptr) io.err[spot.dst] = __fsub_rn(io.w[spot.src], q);
        } else {
            io.out_tiles[spot.dst] = q;
        }
    }
}

// Everything a tile's encode needs besides its labels.
struct LazyCtx {
    LazySmem* sm;
    __half* cost0;
    __half* cost1;
    uint8_t* slot_base;   // this CTA's two scratch slots
    size_t slot_bytes;
    const uint8_t* lut_state;
    const uint8_t* labels;  // the 65,536 state-indexed labels in shared memory (for the chain)
    const TileIO* io;
    int context;
    int tick;             // trellis steps executed by this CTA so far
    int chain_due;        // step at which warp 0 resolves the chain's next link (kNever: none)
};

// Finish the chain in flight, if any: walk its remaining links, then write its tile's results.
// Called by all threads at a point where they are converged.
template <int K, int CHAIN_MODE>
__device__ __forceinline__ void chain_finish(LazyCtx& cx)
{
    Chain* ch = &cx.sm->chain;
    __syncthreads();
    if (ch->state == 0) return;
    if ((threadIdx.x >> 5) == kChainWarp)
        chain_drain<K, CHAIN_MODE>(ch, cx.sm, cx.slot_base, cx.slot_bytes, cx.labels, threadIdx.x & 31);
    __syncthreads();
    store_tile(*cx.io, ch->tile, cx.sm->states[ch->head.slot], cx.lut_state);
    __syncthreads();
    if (threadIdx.x == 0) ch->state = 0;
    __syncthreads();
}

// Encode the tile whose rounded input is in sm->in_h[slot].
// Returns 0: invalid (MODE_FAST met the clamp; encode again with MODE_SAFE),
//         1: sm->states[slot] holds the result,
//         2: the result is being walked by the chain (lazy constrained pass).
template <int K, int MODE, int UNITS, int NL>
__device__ __forceinline__ int encode_tile_lazy(const uint32_t (&L)[UNITS][NL], LazyCtx& cx, int slot,
                                                bool lazy, int64_t tile)
{
    using G = Geo<K>;
    constexpr int THREADS = kUnits / UNITS;
    constexpr int WARPS = THREADS / 32;
    // Chains belong to tiles encoded lazily, i.e. with the fast or the dedicated K2 arithmetic;
    // a tile being re-encoded with MODE_SAFE still advances a MODE_FAST chain.
    constexpr int CHAIN_MODE = MODE == MODE_K2 ? MODE_K2 : MODE_FAST;
    LazySmem* sm = cx.sm;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int context = cx.context;
    __half* cur = cx.cost0;
    __half* inc = cx.cost1;
    uint8_t* slot_rows = cx.slot_base + size_t(slot) * cx.slot_bytes;  // decision rows and cost rows alias
    __half2 track_max = u2h2(0u);

    // lag-2 renormalisation of the dedicated K2 arithmetic (k2 cuh:117-137, 211-230)
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
#define ACS(M, FIRST, CONS, REC, TRACK)                                                                \
    UNIT_LOOP(acs_step<K, M, FIRST, CONS, REC, NL, COSTS>(L[uu], int(threadIdx.x) + uu * THREADS, inc, \
                                                          cur, w, pre_state, shift2, row, TRACK))

    auto run_pass = [&](int roll, int steps, int pre_state, int trace_start, auto constrained_tag,
                        auto costs_tag) {
        constexpr bool CONSTRAINED = decltype(constrained_tag)::value;
        constexpr bool COSTS = decltype(costs_tag)::value;
        constexpr int row_stride = COSTS ? G::edges * 2 : G::row_bytes;
        if constexpr (MODE == MODE_K2) {
            if (threadIdx.x == 0) {
                sm->shift[0] = __ushort_as_half(0);
                sm->shift[1] = __ushort_as_half(0);
            }
            __syncthreads();
        }
        // Every pass has an even number of steps, so the step counter is even after the second
        // step of each pair below: the chain, whose links fall due on even counts, is looked at
        // there only.
        auto step = [&](const int i, auto chain_tag) {
            const int ri = (i + roll) & 255;
            ++cx.tick;
            if constexpr (decltype(chain_tag)::value) {
                if (cx.tick == cx.chain_due) {  // kNever in every warp but the chain's
                    const bool more = chain_link<K, CHAIN_MODE>(&sm->chain, sm, cx.slot_base, cx.slot_bytes,
                                                                cx.labels, lane);
                    cx.chain_due = more ? cx.tick + kChainCadence : kNever;
                }
            }
            __half* t = cur; cur = inc; inc = t;
            const __half w = sm->in_h[slot][ri];
            uint8_t* row = slot_rows + size_t(ri) * row_stride;
            __half2 shift2 = u2h2(0u);
            __half2 step_min2 = u2h2(kInf2);
            if constexpr (MODE == MODE_K2) {
                if (i > 0) k2_fold(i);
                shift2 = __half2half2(sm->shift[i & 1]);
            }
            if (i == 0) {
                if constexpr (MODE == MODE_K2)
                    ACS(MODE, true, CONSTRAINED, CONSTRAINED, step_min2);
                else if constexpr (MODE == MODE_FAST && CONSTRAINED)
                    ACS(MODE_SAFE, true, true, true, track_max);
                else
                    ACS(MODE, true, CONSTRAINED, CONSTRAINED, track_max);
            } else if (i < trace_start) {
                if constexpr (MODE == MODE_K2)
                    ACS(MODE, false, false, false, step_min2);
                else
                    ACS(MODE, false, false, false, track_max);
            } else {
                if constexpr (MODE == MODE_K2) {
                    ACS(MODE, false, false, true, step_min2);
                } else if constexpr (MODE == MODE_FAST && CONSTRAINED) {
                    if (i < kSafeSteps)  // unreachable states exist for the first few constrained steps
                        ACS(MODE_SAFE, false, false, true, track_max);
                    else
                        ACS(MODE, false, false, true, track_max);
                } else {
                    ACS(MODE, false, false, true, track_max);
                }
            }
            if constexpr (MODE == MODE_K2) k2_publish(i, step_min2);
            __syncthreads();
        };
        for (int i = 0; i < steps; i += 2) {
            step(i, std::false_type{});
            step(i + 1, std::true_type{});
        }
    };
    auto clamp_met = [&]() {
        const bool over = !(__hlt(__low2half(track_max), u2h2(kMax2).x) &&
                            __hlt(__high2half(track_max), u2h2(kMax2).x));
        return __syncthreads_or(over) != 0;
    };

    // Primer: 2*C symbols centred on symbol 0, decisions kept for the last C of them.
    run_pass(256 - context, 2 * context, -1, context, std::false_type{}, std::false_type{});
    if constexpr (MODE == MODE_FAST) {
        if (clamp_met()) return 0;
    }
    int boundary;
    if constexpr (MODE == MODE_K2)
        boundary = boundary_argmin<K, false, UNITS>(cur, sm->red);  // final primer step (k2 cuh:282)
    else
        boundary = boundary_argmin<K, K != 2, UNITS>(inc, sm->red);  // step before the last (cuh:375,401)
    const int end_state = traceback<K, UNITS>(slot_rows, reinterpret_cast<uint8_t*>(cx.cost0), context - 1,
                                              boundary, false, sm->states[slot], &sm->edge);

    // Constrained pass: starts from and must return to end_state.
    if (lazy) {
        run_pass(0, 256, end_state, 0, std::true_type{}, std::true_type{});
        if constexpr (MODE == MODE_FAST) {
            if (clamp_met()) return 0;
        }
        chain_finish<K, CHAIN_MODE>(cx);  // the previous tile's chain had this tile's 512 steps
        Chain* ch = &sm->chain;
        if (warp == kChainWarp) {
            if (lane == 0) {
                ch->state = 1;
                ch->pre_state = end_state;
                ch->tile = tile;
                *reinterpret_cast<int4*>(&ch->head) =
                    make_int4(255, end_state, slot, int(__half_as_ushort(sm->in_h[slot][255])));
            }
            __syncwarp();
            chain_issue<K>(ch, 255, end_state, slot_rows, lane);
        }
        cx.chain_due = warp == kChainWarp ? cx.tick + kChainCadence : kNever;
        __syncthreads();
        return 2;
    }
    run_pass(0, 256, end_state, 0, std::true_type{}, std::false_type{});
    if constexpr (MODE == MODE_FAST) {
        if (clamp_met()) return 0;
    }
    traceback<K, UNITS>(slot_rows, reinterpret_cast<uint8_t*>(cx.cost0), 255, end_state, true,
                        sm->states[slot], &sm->edge);
    return 1;
#undef ACS
#undef UNIT_LOOP
}

template <int K>
constexpr size_t lazy_slot_bytes() { return size_t(256) * Geo<K>::edges * 2; }

template <int K, bool DEDICATED, int UNITS>
__global__ void __launch_bounds__(kUnits / UNITS, 1)
viterbi_lazy_kernel(const TileIO io, const uint8_t* __restrict__ lut_pm,
                    const uint8_t* __restrict__ lut_state, uint8_t* scratch_base, int64_t n_tiles,
                    int context)
{
    using G = Geo<K>;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    LazyCtx cx;
    cx.cost0 = reinterpret_cast<__half*>(smem_raw);
    cx.cost1 = cx.cost0 + G::edges;
    cx.sm = reinterpret_cast<LazySmem*>(smem_raw + 2 * G::edges * sizeof(__half));
    uint8_t* labels = smem_raw + 2 * G::edges * sizeof(__half) + sizeof(LazySmem);
    for (int i = threadIdx.x; i < 65536 / 16; i += blockDim.x)
        reinterpret_cast<uint4*>(labels)[i] = reinterpret_cast<const uint4*>(lut_state)[i];
    cx.labels = labels;
    cx.slot_bytes = lazy_slot_bytes<K>();
    cx.slot_base = scratch_base + size_t(blockIdx.x) * 2 * cx.slot_bytes;
    cx.lut_state = lut_state;
    cx.io = &io;
    cx.context = context;
    cx.tick = 0;
    cx.chain_due = kNever;
    if (threadIdx.x == 0) {
        cx.sm->chain.state = 0;
        cx.sm->chain.head.ri = -1;
    }

    constexpr int THREADS = kUnits / UNITS;
    constexpr int NL = UNITS >= 2 ? 32 : 16;
    constexpr int CHAIN_MODE = DEDICATED ? MODE_K2 : MODE_FAST;
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
    __syncthreads();

    int slot = 0;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, slot ^= 1) {
        const bool last = tile + gridDim.x >= n_tiles;
        // the slot's rows, input and states may still belong to a chain (after a tile that
        // started none): finish it before they are overwritten
        if (cx.sm->chain.state != 0 && cx.sm->chain.head.slot == slot) chain_finish<K, CHAIN_MODE>(cx);
        load_tile<DEDICATED>(io, tile, cx.sm->in_h[slot]);
        __syncthreads();
        int result;
        if constexpr (DEDICATED) {
            result = encode_tile_lazy<K, MODE_K2, UNITS, NL>(L, cx, slot, !last, tile);
        } else {
            result = encode_tile_lazy<K, MODE_FAST, UNITS, NL>(L, cx, slot, !last, tile);
            if (result == 0) result = encode_tile_lazy<K, MODE_SAFE, UNITS, NL>(L, cx, slot, false, tile);
        }
        if (result == 1) store_tile(io, tile, cx.sm->states[slot], lut_state);
        __syncthreads();
    }
    chain_finish<K, CHAIN_MODE>(cx);
}

template <int K>
constexpr size_t lazy_smem_bytes()
{
    return 2 * Geo<K>::edges * sizeof(__half) + sizeof(LazySmem) + 65536;  // costs, bookkeeping, labels
}

template <int K, bool DEDICATED, int UNITS>
int launch_lazy(const TileIO& io, int64_t n_tiles, const uint8_t* lut_state, const uint8_t* lut_pm,
                int context, void* scratch, int grid, cudaStream_t stream)
{
    auto kernel = viterbi_lazy_kernel<K, DEDICATED, UNITS>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           int(lazy_smem_bytes<K>()));
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "cudaFuncSetAttribute(viterbi_lazy)");
    kernel<<<dim3(unsigned(grid)), dim3(kUnits / UNITS), lazy_smem_bytes<K>(), stream>>>(
        io, lut_pm, lut_state, static_cast<uint8_t*>(scratch), n_tiles, context);
    err = cudaGetLastError();
    if (err != cudaSuccess) return qsrtb_fail_cuda(err, "viterbi_lazy kernel launch");
    return QSRTB_OK;
}

}  // namespace

size_t qsrtb_lazy_scratch_per_cta(int bits)
{
    return 2 * (size_t(256) << (16 - bits)) * 2;  // two slots of 256 rows of 2^(16-bits) halves
}

int qsrtb_lazy_launch(const qsrtb_vit::TileIO& io, int64_t n_tiles, const uint8_t* lut_state,
                      const uint8_t* lut_pm, int bits, int context, int dedicated, int units,
                      void* scratch, int grid, cudaStream_t stream)
{
    if (bits == 3) {
        if (units == 1)
            return launch_lazy<3, false, 1>(io, n_tiles, lut_state, lut_pm, context, scratch, grid, stream);
        return launch_lazy<3, false, 2>(io, n_tiles, lut_state, lut_pm, context, scratch, grid, stream);
    }
    if (bits == 4) {
        if (units == 1)
            return launch_lazy<4, false, 1>(io, n_tiles, lut_state, lut_pm, context, scratch, grid, stream);
        return launch_lazy<4, false, 2>(io, n_tiles, lut_state, lut_pm, context, scratch, grid, stream);
    }
    if (dedicated) {
        if (units == 1)
            return launch_lazy<2, true, 1>(io, n_tiles, lut_state, lut_pm, context, scratch, grid, stream);
        return launch_lazy<2, true, 2>(io, n_tiles, lut_state, lut_pm, context, scratch, grid, stream);
    }
    if (units == 1)
        return launch_lazy<2, false, 1>(io, n_tiles, lut_state, lut_pm, context, scratch, grid, stream);
    return launch_lazy<2, false, 2>(io, n_tiles, lut_state, lut_pm, context, scratch, grid, stream);
}
