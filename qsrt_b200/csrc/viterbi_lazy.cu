// Tail-biting Viterbi tile encoder with lazily resolved survivor decisions (sm_100a).
//
// Same search, same results as viterbi.cu (and therefore as the reference kernels
//   qsrt/csrc/qsrt_quantize_tiles_kernel.cuh:26-500 and qsrt_quantize_tiles_k2_kernel.cuh:47-366),
// organised so that the trellis steps carry no compare / select / position bookkeeping:
//   * a pass only takes minima and streams the step's path costs (one half per state) to a
//     scratch row in global memory;
//   * a traceback needs the decision of ONE out-edge per step.  It recomputes that decision
//     from the costs of the step before with exactly the arithmetic of the forward pass (same
//     fp16 subtract / fused multiply-add / clamp, lowest predecessor on ties), so a traceback
//     is a chain of dependent links, each a handful of 2-byte reads;
//   * a chain is latency-bound (about a microsecond per link from HBM), so it never runs on its
//     own: one warp advances it by a link every second trellis step of whatever pass the CTA is
//     running (cp.async of the predecessors' cost words into shared memory, consumed two steps
//     later).  One warp walks the constrained pass's chain (256 links, writes the states), the
//     next one the primer's (C links, yields the boundary state);
//   * a primer's boundary state is needed before the same tile's constrained pass can start, so
//     a CTA interleaves its tiles: P(0) P(1) C(0) P(2) C(1) P(3) C(2) ...  The primer chain of
//     tile x+1 is walked during C(x), the constrained chain of tile x during P(x+2) and C(x+1);
//   * the dedicated K2 arithmetic, whose cost rows are 32 KiB, stores every second row only; a
//     link that needs a missing row recomputes the four costs it wants from the row before;
//   * the constrained passes of a CTA's last two tiles keep survivor decisions and the batched
//     traceback of viterbi.cu (nothing follows them to hide a chain behind), as does every pass
//     of a tile that met the fp16 clamp and is re-encoded with the literal arithmetic.
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
constexpr int kNever = 0x7fffffff;
constexpr int kInFlight = 3;      // tiles of a CTA whose input and states are live at a time
constexpr int kPrimerRows = 130;  // cost rows of a primer buffer (C + 1 used, C <= 128)

enum ChainKind { CHAIN_CONSTRAINED = 0, CHAIN_PRIMER = 1 };
// The warp that walks a chain.  With the dedicated K2 arithmetic warp 0 already folds the block
// minimum every step, and the chains go to warps 2 and 3 (K2: 237 k against 228 k tiles/s); the
// other arithmetics measured better with warps 0 and 1 (K3: 348 k against 337 k).
template <int MODE>
constexpr int chain_warp(int kind) { return (MODE == MODE_K2 ? 2 : 0) + kind; }

// A traceback in flight.  `head` is what a link needs and changes with every link; the walking
// warp reads and writes it with one 16-byte access.
struct ChainHead {
    int ri;      // symbol whose decision is resolved next, counting down; -1 when none is pending
    int edge;    // trellis state after that symbol
    int slot;    // which of the in-flight tiles (input, states)
    int w_bits;  // the tile's rounded input at symbol ri (half bits)
};
struct Chain {
    ChainHead head;
    const uint8_t* rows;  // the pass's cost rows; the link at ri reads row ri + row_bias
    int row_bias;         // -1 constrained (costs after symbol ri - 1), 0 primer (rows start one step early)
    int state;            // 0 none, 1 walking, 2 walked
    int pre_state;        // constrained: start (= end) state of the pass
    int result;           // the state before symbol 0, once walked (the primer's boundary state)
    long long tile;
    uint32_t cost_word[16];  // per predecessor: the 4-byte word holding its cost
};

struct TileSlot {
    int end_state;  // boundary state from the primer
    int done;       // the tile was finished out of turn (re-encoded after meeting the clamp)
};

struct LazySmem {
    __half in_h[kInFlight][256];
    uint16_t states[kInFlight][256];
    uint32_t red[32];
    __half warp_mins[2][32];
    __half shift[2];
    int edge;
    int pad;
    TileSlot slot[kInFlight];
    __half shift_hist[2][kInFlight][256];  // dedicated K2: the shift each recorded step subtracted
    __align__(16) Chain chain[2];  // [CHAIN_CONSTRAINED], [CHAIN_PRIMER]: each walked by its own warp
};

// The dedicated K2 arithmetic keeps every second cost row only (a K2 row is 32 KiB, and storing
// all of them costs more than the bookkeeping they replace): a link that needs a missing row
// recomputes the four costs it wants from the row before.
template <int MODE>
constexpr bool half_rows() { return MODE == MODE_K2; }

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

// Issue the reads a link at out-edge e needs: the cost of every predecessor k of e in cost row
// `row` (none for a constrained pass's symbol 0, row -1).  The branch labels come from the copy
// of the state table in shared memory.  The chain's warp only.
template <int K>
__device__ __forceinline__ void chain_issue(Chain* ch, int row, int e, int lane)
{
    using G = Geo<K>;
    if (lane < G::NK && row >= 0) {
        const int pred = (e >> K) + lane * G::pred_stride;
        cp_async4(&ch->cost_word[lane], ch->rows + (size_t(row) * G::edges + (pred & ~1)) * 2);
    }
    cp_async_commit();
}

// Resolve the pending link and issue the reads of the next.  The decision is recomputed exactly
// as acs_step computes the branch metrics of that step (same fp16 operations, same clamp), and
// the lowest predecessor among the minima wins, as in the forward tournament.  Everything the
// link needs sits at fixed shared-memory addresses, so its loads go out together.  The chain's
// warp only, after the link's reads have landed.  Returns false when no link was pending.
template <int K, int MODE, int KIND>
__device__ __forceinline__ bool chain_link(Chain* ch, LazySmem* sm, const uint8_t* labels, int lane)
{
    using G = Geo<K>;
    cp_async_wait_all();
    const int4 h = *reinterpret_cast<const int4*>(&ch->head);
    const uint32_t label = labels[((lane & (G::NK - 1)) << G::Kr) | (h.y & (G::edges - 1))];
    const uint32_t cw = ch->cost_word[lane & 15];
    const int pre_state = ch->pre_state;
    const int row_bias = ch->row_bias;
    const int ri = h.x, e = h.y, slot = h.z;
    if (ri < 0) return false;
    uint32_t key = 0xffffffffu;
    if (lane < G::NK) {
        const __half dh = __hsub(e4m3_to_half(label), __ushort_as_half(static_cast<unsigned short>(h.w)));
        const int pred = (e >> K) + lane * G::pred_stride;
        const __half inf = __ushort_as_half(0x7c00), top = __ushort_as_half(0x7bff);
        __half v;
        if (KIND == CHAIN_CONSTRAINED && ri == 0) {
            v = __hmul(dh, dh);
            if constexpr (MODE != MODE_K2) v = __hmin(v, top);
            if (pred != pre_state) v = inf;
        } else {
            const uint32_t pbits = (pred & 1) ? (cw >> 16) : (cw & 0xffffu);
            v = __hfma(dh, dh, __ushort_as_half(static_cast<unsigned short>(pbits)));
            if constexpr (MODE == MODE_FAST && KIND == CHAIN_CONSTRAINED) {
                if (ri < kSafeSteps) {  // these steps ran the clamped arithmetic
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
    if (next >= 0) chain_issue<K>(ch, next + row_bias, prev, lane);
    if (lane == 0) {
        if constexpr (KIND == CHAIN_CONSTRAINED) sm->states[slot][ri] = uint16_t((prev << K) | e);
        const int w_bits = next >= 0 ? int(__half_as_ushort(sm->in_h[slot][next])) : 0;
        *reinterpret_cast<int4*>(&ch->head) = make_int4(next, prev, slot, w_bits);
        if (next < 0) {
            ch->result = prev;
            ch->state = 2;
        }
    }
    __syncwarp();
    return true;
}

// ---- dedicated K2: every second cost row ------------------------------------------------------
// Cost row q of a pass lives at rows + (q >> 1) rows, for even q only.  Lane 4k + j of the chain's
// warp serves predecessor k of the link's out-edge and, where row q is missing, predecessor j of
// that predecessor.
__device__ __forceinline__ void chain_issue_half(Chain* ch, int q, int e, int lane)
{
    using G = Geo<2>;
    const int k = (lane >> 2) & 3, j = lane & 3;
    const int s_k = (e >> 2) + k * G::pred_stride;
    if (lane < 16 && q >= 0) {
        if (q & 1) {
            const int pp = (s_k >> 2) + j * G::pred_stride;
            cp_async4(&ch->cost_word[lane], ch->rows + (size_t(q >> 1) * G::edges + (pp & ~1)) * 2);
        } else if (j == 0) {
            cp_async4(&ch->cost_word[lane], ch->rows + (size_t(q >> 1) * G::edges + (s_k & ~1)) * 2);
        }
    }
    cp_async_commit();
}

template <int KIND>
__device__ __forceinline__ bool chain_link_half(Chain* ch, LazySmem* sm, const uint8_t* labels, int lane)
{
    using G = Geo<2>;
    cp_async_wait_all();
    const int4 h = *reinterpret_cast<const int4*>(&ch->head);
    const int k = (lane >> 2) & 3, j = lane & 3;
    const int ri = h.x, e = h.y & (G::edges - 1), slot = h.z;
    const int s_k = (e >> 2) + k * G::pred_stride;
    const uint32_t outer_label = labels[(k << G::Kr) | e];
    const uint32_t inner_label = labels[(j << G::Kr) | s_k];
    const uint32_t cw = ch->cost_word[lane & 15];
    const int pre_state = ch->pre_state;
    const int row_bias = ch->row_bias;
    if (ri < 0) return false;
    const int q = ri + row_bias;  // the cost row this link needs
    __half p = __ushort_as_half(0);
    if (q >= 0) {
        if (q & 1) {
            // costs after step q of the four predecessors, from the row before: the forward
            // pass's own metric, minimum and shift (acs_step, MODE_K2)
            const int symbol = KIND == CHAIN_CONSTRAINED ? q : q - 1;
            const __half dh = __hsub(e4m3_to_half(inner_label), sm->in_h[slot][symbol & 255]);
            const int pp = (s_k >> 2) + j * G::pred_stride;
            const uint32_t bits = (pp & 1) ? (cw >> 16) : (cw & 0xffffu);
            __half m = __hfma(dh, dh, __ushort_as_half(static_cast<unsigned short>(bits)));
            m = __hmin(m, __shfl_xor_sync(0xffffffffu, m, 1));
            m = __hmin(m, __shfl_xor_sync(0xffffffffu, m, 2));
            p = __hsub(m, sm->shift_hist[KIND][slot][q & 255]);
        } else {
            const uint32_t bits = (s_k & 1) ? (cw >> 16) : (cw & 0xffffu);
            p = __ushort_as_half(static_cast<unsigned short>(bits));
        }
    }
    uint32_t key = 0xffffffffu;
    if (lane < 16 && j == 0) {
        const __half dh = __hsub(e4m3_to_half(outer_label), __ushort_as_half(static_cast<unsigned short>(h.w)));
        __half v;
        if (KIND == CHAIN_CONSTRAINED && ri == 0) {
            v = __hmul(dh, dh);
            if (s_k != pre_state) v = __ushort_as_half(0x7c00);
        } else {
            v = __hfma(dh, dh, p);
        }
        key = (half_key(__half_as_ushort(v)) << 5) | uint32_t(k);
    }
    key = __reduce_min_sync(0xffffffffu, key);
    const int decision = int(key & 31u);
    const int prev = (decision << (16 - 2 * 2)) | (e >> 2);
    const int next = ri - 1;
    if (next >= 0) chain_issue_half(ch, next + row_bias, prev, lane);
    if (lane == 0) {
        if constexpr (KIND == CHAIN_CONSTRAINED) sm->states[slot][ri] = uint16_t((prev << 2) | e);
        const int w_bits = next >= 0 ? int(__half_as_ushort(sm->in_h[slot][next])) : 0;
        *reinterpret_cast<int4*>(&ch->head) = make_int4(next, prev, slot, w_bits);
        if (next < 0) {
            ch->result = prev;
            ch->state = 2;
        }
    }
    __syncwarp();
    return true;
}

// One link of a chain, whichever row layout its pass has.
template <int K, int MODE, int KIND>
__device__ __forceinline__ bool chain_step(Chain* ch, LazySmem* sm, const uint8_t* labels, int lane)
{
    if constexpr (half_rows<MODE>())
        return chain_link_half<KIND>(ch, sm, labels, lane);
    else
        return chain_link<K, MODE, KIND>(ch, sm, labels, lane);
}

// Walk what is left of a chain without anything to hide the latency behind (normally nothing
// is left).  The chain's warp only.
template <int K, int MODE, int KIND>
__device__ __forceinline__ void chain_drain(Chain* ch, LazySmem* sm, const uint8_t* labels, int lane)
{
    for (int guard = 0; guard < 257; ++guard)
        if (!chain_step<K, MODE, KIND>(ch, sm, labels, lane)) break;
}

// Start a chain at (ri, edge) of the tile in `slot`.  All lanes of the chain's warp.
template <int K, int MODE>
__device__ __forceinline__ void chain_start(Chain* ch, LazySmem* sm, const uint8_t* rows, int row_bias,
                                            int ri, int edge, int slot, int pre_state, long long tile,
                                            int lane)
{
    if (lane == 0) {
        ch->rows = rows;
        ch->row_bias = row_bias;
        ch->state = 1;
        ch->pre_state = pre_state;
        ch->result = -1;
        ch->tile = tile;
        *reinterpret_cast<int4*>(&ch->head) =
            make_int4(ri, edge, slot, int(__half_as_ushort(sm->in_h[slot][ri])));
    }
    __syncwarp();
    if constexpr (half_rows<MODE>())
        chain_issue_half(ch, ri + row_bias, edge, lane);
    else
        chain_issue<K>(ch, ri + row_bias, edge, lane);
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

// Everything the passes of a CTA need besides the labels.
struct LazyCtx {
    LazySmem* sm;
    __half* cost0;
    __half* cost1;
    uint8_t* scratch;       // this CTA's cost rows: two constrained buffers, then two primer buffers
    const uint8_t* lut_state;
    const uint8_t* labels;  // the 65,536 state-indexed labels in shared memory (for the chains)
    const TileIO* io;
    int context;
    int tick;               // trellis steps executed by this CTA so far
    int chain_due;          // step at which this warp resolves its chain's next link (kNever: none)
};

// Finish the constrained chain in flight, if any: walk its remaining links, then write its
// tile's results.  Called by all threads at a point where they are converged.
template <int K, int CHAIN_MODE>
__device__ __forceinline__ void finish_constrained_chain(LazyCtx& cx)
{
    Chain* ch = &cx.sm->chain[CHAIN_CONSTRAINED];
    __syncthreads();
    if (ch->state == 0) return;
    if ((threadIdx.x >> 5) == chain_warp<CHAIN_MODE>(CHAIN_CONSTRAINED))
        chain_drain<K, CHAIN_MODE, CHAIN_CONSTRAINED>(ch, cx.sm, cx.labels, threadIdx.x & 31);
    __syncthreads();
    store_tile(*cx.io, ch->tile, cx.sm->states[ch->head.slot], cx.lut_state);
    __syncthreads();
    if (threadIdx.x == 0) ch->state = 0;
    __syncthreads();
}

// Finish the primer chain in flight, if any, and file its boundary state with its tile.
template <int K, int CHAIN_MODE>
__device__ __forceinline__ void finish_primer_chain(LazyCtx& cx)
{
    Chain* ch = &cx.sm->chain[CHAIN_PRIMER];
    __syncthreads();
    if (ch->state == 0) return;
    if ((threadIdx.x >> 5) == chain_warp<CHAIN_MODE>(CHAIN_PRIMER))
        chain_drain<K, CHAIN_MODE, CHAIN_PRIMER>(ch, cx.sm, cx.labels, threadIdx.x & 31);
    __syncthreads();
    if (threadIdx.x == 0) {
        cx.sm->slot[ch->head.slot].end_state = ch->result;
        ch->state = 0;
    }
    __syncthreads();
}

// One pass over `steps` symbols of the tile in `slot`, starting at symbol `roll`.
//   CONSTRAINED : the pass starts from (and must return to) pre_state;
//   COSTS       : recorded steps store their path costs instead of survivor decisions;
//   recorded steps are those from `record_from` on; their row is `row_of(i, ri)`.
// Returns (block-uniform) whether MODE_FAST met the clamp.
template <int K, int MODE, int UNITS, int NL, bool CONSTRAINED, bool COSTS>
__device__ __forceinline__ bool run_pass(const uint32_t (&L)[UNITS][NL], LazyCtx& cx, int slot, int roll,
                                         int steps, int pre_state, int record_from, uint8_t* rows,
                                         int first_row_step, __half*& cur, __half*& inc)
{
    using G = Geo<K>;
    constexpr int THREADS = kUnits / UNITS;
    constexpr int WARPS = THREADS / 32;
    // Chains belong to passes run with the fast or the dedicated K2 arithmetic; a tile being
    // re-encoded with MODE_SAFE still advances MODE_FAST chains.
    constexpr int CHAIN_MODE = MODE == MODE_K2 ? MODE_K2 : MODE_FAST;
    constexpr int row_stride = COSTS ? G::edges * 2 : G::row_bytes;
    LazySmem* sm = cx.sm;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __half2 track_max = u2h2(0u);

    // lag-2 renormalisation of the dedicated K2 arithmetic (k2 cuh:117-137, 211-230)
    auto k2_fold = [&](int s) {
        if (warp == 0) {
            const __half m = warp_min_half(lane < WARPS ? sm->warp_mins[(s - 1) & 1][lane] : __ushort_as_half(0x7c00));
            if (lane == 0)
                sm->shift[(s + 1) & 1] = __hge(m, __float2half_rn(1024.0f)) ? m : __ushort_as_half(0);
        }
    };
    auto k2_publish = [&](int s, __half2 step_min2) {
        const __half m = warp_min_half(__hmin(__low2half(step_min2), __high2half(step_min2)));
        if (lane == 0) sm->warp_mins[s & 1][warp] = m;
    };

#define UNIT_LOOP(...)                                                        \
    do {                                                                      \
        _Pragma("unroll") for (int uu = 0; uu < UNITS; ++uu) { __VA_ARGS__; } \
    } while (0)
#define ACS(M, FIRST, CONS, REC, TRACK)                                                                \
    UNIT_LOOP(acs_step<K, M, FIRST, CONS, REC, NL, COSTS>(L[uu], int(threadIdx.x) + uu * THREADS, inc, \
                                                          cur, w, pre_state, shift2, row, TRACK))

    if constexpr (MODE == MODE_K2) {
        if (threadIdx.x == 0) {
            sm->shift[0] = __ushort_as_half(0);
            sm->shift[1] = __ushort_as_half(0);
        }
        __syncthreads();
    }
    // Every pass has an even number of steps, so the step counter is even after the second step
    // of each pair below: the chains, whose links fall due on even counts, are looked at there.
    auto step = [&](const int i, auto chain_tag) {
        const int ri = (i + roll) & 255;
        ++cx.tick;
        if constexpr (decltype(chain_tag)::value) {
            if (cx.tick == cx.chain_due) {  // kNever in every warp but the two that walk chains
                bool more;
                if (warp == chain_warp<CHAIN_MODE>(CHAIN_CONSTRAINED))
                    more = chain_step<K, CHAIN_MODE, CHAIN_CONSTRAINED>(&sm->chain[CHAIN_CONSTRAINED], sm,
                                                                        cx.labels, lane);
                else
                    more = chain_step<K, CHAIN_MODE, CHAIN_PRIMER>(&sm->chain[CHAIN_PRIMER], sm, cx.labels,
                                                                   lane);
                cx.chain_due = more ? cx.tick + kChainCadence : kNever;
            }
        }
        __half* t = cur; cur = inc; inc = t;
        const __half w = sm->in_h[slot][ri];
        // a recorded step's row: by symbol for decisions and constrained costs, by step for a
        // primer's costs (which start one step before the first recorded decision)
        const int row_index = COSTS && !CONSTRAINED ? i - first_row_step : ri;
        constexpr bool HALF = COSTS && half_rows<MODE>();
        uint8_t* row = rows + size_t(HALF ? row_index >> 1 : row_index) * row_stride;
        __half2 shift2 = u2h2(0u);
        __half2 step_min2 = u2h2(kInf2);
        if constexpr (MODE == MODE_K2) {
            if (i > 0) k2_fold(i);
            shift2 = __half2half2(sm->shift[i & 1]);
            if constexpr (HALF) {
                if (threadIdx.x == 0 && row_index >= 0)
                    sm->shift_hist[CONSTRAINED ? CHAIN_CONSTRAINED : CHAIN_PRIMER][slot][row_index & 255] =
                        sm->shift[i & 1];
            }
        }
        if (i == 0) {
            if constexpr (MODE == MODE_K2)
                ACS(MODE, true, CONSTRAINED, CONSTRAINED, step_min2);
            else if constexpr (MODE == MODE_FAST && CONSTRAINED)
                ACS(MODE_SAFE, true, true, true, track_max);
            else
                ACS(MODE, true, CONSTRAINED, CONSTRAINED, track_max);
        } else if (i < record_from) {
            if constexpr (MODE == MODE_K2)
                ACS(MODE, false, false, false, step_min2);
            else
                ACS(MODE, false, false, false, track_max);
        } else {
            if constexpr (MODE == MODE_K2) {
                if (HALF && (row_index & 1))  // the row between two stored ones
                    ACS(MODE, false, false, false, step_min2);
                else
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
#undef ACS
#undef UNIT_LOOP
    if constexpr (MODE == MODE_FAST) {
        const bool over = !(__hlt(__low2half(track_max), u2h2(kMax2).x) &&
                            __hlt(__high2half(track_max), u2h2(kMax2).x));
        return __syncthreads_or(over) != 0;
    }
    return false;
}

// Encode the tile in `slot` from scratch with survivor decisions in both passes and the batched
// traceback (the organisation of viterbi.cu); `rows` is a scratch area no chain is reading.
// Leaves the states in sm->states[slot].  Returns false if MODE_FAST met the clamp.
template <int K, int MODE, int UNITS, int NL>
__device__ __forceinline__ bool encode_with_decisions(const uint32_t (&L)[UNITS][NL], LazyCtx& cx, int slot,
                                                      uint8_t* rows)
{
    LazySmem* sm = cx.sm;
    const int context = cx.context;
    __half* cur = cx.cost0;
    __half* inc = cx.cost1;
    if (run_pass<K, MODE, UNITS, NL, false, false>(L, cx, slot, 256 - context, 2 * context, -1, context, rows,
                                                   0, cur, inc))
        return false;
    int boundary;
    if constexpr (MODE == MODE_K2)
        boundary = boundary_argmin<K, false, UNITS>(cur, sm->red);
    else
        boundary = boundary_argmin<K, K != 2, UNITS>(inc, sm->red);
    const int end_state = traceback<K, UNITS>(rows, reinterpret_cast<uint8_t*>(cx.cost0), context - 1,
                                              boundary, false, sm->states[slot], &sm->edge);
    if (run_pass<K, MODE, UNITS, NL, true, false>(L, cx, slot, 0, 256, end_state, 0, rows, 0, cur, inc))
        return false;
    traceback<K, UNITS>(rows, reinterpret_cast<uint8_t*>(cx.cost0), 255, end_state, true, sm->states[slot],
                        &sm->edge);
    return true;
}

// Cost rows per CTA: two constrained and two primer buffers (half of the rows with the dedicated
// K2 arithmetic, which stores every second one).
template <bool DEDICATED>
constexpr int constrained_buffer_rows() { return DEDICATED ? 128 : 256; }
template <bool DEDICATED>
constexpr int primer_buffer_rows() { return DEDICATED ? kPrimerRows / 2 : kPrimerRows; }
template <int K, bool DEDICATED>
constexpr size_t lazy_cta_bytes()
{
    return size_t(2 * constrained_buffer_rows<DEDICATED>() + 2 * primer_buffer_rows<DEDICATED>()) *
           Geo<K>::edges * 2;
}

template <int K, bool DEDICATED, int UNITS>
__global__ void __launch_bounds__(kUnits / UNITS, 1)
viterbi_lazy_kernel(const TileIO io, const uint8_t* __restrict__ lut_pm,
                    const uint8_t* __restrict__ lut_state, uint8_t* scratch_base, int64_t n_tiles,
                    int context)
{
    using G = Geo<K>;
    constexpr int THREADS = kUnits / UNITS;
    constexpr int NL = UNITS >= 2 ? 32 : 16;
    constexpr int MODE = DEDICATED ? MODE_K2 : MODE_FAST;  // arithmetic of every pass but re-encodes
    extern __shared__ __align__(16) uint8_t smem_raw[];
    LazyCtx cx;
    cx.cost0 = reinterpret_cast<__half*>(smem_raw);
    cx.cost1 = cx.cost0 + G::edges;
    cx.sm = reinterpret_cast<LazySmem*>(smem_raw + 2 * G::edges * sizeof(__half));
    LazySmem* sm = cx.sm;
    uint8_t* labels = smem_raw + 2 * G::edges * sizeof(__half) + sizeof(LazySmem);
    for (int i = threadIdx.x; i < 65536 / 16; i += blockDim.x)
        reinterpret_cast<uint4*>(labels)[i] = reinterpret_cast<const uint4*>(lut_state)[i];
    cx.labels = labels;
    cx.scratch = scratch_base + size_t(blockIdx.x) * lazy_cta_bytes<K, DEDICATED>();
    // buffers alternate between consecutive tiles
    auto constrained_rows = [&](int x) {
        return cx.scratch + size_t((x & 1) * constrained_buffer_rows<DEDICATED>()) * (G::edges * 2);
    };
    auto primer_rows = [&](int x) {
        return cx.scratch + size_t(2 * constrained_buffer_rows<DEDICATED>() +
                                   (x & 1) * primer_buffer_rows<DEDICATED>()) * (G::edges * 2);
    };
    cx.lut_state = lut_state;
    cx.io = &io;
    cx.context = context;
    cx.tick = 0;
    cx.chain_due = kNever;
    if (threadIdx.x < 2) {
        sm->chain[threadIdx.x].state = 0;
        sm->chain[threadIdx.x].head.ri = -1;
        sm->chain[threadIdx.x].head.edge = 0;
    }

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

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int count = int((n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x);  // this CTA's tiles
    auto tile_of = [&](int x) { return int64_t(blockIdx.x) + int64_t(x) * gridDim.x; };
    // A primer's chain needs a pass to ride on before its tile's constrained pass: with a single
    // tile there is none.  (With a one-symbol context the primer's first step would have to be
    // a recorded one; that case keeps decisions too.)
    const bool lazy_primers = count >= 2 && context >= 2;

    // Re-encode tile x with the literal arithmetic, out of turn, and write its results.
    auto reencode = [&](int x) {
        const int slot = x % kInFlight;
        // the primer buffer of x is free: its primer was just abandoned, or its chain is finished
        encode_with_decisions<K, MODE_SAFE, UNITS, NL>(L, cx, slot, primer_rows(x));
        store_tile(io, tile_of(x), sm->states[slot], lut_state);
        if (threadIdx.x == 0) sm->slot[slot].done = 1;
        __syncthreads();
    };

    // P(x): load tile x and run its primer; leaves its boundary state with the slot, or starts
    // the primer chain that will.  Returns x if the tile met the clamp and has to be re-encoded,
    // else -1.
    auto primer = [&](int x) -> int {
        const int slot = x % kInFlight;
        // the slot's input and states may still belong to the constrained chain of tile x - 3
        if (sm->chain[CHAIN_CONSTRAINED].state != 0 && sm->chain[CHAIN_CONSTRAINED].head.slot == slot)
            finish_constrained_chain<K, MODE>(cx);
        load_tile<DEDICATED>(io, tile_of(x), sm->in_h[slot]);
        if (threadIdx.x == 0) sm->slot[slot].done = 0;
        __syncthreads();
        __half* cur = cx.cost0;
        __half* inc = cx.cost1;
        uint8_t* rows = primer_rows(x);
        bool over;
        if (lazy_primers)
            over = run_pass<K, MODE, UNITS, NL, false, true>(L, cx, slot, 256 - context, 2 * context, -1,
                                                             context - 1, rows, context - 1, cur, inc);
        else
            over = run_pass<K, MODE, UNITS, NL, false, false>(L, cx, slot, 256 - context, 2 * context, -1,
                                                              context, rows, 0, cur, inc);
        if (over) return x;  // MODE_FAST only
        int boundary;
        if constexpr (MODE == MODE_K2)
            boundary = boundary_argmin<K, false, UNITS>(cur, sm->red);  // final primer step (k2 cuh:282)
        else
            boundary = boundary_argmin<K, K != 2, UNITS>(inc, sm->red);  // step before the last (cuh:375,401)
        if (lazy_primers) {
            finish_primer_chain<K, MODE>(cx);  // tile x - 1's: it had a constrained pass and this primer
            if (warp == chain_warp<MODE>(CHAIN_PRIMER))
                chain_start<K, MODE>(&sm->chain[CHAIN_PRIMER], sm, rows, 0, context - 1, boundary, slot, -1,
                               tile_of(x), lane);
            cx.chain_due = warp == chain_warp<MODE>(CHAIN_PRIMER) ? cx.tick + kChainCadence
                           : warp == chain_warp<MODE>(CHAIN_CONSTRAINED) ? cx.chain_due : kNever;
            __syncthreads();
        } else {
            const int end_state = traceback<K, UNITS>(rows, reinterpret_cast<uint8_t*>(cx.cost0), context - 1,
                                                      boundary, false, sm->states[slot], &sm->edge);
            if (threadIdx.x == 0) sm->slot[slot].end_state = end_state;
            __syncthreads();
        }
        return -1;
    };

    // C(x): the constrained pass of tile x, with path costs and a chain if two more passes
    // follow to walk it during, else with survivor decisions.  Returns x if the tile met the
    // clamp and has to be re-encoded, else -1.
    auto constrained = [&](int x) -> int {
        const int slot = x % kInFlight;
        if (sm->slot[slot].done) return -1;
        if (sm->chain[CHAIN_PRIMER].state != 0 && sm->chain[CHAIN_PRIMER].head.slot == slot)
            finish_primer_chain<K, MODE>(cx);
        const int end_state = sm->slot[slot].end_state;
        const bool lazy = x + 2 < count;
        uint8_t* rows = constrained_rows(x);
        __half* cur = cx.cost0;
        __half* inc = cx.cost1;
        // tile x - 2's chain read these rows; it is finished by the time tile x - 1's starts, but
        // tile x - 1 may have started none
        if (sm->chain[CHAIN_CONSTRAINED].state != 0 && sm->chain[CHAIN_CONSTRAINED].rows == rows)
            finish_constrained_chain<K, MODE>(cx);
        if (lazy) {
            if (run_pass<K, MODE, UNITS, NL, true, true>(L, cx, slot, 0, 256, end_state, 0, rows, 0, cur, inc))
                return x;
            finish_constrained_chain<K, MODE>(cx);  // tile x - 1's: it had a primer and this pass
            if (warp == chain_warp<MODE>(CHAIN_CONSTRAINED))
                chain_start<K, MODE>(&sm->chain[CHAIN_CONSTRAINED], sm, rows, -1, 255, end_state, slot, end_state,
                               tile_of(x), lane);
            cx.chain_due = warp == chain_warp<MODE>(CHAIN_CONSTRAINED) ? cx.tick + kChainCadence
                           : warp == chain_warp<MODE>(CHAIN_PRIMER) ? cx.chain_due : kNever;
            __syncthreads();
        } else {
            if (run_pass<K, MODE, UNITS, NL, true, false>(L, cx, slot, 0, 256, end_state, 0, rows, 0, cur, inc))
                return x;
            traceback<K, UNITS>(rows, reinterpret_cast<uint8_t*>(cx.cost0), 255, end_state, true,
                                sm->states[slot], &sm->edge);
            store_tile(io, tile_of(x), sm->states[slot], lut_state);
            __syncthreads();
        }
        return -1;
    };

    // P(0) P(1) C(0) P(2) C(1) ... : every function above has exactly one call site, so that the
    // labels stay in registers through all of them.
#pragma unroll 1
    for (int turn = 0; turn <= 2 * count; ++turn) {
        int redo = -1;
        if (turn == 0 || (turn & 1)) {
            const int p = (turn + 1) >> 1;  // turns 0, 1, 3, 5, ...: the primers of tiles 0, 1, 2, 3, ...
            if (p < count) redo = primer(p);
        } else {
            redo = constrained((turn >> 1) - 1);  // turns 2, 4, 6, ...: the constrained passes
        }
        if (redo >= 0) reencode(redo);
    }
    finish_constrained_chain<K, MODE>(cx);
    finish_primer_chain<K, MODE>(cx);  // none is left unless its tile was finished out of turn
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

size_t qsrtb_lazy_scratch_per_cta(int bits, int dedicated)
{
    // two constrained and two primer buffers of cost rows, rows of 2^(16-bits) halves
    const size_t rows = (bits == 2 && dedicated) ? 2 * 128 + 2 * (kPrimerRows / 2) : 2 * 256 + 2 * kPrimerRows;
    return rows * (size_t(2) << (16 - bits));
}

int qsrtb_lazy_launch(const qsrtb_vit::TileIO& io, int64_t n_tiles, const uint8_t* lut_state,
                      const uint8_t* lut_pm, int bits, int context, int dedicated, void* scratch, int grid,
                      cudaStream_t stream)
{
    // Always 512 threads with two units each: with 1024 threads the chains' warps (one of eight
    // on their scheduler instead of one of four) fall behind and delay every step's barrier
    // (K3: 304 k against 349 k tiles/s), and 64 registers do not hold the kernel without spills.
    if (bits == 3) return launch_lazy<3, false, 2>(io, n_tiles, lut_state, lut_pm, context, scratch, grid, stream);
    if (bits == 4) return launch_lazy<4, false, 2>(io, n_tiles, lut_state, lut_pm, context, scratch, grid, stream);
    if (dedicated) return launch_lazy<2, true, 2>(io, n_tiles, lut_state, lut_pm, context, scratch, grid, stream);
    return launch_lazy<2, false, 2>(io, n_tiles, lut_state, lut_pm, context, scratch, grid, stream);
}
