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

#include "viterbi_core.cuh"

namespace {

using namespace qsrtb_vit;

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
    // Launches that give a CTA more than one tile keep path costs instead of survivor decisions
    // for half of the steps (viterbi_lazy.cu), which takes two slots of 256 cost rows per CTA.
    const size_t per_cta = n_tiles > sms ? qsrtb_lazy_scratch_per_cta(bits, 1) : 256 * row_bytes;
    *bytes = size_t(grid > 0 ? grid : 1) * per_cta;
    return QSRTB_OK;
}

extern "C" int qsrtb_viterbi_cost_scratch_bytes(int bits, int64_t n_tiles, size_t* bytes)
{
    if (bits < 2 || bits > 4 || !bytes || n_tiles < 0) return qsrtb_fail(QSRTB_EINVAL, "bad scratch query");
    const int sms = resident_ctas();
    if (sms <= 0) return qsrtb_fail(QSRTB_ECUDA, "cannot query the device");
    const int64_t grid = n_tiles < sms ? n_tiles : sms;
    *bytes = size_t(grid > 0 ? grid : 1) * qsrtb_lazy_scratch_per_cta(bits, 0);
    return QSRTB_OK;
}

namespace {

int check_common(int bits, int tailbite_context, int variant, int64_t n_tiles)
{
    if (bits < 2 || bits > 4) return qsrtb_fail(QSRTB_EINVAL, "bits must be 2, 3 or 4");
    if (tailbite_context < 1 || tailbite_context > 128)
        return qsrtb_fail(QSRTB_EINVAL, "tailbite_context must be in 1..128");
    if ((variant & ~0xf1) != 0 || ((variant >> 4) & 3) == 3 || ((variant >> 6) & 3) == 3)
        return qsrtb_fail(QSRTB_EINVAL, "variant: bit 0 selects the dedicated K2 arithmetic, bits 4-5 the thread layout (0, 1 or 2), bits 6-7 the traceback organisation (0, 1 or 2)");
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
    // Traceback organisation (bits 6-7): 1 = survivor decisions for every recorded step, 2 = path
    // costs with the decisions recomputed by the traceback chains (viterbi_lazy.cu), 0 = the
    // latter where it pays: three or four bits or the dedicated K2 arithmetic (the generic K2
    // arithmetic would have to store every 32 KiB cost row, which costs what the bookkeeping
    // saves), full tail-biting context (a chain rides on the 256-step passes that follow), more
    // tiles than CTAs, and scratch for the cost rows.  Same results either way.
    const int organisation = (variant >> 6) & 3;
    variant &= 1;
    if (organisation != 1) {
        const int sms = resident_ctas();
        if (sms <= 0) return qsrtb_fail(QSRTB_ECUDA, "cannot query the device");
        const size_t per_cta = qsrtb_lazy_scratch_per_cta(bits, variant);
        int64_t grid = n_tiles < sms ? n_tiles : sms;
        // the state table is copied to shared memory and the cost rows are written 16 bytes at a time
        const bool aligned = (reinterpret_cast<uintptr_t>(lut_state) & 15) == 0 &&
                             (reinterpret_cast<uintptr_t>(scratch) & 15) == 0;
        const bool fits = aligned && scratch_bytes / per_cta >= size_t(grid);
        if (organisation == 2 && !fits)
            return qsrtb_fail(QSRTB_ESCRATCH, "traceback scratch smaller than the cost rows of the grid, or table / scratch not 16-byte aligned");
        // (the thread layout bits do not apply: that kernel always runs 512 threads)
        if (fits && (organisation == 2 || ((bits != 2 || variant == 1) && context == 128 && n_tiles > sms)))
            return qsrtb_lazy_launch(io, n_tiles, lut_state, lut_pm, bits, context, variant, scratch, int(grid), s);
    }
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
    return dispatch(io, n_tiles, lut_state, lut_pm, bits, tailbite_context, (variant & 0x3f) | (1 << 6),
                    scratch, size_t(QSRTB_STATIC_SCRATCH_BYTES), static_cast<cudaStream_t>(stream));
}
