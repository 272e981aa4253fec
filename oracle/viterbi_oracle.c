/*
 * CPU restatement of the reference's tail-biting trellis tile encoder.
 *
 * TEST INFRASTRUCTURE ONLY: this file is the checker for the CUDA product path (and the
 * timed CPU baseline of the benchmark).  The product never links or calls it.
 *
 * It follows, operation for operation, the two CUDA kernels of the reference
 *   qsrt/csrc/qsrt_quantize_tiles_kernel.cuh:26-500      (generic kernel, any K, E4M3 table)
 *   qsrt/csrc/qsrt_quantize_tiles_k2_kernel.cuh:47-366   (dedicated K2 kernel)
 * and the launcher's choice between them (qsrt/csrc/sqg_quantize.cu:730-748).
 *
 * All path costs are IEEE binary16.  Every half operation of the kernels is single-rounded:
 *   hsub(d, w)      : both operands are multiples of 2^-24 below 2^16, so the difference is
 *                     exact in binary64 and is rounded to half once;
 *   hmul(dh, dh)    : an 11-bit by 11-bit product, exact in binary64, rounded once;
 *   hfma(dh, dh, p) : the exact product plus a half value.  The binary64 sum is exact
 *                     whenever it matters: if the product is so small that binary64 drops
 *                     bits, the exact sum lies within 2^-30 of a half value and far from a
 *                     rounding tie, so rounding the binary64 sum to half gives the single
 *                     rounded result of the fused operation.
 * Ties are resolved exactly as the kernels do (strict less-than, lowest predecessor first,
 * and the kernels' literal warp shuffle reduction trees for the boundary argmin).
 *
 * State convention (cuh:443-468): a 16-bit state is (k << (16-K)) | out_edge where out_edge
 * is the low 16-K bits and k is the decision (the K bits about to be shifted out of the
 * predecessor).  The predecessor edge of out_edge under decision k is
 * (out_edge >> K) + k * 2^(16-2K).  `lut` is indexed by the 16-bit state.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define H_INF 0x7c00u
#define H_MAXF 0x7bffu

/* ---- binary16 helpers --------------------------------------------------------------- */

static double h2d_table[65536];
static int tables_ready = 0;

static double half_bits_to_double(uint16_t h)
{
    int s = h >> 15, e = (h >> 10) & 31, m = h & 1023;
    double v;
    if (e == 0) v = ldexp((double)m, -24);
    else if (e == 31) v = m ? NAN : INFINITY;
    else v = ldexp((double)(1024 + m), e - 25);
    return s ? -v : v;
}

static void init_tables(void)
{
    if (tables_ready) return;
    for (int i = 0; i < 65536; ++i) h2d_table[i] = half_bits_to_double((uint16_t)i);
    tables_ready = 1;
}

/* Round a binary64 value to binary16, round-to-nearest-even, overflow to infinity. */
static inline uint16_t d2h(double x)
{
    uint64_t u;
    memcpy(&u, &x, 8);
    uint16_t sign = (uint16_t)((u >> 48) & 0x8000u);
    u &= 0x7fffffffffffffffULL;
    if (u >= 0x7ff0000000000000ULL)
        return (uint16_t)(sign | (u > 0x7ff0000000000000ULL ? 0x7e00u : 0x7c00u));
    int e = (int)(u >> 52) - 1023;
    if (e >= 16) return (uint16_t)(sign | 0x7c00u);
    if (e < -25) return sign;
    uint64_t m = (u & 0xfffffffffffffULL) | (1ULL << 52);
    int shift = (e >= -14) ? 42 : (42 + (-14 - e));
    uint64_t q = m >> shift;
    uint64_t rem = m & ((1ULL << shift) - 1);
    uint64_t halfway = 1ULL << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1))) q++;
    uint32_t h;
    if (e >= -14) h = (uint32_t)(((uint32_t)(e + 15) << 10) + (q - 1024));
    else h = (uint32_t)q;
    if (h >= 0x7c00u) h = 0x7c00u;
    return (uint16_t)(sign | h);
}

static double e4m3_to_double(uint8_t b)
{
    int s = b >> 7, e = (b >> 3) & 15, m = b & 7;
    double v;
    if (e == 0) v = ldexp((double)m, -9);
    else if (e == 15 && m == 7) v = NAN;
    else v = ldexp((double)(8 + m), e - 10);
    return s ? -v : v;
}

/* Signed ordering of half bit patterns (no NaN reaches these; -0 and +0 compare equal).
 * The generic kernel's costs are never negative; the dedicated K2 kernel's lagged
 * renormalisation (k2 cuh:117-137,211-212) can drive them below zero. */
static inline int hkey(uint16_t h) { return (h & 0x8000u) ? -(int)(h & 0x7fffu) : (int)h; }
static inline int hlt(uint16_t a, uint16_t b) { return hkey(a) < hkey(b); }
static inline uint16_t hmin_(uint16_t a, uint16_t b) { return hkey(a) < hkey(b) ? a : b; }

/* Literal model of the kernels' `for offset = 16..1: shfl_down; if other < mine take other`. */
static void warp_tree(uint16_t* mn, int* ix)
{
    for (int offset = 16; offset > 0; offset >>= 1)
        for (int lane = 0; lane + offset < 32; ++lane)
            if (hlt(mn[lane + offset], mn[lane]))
            {
                mn[lane] = mn[lane + offset];
                ix[lane] = ix[lane + offset];
            }
}

typedef struct
{
    int K;
    int edges;
    int context;
    const uint8_t* lut;      /* state indexed */
    double lutd[256];        /* label byte -> value */
    uint16_t in_h[256];      /* rounded tile */
    uint16_t* cost_a;        /* [edges] */
    uint16_t* cost_b;        /* [edges] */
    uint8_t* dec;            /* [256][edges] */
    uint16_t* cur;           /* written by the latest step  (kernel: temp_costs)     */
    uint16_t* inc;           /* the step before             (kernel: temp_costs_inc) */
} tile_ctx;

/* ---- generic kernel (cuh:79-358) ---------------------------------------------------- */

static void generic_forward(tile_ctx* c, int roll, int steps, int pre_state, int trace_start)
{
    const int K = c->K, Kr = 16 - K, nk = 1 << K, edges = c->edges;
    const int pstep = 1 << (16 - 2 * K);
    double sq[256];
    uint16_t first[256];
    for (int i = 0; i < steps; ++i)
    {
        const int ri = (i + roll) & 255;
        uint16_t* t = c->cur; c->cur = c->inc; c->inc = t;
        const double w = h2d_table[c->in_h[ri]];
        for (int b = 0; b < 256; ++b)
        {
            double dh = h2d_table[d2h(c->lutd[b] - w)];
            sq[b] = dh * dh;
            if (i == 0) first[b] = hmin_(d2h(sq[b]), H_MAXF);
        }
        const int record = (i == 0) ? (trace_start == 0) : (i >= trace_start);
        uint8_t* dec = c->dec + (size_t)ri * edges;
        for (int e = 0; e < edges; ++e)
        {
            uint16_t best = 0;
            int bk = 0;
            int pred = e >> K;
            for (int k = 0; k < nk; ++k, pred += pstep)
            {
                const uint8_t label = c->lut[((uint32_t)k << Kr) | (uint32_t)e];
                uint16_t v;
                if (i == 0)
                {
                    v = first[label];
                    if (pre_state >= 0 && pred != pre_state) v = H_INF;
                }
                else
                {
                    const uint16_t pc = c->inc[pred];
                    v = (pc == H_INF) ? H_INF : hmin_(d2h(sq[label] + h2d_table[pc]), H_MAXF);
                }
                if (k == 0) best = v;
                else if (hlt(v, best)) { best = v; bk = k; }
            }
            c->cur[e] = best;
            if (record) dec[e] = (uint8_t)bk;
        }
    }
}

/* cuh:360-441.  Reads temp_costs_inc, i.e. the costs of the step before the last one. */
static int generic_argmin(tile_ctx* c)
{
    const int edges = c->edges;
    const uint16_t* costs = c->inc;
    uint16_t sh_min[32];
    int sh_idx[32];
    for (int i = 0; i < 32; ++i) { sh_min[i] = 0; sh_idx[i] = 0; }
    if (c->K == 2)
    {
        for (int warp = 0; warp < 32; ++warp)
        {
            uint16_t mn[32]; int ix[32];
            for (int lane = 0; lane < 32; ++lane)
            {
                const int thread = warp * 32 + lane;
                uint16_t lm = H_INF; int li = -1;
                for (int e = thread; e < edges; e += 1024)
                    if (hlt(costs[e], lm)) { lm = costs[e]; li = e; }
                mn[lane] = lm; ix[lane] = li;
            }
            warp_tree(mn, ix);
            sh_min[warp] = mn[0]; sh_idx[warp] = ix[0];
        }
    }
    else
    {
        for (int warp = 0; warp < 16; ++warp)
        {
            uint16_t mn0[32], mn1[32]; int ix0[32], ix1[32];
            for (int lane = 0; lane < 32; ++lane)
            {
                const int thread = warp * 32 + lane;
                uint16_t l0 = H_INF, l1 = H_INF; int i0 = -1, i1 = -1;
                for (int e = thread; e < edges; e += 1024)
                    if (hlt(costs[e], l0)) { l0 = costs[e]; i0 = e; }
                for (int e = thread + 512; e < edges; e += 1024)
                    if (hlt(costs[e], l1)) { l1 = costs[e]; i1 = e; }
                mn0[lane] = l0; ix0[lane] = i0; mn1[lane] = l1; ix1[lane] = i1;
            }
            warp_tree(mn0, ix0);
            warp_tree(mn1, ix1);
            sh_min[warp] = mn0[0]; sh_idx[warp] = ix0[0];
            sh_min[16 + warp] = mn1[0]; sh_idx[16 + warp] = ix1[0];
        }
    }
    warp_tree(sh_min, sh_idx);
    return sh_idx[0];
}

/* cuh:443-487 (and k2 cuh:327-354: identical walk). */
static int backward(tile_ctx* c, int roll, int steps, int write, int edge, float* out, uint16_t* idx)
{
    const int K = c->K, edges = c->edges;
    for (int i = steps - 1; i >= 0; --i)
    {
        const int ri = (i + roll) & 255;
        const int decision = c->dec[(size_t)ri * edges + edge];
        const int prev_edge = (decision << (16 - 2 * K)) | (edge >> K);
        const int encoded = ((prev_edge << K) | edge) & 0xffff;
        edge = prev_edge;
        if (write)
        {
            idx[ri] = (uint16_t)encoded;
            out[ri] = (float)c->lutd[c->lut[encoded]];
        }
        else if (ri == 0) break;
    }
    return edge;
}

/* ---- dedicated K2 kernel (k2 cuh:107-272) ------------------------------------------- */

typedef struct { uint16_t shift[2]; uint16_t step_min[2]; } k2_state;

static void k2_forward(tile_ctx* c, k2_state* s, int roll, int steps, int pre_state,
                       int trace_start, int constrained)
{
    const int edges = c->edges; /* 16384 */
    double sq[256];
    uint16_t first[256];
    for (int i = 0; i < steps; ++i)
    {
        const int ri = (i + roll) & 255;
        uint16_t* t = c->cur; c->cur = c->inc; c->inc = t;
        const int is_first = (i == 0);
        const int record = is_first ? constrained : (i >= trace_start);
        if (!is_first)
        {
            /* Warp 0 folds the previous step's minimum into the shift used by step i+1. */
            const uint16_t m = s->step_min[(i - 1) & 1];
            s->shift[(i + 1) & 1] = (hkey(m) >= 0x6400 /* 1024.0 */) ? m : 0;
        }
        const double w = h2d_table[c->in_h[ri]];
        const uint16_t shift = s->shift[i & 1];
        const double shift_d = h2d_table[shift];
        for (int b = 0; b < 256; ++b)
        {
            double dh = h2d_table[d2h(c->lutd[b] - w)];
            sq[b] = dh * dh;
            if (is_first) first[b] = d2h(sq[b]);
        }
        uint8_t* dec = c->dec + (size_t)ri * edges;
        uint16_t step_min = H_INF;
        for (int e = 0; e < edges; ++e)
        {
            uint16_t best = 0;
            int bk = 0;
            const int q = e >> 2;
            for (int k = 0; k < 4; ++k)
            {
                const uint8_t label = c->lut[((uint32_t)k << 14) | (uint32_t)e];
                uint16_t v;
                if (is_first)
                {
                    v = first[label];
                    if (constrained && q + (k << 12) != pre_state) v = H_INF;
                }
                else
                {
                    const uint16_t pc = c->inc[q + (k << 12)];
                    v = (pc == H_INF) ? H_INF : d2h(sq[label] + h2d_table[pc]);
                }
                if (k == 0) best = v;
                else if (hlt(v, best)) { best = v; bk = k; }
            }
            if (best != H_INF && shift != 0) best = d2h(h2d_table[best] - shift_d);
            c->cur[e] = best;
            step_min = hmin_(step_min, best);
            if (record) dec[e] = (uint8_t)bk;
        }
        s->step_min[i & 1] = step_min;
    }
}

/* k2 cuh:276-325: argmin over the final step's costs, 1024 threads. */
static int k2_argmin(tile_ctx* c)
{
    const int edges = c->edges;
    const uint16_t* costs = c->cur;
    uint16_t sh_min[32];
    int sh_idx[32];
    for (int warp = 0; warp < 32; ++warp)
    {
        uint16_t mn[32]; int ix[32];
        for (int lane = 0; lane < 32; ++lane)
        {
            const int thread = warp * 32 + lane;
            uint16_t lm = H_INF; int li = -1;
            for (int e = thread; e < edges; e += 1024)
                if (hlt(costs[e], lm)) { lm = costs[e]; li = e; }
            mn[lane] = lm; ix[lane] = li;
        }
        warp_tree(mn, ix);
        sh_min[warp] = mn[0]; sh_idx[warp] = ix[0];
    }
    warp_tree(sh_min, sh_idx);
    return sh_idx[0];
}

/* ---- entry points ------------------------------------------------------------------- */

/* Largest |label| of the table; the launcher's K2 routing rule (sqg_quantize.cu:735-737). */
double qsrt_oracle_lut_abs_max(const uint8_t* lut)
{
    double m = 0.0;
    for (int i = 0; i < 65536; ++i)
    {
        double v = fabs(e4m3_to_double(lut[i]));
        if (!(v <= m)) m = v; /* NaN propagates like amax */
    }
    return m;
}

/*
 * variant: 0 = the launcher's rule, 1 = generic kernel, 2 = dedicated K2 kernel.
 * Returns 0, or a negative code for bad arguments.
 */
int qsrt_oracle_quantize_tiles(const float* tiles, long n_tiles, const uint8_t* lut, int K,
                               int tailbite_context, int variant, float* out, uint16_t* idx,
                               int threads)
{
    if (K < 1 || K > 6) return -1;
    if (tailbite_context < 1 || tailbite_context > 128) return -2;
    if (variant < 0 || variant > 2 || (variant == 2 && K != 2)) return -3;
    init_tables();
    int use_k2 = 0;
    if (K == 2)
    {
        if (variant == 2) use_k2 = 1;
        else if (variant == 0)
        {
            double amax = qsrt_oracle_lut_abs_max(lut);
            use_k2 = isfinite(amax) && amax > 0.0 && amax <= 16.0;
        }
    }
    const int edges = 65536 >> K;
    int status = 0;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
#pragma omp parallel
    {
        tile_ctx c;
        c.K = K; c.edges = edges; c.context = tailbite_context; c.lut = lut;
        for (int b = 0; b < 256; ++b) c.lutd[b] = e4m3_to_double((uint8_t)b);
        c.cost_a = (uint16_t*)malloc(sizeof(uint16_t) * edges);
        c.cost_b = (uint16_t*)malloc(sizeof(uint16_t) * edges);
        c.dec = (uint8_t*)malloc((size_t)256 * edges);
        if (!c.cost_a || !c.cost_b || !c.dec)
        {
#pragma omp atomic write
            status = -4;
        }
        else
        {
#pragma omp for schedule(dynamic, 1)
            for (long tile = 0; tile < n_tiles; ++tile)
            {
                const float* in = tiles + 256 * tile;
                float* o = out + 256 * tile;
                uint16_t* ix = idx + 256 * tile;
                memset(c.cost_a, 0, sizeof(uint16_t) * edges);
                memset(c.cost_b, 0, sizeof(uint16_t) * edges);
                c.cur = c.cost_a; c.inc = c.cost_b;
                const int roll = 256 - tailbite_context, steps = 2 * tailbite_context;
                if (use_k2)
                {
                    for (int i = 0; i < 256; ++i)
                    {
                        float w = in[i];
                        w = fmaxf(-64.0f, fminf(w, 64.0f));
                        c.in_h[i] = d2h((double)w);
                    }
                    k2_state s = {{0, 0}, {H_INF, H_INF}};
                    k2_forward(&c, &s, roll, steps, -1, tailbite_context, 0);
                    int end_state = backward(&c, roll, steps, 0, k2_argmin(&c), o, ix);
                    s.shift[0] = s.shift[1] = 0;
                    k2_forward(&c, &s, 0, 256, end_state, 0, 1);
                    backward(&c, 0, 256, 1, end_state, o, ix);
                }
                else
                {
                    for (int i = 0; i < 256; ++i) c.in_h[i] = d2h((double)in[i]);
                    generic_forward(&c, roll, steps, -1, tailbite_context);
                    int end_state = backward(&c, roll, steps, 0, generic_argmin(&c), o, ix);
                    generic_forward(&c, 0, 256, end_state, 0);
                    backward(&c, 0, 256, 1, end_state, o, ix);
                }
            }
        }
        free(c.cost_a); free(c.cost_b); free(c.dec);
    }
    return status;
}

/* Scalar helpers exported so the tests can pin the half arithmetic itself. */
uint16_t qsrt_oracle_d2h(double x) { return d2h(x); }
double qsrt_oracle_h2d(uint16_t h) { return half_bits_to_double(h); }
double qsrt_oracle_e4m3(uint8_t b) { return e4m3_to_double(b); }
