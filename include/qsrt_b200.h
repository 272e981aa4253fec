/*
 * C ABI of the B200 (sm_100a) offline trellis-encoder kernels.
 *
 * Conventions for every entry point:
 *   - returns QSRTB_OK (0) or a negative QSRTB_E* code; nothing is thrown across the ABI;
 *   - every pointer is a DEVICE pointer borrowed from the caller unless named `host_*`;
 *     the callee never allocates or frees device memory and keeps no pointer after return;
 *   - all work is enqueued on the `stream` argument (a cudaStream_t passed as void*) and the
 *     call returns without synchronising unless stated otherwise;
 *   - there is no global mutable state: look-up tables travel as arguments.
 *
 * Each declaration cites the reference interface it stands in for (paths relative to the
 * reference checkout).
 */
#ifndef QSRT_B200_H
#define QSRT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QSRTB_OK 0
#define QSRTB_EINVAL (-1)   /* bad shape / rate / context argument          */
#define QSRTB_ESCRATCH (-2) /* scratch buffer too small                     */
#define QSRTB_ECUDA (-3)    /* a CUDA runtime call failed (see last error)  */
#define QSRTB_ENOTPD (-4)   /* Hessian not positive definite                */

/* Library / build identification. */
int qsrtb_abi_version(void);
const char* qsrtb_last_error(void);

/* Measurement aid (no reference counterpart): runs iters x 8 independent half2 FMAs per thread
 * on a device-filling grid; *fma_lanes (HOST pointer) receives the number of half lanes
 * issued.  Timed by the benchmark to obtain the half2 FMA rate used as ALU roofline. */
int qsrtb_probe_half2_fma(int iters, float* sink, double* fma_lanes, void* stream);

/* ---- V5: look-up table preparation -------------------------------------------------
 * Replaces the table transpose of qsrt/sqg_quantizer.py:611-640.
 * lut_state : 65,536 E4M3 bytes indexed by the 16-bit trellis state.
 * lut_pm    : 65,536 bytes out, laid out [out-edge pair][predecessor][2].
 * abs_max   : one float out, max |label| (the launcher's K2 routing input,
 *             qsrt/csrc/sqg_quantize.cu:735-737).
 */
int qsrtb_lut_prepare(const uint8_t* lut_state, int bits, uint8_t* lut_pm, float* abs_max,
                      void* stream);

/* ---- V1-V4: tail-biting Viterbi tile encoder ------------------------------------------
 * Replaces quantize_tiles_sqg_cuda (qsrt/csrc/sqg_quantize.cu:651-783), i.e. the kernels
 * qsrt/csrc/qsrt_quantize_tiles_kernel.cuh:26-500 (variant 0) and
 * qsrt/csrc/qsrt_quantize_tiles_k2_kernel.cuh:47-366 (variant 1, bits == 2 only), and is
 * bit-identical to them.
 *
 * qsrtb_viterbi_scratch_bytes: bytes of traceback scratch wanted for `n_tiles` tiles on the
 * current device (a persistent grid is used, so this saturates at one slice per resident CTA:
 * 0.5 or 1 MiB of survivor decisions when no CTA gets a second tile, else path-cost rows: 6 MiB
 * at 4 bits, 12 MiB at 3 and at 2 - where only the dedicated arithmetic uses them, storing
 * every second row).  A call given less scratch than
 * that still works: it keeps survivor decisions for every step, on as many CTAs as the scratch
 * has slices.
 */
int qsrtb_viterbi_scratch_bytes(int bits, int64_t n_tiles, size_t* bytes);
/* The scratch an explicit QSRTB_VARIANT_TRACEBACK(2) needs at any rate: two buffers of 256 and
 * two of 130 path-cost rows per resident CTA (6 / 12 / 24 MiB at 4 / 3 / 2 bits). */
int qsrtb_viterbi_cost_scratch_bytes(int bits, int64_t n_tiles, size_t* bytes);

/* `variant` of the search entry points: bit 0 = dedicated K2 arithmetic (bits == 2 only);
 * bits 4-5 = thread layout of the search kernel, a per-call tuning choice without a reference
 * counterpart (0 = the faster one for the rate and traceback organisation, 1 = 1024 threads
 * holding fp8 labels, 2 = 512 threads holding half2 labels in registers; the path-cost
 * organisation below always runs 2); bits 6-7 = what the search keeps for its traceback, also
 * without a reference counterpart (1 = survivor decisions for every recorded step; 2 = path
 * costs, from which the tracebacks recompute the one decision per step they need while the
 * passes of the CTA's next tiles run - all passes but the constrained ones of a CTA's last two
 * tiles; 0 = 2 where it pays: 3 or 4 bits or the dedicated K2 arithmetic, tailbite_context 128,
 * more tiles than SMs, scratch as qsrtb_viterbi_scratch_bytes says; an explicit 2 needs
 * qsrtb_viterbi_cost_scratch_bytes).
 * Results are identical for every layout and organisation. */
#define QSRTB_VARIANT_DEDICATED_K2 1
#define QSRTB_VARIANT_LAYOUT(units) ((units) << 4)
#define QSRTB_VARIANT_TRACEBACK(organisation) ((organisation) << 6)

int qsrtb_quantize_tiles(const float* tiles,        /* [n_tiles, 256] tensor-core order   */
                         int64_t n_tiles,
                         const uint8_t* lut_state,   /* 65,536 bytes, state indexed        */
                         const uint8_t* lut_pm,      /* from qsrtb_lut_prepare             */
                         int bits,                   /* 2, 3 or 4                          */
                         int tailbite_context,       /* 1..128                             */
                         int variant,                /* see QSRTB_VARIANT_* above           */
                         float* out_tiles,           /* [n_tiles, 256] reconstruction      */
                         int16_t* out_states,        /* [n_tiles, 256] 16-bit states       */
                         void* scratch, size_t scratch_bytes,
                         void* stream);

/* Tile search for callers that cannot allocate device memory (no counterpart in the
 * reference, which always allocates its traceback buffers with torch).  Same inputs, outputs
 * and results as qsrtb_quantize_tiles, but the survivor scratch is a fixed 16 MiB array inside
 * the library image on each GPU, so the call performs no allocation of any kind.
 *   - at most 4096 tiles per call (QSRTB_EINVAL beyond that); the small scratch limits the
 *     grid to 16 CTAs (K2, K3) or 32 (K4), so it is slower than the regular entry point;
 *   - the first call on a device looks up the array's device address, and is also the moment
 *     the CUDA runtime may make the library's code and this array resident on that GPU; make
 *     that first call at start-up - outside any stream capture and before a memory pool claims
 *     whatever device memory is left;
 *   - all calls share the array: calls that overlap in time on one GPU race, serialise them.
 */
int qsrtb_quantize_tiles_static(const float* tiles, int64_t n_tiles, const uint8_t* lut_state,
                                const uint8_t* lut_pm, int bits, int tailbite_context,
                                int variant, float* out_tiles, int16_t* out_states, void* stream);

/* ---- H1: calibration Hessian accumulation ------------------------------------------------
 * Replaces the chunked `accumulator.addmm_(x.T, x * w)` of weighted_covariance
 * (qsrt/candidate_hessian.py:70-112) and _accumulate_hessian (qsrt/capture.py:714-731).
 *   qsrtb_hessian_accumulate : lower triangle of  lower (+)= sum_r w[r] * rows[r]^T rows[r]
 *                              (weights may be NULL = 1; accumulate 0 overwrites, 1 adds).
 *   qsrtb_hessian_finish     : divides the lower triangle by weight_sum and mirrors it, giving
 *                              the symmetric float32 covariance ((C + C^T) / 2 of the reference).
 */
int qsrtb_hessian_accumulate(const float* rows, const float* weights, int64_t n_rows, int d,
                             int ld_rows, float* lower, int ld_h, int accumulate, void* stream);
int qsrtb_hessian_finish(float* h, int d, int ld_h, double weight_sum, void* stream);

/* Tensor-core variant of qsrtb_hessian_accumulate (same reference counterpart): tcgen05 TF32
 * MMAs with the accumulator in tensor memory; the float32 inputs are split into TF32 head and
 * tail (three products, float32 accumulation) so the result stays within 1e-5 of float64.
 * Needs d % 128 == 0 and a workspace of qsrtb_hessian_tc_workspace_bytes(n_rows, d).
 * *status_flag (device int, zeroed by the caller) becomes 1 if a bounded wait inside the kernel
 * expired; the output is then undefined but the context stays usable.
 */
int qsrtb_hessian_tc_workspace_bytes(int64_t chunk_rows, int d, size_t* bytes);
int qsrtb_hessian_accumulate_tc(const float* rows, const float* weights, int64_t n_rows, int d,
                                int ld_rows, float* lower, int ld_h, int accumulate, void* workspace,
                                size_t workspace_bytes, int* status_flag, void* stream);

/* ---- R1 / H2 / D1: blockwise 128-point Hadamard with a fused sign/scale vector ----------
 * Replaces blockwise_preapply_had_l_/r_ and preapply_had_l/r together with the vector
 * scaling next to them (qsrt/exl3_encoder_backend.py:275-320, 2654-2675, 2142-2145,
 * 3031-3034; decode side qsrt/exl3_reference.py:230-243, 298-301).  In place on `batch`
 * row-major matrices [rows, cols] (row pitch ld, matrix pitch x_stride).
 *   axis 1: every 128-column block of every row  := block @ Had128 / sqrt(128)  ("had_r")
 *   axis 0: every 128-row block of every column  := Had128 / sqrt(128) @ block  ("had_l")
 *   scale (optional, one vector per matrix, pitch scale_stride): indexed by column when
 *   scale_per_col else by row; divides when scale_divide else multiplies; applied to the
 *   transformed values when scale_after else to the inputs.
 *   row_sumsq (axis 1 only, optional): per-row sum of squares of the result, fixed order.
 */
int qsrtb_hadamard128(float* x, int batch, int rows, int cols, int ld, int64_t x_stride, int axis,
                      const float* scale, int64_t scale_stride, int scale_per_col,
                      int scale_divide, int scale_after, float* row_sumsq, int64_t sumsq_stride,
                      void* stream);

/* ---- R2: signed block Walsh-Hadamard of the coupled gate/up/down coordinates -------------
 * Replaces block_hadamard / signed_block_hadamard (qsrt/qsrt_coupled.py:49-132) on a row-major
 * float32 matrix, in place: along `axis` (1 = within rows, 0 = within columns) every block of
 * `block_size` (128, 256 or 512) becomes H(block * signs) / sqrt(block_size) ("D H",
 * sign_after = 0) or H(block) / sqrt(block_size) * signs (its inverse "H D", sign_after = 1);
 * signs may be NULL.  Butterfly order and the true division match the reference's float32
 * CPU arithmetic bit for bit.
 */
int qsrtb_signed_block_hadamard(float* x, int64_t rows, int cols, int ld, int axis, int block_size,
                                const float* signs, int sign_after, void* stream);

/* The same "D H" transform along the input axis (axis 1) with the source matrix read in its
 * packed MXFP4 storage - packed [rows, cols / 2] E2M1 codes, low nibble first, scale
 * [rows, cols / 32] E8M0 bytes (dequant law of qsrt/io/mxfp4.py:50-63) - so that source ingest and
 * the first coupled transform (qsrt/qsrt_coupled.py:145-196) are one pass and the dequantised
 * matrix is never stored.  Source row r goes to output row r * row_step + row_offset (row_step 2
 * interleaves the gate and up matrices); round_bf16 != 0 rounds every dequantised value to
 * bfloat16 first, as a bf16 checkpoint of the source holds it.  Results equal dequant followed by
 * qsrtb_signed_block_hadamard bit for bit.
 */
int qsrtb_mxfp4_signed_block_hadamard(const uint8_t* packed, const uint8_t* scale, int64_t rows, int cols,
                                      float* out, int ld, int row_step, int row_offset, int block_size,
                                      const float* signs, int round_bf16, void* stream);

/* Column sums of squares of `batch` matrices (the out-channel RMS of regularize,
 * qsrt/exl3_encoder_backend.py:2508-2521, 2634).  workspace: batch*ceil(rows/256)*cols floats. */
int qsrtb_col_sumsq(const float* x, int batch, int rows, int cols, int ld, int64_t x_stride,
                    float* out, int64_t out_stride, float* workspace, size_t workspace_bytes,
                    void* stream);

/* ---- float32-accurate products on the tensor cores -------------------------------------------
 * qsrtb_gemm3x_tc:  D[z] = alpha * A[z] * B[z]^T + beta * D[z]  for z < batch, with A [m, k] and
 * B [n, k] both stored with k contiguous ("K-major").  Stands in for the library float32 GEMMs of
 * the path: the BlockLDLQ feedback `addmm_` / `baddbmm` (qsrt/exl3_encoder_backend.py:494-501,
 * 533-534, 1170-1187), the trailing update inside `torch.linalg.cholesky` (:335) and the
 * `F.linear` products of the routed scoring (qsrt/pooled_calibration.py:734-753).
 * tcgen05 TF32 MMAs with the accumulator in tensor memory; each operand is passed as two planes,
 * the TF32 head and tail of the float32 values (qsrtb_split_tf32), and three products are
 * accumulated in float32, which keeps float32 accuracy.
 *   lda / ldb / ldd : row pitches in floats (multiples of 4; all bases 16-byte aligned);
 *   *_stride        : floats between consecutive matrices of a stack (ignored when batch == 1);
 *   lower_only      : m == n, only the 128 x 128 tiles on or below the diagonal are computed;
 *   transposed_out  : 0 writes D[i * ldd + j], 1 writes D[j * ldd + i];
 *   skip_flag       : optional device int; nonzero at run time makes the launch a no-op;
 *   status_flag     : device int, zeroed by the caller; nonzero afterwards if a bounded wait
 *                     inside the kernel expired (output undefined, context still usable).
 * m, n, k need not be multiples of the tile sizes.
 */
int qsrtb_gemm3x_tc(const float* a_hi, const float* a_lo, int lda, int64_t a_stride,
                    const float* b_hi, const float* b_lo, int ldb, int64_t b_stride,
                    int batch, int m, int n, int k,
                    float* d, int ldd, int64_t d_stride, float alpha, float beta,
                    int lower_only, int transposed_out,
                    const int* skip_flag, int* status_flag, void* stream);

/* Splits `batch` row-major float32 matrices [rows, cols] into their TF32 head and tail planes
 * (x = hi + lo exactly up to the tail's own rounding), optionally transposing: transpose == 0
 * gives planes [rows, cols], transpose == 1 planes [cols, rows]; ld_out is the planes' row pitch.
 * No reference counterpart (operand preparation of qsrtb_gemm3x_tc).
 */
int qsrtb_split_tf32(const float* src, int batch, int rows, int cols, int ld, int64_t src_stride,
                     float* hi, float* lo, int ld_out, int64_t out_stride, int transpose, void* stream);

/* ---- H2: dense Cholesky of the damped Hessian, on the device ------------------------------------
 * Replaces `torch.linalg.cholesky(H)` inside block_ldl (qsrt/exl3_encoder_backend.py:335) and the
 * exception the reference catches for its retry loop (:331-370).  In place: on return the lower
 * triangle of `a` holds L with L L^T = A; the strict upper triangle is scratch.
 *   workspace : qsrtb_cholesky_workspace_bytes(n) bytes;
 *   status    : TWO device ints zeroed by the caller.  status[0] = 0, or the 1-based column of the
 *               first pivot that was not positive (the matrix is not positive definite; the
 *               contents of `a` are then undefined) - nothing is thrown or trapped, the host reads
 *               the word when it chooses and adds damping.  status[1] != 0: a bounded wait of the
 *               tensor-core update expired.
 * Blocked right-looking factorisation: 128-column panels factored and solved by float32 kernels,
 * trailing updates by qsrtb_gemm3x_tc.  n % 16 == 0 (the block size of the block-LDL factor); ld % 4 == 0.
 */
int qsrtb_cholesky_workspace_bytes(int n, size_t* bytes);
int qsrtb_cholesky_blocked(float* a, int n, int ld, void* workspace, size_t workspace_bytes,
                           int* status, void* stream);

/* ---- H2: Cholesky factor -> unit block-lower LDL feedback factor, in place ---------------
 * Replaces the tail of block_ldl and the diagonal clearing after it
 * (qsrt/exl3_encoder_backend.py:372-393, 2152-2153): each 16-column block is multiplied by
 * the inverse of its diagonal block; diagonal blocks and everything above them become 0.
 */
int qsrtb_block_ldl_normalize(float* chol, int n, int ld, void* stream);

/* ---- L1: one 16-row step of the BlockLDLQ loop ----------------------------------------
 * Replaces, for one 16-row block of `batch` stacked row-major matrices, the per-step chain of
 * ldlq / ldlq_batched (qsrt/exl3_encoder_backend.py:502-520, 2040-2062): feedback add
 * (`_apply_ldlq_feedback`, :408-417), reshape to 16x16 tiles, tensor-core permutation (:35-57),
 * tile search, inverse permutation and scatter of the reconstruction.
 *   w, wq, err : pointers to the FIRST of the 16 rows in matrix 0 (row pitch `ld`, matrix
 *                pitch `w_stride`); err (= w - wq) may be NULL.
 *   comp       : compensation rows [16, n] per matrix (pitch comp_ld / comp_stride) or NULL.
 *   out_states : [n/16, 256] states per matrix for this row of tiles (pitch state_stride).
 *   tile_map   : optional device list of the column tiles to encode (tile_map_count of
 *                them, others untouched): one launch per rate of a mixed-rate column map
 *                (ldlq_mixed, qsrt/exl3_encoder_backend.py:898-1082); NULL = all n/16 tiles.
 * Encoder input is w (multiplier 0), w + comp (1) or w + multiplier * comp.
 */
int qsrtb_ldlq_quantize_rows(const float* w, const float* comp, float multiplier, int batch,
                             int n, int ld, int comp_ld, int64_t w_stride, int64_t comp_stride,
                             const uint8_t* lut_state, const uint8_t* lut_pm, int bits,
                             int tailbite_context, int variant, float* wq, float* err,
                             int16_t* out_states, int64_t state_stride, const int32_t* tile_map,
                             int tile_map_count, void* scratch, size_t scratch_bytes,
                             void* stream);

/* Same step for an arbitrary set of live encoder states that share source matrices: the
 * continuation form of ldlq_mixed_batched (qsrt/exl3_encoder_backend.py:1190-1478, its
 * `source_indices` argument) used by the candidate prefix trie (:1645-1830).  members is a DEVICE
 * array of member_count (source, owner) int32 pairs: visited matrix b reads rows of source matrix
 * members[2b] of w and reads/writes matrix members[2b+1] of comp / wq / err / out_states.  All
 * other arguments as qsrtb_ldlq_quantize_rows.
 */
int qsrtb_ldlq_quantize_members(const float* w, const float* comp, float multiplier,
                                const int32_t* members, int member_count, int n, int ld,
                                int comp_ld, int64_t w_stride, int64_t comp_stride,
                                const uint8_t* lut_state, const uint8_t* lut_pm, int bits,
                                int tailbite_context, int variant, float* wq, float* err,
                                int16_t* out_states, int64_t state_stride,
                                const int32_t* tile_map, int tile_map_count, void* scratch,
                                size_t scratch_bytes, void* stream);

/* ---- source ingest: MXFP4 expert weights -> float32 ------------------------------------------
 * Replaces dequant (qsrt/io/mxfp4.py:50-63; unpack_codes :19-30, scale_factors :42-44,
 * code_values :45-48) and the transpose into encoder orientation that follows it.
 * packed uint8 [out_rows, in_cols/2] (low nibble = even input), scale uint8 [out_rows, in_cols/32]
 * (E8M0, 2^(byte-127)).  transposed = 0: dst [out_rows, in_cols]; 1: dst [in_cols, out_rows].
 * Bit-exact with the reference's float32 arithmetic.
 */
int qsrtb_mxfp4_dequant(const uint8_t* packed, const uint8_t* scale, int out_rows, int in_cols,
                        float* dst, int ld, int transposed, void* stream);

/* No reference counterpart: launches one warp that waits on an mbarrier nothing ever arrives on,
 * through the same bounded wait the tensor-core Hessian kernel uses.  After about 20 ms the wait
 * gives up and *status_flag (device int, zeroed by the caller) receives 0x06000000 | lane of the
 * thread that recorded the expiry; the context stays usable.  For tests of the expiry path.
 */
int qsrtb_hessian_tc_wait_probe(int* status_flag, void* stream);

/* ---- C1/C2: per-tile error surfaces for rate allocation ---------------------------------------
 * Replaces tile_squared_error and the final tile reduction of dense_h_tile_error_contributions
 * (qsrt/high_rate_allocation.py:55-73,136-148).  a, b [rows, cols] float32 (row pitches lda, ldb)
 * -> out [rows/16, cols/16] float64: mode 0 sums (b - a)^2, mode 1 sums a * b over each 16x16
 * tile; terms are rounded to float32 and added in float64 as in the reference.
 */
int qsrtb_tile_reduce(const float* a, const float* b, int rows, int cols, int lda, int ldb, int mode,
                      double* out, void* stream);

/* ---- (f)3: dense-H path refinement, scoring and acceptance for one 16-row block -------------
 * Replaces the per-block tail of refine_h2_viterbi_paths (qsrt/h2_viterbi_refine.py:451-505;
 * _conditional_scores :261-279).  All row pointers address the FIRST of the block's 16 rows.
 *   weight, target : float32 [16, n] regularised weights and the conditional target (cast to
 *                    float32, as the reference casts it before the tile search).
 *   recon, states  : stored reconstruction rows [16, n] and payload [n/16, 256]; rewritten for
 *                    accepted tiles.
 *   cand, cand_states : `variants` proposals, [variants, 16, n] (pitches ldc, cand_stride) and
 *                    [variants, n/16, 256] (pitch cand_state_stride), as written by
 *                    qsrtb_ldlq_quantize_rows with batch = variants.
 *   h_block        : the block's 16x16 diagonal Hessian block; col_weights [n]; err [16, n]
 *                    (weight - recon, updated); delta [16, n] receives new err - old err (0 for
 *                    kept tiles).  These four are float32, or float64 when score_is_double.
 *   A tile switches to its first best-scoring proposal when
 *   best + abs_tol + rel_tol * |current| < current.
 *   counters[0] += accepted tiles, counters[1] += distinct payloads per tile (device words).
 */
int qsrtb_refine_select(const float* weight, int ldw, const float* target, int ldt, float* recon,
                        int ldq, int n, const float* cand, int ldc, int64_t cand_stride,
                        int variants, const int16_t* cand_states, int64_t cand_state_stride,
                        int16_t* states, const void* h_block, int ldh, const void* col_weights,
                        void* err, int lde, void* delta, int ldd, double abs_tol, double rel_tol,
                        int score_is_double, unsigned long long* counters, void* stream);

/* ---- P1: bit packer --------------------------------------------------------------------
 * Replaces pack_trellis (qsrt/exl3_encoder_backend.py:2361-2372, third-party
 * ext.pack_trellis) and its torch restatement pack_trellis_edges (qsrt/qsrt.py:861-883).
 * states [n_tiles, 256] int16 -> packed [n_tiles, 16*bits] int16.
 */
int qsrtb_pack_trellis(const int16_t* states, int64_t n_tiles, int bits, int16_t* packed,
                       void* stream);

/* ---- P2: mixed-rate record container and atom-major storage image ------------------------
 * Replaces pack_qsrt_trellis / unpack_qsrt_trellis_edges / unpack_qsrt_trellis_states
 * (qsrt/qsrt.py:1051-1172) and, with layout 1, pack_matrix_atoms + rotate_expert_atoms written
 * straight into a layer image (qsrt/qsrt_storage.py:194-231,347-362,441-462).
 *
 * states [tiles_k, tiles_n, 256] int16.  The rate axis (0 = K/rows, 1 = N/columns) is cut into
 * n_records records of `stripes` tiles; record r is stored with record_bits[r] (HOST array) bits
 * per edge.  layout 0: records back to back, tiles of a record in row-major tile order (the
 * reference's one-dimensional payload).  layout 1: atom (pair p, stripe s) = stripe s of record
 * 2p then stripe s of record 2p+1, stored at dst + ((p*stripes + s + rotation) mod n_atoms) *
 * atom_pitch_bytes; rotation and atom_pitch_bytes are ignored for layout 0.
 * open_paths (device int, may be NULL): incremented once per tile whose states are not the
 * closed cyclic walk of their own low bits (the reference raises ValueError for such input).
 */
int qsrtb_pack_records(const int16_t* states, int tiles_k, int tiles_n, int rate_axis,
                       int n_records, int stripes, const uint8_t* record_bits, int layout,
                       int rotation, int64_t atom_pitch_bytes, int16_t* dst, int64_t dst_bytes,
                       int* open_paths, void* stream);

/* Inverse of qsrtb_pack_records: 16-bit cyclic states and/or the stored K-bit edge symbols, each
 * [tiles_k, tiles_n, 256] int16 (either may be NULL).
 */
int qsrtb_unpack_records(const int16_t* src, int64_t src_bytes, int tiles_k, int tiles_n,
                         int rate_axis, int n_records, int stripes, const uint8_t* record_bits,
                         int layout, int rotation, int64_t atom_pitch_bytes, int16_t* out_states,
                         int16_t* out_edges, void* stream);

/* Moves complete packed tile paths between the record payload and the atom layout without
 * decoding a bit (pack_matrix_atoms / unpack_matrix_atoms, qsrt/qsrt_storage.py:194-289).
 * to_records = 0: records -> atoms; 1: atoms -> records.
 */
int qsrtb_records_atoms(int16_t* records, int64_t records_bytes, int tiles_k, int tiles_n,
                        int rate_axis, int n_records, int stripes, const uint8_t* record_bits,
                        int rotation, int64_t atom_pitch_bytes, int16_t* atoms, int64_t atoms_bytes,
                        int to_records, void* stream);

/* ---- C1: routed-error scoring ------------------------------------------------------------------
 * qsrtb_gated_activation: `gate_up` holds [rows, 2 * inter] pre-activations (gate columns first,
 * then up: one product of the routed rows against the stacked gate and up matrices); writes the
 * middle activation act(gate) * up - activation 0 = SiLU (F.silu(gate) * up,
 * qsrt/glm52_down_construction.py:159-260), 1 = the bounded gated activation of
 * qsrt/tp_simulator.py:82-93 - as TF32 head / tail planes for qsrtb_gemm3x_tc (hi / lo may both be
 * NULL) and / or as float32 rows (`middle` may be NULL).
 *
 * qsrtb_routed_row_sse: per row r, row_sse[r] = sum_j (candidate[r, j] - reference[r, j])^2 and
 * (optional) row_energy[r] = sum_j reference[r, j]^2, accumulated in float64: the row reductions of
 * functional_sse_by_request (qsrt/qsrt_candidates.py:621-654) and _defer_functional_row_sse
 * (qsrt/pack/qsrt_candidates.py:318-349).  Route weights and request grouping stay with the caller.
 */
int qsrtb_gated_activation(const float* gate_up, int64_t rows, int inter, int ld, int activation,
                           float* hi, float* lo, int ld_planes, float* middle, int ld_middle,
                           void* stream);
int qsrtb_routed_row_sse(const float* reference, const float* candidate, int64_t rows, int d,
                         int ld_reference, int ld_candidate, double* row_sse, double* row_energy,
                         void* stream);

/* ---- D1: decoder -------------------------------------------------------------------------
 * Replaces unpack_trellis_states + LUT decode (qsrt/qsrt.py:886-913,
 * qsrt/exl3_reference.py:34-83).  packed [n_tiles, 16*bits] -> states [n_tiles,256] int16
 * (may be NULL) and/or raw E4M3 bytes [n_tiles,256] (may be NULL), tile order unchanged.
 */
int qsrtb_unpack_decode(const int16_t* packed, int64_t n_tiles, int bits,
                        const uint8_t* lut_state, int16_t* out_states, uint8_t* out_e4m3,
                        void* stream);

/* States [tiles_k, tiles_n, 256] (tensor-core element order) -> decoded row-major float32
 * [tiles_k*16, tiles_n*16] in the regularised basis: LUT decode, inverse tile permutation and
 * tile placement of decode_regularized_weight (qsrt/exl3_reference.py:108-140) in one pass.
 */
int qsrtb_states_to_matrix(const int16_t* states, int tiles_k, int tiles_n,
                           const uint8_t* lut_state, float* out, int ld, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* QSRT_B200_H */
