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
 * current device (a persistent grid is used, so this saturates at one slice per resident CTA).
 */
int qsrtb_viterbi_scratch_bytes(int bits, int64_t n_tiles, size_t* bytes);

int qsrtb_quantize_tiles(const float* tiles,        /* [n_tiles, 256] tensor-core order   */
                         int64_t n_tiles,
                         const uint8_t* lut_state,   /* 65,536 bytes, state indexed        */
                         const uint8_t* lut_pm,      /* from qsrtb_lut_prepare             */
                         int bits,                   /* 2, 3 or 4                          */
                         int tailbite_context,       /* 1..128                             */
                         int variant,                /* 0 generic, 1 dedicated K2          */
                         float* out_tiles,           /* [n_tiles, 256] reconstruction      */
                         int16_t* out_states,        /* [n_tiles, 256] 16-bit states       */
                         void* scratch, size_t scratch_bytes,
                         void* stream);

/* ---- P1: bit packer --------------------------------------------------------------------
 * Replaces pack_trellis (qsrt/exl3_encoder_backend.py:2361-2372, third-party
 * ext.pack_trellis) and its torch restatement pack_trellis_edges (qsrt/qsrt.py:861-883).
 * states [n_tiles, 256] int16 -> packed [n_tiles, 16*bits] int16.
 */
int qsrtb_pack_trellis(const int16_t* states, int64_t n_tiles, int bits, int16_t* packed,
                       void* stream);

/* ---- D1: decoder -------------------------------------------------------------------------
 * Replaces unpack_trellis_states + LUT decode (qsrt/qsrt.py:886-913,
 * qsrt/exl3_reference.py:34-83).  packed [n_tiles, 16*bits] -> states [n_tiles,256] int16
 * (may be NULL) and/or raw E4M3 bytes [n_tiles,256] (may be NULL), tile order unchanged.
 */
int qsrtb_unpack_decode(const int16_t* packed, int64_t n_tiles, int bits,
                        const uint8_t* lut_state, int16_t* out_states, uint8_t* out_e4m3,
                        void* stream);

#ifdef __cplusplus
}
#endif
#endif /* QSRT_B200_H */
