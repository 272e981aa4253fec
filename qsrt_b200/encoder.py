"""BlockLDLQ trellis encoder: the ``quantizer_module`` entry points on B200.

Host-side mirror of the reference's encoder backend (``qsrt/exl3_encoder_backend.py``): the
same function names, argument meaning, ``quant_args`` / ``H_data`` mutation contract and error
behaviour, so a caller that holds the reference's ``quantizer_module`` can hold this module
instead.  The numerical work is done by the hand-written kernels of ``libqsrt_b200.so``:

* ``qsrtb_hadamard128``  - 128-point block Hadamards fused with the sign/scale vectors,
* ``qsrtb_col_sumsq``    - out-channel RMS,
* ``qsrtb_block_ldl_normalize`` - Cholesky factor -> block-LDL feedback factor,
* ``qsrtb_ldlq_quantize_rows``  - one 16-row LDLQ step (feedback add, tile gather, Viterbi,
  scatter) in a single launch,
* ``qsrtb_quantize_tiles`` / ``qsrtb_pack_trellis``.

* ``qsrtb_cholesky_blocked`` - the dense Cholesky inside ``block_ldl`` (panels in float32
  kernels, trailing updates on the tensor cores, a status word instead of an exception).

PyTorch supplies device memory, streams, the seeded sign draws (which must come from torch's
CUDA generator to match the reference, ``qsrt/rng.py:16-20``) and the plain feedback GEMMs
(cuBLAS, the very calls the reference issues, which keeps the float32 rounding of the feedback
identical).
"""

from __future__ import annotations

import ctypes
import math
import threading

import torch

from . import _lib
from . import linalg as _linalg
from . import tiles as _tiles
from .tiles import _stream_ptr, encode_tiles, prepared_table, quantize_tiles, traceback_scratch, K2_DEDICATED_MAX_LABEL

had_k, had_n = 128, 128
codebook_scale = 1.24371088
SIGMA_REG = 0.025

# The reference parks the damped Hessian (and, in quantize_qsrt, the factor) in host memory to
# save VRAM (exl3_encoder_backend.py:336-341, 2155-2157, 2829-2830): two 205 MB transfers through
# pageable memory per 7168-wide Hessian.  With 180 GB of HBM they can stay on the device; set
# this to False to reproduce the reference's placement exactly.
KEEP_HESSIAN_ON_DEVICE = True

# Feedback products of the BlockLDLQ recursion: True = this library's tensor-core products
# (tcgen05, float32 accuracy from three TF32 products; the result of a product does not depend on
# how matrices are batched, so stacked and one-by-one encodes agree bit for bit), False = the
# float32 library GEMMs the reference itself calls.  ``quant_args["ldlq_tensor_cores"]`` overrides
# it per call.
LDLQ_TENSOR_CORES = True

finalize_capture_H_mutex = threading.Lock()
_SHARED_INPUT_SCALES: dict = {}


# --------------------------------------------------------------------------------------
# kernel wrappers
# --------------------------------------------------------------------------------------

def _hadamard(x: torch.Tensor, axis: int, scale: torch.Tensor | None = None, *, per_col: bool = False,
              divide: bool = False, after: bool = False, row_sumsq: torch.Tensor | None = None) -> None:
    """In-place blockwise Hadamard of a [rows, cols] or stacked [B, rows, cols] float32 tensor."""

    if x.dtype != torch.float32 or not x.is_cuda:
        raise TypeError("Hadamard input must be a CUDA float32 tensor")
    if x.ndim == 2:
        batch, (rows, cols) = 1, x.shape
    elif x.ndim == 3:
        batch, rows, cols = x.shape
    else:
        raise ValueError("Hadamard input must be a matrix or a stack of matrices")
    if not x.is_contiguous():
        raise ValueError("Hadamard input must be contiguous")
    if scale is not None:
        scale = scale.reshape(batch, -1)
        if scale.dtype != torch.float32 or not scale.is_contiguous() or scale.device != x.device:
            raise TypeError("scale vector must be contiguous float32 on the matrix device")
        if scale.shape[1] != (cols if per_col else rows):
            raise ValueError("scale vector length does not match the scaled axis")
    with torch.cuda.device(x.device):
        _lib.check(
            _lib.lib().qsrtb_hadamard128(
                x.data_ptr(), batch, rows, cols, cols, rows * cols, axis,
                scale.data_ptr() if scale is not None else None,
                scale.shape[1] if scale is not None else 0,
                int(per_col), int(divide), int(after),
                row_sumsq.data_ptr() if row_sumsq is not None else None, rows,
                _stream_ptr(x.device),
            ),
            "qsrtb_hadamard128",
        )


def preapply_had_l(x: torch.Tensor, had_dim: int) -> torch.Tensor:
    """``had @ x`` per block of 128 rows (exl3_encoder_backend.py:275-282), out of place."""

    if had_dim != 128:
        raise ValueError("the B200 encoder implements the 128-point block Hadamard")
    out = x.to(torch.float32).contiguous().clone()
    _hadamard(out, 0)
    return out.to(x.dtype)


def preapply_had_r(x: torch.Tensor, had_dim: int) -> torch.Tensor:
    """``x @ had`` per block of 128 columns (exl3_encoder_backend.py:285-292), out of place."""

    if had_dim != 128:
        raise ValueError("the B200 encoder implements the 128-point block Hadamard")
    out = x.to(torch.float32).contiguous().clone()
    _hadamard(out, 1)
    return out.to(x.dtype)


def blockwise_preapply_had_l_(x: torch.Tensor, had_dim: int) -> None:
    assert x.shape[0] % had_dim == 0 and x.dtype == torch.float and had_dim == 128
    _hadamard(x, 0)


def blockwise_preapply_had_r_(x: torch.Tensor, had_dim: int) -> None:
    assert x.shape[1] % had_dim == 0 and x.dtype == torch.float and had_dim == 128
    _hadamard(x, 1)


def _col_sumsq(x: torch.Tensor) -> torch.Tensor:
    rows, cols = x.shape
    out = torch.empty(cols, dtype=torch.float32, device=x.device)
    chunks = max(1, (rows + 255) // 256)
    work = torch.empty(chunks * cols, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(
            _lib.lib().qsrtb_col_sumsq(
                x.data_ptr(), 1, rows, cols, cols, rows * cols, out.data_ptr(), cols,
                work.data_ptr(), work.numel() * 4, _stream_ptr(x.device),
            ),
            "qsrtb_col_sumsq",
        )
    return out


def seeded_normal(length: int, *, device: torch.device, seed: int | None) -> torch.Tensor:
    """Device-local seeded normal draw (qsrt/rng.py:8-20)."""

    generator = None
    if seed is not None:
        generator = torch.Generator(device=device)
        generator.manual_seed(seed)
    return torch.randn(length, device=device, generator=generator)


def _signs(length: int, device: torch.device, seed: int | None) -> torch.Tensor:
    return (seeded_normal(length, device=device, seed=seed).sign() + 1e-5).sign().to(torch.float)


def output_signs(n: int, device: torch.device, quant_args: dict) -> torch.Tensor:
    """exl3_encoder_backend.py:2562-2577."""

    return _signs(n, device, quant_args.get("sv_seed")).unsqueeze(0)


def make_shared_h(in_features: int, device: torch.device, hessian: torch.Tensor | None = None) -> dict:
    """Mutable Hessian wrapper consumed by the encoder (qsrt/ldlq.py:11-36)."""

    if hessian is None:
        hessian = torch.eye(in_features, dtype=torch.float32)
    if tuple(hessian.shape) != (in_features, in_features):
        raise ValueError(f"Hessian shape {tuple(hessian.shape)} does not match {in_features}")
    canonical = hessian.to(device=device, dtype=torch.float32, copy=True).contiguous()
    return {
        "H": canonical.clone(),
        "error_H": canonical,
        "first_key": f"h{in_features}",
        "count": 1,
        "finalized": False,
        "num_total": 1,
        "inf_nan": torch.zeros(2, dtype=torch.long, device=device),
        "device": device,
    }


# --------------------------------------------------------------------------------------
# H2: Hessian damping, congruence and block LDL
# --------------------------------------------------------------------------------------

def block_ldl(H: torch.Tensor, b: int, quant_args: dict, verbose: bool):
    """Block LDL of a damped Hessian (exl3_encoder_backend.py:323-393).

    Returns ``(L, H_copy)``: ``L`` (unit block-lower: identity diagonal blocks, zeros above them)
    overwrites H's device storage, ``H_copy`` is the matrix that was factored, extra damping
    included.  The dense Cholesky runs on the device in this library's kernels
    (``linalg.cholesky_``); a matrix that is not positive definite comes back as a status word, not
    an exception, and is retried up to ten times with ``2 * sigma_reg * mean(diag)`` of extra
    damping before ``LinAlgError`` is raised, as in the reference."""

    if b != 16:
        raise ValueError("the B200 encoder factors in 16x16 blocks")
    n = H.shape[0]
    assert n % b == 0
    H_copy = H.clone() if KEEP_HESSIAN_ON_DEVICE else H.cpu()
    retries = 0
    while True:
        info = _linalg.cholesky_(H)
        if info == 0:
            break
        retries += 1
        if retries > 10:
            print(" ## Cholesky decomp. failed, number of retries exceeded")
            raise torch.linalg.LinAlgError(
                f"linalg.cholesky: the input is not positive-definite (leading minor {info})"
            )
        print(f" !! Cholesky decomp. failed, increasing diagonal damping, attempt {retries}/10")
        H.copy_(H_copy)   # the failed factorisation left H undefined
        H.diagonal().add_(2.0 * quant_args.get("sigma_reg", SIGMA_REG) * H.diagonal().mean())
        H_copy.diagonal().copy_(H.diagonal())
    with torch.cuda.device(H.device):
        _lib.check(
            _lib.lib().qsrtb_block_ldl_normalize(H.data_ptr(), n, H.stride(0), _stream_ptr(H.device)),
            "qsrtb_block_ldl_normalize",
        )
    H.diagonal().fill_(1.0)   # identity diagonal blocks (exl3_encoder_backend.py:387-391)
    return H, H_copy


def _prepare_capture_H(H_data: dict, quant_args: dict, verbose: bool):
    """Normalise and damp (exl3_encoder_backend.py:2077-2122); draws the input signs."""

    H = H_data["H"]
    count = H_data["count"]
    if count == 0:
        q_fallback = True
        diag_mean = 0.0
    else:
        H /= count
        diag_mean = torch.diag(H).mean()
        q_fallback = diag_mean.item() < 1e-20
    H.diagonal().add_(quant_args.get("sigma_reg", SIGMA_REG) * diag_mean)
    diag = H.diagonal().clone()
    su = _signs(H.shape[0], H.device, quant_args.get("seed")).unsqueeze(1)
    H_data["su"] = su
    H_data["diag"] = diag
    H_data["q_fallback"] = q_fallback
    return q_fallback, H, su, diag


def _factor_capture_H(H_data: dict, H: torch.Tensor, su: torch.Tensor, quant_args: dict, verbose: bool):
    """Decoder-input congruence and block factorisation (exl3_encoder_backend.py:2125-2160)."""

    if su.shape != (H.shape[0], 1) or su.dtype != torch.float:
        raise ValueError("input conditioning must be float32 [input, 1]")
    if su.device != H.device:
        su = su.to(H.device)
    flat = su.reshape(-1).contiguous()
    _hadamard(H, 1, flat, per_col=True)    # H *= su.T ; had_r
    _hadamard(H, 0, flat, per_col=False)   # H *= su   ; had_l
    q_fallback = bool(H_data["q_fallback"])
    if q_fallback:
        L = None
    else:
        L, H = block_ldl(H, 16, quant_args, verbose)
        L.diagonal().zero_()   # exl3_encoder_backend.py:2152-2153
    H_data["L"] = L
    if not KEEP_HESSIAN_ON_DEVICE:
        H = H.cpu()
    H_data["H"] = H
    H_data["su"] = su
    H_data["finalized"] = True
    return q_fallback, H, L, su, H_data["diag"]


def prepare_capture_H_for_conditioning(H_data: dict, quant_args: dict, verbose: bool):
    """First half of the two-stage preparation (exl3_encoder_backend.py:2163-2182)."""

    with finalize_capture_H_mutex:
        if H_data["H"].is_meta:
            raise ValueError("conditioned QSRT requires a materialized dense Hessian")
        if "H_swap_device" in H_data:
            H_data["H"] = H_data["H"].to(H_data["H_swap_device"])
            del H_data["H_swap_device"]
        if H_data.get("_conditioning_pending"):
            raise ValueError("conditioned Hessian preparation is already pending")
        if H_data["finalized"]:
            raise ValueError("conditioned QSRT Hessian was already finalized")
        q_fallback, H, su, diag = _prepare_capture_H(H_data, quant_args, verbose)
        H_data["_conditioning_pending"] = True
        return q_fallback, H, su, diag


def finalize_capture_H_with_conditioning(H_data: dict, su: torch.Tensor, quant_args: dict, verbose: bool):
    """Second half: factor with regularize's complete ``su`` (exl3_encoder_backend.py:2185-2198)."""

    with finalize_capture_H_mutex:
        if not H_data.pop("_conditioning_pending", False):
            raise ValueError("conditioned Hessian preparation was not started")
        return _factor_capture_H(H_data, H_data["H"], su, quant_args, verbose)


def finalize_capture_H(H_data: dict, quant_args: dict, verbose: bool):
    """exl3_encoder_backend.py:2201-2243."""

    with finalize_capture_H_mutex:
        if H_data["H"].is_meta:
            H_data["L"] = None
            H_data["finalized"] = True
            H_data["diag"] = None
            H_data["q_fallback"] = True
            su = _signs(H_data["H"].shape[0], torch.device(H_data["device"]), quant_args.get("seed")).unsqueeze(1)
            H_data["su"] = su
            return True, None, None, su, None
        if "H_swap_device" in H_data:
            H_data["H"] = H_data["H"].to(H_data["H_swap_device"])
            del H_data["H_swap_device"]
        H = H_data["H"]
        if H_data["finalized"]:
            return H_data["q_fallback"], H, H_data["L"], H_data["su"], H_data["diag"]
        if H_data.get("_conditioning_pending"):
            raise ValueError("cannot use ordinary finalization during QSRT conditioning")
        q_fallback, H, su, _ = _prepare_capture_H(H_data, quant_args, verbose)
        return _factor_capture_H(H_data, H, su, quant_args, verbose)


# --------------------------------------------------------------------------------------
# X1 / S1: tile order and global-scale search
# --------------------------------------------------------------------------------------

_perm_cache: dict[str, tuple[torch.Tensor, torch.Tensor]] = {}


def tensor_core_perm(device) -> torch.Tensor:
    """Row-major 16x16 tile -> tensor-core element order (exl3_encoder_backend.py:35-57)."""

    key = str(device)
    if key not in _perm_cache:
        perm = [0] * 256
        for lane in range(32):
            r0 = (lane % 4) * 2
            c0 = lane // 4
            for j, row in enumerate((r0, r0 + 1, r0 + 8, r0 + 9)):
                perm[lane * 8 + j] = row * 16 + c0
                perm[lane * 8 + 4 + j] = row * 16 + c0 + 8
        p = torch.tensor(perm, dtype=torch.int, device=device)
        _perm_cache[key] = (p, torch.argsort(p))
    return _perm_cache[key][0]


def tensor_core_perm_i(device) -> torch.Tensor:
    tensor_core_perm(device)
    return _perm_cache[str(device)][1]


def sample_scale_tiles(weight_r: torch.Tensor, width: int = 3) -> torch.Tensor:
    """Tiles sampled for the global-scale search (exl3_encoder_backend.py:2383-2410): a
    wrapped diagonal of the given width plus the tiles of highest and lowest RMS."""

    device = weight_r.device
    tiles_k = weight_r.shape[0] // 16
    tiles_n = weight_r.shape[1] // 16
    w4 = weight_r.view(tiles_k, 16, tiles_n, 16)
    diag_len = max(tiles_k, tiles_n)
    ii = torch.arange(diag_len, device=device).repeat_interleave(width)
    ww = torch.arange(width, device=device).repeat(diag_len)
    kk = ii % tiles_k
    nn = (ii + ww) % tiles_n
    num_x = max(8, (diag_len * width) // 16)
    tile_ms = w4.square().mean(dim=(1, 3)).flatten()
    num_x = min(num_x, (tile_ms.shape[0] + 1) // 2)
    hi = torch.topk(tile_ms, num_x).indices
    lo = torch.topk(tile_ms, num_x, largest=False).indices
    xk = torch.cat((hi, lo)) // tiles_n
    xn = torch.cat((hi, lo)) % tiles_n
    tiles = w4[torch.cat((kk, xk)), :, torch.cat((nn, xn)), :].reshape(-1, 256)
    return tiles[:, tensor_core_perm(device)].contiguous()


def g_scale_search_batch(samples: list[torch.Tensor], quant_args: dict) -> list[tuple[float, torch.Tensor]]:
    """Coarse grid, fine grid, parabolic refinement (exl3_encoder_backend.py:2413-2476).

    Every (tensor, scale) evaluation of a stage goes through as few tile-encoder launches as
    the 65,536-tile batch limit allows; the host synchronises twice per group.
    """

    n_t = len(samples)
    device = samples[0].device
    max_tiles = 65536

    def eval_pairs(pairs, tile_sets):
        out = torch.empty(len(pairs), dtype=torch.float, device=device)
        i = 0
        while i < len(pairs):
            j, tot = i, 0
            while j < len(pairs) and tot + tile_sets[pairs[j][0]].shape[0] <= max_tiles:
                tot += tile_sets[pairs[j][0]].shape[0]
                j += 1
            j = max(j, i + 1)
            batch = torch.cat([tile_sets[t] * s for t, s in pairs[i:j]])
            quant_w, _ = quantize_tiles(batch, quant_args)
            offset = 0
            for p, (t, s) in enumerate(pairs[i:j]):
                cnt = tile_sets[t].shape[0]
                out[i + p] = (quant_w[offset:offset + cnt] / s - tile_sets[t]).square().mean()
                offset += cnt
            i = j
        return out

    coarse = [0.1 + 0.2 * i for i in range(10)]
    subs = [s[::3] for s in samples]
    pairs1 = [(t, s) for t in range(n_t) for s in coarse]
    mse1 = eval_pairs(pairs1, subs).view(n_t, len(coarse))
    centers = [coarse[c] for c in mse1.argmin(dim=1).tolist()]
    step = 0.075
    fine = [[c + step * (i - 2) for i in range(5)] for c in centers]
    pairs2 = [(t, s) for t in range(n_t) for s in fine[t]]
    mse2 = eval_pairs(pairs2, samples).view(n_t, 5)
    mse2_h = mse2.tolist()
    results = []
    for t in range(n_t):
        best = min(range(5), key=lambda i: mse2_h[t][i])
        if 0 < best < 4:
            y0, y1, y2 = mse2_h[t][best - 1], mse2_h[t][best], mse2_h[t][best + 1]
            denom = y0 - 2.0 * y1 + y2
            offset = 0.5 * (y0 - y2) / denom if denom > 0 else 0.0
            offset = max(-0.5, min(0.5, offset))
        else:
            offset = 0.0
        best_scale = max(fine[t][best] + offset * step, 0.01)
        results.append((best_scale, mse2[t, best]))
    return results


def g_scale_gss(weight_r: torch.Tensor, verbose: bool, quant_args: dict, width: int = 3, pb=None):
    """exl3_encoder_backend.py:2479-2505."""

    tiles = sample_scale_tiles(weight_r, width)
    best_scale, best_mse = g_scale_search_batch([tiles], quant_args)[0]
    if verbose:
        print(f"     - scale search: min = {best_scale:.6f}, mse: {best_mse.item():.6f}")
    return best_scale, best_mse


# --------------------------------------------------------------------------------------
# R1: regularisation
# --------------------------------------------------------------------------------------

def apply_g_scale(weight, su, sv, g_scale: float, *, into_sv: bool = False):
    """exl3_encoder_backend.py:2727-2751."""

    if not math.isfinite(float(g_scale)) or float(g_scale) <= 0.0:
        raise ValueError("g_scale must be positive and finite")
    weight *= g_scale
    if into_sv:
        sv /= g_scale
    else:
        su /= g_scale
    return weight, su, sv


def relocate_g_scale_to_sv(su: torch.Tensor, sv: torch.Tensor, g_scale: float):
    """exl3_encoder_backend.py:2711-2724."""

    if not math.isfinite(float(g_scale)) or float(g_scale) <= 0.0:
        raise ValueError("g_scale must be positive and finite")
    return su * g_scale, sv / g_scale


def prime_shared_input_scales(weight: torch.Tensor, quant_args: dict, H_diag: torch.Tensor | None = None) -> torch.Tensor:
    """Seed the shared input-scale profile of ``quant_args["shared_input_scales_key"]`` from
    ``weight`` ([in, out], left untouched) and return it.

    In shared-su mode the first tensor encoded with a key defines the per-input-channel scale
    profile of every later tensor with that key (exl3_encoder_backend.py:2664-2672); in a canonical
    full-layer encode that tensor is expert zero's.  A worker that holds only a shard of the
    experts obtains the same profile by running expert zero's matrices through this function
    before its first encode.  The reference's split workers repeat expert zero's whole encode for
    that and discard the payload (scripts/pack_qsrt_candidates.py:1413-1425); the profile only
    depends on the first half of ``regularize``, which is all that runs here."""

    key = quant_args.get("shared_input_scales_key")
    if key is None:
        raise ValueError("quant_args carries no shared_input_scales_key")
    work = weight.to(torch.float32).contiguous().clone()
    scratch_args = dict(quant_args)
    su = torch.ones((work.shape[0], 1), dtype=torch.float32, device=work.device)
    sv = output_signs(work.shape[1], work.device, scratch_args)
    _regularize_head(work, su, sv, scratch_args, False, H_diag, False)
    return _SHARED_INPUT_SCALES[key]


def clear_shared_input_scales() -> None:
    """Forget every shared input-scale profile (between layers, or between tests)."""

    _SHARED_INPUT_SCALES.clear()


def regularize(weight: torch.Tensor, su: torch.Tensor, sv: torch.Tensor, quant_args: dict, verbose: bool,
               H_diag: torch.Tensor | None, pb, skip_g_scale: bool = False, q_fallback: bool = False):
    """Sign flips, channel scales, both Hadamards and the global scale
    (exl3_encoder_backend.py:2580-2708).  ``weight`` [in, out] is transformed in place by two
    fused kernels (divide-by-sv + output Hadamard + row sums; divide-by-su + input Hadamard)."""

    apply_out_scales, su, sv = _regularize_head(weight, su, sv, quant_args, verbose, H_diag, q_fallback)

    # weight /= su ; input Hadamard
    _hadamard(weight, 0, su.reshape(-1).contiguous(), per_col=False, divide=True)

    if not skip_g_scale:
        override = quant_args.get("g_scale_override")
        if override is None:
            g_scale, mse_scale = g_scale_gss(weight, False, quant_args, pb=pb)
        else:
            if isinstance(override, bool) or not isinstance(override, (int, float)):
                raise TypeError("g_scale_override must be a real number")
            g_scale = float(override)
            if not math.isfinite(g_scale) or g_scale <= 0.0:
                raise ValueError("g_scale_override must be positive and finite")
            mse_scale = torch.tensor(float("nan"), device=weight.device)
    else:
        g_scale = 1.0
    weight, su, sv = apply_g_scale(weight, su, sv, g_scale, into_sv=bool(quant_args.get("g_scale_into_sv")))
    if verbose:
        print(f"     - su/sv std: {su.std().item():.6f}   {sv.std().item():.6f}")
        print(f"     - global scale: {g_scale:.6f}")
        print(f"     - apply_out_scales: {str(apply_out_scales)}")
    return apply_out_scales, weight, g_scale, su, sv


def _regularize_head(weight, su, sv, quant_args, verbose, H_diag, q_fallback):
    """First half of ``regularize``: output scales and signs, output Hadamard, input-channel scale
    profile (shared or own) folded into ``su``.  Returns ``(apply_out_scales, su, sv)``."""

    force_out_scales = quant_args["apply_out_scales"]
    if not q_fallback and H_diag is not None:
        diag = H_diag.sqrt()
        diag, _ = torch.sort(diag, descending=True)
        cutoff = diag.shape[0] // 50
        skew_factor = diag[:cutoff].sum() / diag.sum()
        if verbose:
            print(f"     - input state skew: {skew_factor.item():.6f}")
        if force_out_scales is None:
            apply_out_scales = skew_factor.item() < 0.15
        else:
            apply_out_scales = force_out_scales
    else:
        apply_out_scales = True if force_out_scales is None else force_out_scales
    if q_fallback:
        apply_out_scales = force_out_scales

    k, n = weight.shape
    out_channel_scales = (_col_sumsq(weight) / k).sqrt().unsqueeze(0)
    mean = out_channel_scales.mean().item()
    if mean > 1e-30:
        out_channel_scales /= mean
        quant_args["zeros"] = False
    else:
        quant_args["zeros"] = True
        if force_out_scales is not None:
            apply_out_scales = True
    zero_out_scales = out_channel_scales.abs() < 1e-30
    if apply_out_scales:
        out_channel_scales[zero_out_scales] = 0.1
        sv = (sv * out_channel_scales + 1e-10).float()

    # weight /= sv ; output Hadamard ; per-input-channel sums of squares of the result
    row_sumsq = torch.empty(k, dtype=torch.float32, device=weight.device)
    _hadamard(weight, 1, sv.reshape(-1).contiguous(), per_col=True, divide=True, row_sumsq=row_sumsq)
    sv[zero_out_scales] = 0.0

    in_channel_scales = (row_sumsq / n).sqrt().unsqueeze(1)
    in_channel_scales[in_channel_scales.abs() < 1e-30] = 0.1
    shared_key = quant_args.get("shared_input_scales_key")
    if shared_key is not None:
        in_channel_scales = _SHARED_INPUT_SCALES.setdefault(shared_key, in_channel_scales)
    su = (su * in_channel_scales / (-codebook_scale) + 1e-10).float()
    return apply_out_scales, su, sv


# --------------------------------------------------------------------------------------
# L1: BlockLDLQ feedback loop
# --------------------------------------------------------------------------------------

def _ldlq_feedback_multiplier(quant_args: dict) -> float:
    value = quant_args.get("ldlq_feedback_multiplier", 1.0)
    if (
        isinstance(value, bool)
        or not isinstance(value, (int, float))
        or not math.isfinite(float(value))
        or not 0.0 <= float(value) <= 1.0
    ):
        raise ValueError("ldlq_feedback_multiplier must be a real number in [0, 1]")
    return float(value)


def _codebook_for(quant_args: dict, bits: int) -> torch.Tensor:
    codebook = quant_args.get("sqg_e4m3_lut")
    by_bits = quant_args.get("sqg_e4m3_luts_by_bits")
    if codebook is None and by_bits is not None:
        if bits not in by_bits:
            raise ValueError(f"missing rate-specific SQG K{bits} LUT")
        codebook = by_bits[bits]
    if codebook is None:
        raise ValueError("the B200 encoder needs a QSRT table (sqg_e4m3_lut or sqg_e4m3_luts_by_bits)")
    return codebook


def _quantize_rows(w_rows, comp_rows, multiplier, wq_rows, err_rows, states_row, quant_args, bits,
                   *, batch, n, ld, w_stride, comp_ld, comp_stride, state_stride, tile_map=None):
    """One launch of ``qsrtb_ldlq_quantize_rows`` on views that start at the step's first row."""

    device = w_rows.device
    lut, lut_pm, abs_max = prepared_table(_codebook_for(quant_args, bits), bits, device)
    dedicated = bits == 2 and abs_max == abs_max and 0.0 < abs_max <= K2_DEDICATED_MAX_LABEL
    variant, cost_rows = _tiles.search_variant(dedicated, quant_args)
    scratch = traceback_scratch(device, bits, cost_rows=cost_rows)
    visited = tile_map.numel() if tile_map is not None else n // 16
    with torch.cuda.device(device), _tiles.timed_search(device, batch * visited, bits):
        _lib.check(
            _lib.lib().qsrtb_ldlq_quantize_rows(
                w_rows.data_ptr(), comp_rows.data_ptr() if comp_rows is not None else None,
                float(multiplier), batch, n, ld, comp_ld, w_stride, comp_stride,
                lut.data_ptr(), lut_pm.data_ptr(), bits, int(quant_args.get("tailbite_context", 128)),
                variant, wq_rows.data_ptr(),
                err_rows.data_ptr() if err_rows is not None else None,
                states_row.data_ptr(), state_stride,
                tile_map.data_ptr() if tile_map is not None else None,
                tile_map.numel() if tile_map is not None else 0,
                scratch.data_ptr(), scratch.numel(),
                _stream_ptr(device),
            ),
            "qsrtb_ldlq_quantize_rows",
        )


def mixed_rate_spec(size_k: int, size_n: int, quant_args: dict):
    """Validate a per-tile rate map (exl3_encoder_backend.py:737-772)."""

    rate_axis = quant_args.get("mixed_rate_axis")
    if rate_axis not in ("k", "n", "tile"):
        raise ValueError("mixed_rate_axis must be 'k', 'n', or 'tile'")
    if size_k % 16 or size_n % 16:
        raise ValueError("mixed-rate LDLQ input must be 16x16 tile aligned")
    raw_tile_bits = quant_args.get("mixed_tile_bits")
    if raw_tile_bits is None:
        raise ValueError("mixed_tile_bits is required for mixed-rate LDLQ")
    tile_bits = tuple(raw_tile_bits)
    if rate_axis == "tile":
        rate_tiles = (size_k // 16) * (size_n // 16)
    else:
        rate_tiles = size_k // 16 if rate_axis == "k" else size_n // 16
    if len(tile_bits) != rate_tiles:
        raise ValueError(f"mixed_tile_bits has {len(tile_bits)} entries; expected {rate_tiles}")
    if any(isinstance(bits, bool) or not isinstance(bits, int) or bits not in (1, 2, 3, 4) for bits in tile_bits):
        raise ValueError("mixed-rate LDLQ supports only integer K1 through K4")
    return rate_axis, tile_bits


def _uniform_plan(bits: int):
    return lambda row_tile: [(bits, None)]


def _mixed_plan(size_k: int, size_n: int, quant_args: dict, device):
    """Per row of tiles: [(bits, device list of column tiles or None for all)]."""

    rate_axis, tile_bits = mixed_rate_spec(size_k, size_n, quant_args)
    if quant_args.get("mixed_tile_codebook_ids") is not None or quant_args.get("sqg_e4m3_lut_banks_by_bits") is not None:
        raise NotImplementedError("per-tile codebook banks are a research hook outside the B200 hot path")
    if 1 in tile_bits:
        raise NotImplementedError("K1 tiles are outside the B200 tile encoder (K2, K3, K4)")
    tiles_n = size_n // 16

    def positions(row_bits):
        return [
            (bits, torch.tensor([i for i, b in enumerate(row_bits) if b == bits], dtype=torch.int32, device=device))
            for bits in sorted(set(row_bits))
        ]

    if rate_axis == "k":
        return lambda row_tile: [(tile_bits[row_tile], None)]
    if rate_axis == "n":
        fixed = positions(tile_bits)
        if len(fixed) == 1:
            fixed = [(fixed[0][0], None)]
        return lambda row_tile: fixed
    cache: dict[tuple, list] = {}

    def per_tile(row_tile):
        row_bits = tuple(tile_bits[row_tile * tiles_n:(row_tile + 1) * tiles_n])
        if row_bits not in cache:
            cache[row_bits] = positions(row_bits)
        return cache[row_bits]

    return per_tile


def _ldlq_steps(weights: torch.Tensor, Ls: torch.Tensor, quant_args: dict, plan, out: dict):
    """Generator form of the reference's reverse block recursion
    (exl3_encoder_backend.py:470-539, 2020-2068): spans of ``buf_size_k`` rows from the bottom
    up, 16-row blocks inside a span, the same two GEMM calls, and one fused encode launch per
    rate present in the 16-row step.  Yields after every 16-row step (nothing synchronises), so
    several recursions can be interleaved on different streams; ``out`` receives
    ``weight_q`` and ``encoded``."""

    assert weights.ndim == 3 and Ls.ndim == 3
    batch, size_k, size_n = weights.shape
    assert size_k % 16 == 0 and size_n % 128 == 0
    device = weights.device
    multiplier = _ldlq_feedback_multiplier(quant_args)
    buf_size_k = max(quant_args.get("buf_size_k", 128), 16)
    assert buf_size_k % 16 == 0 and size_k % buf_size_k == 0
    tiles_k, tiles_n = size_k // 16, size_n // 16
    tf32 = bool(quant_args.get("ldlq_tf32", False))

    prod_cache = torch.zeros((batch, size_k, size_n), dtype=torch.float, device=device)
    weight_q = torch.zeros((batch, size_k, size_n), dtype=torch.float, device=device)
    err = torch.zeros((batch, size_k, size_n), dtype=torch.float, device=device)
    encoded = torch.zeros((batch, tiles_k, tiles_n, 256), dtype=torch.short, device=device)
    out["weight_q"], out["encoded"] = weight_q, encoded

    tensor_cores = bool(quant_args.get("ldlq_tensor_cores", LDLQ_TENSOR_CORES))
    if tensor_cores and (size_k % 4 or buf_size_k % 4):
        raise ValueError("the tensor-core feedback products need row counts that are multiples of 4")
    if tensor_cores:
        # Operands of the feedback products, both stored with the contraction index (a row of the
        # current span) contiguous: the transposed factor, split once, and the transposed error
        # rows of the span, split after every 16-row step.  A product only ever contracts over rows
        # that are already encoded, so neither the diagonal blocks of the factor nor error rows
        # left over from the previous span are read.
        factor_t = _linalg.split_tf32(Ls, transpose=True)                       # [B, column, row]
        err_t = _linalg.Planes(torch.zeros((batch, size_n, buf_size_k), dtype=torch.float, device=device),
                               torch.zeros((batch, size_n, buf_size_k), dtype=torch.float, device=device))

        def view(planes, rows, cols):
            return _linalg.Planes(planes.hi[:, rows, cols], planes.lo[:, rows, cols])

    def gemm(target, a, b):
        allow = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = tf32
        try:
            target.baddbmm_(a, b)
        finally:
            torch.backends.cuda.matmul.allow_tf32 = allow

    for j in range(size_k, 0, -buf_size_k):
        i = j - buf_size_k
        for bj in range(buf_size_k, 0, -16):
            bi = bj - 16
            comp = prod_cache[:, i + bi:i + bj]
            if bj < buf_size_k:
                # compensation from the rows already encoded inside this span
                if tensor_cores:
                    _linalg.gemm_nt(view(err_t, slice(None), slice(bj, buf_size_k)),
                                    view(factor_t, slice(i + bi, i + bj), slice(i + bj, j)), comp,
                                    beta=1.0, transposed_out=True)
                else:
                    gemm(comp, Ls[:, i + bj:j, i + bi:i + bj].transpose(1, 2), err[:, i + bj:j])
            for bits, tile_map in plan((i + bi) // 16):
                _quantize_rows(
                    weights[:, i + bi:], comp, multiplier, weight_q[:, i + bi:], err[:, i + bi:],
                    encoded[:, (i + bi) // 16], quant_args, bits,
                    batch=batch, n=size_n, ld=size_n, w_stride=size_k * size_n,
                    comp_ld=size_n, comp_stride=size_k * size_n,
                    state_stride=tiles_k * tiles_n * 256, tile_map=tile_map,
                )
            if tensor_cores:
                _linalg.split_tf32(err[:, i + bi:i + bj], transpose=True,
                                   out=view(err_t, slice(None), slice(bi, bj)))
            if bj == 16 and i > 0:
                # cache the span's error for every row block still to be encoded
                if tensor_cores:
                    _linalg.gemm_nt(view(factor_t, slice(0, i), slice(i, j)), err_t, prod_cache[:, :i], beta=1.0)
                else:
                    gemm(prod_cache[:, :i], Ls[:, i:j, :i].transpose(1, 2), err[:, i:j])
            yield
    if tensor_cores:
        _linalg.check_status(device)


def _ldlq_core(weights: torch.Tensor, Ls: torch.Tensor, quant_args: dict, plan, pb=None):
    out: dict = {}
    for step, _ in enumerate(_ldlq_steps(weights, Ls, quant_args, plan, out), start=1):
        if pb:
            pb.update(step)
    return out["weight_q"], out["encoded"]


_side_stream_cache: dict[str, list] = {}


def _side_streams(device: torch.device, count: int) -> list:
    """Long-lived side streams (their survivor scratch and cuBLAS workspaces are created once)."""

    pool = _side_stream_cache.setdefault(str(device), [])
    while len(pool) < count:
        pool.append(torch.cuda.Stream(device=device))
    return pool[:count]


def ldlq_concurrent(jobs: list[tuple], max_streams: int = 4):
    """Run several independent stacked LDLQ recursions at once, each on its own stream.

    A 16-row step offers only ``batch * n / 16`` tiles; one persistent search launch then leaves
    part of the GPU idle in its last wave.  Interleaving independent recursions (for example the
    gate/up stack and the down stack of an expert batch) lets the CTAs of one launch fill the
    tail of the other.  Returns ``[(weight_q, encoded), ...]`` in job order; on return the
    current stream has been made to wait for all of them."""

    if not jobs:
        return []
    if len(jobs) > max_streams:
        done: list = []
        for begin in range(0, len(jobs), max_streams):
            done.extend(ldlq_concurrent(jobs[begin:begin + max_streams], max_streams))
        return done
    device = jobs[0][0].device
    current = torch.cuda.current_stream(device)
    ready = torch.cuda.Event()
    ready.record(current)
    streams = _side_streams(device, len(jobs)) if len(jobs) > 1 else [current]
    outs: list[dict] = [{} for _ in jobs]
    gens = []
    for job, stream, out in zip(jobs, streams, outs):
        weights, Ls, quant_args = job[:3]
        plan = job[3] if len(job) > 3 else _uniform_plan(int(quant_args["K"]))
        if stream is not current:
            stream.wait_event(ready)
        with torch.cuda.stream(stream):
            gens.append(_ldlq_steps(weights, Ls, quant_args, plan, out))
    alive = list(range(len(jobs)))
    # advance the longer recursions proportionally more often so that all finish together
    lengths = [job[0].shape[1] // 16 for job in jobs]
    progress = [0] * len(jobs)
    while alive:
        k = min(alive, key=lambda idx: (progress[idx] / lengths[idx], idx))
        with torch.cuda.stream(streams[k]):
            try:
                next(gens[k])
                progress[k] += 1
            except StopIteration:
                alive.remove(k)
    for stream, job, out in zip(streams, jobs, outs):
        weights, Ls = job[0], job[1]
        if stream is not current:
            done = torch.cuda.Event()
            done.record(stream)
            current.wait_event(done)
            for t in (weights, Ls):
                t.record_stream(stream)      # allocated on the caller's stream, read on the side stream
            for t in (out["weight_q"], out["encoded"]):
                t.record_stream(current)     # allocated on the side stream, consumed by the caller
    return [(o["weight_q"], o["encoded"]) for o in outs]


def ldlq_batched(weights: torch.Tensor, Ls: torch.Tensor, quant_args: dict, pb=None):
    """LDLQ over a stack of same-shape tensors with per-tensor L
    (exl3_encoder_backend.py:1980-2071): every 16-row step encodes all tensors' tiles in one
    launch.  Returns (weight_q [B, k, n], encoded [B, k/16, n/16, 256])."""

    return _ldlq_core(weights, Ls, quant_args, _uniform_plan(int(quant_args["K"])), pb)


def ldlq_mixed(weight: torch.Tensor, L: torch.Tensor, quant_args: dict, pb=None):
    """Dense-H LDLQ with the rate chosen per tile on one matrix axis
    (exl3_encoder_backend.py:898-1082).  One traversal; a step launches once per rate present."""

    size_k, size_n = weight.shape
    plan = _mixed_plan(size_k, size_n, quant_args, weight.device)
    weight_q, encoded = _ldlq_core(weight.unsqueeze(0), L.unsqueeze(0), quant_args, plan, pb)
    return weight_q[0], encoded[0]


def ldlq(weight: torch.Tensor, L: torch.Tensor, quant_args: dict, pb=None):
    """exl3_encoder_backend.py:420-539: returns (weight_q [k, n], encoded [k/16, n/16, 256])."""

    weight_q, encoded = ldlq_batched(weight.unsqueeze(0), L.unsqueeze(0), quant_args, pb)
    return weight_q[0], encoded[0]


def fallback_quant(weight: torch.Tensor, device, quant_args: dict, pb=None):
    """Plain tile-by-tile encode without feedback, used when the Hessian is unusable
    (exl3_encoder_backend.py:1833-1948).  Returns (weight_q, encoded, mse)."""

    size_k, size_n = weight.shape
    zero = torch.zeros((1, 1, 1), dtype=torch.float, device=weight.device)
    args = dict(quant_args)
    args["ldlq_feedback_multiplier"] = 0.0
    bits = int(quant_args["K"])
    weight_q = torch.zeros_like(weight)
    encoded = torch.zeros((size_k // 16, size_n // 16, 256), dtype=torch.short, device=weight.device)
    for row in range(0, size_k, 16):
        _quantize_rows(
            weight[row:], None, 0.0, weight_q[row:], None, encoded[row // 16], args, bits,
            batch=1, n=size_n, ld=size_n, w_stride=0, comp_ld=size_n, comp_stride=0, state_stride=0,
        )
    del zero
    # mean squared error of the regularised weight, summed in float64 (:1923-1946)
    mse = (torch.sum((weight.float() - weight_q.float()).pow(2), dtype=torch.float64) / weight.numel()).item()
    return weight_q, encoded, mse


def block_trace_parts(A, B, block_size=1024):
    """Column-block terms of trace(A.T @ B @ A) (exl3_encoder_backend.py:1951-1964)."""

    return torch.stack(
        [
            torch.einsum(
                "ik,ij,jk->",
                A,
                B[:, j_start:min(j_start + block_size, B.shape[1])],
                A[j_start:min(j_start + block_size, B.shape[1]), :],
            )
            for j_start in range(0, B.shape[1], block_size)
        ]
    )


def block_trace(A, B, block_size=1024):
    """exl3_encoder_backend.py:1967-1977."""

    total = 0.0
    for partial in block_trace_parts(A, B, block_size).cpu():
        total += partial.item()
    return total


class HessianTrace:
    """``trace(A.T @ H @ A)`` for several ``A`` against one symmetric ``H`` (the proxy error's
    numerator and denominator, exl3_encoder_backend.py:2994-3025): ``H @ A`` is one tensor-core
    product per ``A`` (``H`` is split into its operand planes once, its rows being its columns),
    the contraction with ``A`` a float64 sum.  Returns 0-d float64 device tensors, so that a
    caller can collect many traces before it synchronises."""

    def __init__(self, H: torch.Tensor) -> None:
        if H.ndim != 2 or H.shape[0] != H.shape[1] or not H.is_cuda or H.shape[0] % 4:
            raise ValueError("the trace needs a square CUDA matrix whose size is a multiple of 4")
        self.planes = _linalg.split_tf32(H.float().contiguous())

    def __call__(self, A: torch.Tensor) -> torch.Tensor:
        A = A.float()
        product = torch.empty_like(A, memory_format=torch.contiguous_format)
        _linalg.gemm_nt(self.planes, _linalg.split_tf32(A, transpose=True), product)
        return torch.sum(product * A, dtype=torch.float64)


def pack_trellis(encoded: torch.Tensor, quant_args: dict) -> torch.Tensor:
    """States [K/16, N/16, 256] -> packed words [K/16, N/16, 16*K] (exl3_encoder_backend.py:2361-2372)."""

    K = quant_args["K"]
    shape = encoded.shape
    assert len(shape) == 3 and shape[2] == 256
    assert encoded.dtype == torch.int16
    encoded = encoded.contiguous()
    packed = torch.empty((shape[0], shape[1], 256 * K // 16), dtype=torch.int16, device=encoded.device)
    with torch.cuda.device(encoded.device):
        _lib.check(
            _lib.lib().qsrtb_pack_trellis(
                encoded.data_ptr(), shape[0] * shape[1], int(K), packed.data_ptr(), _stream_ptr(encoded.device)
            ),
            "qsrtb_pack_trellis",
        )
    return packed


# --------------------------------------------------------------------------------------
# Entry points of the quantizer_module boundary
# --------------------------------------------------------------------------------------

_OUT_OF_SCOPE_ARGS = {
    "output_hessian": "two-sided (output-Hessian) feedback",
    "use_two_sided_traversal_without_output_feedback": "two-sided traversal controls",
    "periodic_rate_schedules": "periodic (within-tile variable) rates",
    "mcg": "the procedural MCG codebook",
    "mul1": "the procedural MUL1 codebook",
    "return_trellis_diagnostics": "the on-GPU trellis diagnostics accumulator (qsrt/sqg_quantizer.py:90-139)",
}


def _reject_out_of_scope(quant_args: dict) -> None:
    for key, what in _OUT_OF_SCOPE_ARGS.items():
        if quant_args.get(key):
            raise NotImplementedError(f"{what} is a research arm outside the B200 encoder hot path")


def _refine():
    from . import refine  # late: refine reaches back into this module for the row kernel

    return refine


def _deregularize(weight_q: torch.Tensor, su: torch.Tensor, sv: torch.Tensor) -> torch.Tensor:
    """had_l, *su, had_r, *sv (exl3_encoder_backend.py:3030-3034) with the scales fused."""

    out = weight_q.contiguous().clone()
    _hadamard(out, 0, su.reshape(-1).float().contiguous(), per_col=False, after=True)
    _hadamard(out, 1, sv.reshape(-1).float().contiguous(), per_col=True, after=True)
    return out


def quantize_qsrt(weight: torch.Tensor, H_data: dict, quant_args: dict, return_weight_q: bool,
                  progress_str: str | None = None, verbose: bool = False,
                  swap_to_device: torch.device | None = None, save_reg: str | None = None):
    """Encode one ``[in_features, out_features]`` float32 matrix
    (exl3_encoder_backend.py:2754-3073).

    Returns ``(weight_q, proxy_err, out_tensors)`` with ``out_tensors = {"suh", "svh",
    "trellis"}``; ``weight`` is transformed in place, ``H_data`` gains ``L``/``su``/``diag``/
    ``q_fallback``/``finalized`` and ``quant_args`` gains ``apply_out_scales``/``g_scale``/
    ``q_fallback``/``zeros``/``h2_viterbi_refine_receipt`` exactly as in the reference.
    """

    _reject_out_of_scope(quant_args)
    assert weight.dtype == torch.float
    devices = quant_args["devices"]
    if weight.device != torch.device(devices[0]):
        weight = weight.to(devices[0])
    device = weight.device if swap_to_device is None else swap_to_device
    k, n = weight.shape

    q_fallback, H, L, su, H_diag = finalize_capture_H(H_data, quant_args, verbose)
    if L is not None:
        L = L.to(device)
    su = su.to(device)
    if H_diag is not None:
        H_diag = H_diag.to(device)
    sv = output_signs(n, device, quant_args)
    if H_data["L"] is not None and not KEEP_HESSIAN_ON_DEVICE:
        H_data["L"] = H_data["L"].cpu()
    if swap_to_device is not None:
        weight = weight.to(swap_to_device)
    weight_r = weight
    del weight

    apply_out_scales, weight_r, g_scale, su, sv = regularize(
        weight_r, su, sv, quant_args, verbose, H_diag, None, q_fallback=q_fallback
    )

    mixed_rate = "mixed_rate_axis" in quant_args or "mixed_tile_bits" in quant_args
    if not q_fallback:
        if mixed_rate:
            weight_q, encoded_q = ldlq_mixed(weight_r, L, quant_args)
        else:
            weight_q, encoded_q = ldlq(weight_r, L, quant_args)
        del L
        # dense-H path refinement of the finished candidate (exl3_encoder_backend.py:2970-2979)
        weight_q, encoded_q, quant_args["h2_viterbi_refine_receipt"] = _refine().refine_uniform_h2_candidate(
            weight_r, H, weight_q, encoded_q, quant_args)
    else:
        if mixed_rate:
            raise ValueError("variable-rate quantization requires a non-fallback dense Hessian")
        weight_q, encoded_q, mse_err = fallback_quant(weight_r, device, quant_args)

    if not q_fallback:
        trace = HessianTrace(H.to(device))
        num, den = torch.stack((trace(weight_r - weight_q), trace(weight_r))).tolist()
        del trace
        proxy_err = num / max(den, 1e-8)
    else:
        proxy_err = mse_err

    if return_weight_q or verbose:
        weight_q = _deregularize(weight_q.to(device), su, sv)

    suh = su.flatten().contiguous().to(dtype=torch.half, copy=True)
    svh = sv.flatten().contiguous().to(dtype=torch.half, copy=True)
    pack_trellis_fn = quant_args.get("pack_trellis_fn", pack_trellis)
    trellis = pack_trellis_fn(encoded_q.to(device), quant_args)
    out_tensors = {"suh": suh, "svh": svh, "trellis": trellis}
    quant_args.update({"apply_out_scales": apply_out_scales, "g_scale": g_scale, "q_fallback": q_fallback})
    return weight_q, proxy_err, out_tensors


def quantize_uniform_batch(weights: list[torch.Tensor], H_datas: list[dict], quant_args_list: list[dict],
                           progress_str: str | None = None, verbose: bool = False):
    """Encode a group of same-K matrices together (exl3_encoder_backend.py:3397-3620).

    Shared Hessian (the same ``H_data`` object for every tensor): the regularised weights are
    concatenated along out_features and run through one LDLQ pass.  Distinct Hessians over
    same-shape tensors: the tensors are stacked and every 16-row step encodes all of their
    tiles in one launch.  (Generalisation: runs of tensors that share an ``H_data`` object are
    concatenated, and equally shaped runs are stacked - e.g. the gate/up pairs of several
    experts.)  Returns ``[(proxy_err, out_tensors), ...]``.
    """

    return quantize_uniform_groups([(weights, H_datas, quant_args_list)], verbose=verbose)[0]


def quantize_uniform_groups(groups: list[tuple[list[torch.Tensor], list[dict], list[dict]]], verbose: bool = False):
    """Several ``quantize_uniform_batch`` groups whose LDLQ recursions run concurrently on
    separate streams (``ldlq_concurrent``).  Per group the semantics are exactly those of
    ``quantize_uniform_batch``; the groups must be independent of each other."""

    states = [_uniform_prepare(w, h, q, verbose) for w, h, q in groups]
    jobs, owners = [], []
    for gi, st in enumerate(states):
        if st["job"] is not None:
            jobs.append(st["job"])
            owners.append(gi)
    for gi, (weight_q, encoded) in zip(owners, ldlq_concurrent(jobs)):
        states[gi]["weight_q"], states[gi]["encoded"] = weight_q, encoded
    return [_uniform_finish(st) for st in states]


def _uniform_prepare(weights, H_datas, quant_args_list, verbose):
    if any("mixed_rate_axis" in qa or "mixed_tile_bits" in qa for qa in quant_args_list):
        raise ValueError("mixed-rate LDLQ is currently supported by quantize_qsrt, not the same-K batch API")
    for qa in quant_args_list:
        _reject_out_of_scope(qa)
        if int(qa.get("h2_viterbi_refine_sweeps", 0) or 0) > 0:
            raise NotImplementedError("dense-H path refinement runs in quantize_qsrt and quantize_qsrt_batch, "
                                      "not in the same-K batch API")
    n_t = len(weights)
    qa0 = quant_args_list[0]
    device = torch.device(qa0["devices"][0])
    assert all(w.shape[0] == weights[0].shape[0] for w in weights)
    assert all(qa["K"] == qa0["K"] for qa in quant_args_list)
    results: list = [None] * n_t

    finalized, batch_idx = [], []
    for t in range(n_t):
        q_fallback, H, L, su, H_diag = finalize_capture_H(H_datas[t], quant_args_list[t], verbose)
        if q_fallback:
            finalized.append(None)
        else:
            finalized.append((H, L, su, H_diag))
            batch_idx.append(t)
    for t in range(n_t):
        if finalized[t] is None:
            results[t] = quantize_qsrt(weights[t], H_datas[t], quant_args_list[t], False, None, verbose)[1:]
    state = {"results": results, "batch_idx": batch_idx, "finalized": finalized, "job": None,
             "quant_args_list": quant_args_list, "device": device}
    if not batch_idx:
        return state

    regs = {}
    for t in batch_idx:
        qa = quant_args_list[t]
        H, L, su, H_diag = finalized[t]
        weight = weights[t]
        if weight.device != device:
            weight = weight.to(device)
        su = su.to(device)
        if H_diag is not None:
            H_diag = H_diag.to(device)
        sv = output_signs(weight.shape[1], device, qa)
        apply_out_scales, weight_r, _, su, sv = regularize(weight, su, sv, qa, verbose, H_diag, None, skip_g_scale=True)
        regs[t] = [weight_r, su, sv, apply_out_scales]
        weights[t] = None

    samples = [sample_scale_tiles(regs[t][0]) for t in batch_idx]
    scales = g_scale_search_batch(samples, qa0)
    del samples
    g_scales = {}
    for t, (g_scale, _) in zip(batch_idx, scales):
        regs[t][0] *= g_scale
        if quant_args_list[t].get("g_scale_into_sv"):
            regs[t][2] /= g_scale
        else:
            regs[t][1] /= g_scale
        g_scales[t] = g_scale

    # runs of consecutive tensors sharing one H_data object are concatenated along out_features
    runs: list[list[int]] = []
    for t in batch_idx:
        if runs and H_datas[runs[-1][0]] is H_datas[t]:
            runs[-1].append(t)
        else:
            runs.append([t])
    cats = [torch.cat([regs[t][0] for t in run], dim=1) if len(run) > 1 else regs[run[0]][0] for run in runs]
    assert all(c.shape == cats[0].shape for c in cats), "tensor groups with distinct Hessians must have one shape"
    for t in batch_idx:
        regs[t][0] = None
    weight_r_stack = torch.stack(cats) if len(cats) > 1 else cats[0].unsqueeze(0)
    del cats
    Ls = [finalized[run[0]][1].to(device) for run in runs]
    Ls_stack = torch.stack(Ls) if len(Ls) > 1 else Ls[0].unsqueeze(0)
    del Ls
    state.update({"regs": regs, "g_scales": g_scales, "runs": runs, "weight_r": weight_r_stack,
                  "job": (weight_r_stack, Ls_stack, qa0)})
    return state


def _uniform_finish(state):
    results = state["results"]
    if state["job"] is None:
        return results
    device = state["device"]
    quant_args_list = state["quant_args_list"]
    finalized, regs, runs = state["finalized"], state["regs"], state["runs"]
    weight_r_stack, weight_q_stack, encoded_stack = state["weight_r"], state["weight_q"], state["encoded"]
    state["job"] = None  # drop the stacked factors
    for ri, run in enumerate(runs):
        trace = HessianTrace(finalized[run[0]][0].to(device))
        col = 0
        for t in run:
            qa = quant_args_list[t]
            _, su, sv, apply_out_scales = regs[t]
            width = sv.shape[1]
            w_r = weight_r_stack[ri, :, col:col + width]
            w_q = weight_q_stack[ri, :, col:col + width]
            enc = encoded_stack[ri, :, col // 16:(col + width) // 16]
            col += width
            num, den = torch.stack((trace(w_r - w_q), trace(w_r))).tolist()
            proxy_err = num / max(den, 1e-8)
            suh = su.flatten().contiguous().to(dtype=torch.half, copy=True)
            svh = sv.flatten().contiguous().to(dtype=torch.half, copy=True)
            trellis = pack_trellis(enc.contiguous(), qa)
            qa.update({"apply_out_scales": apply_out_scales, "g_scale": state["g_scales"][t], "q_fallback": False})
            results[t] = (proxy_err, {"suh": suh, "svh": svh, "trellis": trellis})
        del trace
    return results


def quantize_qsrt_batch(weights: list[torch.Tensor], H_datas: list[dict], quant_args_groups: list[list[dict]], *,
                        return_weight_q: bool = True, verbose: bool = False):
    """Prepare each source once and encode all of its mixed-rate candidates
    (exl3_encoder_backend.py:3076-3394).

    Per source: two-stage Hessian preparation with the complete conditioned ``su``, one
    regularisation, one batched global-scale search; then the candidates' BlockLDLQ recursions over
    their tile-rate maps, batched.  Returns one
    list per source of ``{"weight_q", "encoded", "suh", "svh", "proxy", "g_scale",
    "h2_viterbi_refine"}``; the payload is not packed, as in the reference.  Candidates are encoded
    through the reference's reuse schedules where their maps allow it (``:3245-3293``): shared
    K3 columns once for output-axis maps over an all-K3 first candidate, the shared backwards
    prefix once for input-axis maps, a plain batch over shared sources otherwise.
    """

    source_count = len(weights)
    if source_count <= 0 or len(H_datas) != source_count or len(quant_args_groups) != source_count:
        raise ValueError("QSRT batch inputs must have equal nonzero lengths")
    if any(not group for group in quant_args_groups):
        raise ValueError("every QSRT source needs at least one rate candidate")
    if any(weight.ndim != 2 or weight.dtype != torch.float for weight in weights):
        raise TypeError("QSRT batch weights must be float32 matrices")
    shape = weights[0].shape
    if any(weight.shape != shape for weight in weights):
        raise ValueError("QSRT batch sources must have one matrix shape")
    preparation_keys = (
        "K", "seed", "sv_seed", "sigma_reg", "devices", "device_ratios", "apply_out_scales", "mcg", "mul1",
        "shared_input_scales_key", "g_scale_into_sv", "buf_size_k", "ldlq_tf32", "tailbite_context",
        "g_scale_override",
    )
    for group in quant_args_groups:
        reference = group[0]
        for args in group:
            _reject_out_of_scope(args)
            mixed_rate_spec(shape[0], shape[1], args)
            for key in preparation_keys:
                if args.get(key) != reference.get(key):
                    raise ValueError(f"QSRT candidates changed preparation argument {key}")
    devices = quant_args_groups[0][0]["devices"]
    device = torch.device(devices[0])
    if any(group[0].get("devices") != devices for group in quant_args_groups):
        raise ValueError("QSRT source groups must share devices")
    if any(weight.device != device for weight in weights):
        raise ValueError("QSRT batch weights must already be on the quant device")

    prepared = []
    for weight, H_data, group in zip(weights, H_datas, quant_args_groups):
        args = group[0]
        q_fallback, _, su, H_diag = prepare_capture_H_for_conditioning(H_data, args, verbose)
        if q_fallback:
            raise ValueError("mixed-rate batching requires a non-fallback dense Hessian")
        su = su.to(device)
        sv = output_signs(weight.shape[1], device, args)
        apply_out_scales, weight_r, _, su, sv = regularize(
            weight, su, sv, args, verbose, H_diag.to(device) if H_diag is not None else None, None,
            skip_g_scale=True, q_fallback=False,
        )
        q_fallback, H, L, su, _ = finalize_capture_H_with_conditioning(H_data, su, args, verbose)
        if q_fallback or H is None or L is None:
            raise ValueError("mixed-rate batching requires a non-fallback dense Hessian")
        prepared.append({"H": H.to(device), "L": L.to(device), "weight_r": weight_r, "su": su.to(device),
                         "sv": sv, "apply_out_scales": apply_out_scales})

    scales: list = [None] * source_count
    search_sources, search_samples = [], []
    for source, (item, group) in enumerate(zip(prepared, quant_args_groups)):
        override = group[0].get("g_scale_override")
        if override is None:
            search_sources.append(source)
            search_samples.append(sample_scale_tiles(item["weight_r"]))
        else:
            if (isinstance(override, bool) or not isinstance(override, (int, float))
                    or not math.isfinite(float(override)) or float(override) <= 0.0):
                raise ValueError("g_scale_override must be positive and finite")
            scales[source] = (float(override), None)
    if search_samples:
        searched = g_scale_search_batch(search_samples, quant_args_groups[search_sources[0]][0])
        for source, result in zip(search_sources, searched):
            scales[source] = result
    for item, group, result in zip(prepared, quant_args_groups, scales):
        g_scale, _ = result
        item["weight_r"], item["su"], item["sv"] = apply_g_scale(
            item["weight_r"], item["su"], item["sv"], g_scale, into_sv=bool(group[0].get("g_scale_into_sv")))
        item["g_scale"] = g_scale

    members = [(source, candidate) for source, group in enumerate(quant_args_groups) for candidate in range(len(group))]
    axes = [[mixed_rate_spec(shape[0], shape[1], args) for args in group] for group in quant_args_groups]
    source_weights = torch.stack([item["weight_r"] for item in prepared])
    source_Ls = torch.stack([item["L"] for item in prepared])
    if all(all(axis == "n" for axis, _ in group) and group[0][1] == (3,) * (shape[1] // 16) for group in axes):
        # output-axis maps over an all-K3 first candidate: encode the shared columns once
        weights_q, encoded_q = ldlq_mixed_n_candidates_reuse(source_weights, source_Ls, quant_args_groups)
    elif any(len(group) > 1 for group in axes) and all(all(axis == "k" for axis, _ in group) for group in axes):
        # input-axis maps: encode the rows the candidates agree on once, then a trie of states
        weights_q, encoded_q = ldlq_mixed_k_candidates_prefix_reuse(source_weights, source_Ls, quant_args_groups)
    else:
        weights_q, encoded_q = ldlq_mixed_batched(
            source_weights, source_Ls, [quant_args_groups[s][c] for s, c in members],
            source_indices=torch.tensor([s for s, _ in members], dtype=torch.long, device=device),
        )
    del source_Ls
    encoded_all = [(weights_q[i:i + 1], encoded_q[i:i + 1]) for i in range(len(members))]

    results: list[list[dict]] = [[] for _ in range(source_count)]
    traces = [HessianTrace(item["H"]) for item in prepared]
    denominators = [float(trace(item["weight_r"])) for trace, item in zip(traces, prepared)]
    for (source, candidate), (weight_q, encoded) in zip(members, encoded_all):
        item = prepared[source]
        args = quant_args_groups[source][candidate]
        # dense-H path refinement per finished candidate (exl3_encoder_backend.py:3296-3312)
        weight_q, encoded, receipt = _refine().refine_uniform_h2_candidate(
            item["weight_r"], item["H"], weight_q[0], encoded[0], args)
        numerator = float(traces[source](item["weight_r"] - weight_q))
        if "suh" not in item:
            item["suh"] = item["su"].flatten().contiguous().to(dtype=torch.half, copy=True)
            item["svh"] = item["sv"].flatten().contiguous().to(dtype=torch.half, copy=True)
        reconstruction = None
        if return_weight_q:
            reconstruction = _deregularize(weight_q, item["suh"].float(), item["svh"].float())
        args.update({"apply_out_scales": item["apply_out_scales"], "g_scale": item["g_scale"], "q_fallback": False,
                     "zeros": quant_args_groups[source][0].get("zeros", False)})
        results[source].append({
            "weight_q": reconstruction,
            "encoded": encoded.contiguous(),
            "suh": item["suh"],
            "svh": item["svh"],
            "proxy": numerator / max(denominators[source], 1e-8),
            "g_scale": item["g_scale"],
            "h2_viterbi_refine": receipt,
        })
    return results


# candidate-grid entry points of the quantizer module (defined in their own file)
from .candidates import (  # noqa: E402
    ldlq_mixed_batched,
    ldlq_mixed_k_candidates_prefix_reuse,
    ldlq_mixed_n_candidates_reuse,
)

# dense-H path refinement, part of the reference module's surface (exl3_encoder_backend.py:20-23, 840)
from .refine import refine_h2_viterbi_paths, refine_uniform_h2_candidate  # noqa: E402
