"""CPU restatement (numpy, float32) of the reference's BlockLDLQ encoder around the tile search.

TEST INFRASTRUCTURE ONLY: the checker for the product's ``quantize_qsrt`` path.  The product
never imports it.

Parity status: the reference module these functions restate
(``qsrt/exl3_encoder_backend.py``) cannot be imported without the un-vendored ExLlamaV3
package and a CUDA device, so this restatement is pinned only indirectly: its algebra against
the reference's FP64 proofs (``qsrt/blockldlq_proof.py``), its decode/pack helpers against the
reference's own importable modules (fixtures in ``tests/golden``), and its tile search against
the reference CUDA kernel.  The float32 summation order of cuBLAS cannot be restated, which the
reference itself documents as "not a bit-exact batching contract"
(``exl3_encoder_backend.py:1213-1221``).

Random signs: the reference draws ``su``/``sv`` from a CUDA generator
(``qsrt/rng.py:16-20``); here they are inputs.
"""

from __future__ import annotations

import math

import numpy as np

from . import qsrt_oracle as base

CODEBOOK_SCALE = 1.24371088
F32 = np.float32


def block_rms(x: np.ndarray, axis: int) -> np.ndarray:
    """exl3_encoder_backend.py:2508-2521 (sum of squares in blocks of 32, then mean, sqrt)."""

    n = x.shape[axis]
    sq = None
    for start in range(0, n, 32):
        block = np.take(x, range(start, min(start + 32, n)), axis=axis)
        part = np.square(block, dtype=F32).sum(axis=axis, keepdims=True, dtype=F32)
        sq = part if sq is None else (sq + part).astype(F32)
    return np.sqrt(sq / F32(n)).astype(F32)


def prepare_hessian(h: np.ndarray, count: float, sigma_reg: float):
    """_prepare_capture_H (exl3_encoder_backend.py:2077-2122) without the sign draw."""

    h = (h.astype(F32) / F32(count)).astype(F32)
    diag_mean = F32(np.diag(h).mean(dtype=F32))
    q_fallback = float(diag_mean) < 1e-20
    h = h.copy()
    h[np.diag_indices_from(h)] += F32(sigma_reg) * diag_mean
    return q_fallback, h, np.diag(h).copy()


def block_ldl(h: np.ndarray, b: int = 16, sigma_reg: float = 0.025):
    """block_ldl (exl3_encoder_backend.py:323-393): Cholesky, then unit block-lower factor."""

    n = h.shape[0]
    m = n // b
    h = h.astype(F32).copy()
    retries = 0
    while True:
        try:
            chol = np.linalg.cholesky(h.astype(np.float64)).astype(F32)
            break
        except np.linalg.LinAlgError:
            retries += 1
            if retries > 10:
                raise
            h[np.diag_indices_from(h)] += F32(2.0 * sigma_reg) * F32(np.diag(h).mean(dtype=F32))
    out = chol.copy()
    for i in range(m):
        dl = chol[i * b:(i + 1) * b, i * b:(i + 1) * b]
        inv = np.linalg.inv(dl.astype(np.float64)).astype(F32)
        out[:, i * b:(i + 1) * b] = chol[:, i * b:(i + 1) * b] @ inv
    for i in range(m):
        out[i * b:(i + 1) * b, i * b:(i + 1) * b] = np.eye(b, dtype=F32)
    return out, h


def factor_hessian(h: np.ndarray, su: np.ndarray, sigma_reg: float = 0.025):
    """_factor_capture_H (exl3_encoder_backend.py:2125-2160): congruence, LDL, zero diagonal."""

    su = su.reshape(-1, 1).astype(F32)
    h = (h * su.T).astype(F32)
    h = base.hadamard_right(h)
    h = (h * su).astype(F32)
    h = base.hadamard_left(h)
    factor, h = block_ldl(h, 16, sigma_reg)
    factor[np.diag_indices_from(factor)] = 0
    return factor, h


def sample_scale_tiles(weight_r: np.ndarray, width: int = 3) -> np.ndarray:
    """sample_scale_tiles (exl3_encoder_backend.py:2383-2410)."""

    tiles_k, tiles_n = weight_r.shape[0] // 16, weight_r.shape[1] // 16
    w4 = weight_r.reshape(tiles_k, 16, tiles_n, 16)
    diag_len = max(tiles_k, tiles_n)
    ii = np.repeat(np.arange(diag_len), width)
    ww = np.tile(np.arange(width), diag_len)
    kk, nn = ii % tiles_k, (ii + ww) % tiles_n
    num_x = max(8, (diag_len * width) // 16)
    tile_ms = np.square(w4, dtype=F32).mean(axis=(1, 3), dtype=F32).reshape(-1)
    num_x = min(num_x, (tile_ms.shape[0] + 1) // 2)
    order = np.argsort(-tile_ms, kind="stable")
    hi = order[:num_x]
    lo = np.argsort(tile_ms, kind="stable")[:num_x]
    flat = np.concatenate((hi, lo))
    xk, xn = flat // tiles_n, flat % tiles_n
    rows = np.concatenate((kk, xk))
    cols = np.concatenate((nn, xn))
    tiles = w4[rows, :, cols, :].reshape(-1, 256)
    return np.ascontiguousarray(tiles[:, base.tensor_core_perm()])


def g_scale_search(samples: np.ndarray, lut: np.ndarray, bits: int, context: int = 128):
    """g_scale_search_batch for one tensor (exl3_encoder_backend.py:2413-2476)."""

    def mse_at(tiles: np.ndarray, scale: float) -> float:
        scaled = (tiles * F32(scale)).astype(F32)
        quant, _ = base.quantize_tiles(scaled, lut, bits, context)
        return float(np.square(quant / F32(scale) - tiles, dtype=F32).mean(dtype=F32))

    coarse = [0.1 + 0.2 * i for i in range(10)]
    sub = samples[::3]
    mse1 = [mse_at(sub, s) for s in coarse]
    center = coarse[int(np.argmin(np.array(mse1, dtype=F32)))]
    step = 0.075
    fine = [center + step * (i - 2) for i in range(5)]
    mse2 = [mse_at(samples, s) for s in fine]
    best = min(range(5), key=lambda i: mse2[i])
    if 0 < best < 4:
        y0, y1, y2 = mse2[best - 1], mse2[best], mse2[best + 1]
        denom = y0 - 2.0 * y1 + y2
        offset = 0.5 * (y0 - y2) / denom if denom > 0 else 0.0
        offset = max(-0.5, min(0.5, offset))
    else:
        offset = 0.0
    return max(fine[best] + offset * step, 0.01), mse2[best]


def regularize(
    weight: np.ndarray,
    su_sign: np.ndarray,
    sv_sign: np.ndarray,
    *,
    lut: np.ndarray,
    bits: int,
    context: int = 128,
    apply_out_scales: bool | None = False,
    h_diag: np.ndarray | None = None,
    g_scale_override: float | None = None,
    g_scale_into_sv: bool = False,
    skip_g_scale: bool = False,
    shared_in_scales: np.ndarray | None = None,
):
    """regularize + apply_g_scale (exl3_encoder_backend.py:2580-2751), q_fallback False.

    Returns (apply_out_scales, weight_r, g_scale, su, sv, zeros, in_channel_scales).
    """

    weight = weight.astype(F32).copy()
    su = su_sign.reshape(-1, 1).astype(F32)
    sv = sv_sign.reshape(1, -1).astype(F32)
    force = apply_out_scales
    if h_diag is not None:
        diag = np.sort(np.sqrt(h_diag.astype(F32)))[::-1]
        cutoff = diag.shape[0] // 50
        skew = diag[:cutoff].sum(dtype=F32) / diag.sum(dtype=F32)
        apply = (float(skew) < 0.15) if force is None else bool(force)
    else:
        apply = True if force is None else bool(force)
    out_scales = block_rms(weight, 0)
    mean = float(out_scales.mean(dtype=F32))
    zeros = not mean > 1e-30
    if not zeros:
        out_scales = (out_scales / F32(mean)).astype(F32)
    elif force is not None:
        apply = True
    zero_out = np.abs(out_scales) < 1e-30
    if apply:
        out_scales = np.where(zero_out, F32(0.1), out_scales).astype(F32)
        sv = (sv * out_scales + F32(1e-10)).astype(F32)
    weight = (weight / sv).astype(F32)
    sv = np.where(zero_out, F32(0.0), sv).astype(F32)
    weight = base.hadamard_right(weight)
    in_scales = block_rms(weight, 1)
    in_scales = np.where(np.abs(in_scales) < 1e-30, F32(0.1), in_scales).astype(F32)
    if shared_in_scales is not None:
        in_scales = shared_in_scales.reshape(-1, 1).astype(F32)
    su = (su * in_scales / F32(-CODEBOOK_SCALE) + F32(1e-10)).astype(F32)
    weight = (weight / su).astype(F32)
    weight = base.hadamard_left(weight)
    if skip_g_scale:
        g_scale = 1.0
    elif g_scale_override is not None:
        g_scale = float(g_scale_override)
    else:
        g_scale, _ = g_scale_search(sample_scale_tiles(weight), lut, bits, context)
    weight = (weight * F32(g_scale)).astype(F32)
    if g_scale_into_sv:
        sv = (sv / F32(g_scale)).astype(F32)
    else:
        su = (su / F32(g_scale)).astype(F32)
    return apply, weight, g_scale, su, sv, zeros, in_scales


def ldlq(
    weight: np.ndarray,
    factor: np.ndarray,
    lut: np.ndarray,
    bits: int,
    context: int = 128,
    *,
    buf_size_k: int = 128,
    feedback_multiplier: float = 1.0,
    forced_weight_q: np.ndarray | None = None,
):
    """ldlq (exl3_encoder_backend.py:420-539).

    With ``forced_weight_q`` (teacher forcing) the error fed back is computed from the given
    reconstruction instead of this run's, so each step's tiles can be compared in isolation;
    the returned ``targets`` are the rows handed to the tile search at every step.
    """

    size_k, size_n = weight.shape
    tiles_n = size_n // 16
    buf = max(buf_size_k, 16)
    weight = weight.astype(F32)
    prod_cache = np.zeros((size_k, size_n), dtype=F32)
    weight_q = np.zeros((size_k, size_n), dtype=F32)
    feedback_q = weight_q if forced_weight_q is None else forced_weight_q.astype(F32)
    encoded = np.zeros((size_k // 16, tiles_n, 256), dtype=np.int16)
    targets = np.zeros((size_k, size_n), dtype=F32)
    perm, perm_i = base.tensor_core_perm(), base.tensor_core_perm_inverse()
    for j in range(size_k, 0, -buf):
        i = j - buf
        for bj in range(buf, 0, -16):
            bi = bj - 16
            err = (weight[i + bj:j] - feedback_q[i + bj:j]).astype(F32)
            part = factor[i + bj:j, i + bi:i + bj]
            comp = (prod_cache[i + bi:i + bj] + part.T @ err).astype(F32)
            prod_cache[i + bi:i + bj] = comp
            if feedback_multiplier == 0.0:
                rows = weight[i + bi:i + bj]
            elif feedback_multiplier == 1.0:
                rows = (weight[i + bi:i + bj] + comp).astype(F32)
            else:
                rows = (weight[i + bi:i + bj] + F32(feedback_multiplier) * comp).astype(F32)
            targets[i + bi:i + bj] = rows
            tiles = rows.reshape(16, tiles_n, 16).transpose(1, 0, 2).reshape(tiles_n, 256)[:, perm]
            quant_w, quant_i = base.quantize_tiles(np.ascontiguousarray(tiles), lut, bits, context)
            quant_w = quant_w[:, perm_i].reshape(tiles_n, 16, 16).transpose(1, 0, 2).reshape(16, size_n)
            weight_q[i + bi:i + bj] = quant_w
            encoded[(i + bi) // 16] = quant_i
        span_err = (weight[i:j] - feedback_q[i:j]).astype(F32)
        prod_cache += (factor[i:j].T @ span_err).astype(F32)
    return weight_q, encoded, targets


def block_trace(a: np.ndarray, b: np.ndarray) -> float:
    """trace(A^T B A) (exl3_encoder_backend.py:1951-1977), accumulated in float64 here."""

    a64 = a.astype(np.float64)
    return float(np.sum((b.astype(np.float64) @ a64) * a64))


def quantize_qsrt(
    weight: np.ndarray,
    hessian: np.ndarray,
    su_sign: np.ndarray,
    sv_sign: np.ndarray,
    *,
    lut: np.ndarray,
    bits: int,
    sigma_reg: float = 0.025,
    context: int = 128,
    count: float = 1.0,
    apply_out_scales: bool | None = False,
    g_scale_override: float | None = None,
    feedback_multiplier: float = 1.0,
):
    """quantize_qsrt (exl3_encoder_backend.py:2754-3073), uniform rate, Hessian present.

    ``weight`` is [in, out].  Returns a dict with weight_q (de-regularised), proxy_err, suh,
    svh, trellis (packed int16 [in/16, out/16, 16*bits]), encoded states, weight_r, g_scale.
    """

    q_fallback, h, h_diag = prepare_hessian(hessian, count, sigma_reg)
    if q_fallback:
        raise ValueError("the oracle covers the dense-Hessian path only")
    factor, h_work = factor_hessian(h, su_sign, sigma_reg)
    apply, weight_r, g_scale, su, sv, zeros, _ = regularize(
        weight, su_sign, sv_sign, lut=lut, bits=bits, context=context,
        apply_out_scales=apply_out_scales, h_diag=h_diag, g_scale_override=g_scale_override,
    )
    weight_q, encoded, _ = ldlq(
        weight_r, factor, lut, bits, context, feedback_multiplier=feedback_multiplier
    )
    num = block_trace(weight_r - weight_q, h_work)
    den = block_trace(weight_r, h_work)
    proxy = num / max(den, 1e-8)
    recon = base.hadamard_left(weight_q)
    recon = (recon * su).astype(F32)
    recon = base.hadamard_right(recon)
    recon = (recon * sv).astype(F32)
    return {
        "weight_q": recon,
        "weight_q_work": weight_q,
        "weight_r": weight_r,
        "proxy_err": proxy,
        "suh": su.reshape(-1).astype(np.float16),
        "svh": sv.reshape(-1).astype(np.float16),
        "trellis": base.pack_trellis_edges(encoded, bits),
        "encoded": encoded,
        "g_scale": g_scale,
        "apply_out_scales": apply,
        "zeros": zeros,
        "factor": factor,
    }
