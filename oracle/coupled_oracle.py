"""CPU restatement (numpy float32) of the coupled signed block-Hadamard coordinates.

TEST INFRASTRUCTURE ONLY.  Follows ``qsrt/qsrt_coupled.py``: ``block_hadamard`` (:49-84),
``rotation_signs`` (:87-107, torch CPU generator: the draw itself is reproduced with torch),
``signed_block_hadamard`` (:110-132), ``encode_coupled_weights`` (:145-196) and the
``CoupledHadamardExecution`` transforms (:347-543).  Pinned bit for bit against the reference
through the SHA-256 fixture ``tests/golden/coupled_golden.json``.
"""

from __future__ import annotations

import math

import numpy as np

F32 = np.float32


def block_hadamard(values: np.ndarray, block_size: int, axis: int = -1) -> np.ndarray:
    out = np.moveaxis(np.asarray(values, dtype=F32), axis, -1).copy()
    shape = out.shape
    out = out.reshape(*shape[:-1], shape[-1] // block_size, block_size)
    width = 1
    while width < block_size:
        paired = out.reshape(*out.shape[:-1], -1, 2, width)
        left = paired[..., 0, :].copy()
        right = paired[..., 1, :].copy()
        paired[..., 0, :] = left + right
        paired[..., 1, :] = left - right
        out = paired.reshape(*out.shape)
        width *= 2
    out = (out / F32(math.sqrt(block_size))).astype(F32)
    return np.ascontiguousarray(np.moveaxis(out.reshape(shape), -1, axis))


def rotation_signs(length: int, draw: int, axis: int) -> np.ndarray:
    if draw == 0:
        return np.ones(length, dtype=F32)
    import torch

    g = torch.Generator(device="cpu")
    g.manual_seed((0x6A09E667F3BCC909 * draw + 0xBB67AE8584CAA73B * axis) & ((1 << 63) - 1))
    return torch.randint(0, 2, (length,), generator=g).mul_(2).sub_(1).float().numpy()


def signed_block_hadamard(values, block_size, signs, axis=-1, inverse=False):
    values = np.asarray(values, dtype=F32)
    shape = [1] * values.ndim
    shape[axis % values.ndim] = signs.size
    expanded = signs.astype(F32).reshape(shape)
    if inverse:
        return (block_hadamard(values, block_size, axis) * expanded).astype(F32)
    return block_hadamard((values * expanded).astype(F32), block_size, axis)


def encode_coupled_weights(w1, w3, w2, *, residual=512, pre=128, post=128, intermediate_draw=0):
    inter, hidden = w1.shape
    s_in = rotation_signs(hidden, 0, 0)
    s_pre = rotation_signs(2 * inter, intermediate_draw, 1)
    s_post = rotation_signs(inter, intermediate_draw, 2)
    s_out = rotation_signs(hidden, 0, 3)
    interleaved = np.stack((w1, w3), axis=1).reshape(2 * inter, hidden)
    up = signed_block_hadamard(signed_block_hadamard(interleaved, residual, s_in, 1), pre, s_pre, 0)
    down = signed_block_hadamard(signed_block_hadamard(w2, post, s_post, 1), residual, s_out, 0)
    return np.ascontiguousarray(up[:inter]), np.ascontiguousarray(up[inter:]), np.ascontiguousarray(down)
