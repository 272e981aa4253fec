"""MXFP4 source weights -> float32 on the device.

Mirrors ``qsrt/io/mxfp4.py`` (``unpack_codes`` ``:19-30``, ``pack_codes`` ``:33-39``,
``scale_factors`` ``:42-44``, ``code_values`` ``:45-48``, ``dequant`` ``:50-63``) with the same
names and argument meaning.  ``dequant`` is one kernel (``qsrtb_mxfp4_dequant``) instead of a
chain of torch ops that materialises the unpacked codes, their values and the scale factors;
``dequant_encoder_orientation`` writes the ``[in, out]`` matrix the encoder consumes directly.
"""

from __future__ import annotations

import torch

from . import _lib
from .tiles import _stream_ptr

MXFP4_BLOCK = 32
E8M0_BIAS = 127
E2M1_LUT = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def unpack_codes(packed: torch.Tensor) -> torch.Tensor:
    """uint8 ``[..., K/2]`` -> uint8 codes ``[..., K]``; the low nibble is the even index."""

    if packed.dtype != torch.uint8:
        raise TypeError(f"expected uint8, got {packed.dtype}")
    return torch.stack((packed & 0x0F, packed >> 4), dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)


def pack_codes(codes: torch.Tensor) -> torch.Tensor:
    """uint8 codes ``[..., K]`` -> uint8 ``[..., K/2]``."""

    if codes.shape[-1] % 2:
        raise ValueError("K must be even")
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).to(torch.uint8)


def scale_factors(scale: torch.Tensor) -> torch.Tensor:
    """uint8 E8M0 ``[..., K/32]`` -> float32 ``2^(e-127)``."""

    return torch.exp2(scale.to(torch.float32) - E8M0_BIAS)


def code_values(codes: torch.Tensor) -> torch.Tensor:
    """uint8 codes -> float32 E2M1 values (unscaled)."""

    return torch.tensor(E2M1_LUT, dtype=torch.float32, device=codes.device)[codes.long()]


def _dequant(packed: torch.Tensor, scale: torch.Tensor, transposed: bool) -> torch.Tensor:
    if packed.dtype != torch.uint8 or scale.dtype != torch.uint8:
        raise TypeError(f"expected uint8, got {packed.dtype} and {scale.dtype}")
    if packed.ndim != 2 or scale.ndim != 2 or packed.shape[0] != scale.shape[0]:
        raise ValueError("packed codes and scales must be matrices with the same rows")
    k = packed.shape[-1] * 2
    if scale.shape[-1] * MXFP4_BLOCK != k:
        raise ValueError(f"scale blocks {scale.shape[-1]} do not cover K={k} at block {MXFP4_BLOCK}")
    if not packed.is_cuda or scale.device != packed.device:
        raise ValueError("packed codes and scales must be on one CUDA device (there is no CPU path)")
    packed, scale = packed.contiguous(), scale.contiguous()
    rows = packed.shape[0]
    out = torch.empty((k, rows) if transposed else (rows, k), dtype=torch.float32, device=packed.device)
    with torch.cuda.device(packed.device):
        _lib.check(
            _lib.lib().qsrtb_mxfp4_dequant(packed.data_ptr(), scale.data_ptr(), rows, k, out.data_ptr(),
                                           out.shape[1], int(transposed), _stream_ptr(packed.device)),
            "qsrtb_mxfp4_dequant",
        )
    return out


def dequant(packed: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Packed codes ``[out, K/2]`` + E8M0 scales ``[out, K/32]`` -> float32 ``[out, K]``."""

    return _dequant(packed, scale, transposed=False)


def dequant_encoder_orientation(packed: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """The same values as ``dequant(...).T.contiguous()``: ``[K = in, N = out]`` float32."""

    return _dequant(packed, scale, transposed=True)
