"""Bitstream packer and decoder entry points (device resident).

Mirrors the reference's pack / unpack / decode helpers with the same names and argument
meaning:

* ``pack_trellis_edges`` / ``unpack_trellis_edges`` / ``unpack_trellis_states``
  (``qsrt/qsrt.py:861-913``), ``pack_uniform_trellis_edges`` / ``unpack_uniform_trellis_states``
  (``qsrt/qsrt_codec_pilot.py:220-280``),
* ``reconstruct_trellis_states``, ``decode_regularized_weight``, ``decode_exl3_weight``
  (``qsrt/exl3_reference.py:34-58, 108-140, 280-302``),
* ``decode_e4m3``: the "decode to FP8" target, one raw E4M3 byte per weight.

All tensors must live on a CUDA device; the kernels are ``qsrtb_pack_trellis``,
``qsrtb_unpack_decode``, ``qsrtb_states_to_matrix`` and ``qsrtb_hadamard128``.
"""

from __future__ import annotations

import torch

from . import _lib
from .encoder import _hadamard
from .tables import sqg_codebook_bytes
from .tiles import _stream_ptr

TILE_VALUES = 256


def _validate_k(bits: int) -> None:
    if isinstance(bits, bool) or not isinstance(bits, int) or bits not in (2, 3, 4):
        raise ValueError("QSRT supports K=2, K=3, or K=4")


def _require_cuda(tensor: torch.Tensor, what: str) -> None:
    if not tensor.is_cuda:
        raise ValueError(f"{what} must be on a CUDA device (there is no CPU path)")


def pack_trellis_edges(indices: torch.Tensor, bits: int) -> torch.Tensor:
    """Low K bits of every state, MSB first, native word order (qsrt/qsrt.py:861-883)."""

    _validate_k(bits)
    if indices.ndim < 1 or indices.shape[-1] != TILE_VALUES:
        raise ValueError("indices must have a final dimension of 256")
    if indices.dtype == torch.bool or indices.is_floating_point():
        raise TypeError("indices must use an integer dtype")
    _require_cuda(indices, "indices")
    states = indices.to(torch.int16).contiguous()
    lead = states.shape[:-1]
    n_tiles = states.numel() // TILE_VALUES
    packed = torch.empty((*lead, 16 * bits), dtype=torch.int16, device=states.device)
    with torch.cuda.device(states.device):
        _lib.check(
            _lib.lib().qsrtb_pack_trellis(states.data_ptr(), n_tiles, bits, packed.data_ptr(), _stream_ptr(states.device)),
            "qsrtb_pack_trellis",
        )
    return packed


pack_uniform_trellis_edges = pack_trellis_edges


def _unpack(packed: torch.Tensor, bits: int, lut: torch.Tensor | None, want_states: bool, want_bytes: bool):
    _validate_k(bits)
    if packed.ndim < 1 or packed.shape[-1] != 16 * bits:
        raise ValueError(f"packed tiles must end in {16 * bits} int16 words")
    if packed.dtype != torch.int16:
        raise TypeError("packed trellis words must use torch.int16")
    _require_cuda(packed, "packed")
    packed = packed.contiguous()
    lead = packed.shape[:-1]
    n_tiles = packed.numel() // (16 * bits)
    states = torch.empty((*lead, TILE_VALUES), dtype=torch.int16, device=packed.device) if want_states else None
    raw = torch.empty((*lead, TILE_VALUES), dtype=torch.uint8, device=packed.device) if want_bytes else None
    if lut is not None:
        lut = lut.to(device=packed.device, dtype=torch.uint8).contiguous()
    with torch.cuda.device(packed.device):
        _lib.check(
            _lib.lib().qsrtb_unpack_decode(
                packed.data_ptr(), n_tiles, bits, lut.data_ptr() if lut is not None else None,
                states.data_ptr() if states is not None else None,
                raw.data_ptr() if raw is not None else None, _stream_ptr(packed.device),
            ),
            "qsrtb_unpack_decode",
        )
    return states, raw


def unpack_trellis_states(packed: torch.Tensor, bits: int) -> torch.Tensor:
    """Packed words -> cyclic 16-bit states (qsrt/qsrt.py:910-913)."""

    return _unpack(packed, bits, None, True, False)[0]


unpack_uniform_trellis_states = unpack_trellis_states


def unpack_trellis_edges(packed: torch.Tensor, bits: int) -> torch.Tensor:
    """Packed words -> stored K-bit edge symbols (qsrt/qsrt.py:886-907)."""

    return unpack_trellis_states(packed, bits) & ((1 << bits) - 1)


def reconstruct_trellis_states(edge_symbols: torch.Tensor, bits: int) -> torch.Tensor:
    """Edges -> states (qsrt/exl3_reference.py:34-58), via a pack/unpack round trip on device."""

    return unpack_trellis_states(pack_trellis_edges(edge_symbols, bits), bits)


def decode_e4m3(packed: torch.Tensor, bits: int, lut: torch.Tensor) -> torch.Tensor:
    """Packed bitstream -> raw E4M3 bytes, one per weight, tile order unchanged."""

    return _unpack(packed, bits, lut, False, True)[1]


def decode_regularized_weight(states: torch.Tensor, *, lut: torch.Tensor) -> torch.Tensor:
    """``[K/16, N/16, 256]`` states -> regularised ``[K, N]`` float32 (exl3_reference.py:108-140)."""

    if states.ndim != 3 or states.shape[-1] != TILE_VALUES:
        raise ValueError("states must have shape [K/16, N/16, 256]")
    _require_cuda(states, "states")
    states = states.to(torch.int16).contiguous()
    lut = lut.to(device=states.device, dtype=torch.uint8).contiguous()
    kt, nt, _ = states.shape
    out = torch.empty((kt * 16, nt * 16), dtype=torch.float32, device=states.device)
    with torch.cuda.device(states.device):
        _lib.check(
            _lib.lib().qsrtb_states_to_matrix(
                states.data_ptr(), kt, nt, lut.data_ptr(), out.data_ptr(), nt * 16, _stream_ptr(states.device)
            ),
            "qsrtb_states_to_matrix",
        )
    return out


def decode_exl3_weight(states: torch.Tensor, suh: torch.Tensor, svh: torch.Tensor, *,
                       codebook: str = "sqg_xor_cheb_t12", bits: int | None = None,
                       lut: torch.Tensor | None = None) -> torch.Tensor:
    """States + fp16 scales -> ``[K, N]`` float32 weight (exl3_reference.py:280-302)."""

    if lut is None:
        if bits is None:
            raise ValueError("SQG reconstruction requires an explicit trellis rate")
        lut = sqg_codebook_bytes(bits, codebook)
    weight = decode_regularized_weight(states, lut=lut)
    if suh.ndim != 1 or suh.numel() != weight.shape[0]:
        raise ValueError("suh length does not match the EXL K dimension")
    if svh.ndim != 1 or svh.numel() != weight.shape[1]:
        raise ValueError("svh length does not match the EXL N dimension")
    _hadamard(weight, 0, suh.to(device=weight.device, dtype=torch.float32).contiguous(), per_col=False, after=True)
    _hadamard(weight, 1, svh.to(device=weight.device, dtype=torch.float32).contiguous(), per_col=True, after=True)
    return weight
