"""Reconstruction tables of the QSRT trellis codebooks (one-time host set-up).

Mirrors the table builders of the reference (``qsrt/sqg_e4m3.py:196-301``): the primary
``sqg_xor_cheb_t12`` law maps each 16-bit trellis state through a carry-mixed rank
permutation into a 4 KiB modal compression of the E4M3-rounded normal quantile staircase.
The tables are pinned by SHA-256 in the tests.
"""

from __future__ import annotations

from functools import lru_cache

import torch

SQG_XOR_CHEB_T12 = "sqg_xor_cheb_t12"
_STATES = 1 << 16


def _validate_bits(bits: int) -> None:
    if isinstance(bits, bool) or not isinstance(bits, int) or bits not in range(1, 7):
        raise ValueError("SQG supports integer K1 through K6")


@lru_cache(maxsize=None)
def sqg_xor_rank_permutation(bits: int) -> torch.Tensor:
    """Rank of every 16-bit codeword (``qsrt/sqg_e4m3.py:259-284``), int64 [65536]."""

    _validate_bits(bits)
    width = 16 - bits
    low = (1 << width) - 1
    word = torch.arange(_STATES, dtype=torch.int64)
    history, branch = word >> bits, word & ((1 << bits) - 1)
    mixed = history ^ (history >> 11)
    mixed = mixed ^ ((mixed << 11) & low)
    product = (mixed * 0x3FA7D929 + 0xC928FD8E) & 0xFFFFFFFF
    reversed_branch = torch.zeros_like(branch)
    for bit in range(bits):
        reversed_branch |= ((branch >> bit) & 1) << (bits - 1 - bit)
    stratum = reversed_branch ^ (product >> (32 - bits))
    return ((stratum << width) | (product & low)).contiguous()


@lru_cache(maxsize=1)
def sqg_cheb_normal_rank_e4m3_bytes() -> torch.Tensor:
    """E4M3 staircase of 1.5 * Phi^-1 at the 65,536 mid-rank quantiles (``:216-229``)."""

    ranks = torch.arange(_STATES, dtype=torch.float64)
    values = 1.5 * torch.special.ndtri((ranks + 0.5) / _STATES)
    raw = values.float().to(torch.float8_e4m3fn).view(torch.uint8).clone()
    raw[(raw & 0x7F) == 0] = 0  # one canonical zero
    decoded = raw.view(torch.float8_e4m3fn).float()
    if not bool(torch.isfinite(decoded).all()) or not bool(torch.all(decoded[1:] >= decoded[:-1])):
        raise RuntimeError("rank law is not a finite monotone E4M3 staircase")
    return raw.contiguous()


@lru_cache(maxsize=1)
def sqg_xor_cheb_t12_rank_lut_bytes() -> torch.Tensor:
    """Modal byte of each run of 16 ranks, ties to the lower raw byte (``:241-256``)."""

    blocks = sqg_cheb_normal_rank_e4m3_bytes().reshape(1 << 12, 16)
    counts = (blocks[:, :, None] == blocks[:, None, :]).sum(dim=-1)
    modal = counts == counts.max(dim=1, keepdim=True).values
    candidates = torch.where(modal, blocks.to(torch.int16), torch.tensor(256, dtype=torch.int16))
    return candidates.min(dim=1).values.to(torch.uint8).contiguous()


@lru_cache(maxsize=None)
def _t12_cpu(bits: int) -> torch.Tensor:
    return sqg_xor_cheb_t12_rank_lut_bytes().index_select(0, sqg_xor_rank_permutation(bits) >> 4).contiguous()


def sqg_xor_cheb_t12_bytes(bits: int, *, device: torch.device | str = "cpu") -> torch.Tensor:
    """State-indexed E4M3 labels of the primary codebook (``:287-301``)."""

    _validate_bits(bits)
    return _t12_cpu(bits).to(device=device).contiguous()


def sqg_codebook_bytes(
    bits: int,
    codebook: str,
    *,
    rate_axis: str | None = None,
    device: torch.device | str = "cpu",
) -> torch.Tensor:
    """Named codebook -> state-indexed raw E4M3 labels (``:304-319``)."""

    if codebook == SQG_XOR_CHEB_T12:
        return sqg_xor_cheb_t12_bytes(bits, device=device)
    raise ValueError(f"unsupported SQG codebook: {codebook!r}")


def sqg_codebook(
    bits: int,
    codebook: str,
    *,
    rate_axis: str | None = None,
    device: torch.device | str = "cpu",
    dtype: torch.dtype = torch.float16,
) -> torch.Tensor:
    if not dtype.is_floating_point:
        raise TypeError("SQG codebook dtype must be floating point")
    raw = sqg_codebook_bytes(bits, codebook, rate_axis=rate_axis, device=device)
    return raw.view(torch.float8_e4m3fn).to(dtype=dtype).contiguous()
