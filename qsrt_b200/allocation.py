"""Equal-byte K2 / K3 / K4 allocation for the high-rate profile, and the tile error surfaces it
ranks (device resident where the data is large).

Mirrors ``qsrt/high_rate_allocation.py`` with the same names, argument meaning and error
behaviour: ``tile_squared_error`` (``:55-73``), ``dense_h_tile_error_contributions``
(``:76-148``), ``high_rate_record_bits`` (``:229-243``), ``record_rate_map`` (``:246-268``),
``rate_map_proxy_cost`` (``:271-303``), ``select_record_rate_allocation`` (``:306-327``),
``tile_p24_allocation`` (``:369-441``), ``triplet_tile_selector_bytes`` (``:444-449``).

Every 16-channel strip of a Kimi-K3 expert matrix holds 24 rate records; the 3.083333-bpw
profile gives it 74 trellis bits (22 x K3 + 2 x K4), and every exchange considered here (one K3
record to K2, another to K4) keeps that count.  The per-tile error surfaces come from one
reduction kernel (``qsrtb_tile_reduce``), the two 128-point Hadamards of the dense-H decomposition
from ``qsrtb_hadamard128``; the allocation itself works on ``[192, 224]`` cost surfaces with a
few torch operations, as in the reference.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping, Sequence

import torch

from . import _lib
from .records import RECORDS_PER_EXPERT, TILES_PER_RECORD_AXIS
from .tiles import _stream_ptr

HIGH_RATE_STRIP_BITS = 74
FIXED_K4_RECORDS = 2
TRANSFERABLE_RECORD_PAIRS = (RECORDS_PER_EXPERT - FIXED_K4_RECORDS) // 2


@dataclass(frozen=True)
class TileRateAllocation:
    """One flattened matrix tile-rate map and its selector cost."""

    tile_bits: tuple[int, ...]
    selected_p24_tiles: int
    candidate_p24_tiles: int
    selector_bytes: int

    @property
    def selected_fraction(self) -> float:
        return self.selected_p24_tiles / self.candidate_p24_tiles


@dataclass(frozen=True)
class RecordRateAllocation:
    """Best record-contiguous 74-bit schedule under tile cost surfaces."""

    donor_records: int
    tile_bits: tuple[int, ...]
    proxy_cost: float
    costs_by_donor_records: tuple[float, ...]


def _tile_reduce(a: torch.Tensor, b: torch.Tensor, mode: int) -> torch.Tensor:
    if not a.is_cuda or b.device != a.device:
        raise ValueError("tile error inputs must be on one CUDA device (there is no CPU path)")
    a, b = a.float().contiguous(), b.float().contiguous()
    rows, cols = a.shape
    out = torch.empty((rows // 16, cols // 16), dtype=torch.float64, device=a.device)
    with torch.cuda.device(a.device):
        _lib.check(
            _lib.lib().qsrtb_tile_reduce(a.data_ptr(), b.data_ptr(), rows, cols, cols, cols, mode, out.data_ptr(),
                                         _stream_ptr(a.device)),
            "qsrtb_tile_reduce",
        )
    return out


def tile_squared_error(reference: torch.Tensor, reconstruction: torch.Tensor) -> torch.Tensor:
    """One squared-error cost per 16-by-16 encoder tile, ``[K/16, N/16]`` float64."""

    if reference.ndim != 2 or reconstruction.shape != reference.shape:
        raise ValueError("tile error inputs must be aligned matrices")
    if reference.shape[0] % 16 or reference.shape[1] % 16:
        raise ValueError("tile error inputs must be 16-by-16 aligned")
    if not all(torch.is_floating_point(v) for v in (reference, reconstruction)):
        raise TypeError("tile error inputs must be floating point")
    return _tile_reduce(reference, reconstruction, 0)


def dense_h_tile_error_contributions(reference: torch.Tensor, reconstruction: torch.Tensor, hessian: torch.Tensor,
                                     suh: torch.Tensor, svh: torch.Tensor) -> torch.Tensor:
    """Partition ``trace(Eᵀ H E)`` of the physical error ``E`` over the encoder's tiles.

    ``reference`` / ``reconstruction`` are in the regularised ``[K, N]`` coordinates, ``hessian`` is
    the dense input covariance before conditioning.  The error is taken back to physical
    coordinates (had_l, ·suh, had_r, ·svh), multiplied by H, and the adjoint transform of that
    gradient is multiplied element by element with the regularised error; the tile sums add up
    to the complete quadratic form (individual tiles may be negative).
    """

    from .encoder import _hadamard

    if reference.ndim != 2 or reconstruction.shape != reference.shape:
        raise ValueError("dense-H tile inputs must be aligned matrices")
    if reference.shape[0] % 128 or reference.shape[1] % 128:
        raise ValueError("dense-H tile inputs must be 128-by-128 aligned")
    if hessian.shape != (reference.shape[0], reference.shape[0]):
        raise ValueError("dense-H input covariance does not match the K dimension")
    if suh.shape != (reference.shape[0],) or svh.shape != (reference.shape[1],):
        raise ValueError("dense-H scale vectors do not match the encoder matrix")
    values = (reference, reconstruction, hessian, suh, svh)
    if not all(torch.is_floating_point(v) for v in values):
        raise TypeError("dense-H tile inputs must be floating point")
    if not reference.is_cuda:
        raise ValueError("dense-H tile inputs must be on a CUDA device (there is no CPU path)")
    if not all(bool(torch.all(torch.isfinite(v))) for v in values):
        raise ValueError("dense-H tile inputs must be finite")
    if bool(torch.any(suh == 0)) or bool(torch.any(svh == 0)):
        raise ValueError("dense-H scale vectors must be nonzero")

    device = reference.device
    su = suh.to(device=device, dtype=torch.float32).contiguous()
    sv = svh.to(device=device, dtype=torch.float32).contiguous()
    error = reconstruction.float() - reference.float()
    physical = error.clone()
    _hadamard(physical, 0, su, per_col=False, divide=False, after=True)    # had_l, then rows * suh
    _hadamard(physical, 1, sv, per_col=True, divide=False, after=True)     # had_r, then columns * svh
    gradient = hessian.to(device=device, dtype=torch.float32) @ physical
    _hadamard(gradient, 1, sv, per_col=True, divide=False)                 # columns * svh, then had_r
    _hadamard(gradient, 0, su, per_col=False, divide=False)                # rows * suh, then had_l
    return _tile_reduce(error, gradient, 1)


def high_rate_record_bits(donor_records: int) -> tuple[int, ...]:
    """``N x K2, (22 - 2N) x K3, (N + 2) x K4``: always 74 bits per strip."""

    if not 0 <= donor_records <= TRANSFERABLE_RECORD_PAIRS:
        raise ValueError(f"donor records must lie in 0..{TRANSFERABLE_RECORD_PAIRS}")
    bits = (2,) * donor_records + (3,) * (22 - 2 * donor_records) + (4,) * (donor_records + FIXED_K4_RECORDS)
    if len(bits) != RECORDS_PER_EXPERT or sum(bits) != HIGH_RATE_STRIP_BITS:
        raise AssertionError("high-rate record schedule violated its bit budget")
    return bits


def record_rate_map(shape: tuple[int, int], *, rate_axis: str, donor_records: int) -> tuple[int, ...]:
    """One record-contiguous schedule expanded over a matrix's tile grid, row-major."""

    tiles_k, tiles_n = (dimension // 16 for dimension in shape)
    if rate_axis not in ("k", "n"):
        raise ValueError("rate axis must be 'k' or 'n'")
    rate_tiles, orthogonal = (tiles_k, tiles_n) if rate_axis == "k" else (tiles_n, tiles_k)
    if rate_tiles != RECORDS_PER_EXPERT * TILES_PER_RECORD_AXIS:
        raise ValueError("matrix does not contain Kimi-K3's 24 rate records")
    along = [b for b in high_rate_record_bits(donor_records) for _ in range(TILES_PER_RECORD_AXIS)]
    if rate_axis == "n":
        return tuple(along * orthogonal)
    return tuple(b for b in along for _ in range(orthogonal))


def _combined_costs(cost_surfaces: Sequence[Mapping[int, torch.Tensor]], what: str) -> dict[int, torch.Tensor]:
    if not cost_surfaces:
        raise ValueError(f"{what} requires at least one cost surface")
    shape = tuple(cost_surfaces[0][3].shape)
    for surface in cost_surfaces:
        if set(surface) != {2, 3, 4} or any(tuple(surface[b].shape) != shape for b in (2, 3, 4)):
            raise ValueError("K2/K3/K4 cost surfaces must share one shape")
    return {b: torch.stack([s[b].detach().double() for s in cost_surfaces]).sum(dim=0) for b in (2, 3, 4)}


def rate_map_proxy_cost(cost_surfaces: Sequence[Mapping[int, torch.Tensor]], tile_bits: Sequence[int]) -> torch.Tensor:
    """Sum of the tile costs a complete rate map selects (gate and up may both contribute)."""

    if not cost_surfaces:
        raise ValueError("rate-map scoring requires at least one cost surface")
    combined = _combined_costs(cost_surfaces, "rate-map scoring")
    shape = combined[3].shape
    if len(tile_bits) != shape[0] * shape[1] or any(isinstance(b, bool) or b not in (2, 3, 4) for b in tile_bits):
        raise ValueError("rate map does not cover the tile grid with K2/K3/K4")
    chosen = torch.tensor([int(b) for b in tile_bits], dtype=torch.int64, device=combined[3].device)
    table = torch.stack([combined[b].flatten() for b in (2, 3, 4)])
    return table.gather(0, (chosen - 2).unsqueeze(0)).sum()


def select_record_rate_allocation(cost_surfaces: Sequence[Mapping[int, torch.Tensor]], *, shape: tuple[int, int],
                                  rate_axis: str) -> RecordRateAllocation:
    """The cheapest of the twelve ``N K2, 22 - 2N K3, N + 2 K4`` schedules, N = 0..11 (ties to fewer donors)."""

    maps = [record_rate_map(shape, rate_axis=rate_axis, donor_records=n) for n in range(TRANSFERABLE_RECORD_PAIRS + 1)]
    costs = tuple(float(rate_map_proxy_cost(cost_surfaces, m)) for m in maps)
    best = min(range(len(costs)), key=lambda i: (costs[i], i))
    return RecordRateAllocation(donor_records=best, tile_bits=maps[best], proxy_cost=costs[best],
                                costs_by_donor_records=costs)


def _as_strips(value: torch.Tensor, *, rate_axis: str) -> torch.Tensor:
    """Tile costs ``[K/16, N/16]`` -> ``[strips, 24]``: one row per 16-channel strip."""

    if value.ndim != 2:
        raise ValueError("tile cost surfaces must be matrices")
    tiles_k, tiles_n = value.shape
    rate_tiles, orthogonal = (tiles_k, tiles_n) if rate_axis == "k" else (tiles_n, tiles_k)
    if rate_tiles != RECORDS_PER_EXPERT * TILES_PER_RECORD_AXIS:
        raise ValueError("tile costs do not contain 24 rate records")
    if rate_axis == "n":
        return value.reshape(orthogonal, RECORDS_PER_EXPERT, TILES_PER_RECORD_AXIS).permute(0, 2, 1).reshape(
            -1, RECORDS_PER_EXPERT)
    return value.reshape(RECORDS_PER_EXPERT, TILES_PER_RECORD_AXIS, orthogonal).permute(2, 1, 0).reshape(
        -1, RECORDS_PER_EXPERT)


def _from_strips(strips: torch.Tensor, *, rate_axis: str, shape: tuple[int, int]) -> torch.Tensor:
    tiles_k, tiles_n = shape
    orthogonal = tiles_n if rate_axis == "k" else tiles_k
    if tuple(strips.shape) != (orthogonal * TILES_PER_RECORD_AXIS, RECORDS_PER_EXPERT):
        raise ValueError("strip rates have the wrong matrix geometry")
    cube = strips.reshape(orthogonal, TILES_PER_RECORD_AXIS, RECORDS_PER_EXPERT)
    return (cube.permute(0, 2, 1) if rate_axis == "n" else cube.permute(2, 1, 0)).reshape(shape)


def tile_p24_allocation(cost_surfaces: Sequence[Mapping[int, torch.Tensor]], *, rate_axis: str,
                        force_fraction: float | None = None) -> TileRateAllocation:
    """P33 or P24 for every transferable tile pair of every strip.

    Records 22 and 23 stay K4; the others pair up as (0, 21), (1, 20), ... (10, 11).  Turning a pair
    from 3 + 3 into 2 + 4 keeps the strip at 74 bits and is taken where it lowers the summed cost
    (``c2[low] + c4[high] - c3[low] - c3[high] < 0``), or for the ``force_fraction`` of pairs with
    the smallest such difference.
    """

    if rate_axis not in ("k", "n"):
        raise ValueError("rate axis must be 'k' or 'n'")
    if not cost_surfaces:
        raise ValueError("tile allocation requires at least one cost surface")
    if force_fraction is not None and not 0 <= force_fraction <= 1:
        raise ValueError("forced P24 fraction must lie in [0, 1]")
    costs = _combined_costs(cost_surfaces, "tile allocation")
    shape = tuple(costs[3].shape)
    strips = {b: _as_strips(v, rate_axis=rate_axis) for b, v in costs.items()}
    lows = torch.arange(TRANSFERABLE_RECORD_PAIRS, device=strips[3].device)
    highs = 21 - lows
    delta = strips[2][:, lows] + strips[4][:, highs] - strips[3][:, lows] - strips[3][:, highs]
    if force_fraction is None:
        selected = delta < 0
    else:
        count = int(round(delta.numel() * force_fraction))
        selected = torch.zeros_like(delta, dtype=torch.bool)
        if count:
            selected.flatten()[torch.argsort(delta.flatten(), stable=True)[:count]] = True
    rates = torch.full_like(strips[3], 3, dtype=torch.int8)
    rates[:, 22:24] = 4
    rates[:, lows] = torch.where(selected, 2, 3).to(torch.int8)
    rates[:, highs] = torch.where(selected, 4, 3).to(torch.int8)
    if not bool(torch.all(rates.sum(dim=1) == HIGH_RATE_STRIP_BITS)):
        raise AssertionError("tile allocation violated the strip bit budget")
    candidate_tiles = strips[3].shape[0] * TRANSFERABLE_RECORD_PAIRS
    rate_map = _from_strips(rates, rate_axis=rate_axis, shape=shape)
    return TileRateAllocation(
        tile_bits=tuple(int(v) for v in rate_map.flatten().cpu()),
        selected_p24_tiles=int(torch.count_nonzero(selected)),
        candidate_p24_tiles=candidate_tiles,
        selector_bytes=(candidate_tiles + 7) // 8,    # one bit per transferable pair
    )


def triplet_tile_selector_bytes(*, upstream_shared: bool = True) -> int:
    """Bitmap bytes for one Kimi expert's three matrices (gate and up may share one map)."""

    one_map = (224 * TILES_PER_RECORD_AXIS * TRANSFERABLE_RECORD_PAIRS + 7) // 8
    return one_map * (2 if upstream_shared else 3)
