"""High-rate equal-byte allocation and the tile error surfaces it ranks, against values the
reference's own CPU code produced (tests/golden/allocation_golden.npz, made by
tests/golden/make_allocation_golden.py), following the reference's tests/test_high_rate_allocation.py.
"""

import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

from qsrt_b200 import allocation as al
from tests.helpers import allocation_cost_surfaces, allocation_inputs

GOLDEN = np.load(Path(__file__).parent / "golden" / "allocation_golden.npz")


def digest(bits) -> bytes:
    return hashlib.sha256(np.asarray(bits, dtype=np.uint8).tobytes()).digest()


def test_record_schedules_keep_the_74_bit_budget():
    for donors in range(al.TRANSFERABLE_RECORD_PAIRS + 1):
        bits = al.high_rate_record_bits(donors)
        assert len(bits) == 24 and sum(bits) == 74 == al.HIGH_RATE_STRIP_BITS
        assert bits.count(2) == donors and bits.count(4) == donors + 2
    with pytest.raises(ValueError):
        al.high_rate_record_bits(12)
    assert al.triplet_tile_selector_bytes() == 4928 and al.triplet_tile_selector_bytes(upstream_shared=False) == 7392
    with pytest.raises(ValueError, match="24 rate records"):
        al.record_rate_map((3072, 3584), rate_axis="n", donor_records=0)
    with pytest.raises(ValueError, match="rate axis"):
        al.record_rate_map((3072, 3584), rate_axis="x", donor_records=0)


@pytest.mark.parametrize(("axis", "shape"), [("k", (3072, 3584)), ("n", (3584, 3072))])
def test_allocations_match_the_reference(axis, shape):
    surfaces = allocation_cost_surfaces(axis)
    record = al.select_record_rate_allocation(surfaces, shape=shape, rate_axis=axis)
    assert record.donor_records == int(GOLDEN[f"record_{axis}_donors"])
    assert np.array_equal(np.asarray(record.costs_by_donor_records), GOLDEN[f"record_{axis}_costs"])
    assert digest(record.tile_bits) == GOLDEN[f"record_{axis}_map"].tobytes()
    assert record.proxy_cost == min(record.costs_by_donor_records)
    assert float(al.rate_map_proxy_cost(surfaces, record.tile_bits)) == record.proxy_cost
    for name, fraction in (("free", None), ("quarter", 0.25)):
        tile = al.tile_p24_allocation(surfaces, rate_axis=axis, force_fraction=fraction)
        assert tile.selected_p24_tiles == int(GOLDEN[f"tile_{axis}_{name}_selected"])
        assert digest(tile.tile_bits) == GOLDEN[f"tile_{axis}_{name}_map"].tobytes()
        assert tile.candidate_p24_tiles == 224 * 8 * 11 and tile.selector_bytes == 2464
        grid = np.asarray(tile.tile_bits).reshape(surfaces[0][3].shape)
        strips = grid if axis == "n" else grid.T            # one row per orthogonal tile
        assert (strips.reshape(224, 24, 8).sum(axis=1) == 74).all()
    assert al.tile_p24_allocation(surfaces, rate_axis=axis, force_fraction=0.0).selected_p24_tiles == 0
    free = al.tile_p24_allocation(surfaces, rate_axis=axis)
    # a tile-local choice can only improve on the all-P33 map it starts from
    assert float(al.rate_map_proxy_cost(surfaces, free.tile_bits)) <= record.costs_by_donor_records[0]


def test_allocation_argument_errors():
    surfaces = allocation_cost_surfaces("k")
    with pytest.raises(ValueError, match="at least one cost surface"):
        al.tile_p24_allocation([], rate_axis="k")
    with pytest.raises(ValueError, match="fraction"):
        al.tile_p24_allocation(surfaces, rate_axis="k", force_fraction=1.5)
    with pytest.raises(ValueError, match="share one shape"):
        al.tile_p24_allocation([{2: surfaces[0][2], 3: surfaces[0][3]}], rate_axis="k")
    with pytest.raises(ValueError, match="cover the tile grid"):
        al.rate_map_proxy_cost(surfaces, (3,) * 10)
    with pytest.raises(ValueError, match="24 rate records"):
        al.tile_p24_allocation(surfaces, rate_axis="n")
    with pytest.raises(ValueError, match="CUDA"):
        al.tile_squared_error(torch.zeros(16, 16), torch.zeros(16, 16))


@pytest.mark.gpu
def test_tile_squared_error_matches_the_reference(cuda_device):
    reference, reconstruction, _, _, _ = allocation_inputs()
    got = al.tile_squared_error(reference.to(cuda_device), reconstruction.to(cuda_device))
    assert got.dtype == torch.float64 and tuple(got.shape) == (16, 24)
    np.testing.assert_allclose(got.cpu().numpy(), GOLDEN["tile_squared_error"], rtol=1e-13, atol=0)
    # physical 16 x 16 tiles: a single perturbed element moves exactly one tile's cost
    bumped = reconstruction.clone()
    bumped[37, 201] += 1.0
    moved = al.tile_squared_error(reference.to(cuda_device), bumped.to(cuda_device)) - got
    assert int((moved != 0).sum()) == 1 and float(moved[2, 12]) > 0
    with pytest.raises(ValueError, match="16-by-16"):
        al.tile_squared_error(reference[:250].to(cuda_device), reconstruction[:250].to(cuda_device))
    with pytest.raises(TypeError):
        al.tile_squared_error(reference.to(cuda_device).int(), reconstruction.to(cuda_device).int())


@pytest.mark.gpu
def test_dense_h_contributions_match_the_reference_and_sum_to_the_quadratic_form(cuda_device):
    reference, reconstruction, hessian, suh, svh = allocation_inputs()
    dev = [t.to(cuda_device) for t in (reference, reconstruction, hessian, suh, svh)]
    got = al.dense_h_tile_error_contributions(*dev).cpu().numpy()
    want = GOLDEN["dense_h"]
    # float32 GEMM and transforms on both sides: tolerance relative to the surface's scale
    assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max()
    # the tile contributions add up to trace(E^T H E) of the physical error (FP64 check)
    from oracle.qsrt_oracle import normalized_hadamard

    had = torch.from_numpy(normalized_hadamard(128)).double()
    error = (reconstruction - reference).double()
    physical = torch.matmul(had, error.reshape(-1, 128, error.shape[1])).reshape_as(error) * suh.double()[:, None]
    physical = torch.matmul(physical.reshape(error.shape[0], -1, 128), had).reshape_as(error) * svh.double()[None, :]
    total = float(torch.sum(physical * (hessian.double() @ physical)))
    assert abs(got.sum() - total) <= 2e-5 * abs(total)
    with pytest.raises(ValueError, match="nonzero"):
        al.dense_h_tile_error_contributions(dev[0], dev[1], dev[2], torch.zeros_like(dev[3]), dev[4])
    with pytest.raises(ValueError, match="128-by-128"):
        al.dense_h_tile_error_contributions(dev[0][:, :368], dev[1][:, :368], dev[2], dev[3], dev[4][:368])
