"""MXFP4 source ingest against SHA-256 digests of the reference's own dequant output."""

import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import mxfp4_oracle as mo
from qsrt_b200 import mxfp4

GOLDEN = json.loads((Path(__file__).parent / "golden" / "mxfp4_golden.json").read_text())


def sha(a) -> str:
    if isinstance(a, torch.Tensor):
        a = a.detach().cpu().contiguous().numpy()
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_oracle_matches_reference_digests(name):
    case = GOLDEN[name]
    packed, scale = mo.seeded_source(case["rows"], case["cols"], case["seed"], corner_cases=case["corner_cases"])
    w = mo.dequant(packed, scale)
    assert sha(w) == case["plain"]
    assert sha(w.T) == case["transposed"]


def test_host_helpers_round_trip():
    codes = torch.randint(0, 16, (5, 64), dtype=torch.uint8, generator=torch.Generator().manual_seed(1))
    packed = mxfp4.pack_codes(codes)
    assert torch.equal(mxfp4.unpack_codes(packed), codes)
    assert torch.equal(mxfp4.code_values(torch.tensor([5, 13], dtype=torch.uint8)), torch.tensor([3.0, -3.0]))
    assert torch.equal(mxfp4.scale_factors(torch.tensor([127, 121], dtype=torch.uint8)), torch.tensor([1.0, 2.0 ** -6]))
    with pytest.raises(TypeError):
        mxfp4.unpack_codes(codes.int())
    with pytest.raises(ValueError):
        mxfp4.pack_codes(codes[:, :63])
    with pytest.raises(ValueError, match="CUDA"):
        mxfp4.dequant(packed, torch.full((5, 2), 127, dtype=torch.uint8))


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_kernel_matches_reference_digests_in_both_orientations(name):
    case = GOLDEN[name]
    packed, scale = mo.seeded_source(case["rows"], case["cols"], case["seed"], corner_cases=case["corner_cases"])
    p, s = torch.from_numpy(packed).cuda(), torch.from_numpy(scale).cuda()
    plain = mxfp4.dequant(p, s)
    assert plain.shape == (case["rows"], case["cols"]) and plain.dtype == torch.float32
    turned = mxfp4.dequant_encoder_orientation(p, s)
    assert turned.shape == (case["cols"], case["rows"])
    if case["corner_cases"]:
        # 0 * inf: the GPU's NaN has another payload than the host's, so digests cannot match;
        # every other value (subnormals, infinities, signed zeros) must agree in its bits with
        # the restatement that the reference digest pins on the CPU
        want = mo.dequant(packed, scale)
        for got, ref in ((plain.cpu().numpy(), want), (turned.cpu().numpy(), np.ascontiguousarray(want.T))):
            nan = np.isnan(ref)
            assert nan.any() and np.array_equal(np.isnan(got), nan)
            assert np.array_equal(got.view(np.uint32)[~nan], ref.view(np.uint32)[~nan])
        return
    assert sha(plain) == case["plain"]
    assert sha(turned) == case["transposed"]


@pytest.mark.gpu
def test_kernel_rejects_ragged_inputs_and_handles_empty():
    p = torch.zeros((4, 24), dtype=torch.uint8, device="cuda")   # 48 inputs: not a multiple of 32
    with pytest.raises(ValueError, match="do not cover"):
        mxfp4.dequant(p, torch.zeros((4, 1), dtype=torch.uint8, device="cuda"))
    with pytest.raises(ValueError):
        mxfp4.dequant(p[:, :16], torch.zeros((3, 1), dtype=torch.uint8, device="cuda"))
    with pytest.raises(TypeError):
        mxfp4.dequant(p.int(), torch.zeros((4, 1), dtype=torch.uint8, device="cuda"))
    empty = mxfp4.dequant(torch.zeros((0, 16), dtype=torch.uint8, device="cuda"),
                          torch.zeros((0, 1), dtype=torch.uint8, device="cuda"))
    assert empty.shape == (0, 32)
    # a row count that is not a multiple of the 32-row transposition tile
    packed, scale = mo.seeded_source(45, 160, 9)
    got = mxfp4.dequant_encoder_orientation(torch.from_numpy(packed).cuda(), torch.from_numpy(scale).cuda())
    assert np.array_equal(got.cpu().numpy(), mo.dequant(packed, scale).T, equal_nan=True)


@pytest.mark.gpu
@pytest.mark.parametrize("round_bf16", [True, False])
def test_fused_ingest_into_coupled_coordinates_is_bit_identical(round_bf16):
    """MXFP4 source -> coupled coordinates in one pass per matrix equals dequantising (pinned
    above to the reference's digests), optionally rounding to bfloat16 as a checkpoint holds the
    source, and then ``encode_coupled_weights`` (pinned to the reference's digests in
    tests/test_coupled.py), bit for bit."""

    from qsrt_b200 import coupled

    hidden, inter = 1024, 256
    sources, dense = [], []
    for index, (rows, cols) in enumerate(((inter, hidden), (inter, hidden), (hidden, inter))):
        packed, scale = mo.seeded_source(rows, cols, 40 + index)
        p, s = torch.from_numpy(packed).cuda(), torch.from_numpy(scale).cuda()
        sources.append((p, s))
        w = mxfp4.dequant(p, s)
        dense.append(w.to(torch.bfloat16).float() if round_bf16 else w)
    for draw in (0, 3):
        spec = coupled.CoupledHadamardSpec(intermediate_draw=draw)
        want = coupled.encode_coupled_weights(tuple(dense), spec)
        got = coupled.encode_coupled_weights_mxfp4(tuple(sources), spec, round_bf16=round_bf16)
        for a, b in zip(got, want):
            assert a.shape == b.shape and torch.equal(a, b)
    with pytest.raises(ValueError):
        coupled.encode_coupled_weights_mxfp4((sources[0], sources[1], sources[1]), coupled.CoupledHadamardSpec())
    with pytest.raises(TypeError):
        coupled.encode_coupled_weights_mxfp4(((sources[0][0].float(), sources[0][1]), sources[1], sources[2]),
                                             coupled.CoupledHadamardSpec())
