"""Coupled signed block-Hadamard coordinates: CPU pin of the oracle, GPU parity of the kernels."""

import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import coupled_oracle as co
from tests.helpers import coupled_inputs

GOLDEN = json.loads((Path(__file__).resolve().parent / "golden" / "coupled_golden.json").read_text())


def _sha(a) -> str:
    return hashlib.sha256(np.ascontiguousarray(a, dtype=np.float32).tobytes()).hexdigest()


@pytest.mark.parametrize("draw", [0, 3])
def test_oracle_matches_reference_digests(draw):
    """Digests produced by the reference's qsrt.qsrt_coupled (tests/golden/make_coupled_golden.py)."""

    w1, w3, w2, rows, h13, h2 = [t.numpy() for t in coupled_inputs()]
    g = GOLDEN[f"draw{draw}"]
    c1, c3, c2 = co.encode_coupled_weights(w1, w3, w2, intermediate_draw=draw)
    assert (_sha(c1), _sha(c3), _sha(c2)) == (g["w1"], g["w3"], g["w2"])
    s0, s2, s3 = co.rotation_signs(512, 0, 0), co.rotation_signs(128, draw, 2), co.rotation_signs(512, 0, 3)
    assert _sha(co.signed_block_hadamard(rows, 512, s0, 1)) == g["inputs"]
    assert _sha(co.signed_block_hadamard(co.signed_block_hadamard(h13, 512, s0, 0), 512, s0, 1)) == g["h13"]
    assert _sha(co.signed_block_hadamard(co.signed_block_hadamard(h2, 128, s2, 0), 128, s2, 1)) == g["h2"]
    assert _sha(co.signed_block_hadamard(rows[:, :128], 128, s2, 1)) == g["post_rows"]
    assert _sha(co.signed_block_hadamard(rows, 512, s3, 1, inverse=True)) == g["decode_output"]


@pytest.mark.gpu
@pytest.mark.parametrize("draw", [0, 3])
def test_kernels_match_reference_digests_bit_for_bit(cuda_device, draw):
    from qsrt_b200 import coupled

    w1, w3, w2, rows, h13, h2 = [t.to(cuda_device) for t in coupled_inputs()]
    g = GOLDEN[f"draw{draw}"]
    spec = coupled.CoupledHadamardSpec(intermediate_draw=draw)
    c1, c3, c2 = coupled.encode_coupled_weights((w1, w3, w2), spec)
    assert (_sha(c1.cpu().numpy()), _sha(c3.cpu().numpy()), _sha(c2.cpu().numpy())) == (g["w1"], g["w3"], g["w2"])
    ex = coupled.CoupledHadamardExecution(hidden=512, intermediate=128, spec=spec)
    assert _sha(ex.transform_inputs(rows).cpu().numpy()) == g["inputs"]
    assert _sha(ex.transform_h13(h13).cpu().numpy()) == g["h13"]
    assert _sha(ex.transform_h2(h2).cpu().numpy()) == g["h2"]
    assert _sha(ex.transform_postactivation_rows(rows[:, :128]).cpu().numpy()) == g["post_rows"]
    assert _sha(ex.decode_output(rows).cpu().numpy()) == g["decode_output"]


@pytest.mark.gpu
def test_coupled_execution_closes(cuda_device):
    """Transformed weights executed in transformed coordinates reproduce the source expert
    (closure property of tests/test_qsrt_coupled.py in the reference), and congruence
    preserves quadratic forms."""

    from qsrt_b200 import coupled, pipeline

    w1, w3, w2, rows, h13, _ = [t.to(cuda_device) for t in coupled_inputs()]
    spec = coupled.CoupledHadamardSpec(intermediate_draw=5)
    ex = coupled.CoupledHadamardExecution(hidden=512, intermediate=128, spec=spec)
    coupled_weights = coupled.encode_coupled_weights((w1, w3, w2), spec)
    got = ex.execute(rows, coupled_weights)
    expect = pipeline.situ(rows @ w1.T, rows @ w3.T) @ w2.T
    assert float((got - expect).norm() / expect.norm()) < 1e-5
    x = ex.transform_inputs(rows)
    q_src = torch.einsum("ri,ij,rj->r", rows.double(), h13.double(), rows.double())
    q_new = torch.einsum("ri,ij,rj->r", x.double(), ex.transform_h13(h13).double(), x.double())
    assert float((q_src - q_new).abs().max() / q_src.abs().max()) < 1e-5
    for block in (128, 256, 512):
        y = coupled.block_hadamard(coupled.block_hadamard(rows, block_size=block, dim=1), block_size=block, dim=1)
        assert float((y - rows).abs().max()) < 1e-5
        m = torch.randn((1024, 96), device=cuda_device)
        z = coupled.block_hadamard(coupled.block_hadamard(m, block_size=block, dim=0), block_size=block, dim=0)
        assert float((z - m).abs().max()) < 1e-5
        ref = torch.from_numpy(co.block_hadamard(m.cpu().numpy(), block, 0))
        assert torch.equal(coupled.block_hadamard(m, block_size=block, dim=0).cpu(), ref)
    with pytest.raises(ValueError):
        coupled.block_hadamard(rows[:, :100], block_size=128, dim=1)
    with pytest.raises(ValueError):
        coupled.CoupledHadamardSpec(residual_draw=1)
