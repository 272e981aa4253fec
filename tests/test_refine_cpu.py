"""Host-side logic of the dense-H path refinement: configuration, guidance validation, objectives,
and the refusal to run without the CUDA kernels."""

import pytest
import torch

from qsrt_b200 import refine
from tests import helpers


def test_config_from_quant_args_maps_every_key():
    config = refine.config_from_quant_args({
        "h2_viterbi_refine_sweeps": 3, "h2_viterbi_refine_alternate_order": False,
        "h2_viterbi_refine_dither_scales": [0.1, 0.2], "h2_viterbi_refine_patterns": 4,
        "h2_viterbi_refine_seed": 9, "h2_viterbi_refine_max_batch": 32, "h2_viterbi_refine_fp64_score": True,
    })
    assert config == refine.H2ViterbiRefineConfig(
        sweeps=3, alternate_sweep_order=False, dither_scales=(0.1, 0.2), num_dither_patterns=4, seed=9,
        max_quantizer_batch=32, score_dtype=torch.float64)
    assert refine.config_from_quant_args({}) == refine.H2ViterbiRefineConfig()


def test_dense_h_objective_matches_direct_expression():
    g = torch.Generator().manual_seed(1)
    weight, recon = torch.randn((32, 48), generator=g), torch.randn((32, 48), generator=g)
    hessian = helpers.spd_hessian(32, 3.0, 2)
    column_weights = torch.rand(48, generator=g)
    error = (weight - recon).double()
    direct = float(torch.sum(error * (hessian.double() @ error) * column_weights.double()))
    assert abs(refine.dense_h_objective(weight, recon, hessian, column_weights=column_weights,
                                        chunk_columns=20) - direct) < 1e-9 * abs(direct)
    guidance = refine.ViterbiGradientGuidance(gradient=torch.randn((32, 48), generator=g), anchor=weight,
                                              anchor_id="a", objective_id="o", strength=0.25)
    quadratic, linear, total = refine.dense_h_guided_objective(weight, recon, hessian, guidance)
    want = 0.25 * float(torch.sum(guidance.gradient.double() * (recon.double() - weight.double())))
    assert abs(linear - want) < 1e-9 * abs(want) and total == quadratic + linear
    with pytest.raises(ValueError, match="one rank-2 shape"):
        refine.dense_h_objective(weight, recon[:-1], hessian)
    with pytest.raises(ValueError, match="Hessian shape"):
        refine.dense_h_objective(weight, recon, hessian[:-1])
    with pytest.raises(ValueError, match="chunk_columns"):
        refine.dense_h_objective(weight, recon, hessian, chunk_columns=0)
    with pytest.raises(ValueError, match="nonnegative"):
        refine.dense_h_objective(weight, recon, hessian, column_weights=-column_weights)


def test_guidance_validation_and_low_rank_linear_term():
    g = torch.Generator().manual_seed(2)
    left, right = torch.randn((16, 3), generator=g), torch.randn((3, 32), generator=g)
    anchor, candidate = torch.randn((16, 32), generator=g), torch.randn((16, 32), generator=g)
    low = refine.LowRankViterbiGradientGuidance(left=left, right=right, anchor=anchor, anchor_id="a",
                                                objective_id="o", strength=2.0)
    low.validate((16, 32))
    want = 2.0 * float(torch.sum((left.double() @ right.double()) * (candidate.double() - anchor.double())))
    assert abs(low.linear_term(candidate, dtype=torch.float64) - want) < 1e-9 * abs(want)
    assert torch.allclose(low.rows(slice(0, 16), device="cpu", dtype=torch.float32), left @ right)
    with pytest.raises(ValueError, match="incompatible geometry"):
        low.validate((16, 48))
    dense = refine.ViterbiGradientGuidance(gradient=anchor, anchor=anchor, anchor_id="", objective_id="o")
    with pytest.raises(ValueError, match="identities"):
        dense.validate((16, 32))
    with pytest.raises(ValueError, match="do not match the encoded matrix"):
        dense.validate((32, 32))
    bad = refine.ViterbiGradientGuidance(gradient=anchor, anchor=anchor, anchor_id="a", objective_id="o", strength=-1.0)
    with pytest.raises(ValueError, match="finite and nonnegative"):
        bad.validate((16, 32))
    integer = refine.ViterbiGradientGuidance(gradient=anchor.long(), anchor=anchor, anchor_id="a", objective_id="o")
    with pytest.raises(TypeError):
        integer.validate((16, 32))


def test_refinement_refuses_cpu_tensors():
    weight = torch.zeros((16, 16))
    with pytest.raises(ValueError, match="requires CUDA"):
        refine.refine_h2_viterbi_paths(weight, torch.eye(16), weight, torch.zeros((1, 1, 256), dtype=torch.int16), {})


def test_target_shifts_complete_the_square():
    g = torch.Generator().manual_seed(3)
    target, gradient = torch.randn((8, 12), generator=g), torch.randn((8, 12), generator=g)
    weight = torch.rand((8, 12), generator=g) + 0.5
    shifted = refine.shift_elementwise_target(target, gradient, strength=0.8, quadratic_weight=weight)
    # stationarity of a (q - t)^2 + s g q at q = shifted
    assert torch.allclose(2 * weight * (shifted - target) + 0.8 * gradient, torch.zeros_like(target), atol=1e-6)
    assert torch.equal(refine.shift_elementwise_target(target, gradient, strength=0.0), target)
    with pytest.raises(ValueError, match="matching shapes"):
        refine.shift_elementwise_target(target, gradient[:-1], strength=1.0)
    with pytest.raises(ValueError, match="finite and positive"):
        refine.shift_elementwise_target(target, gradient, strength=1.0, quadratic_weight=0.0)
    with pytest.raises(TypeError):
        refine.shift_elementwise_target(target.long(), gradient, strength=1.0)

    row, column = helpers.spd_hessian(8, 4.0, 5).double(), helpers.spd_hessian(12, 6.0, 6).double()
    t64, g64 = target.double(), gradient.double()
    two = refine.shift_two_sided_target(t64, g64, row, column, strength=0.6)
    # gradient of tr(E^T R E C) + s <G, Q> vanishes at Q = two
    residual = 2 * row @ (two - t64) @ column + 0.6 * g64
    assert float(residual.abs().max()) < 1e-10
    anchor = torch.zeros_like(t64)
    quadratic, linear, total = refine.two_sided_guided_objective(t64, two, anchor, g64, row, column, strength=0.6)
    assert float(total) == float(quadratic + linear)
    bumped = two + 1e-3 * torch.randn(two.shape, generator=g, dtype=torch.float64)
    assert float(refine.two_sided_guided_objective(t64, bumped, anchor, g64, row, column, strength=0.6)[2]) > float(total)
    with pytest.raises(ValueError, match="row Hessian"):
        refine.shift_two_sided_target(t64, g64, column, column, strength=0.6)
