"""Host-side scoring logic on the CPU: the float64 pooled statistics, the pooled error forms and
the OAS-shrunk candidate covariance against the reference-made golden
(``tests/golden/scoring_golden.json``), and the request-epoch mask of the capture reducer.
The float32 products and the row reductions are device kernels and are covered by the GPU tests."""

import json
from pathlib import Path

import pytest
import torch
import torch.nn.functional as F

from qsrt_b200 import hessian, pipeline, scoring
from tests import helpers

GOLDEN = json.loads((Path(__file__).parent / "golden" / "scoring_golden.json").read_text())


def _middle(x, triplet):
    return pipeline.situ(F.linear(x, triplet[0]), F.linear(x, triplet[1]))


def test_float64_statistics_and_pooled_forms_match_reference():
    source, candidates, x, gates, _ = helpers.scoring_inputs()
    source_middle, candidate_middle = _middle(x, source), _middle(x, candidates["coarse"])
    stats = scoring.CandidateHiddenStatistics.zeros(256)
    stats.update(candidate_middle[:40], source_middle[:40], gates[:40])
    other = scoring.CandidateHiddenStatistics.zeros(256)
    other.update(candidate_middle[40:], source_middle[40:], gates[40:])
    stats.merge_(other)
    want = GOLDEN["statistics_float64"]
    assert stats.rows == want["rows"]
    for got, key in ((stats.weight_sum, "weight_sum"), (stats.weight_square_sum, "weight_square_sum"),
                     (stats.effective_sample_size, "effective_sample_size"),
                     (float(stats.candidate_gram.trace()), "candidate_gram_trace"),
                     (float(stats.hidden_residual_gram.trace()), "hidden_residual_gram_trace")):
        assert got == pytest.approx(want[key], rel=1e-6), key
    down = scoring.decoded_down_sse(stats, candidates["coarse"][2].T, source[2].T)
    assert float(down) == pytest.approx(want["decoded_down_sse"], rel=1e-5)
    difference = scoring.decoded_down_sse_difference(stats, candidates["coarse"][2].T, candidates["fine"][2].T, source[2].T)
    assert float(difference) == pytest.approx(want["decoded_down_sse_difference"], rel=1e-5)
    h2, evidence = scoring.candidate_h2(stats)
    assert float(h2.trace()) == pytest.approx(want["h2_trace"], rel=1e-6)
    for key, value in want["h2_evidence"].items():
        assert evidence[key] == pytest.approx(value, rel=1e-6), key
    moved = stats.to(device="cpu", dtype=torch.float32)
    assert moved.candidate_gram.dtype == torch.float32 and moved.rows == stats.rows
    lean = scoring.CandidateHiddenStatistics.zeros(256, retain_source_gram=False)
    lean.update(candidate_middle, source_middle, gates)
    with pytest.raises(ValueError):
        scoring.decoded_down_sse(lean, candidates["coarse"][2].T, source[2].T)
    with pytest.raises(ValueError):
        stats.merge_(lean)
    with pytest.raises(ValueError):
        scoring.candidate_h2(scoring.CandidateHiddenStatistics.zeros(8))
    with pytest.raises(ValueError):
        scoring.PooledPortfolioEvaluation({}, 1.0, 1)


def test_request_step_mask():
    observations = (torch.tensor([0, 1, 2, 5, 9, 10, 12], dtype=torch.int64) << 32) | torch.arange(7)
    mask = hessian.request_step_mask(observations, request_step_min=2, request_step_max=9, request_steps=None)
    assert mask.tolist() == [False, False, True, True, True, False, False]
    mask = hessian.request_step_mask(observations, request_step_min=0, request_step_max=None, request_steps=[1, 12])
    assert mask.tolist() == [False, True, False, False, False, False, True]
    with pytest.raises(ValueError):
        hessian.StreamingHessianReducer(128, [0], device=torch.device("cpu"))
