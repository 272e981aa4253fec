"""Routed-error scoring on the device against numbers the reference's own evaluators produced.

``tests/golden/scoring_golden.json`` is written by ``tests/golden/make_scoring_golden.py`` from
``qsrt.qsrt_candidates.functional_sse_by_request`` and ``qsrt.pooled_calibration`` run on the CPU.
Tolerances: the products here and in the reference are float32 sums in different orders (relative
error about 5e-7 of an output's norm); an SSE is a difference of two such outputs, so its relative
error grows by the ratio output / difference (up to 14 for the finer candidate): 1e-4 is asserted
for SSEs, 2e-5 for energies and second-moment statistics.
"""

import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import qsrt_oracle as oracle
from qsrt_b200 import coupled, linalg, pipeline, scoring, tables
from tests import helpers

pytestmark = pytest.mark.gpu

GOLDEN = json.loads((Path(__file__).parent / "golden" / "scoring_golden.json").read_text())


def _close(got, want, tolerance):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert np.all(np.abs(got - want) <= tolerance * np.abs(want)), (got, want)


def _case(device):
    source, candidates, x, gates, steps = helpers.scoring_inputs()
    move = lambda triplet: tuple(t.to(device) for t in triplet)   # noqa: E731
    return move(source), {k: move(v) for k, v in candidates.items()}, x.to(device), gates.to(device), steps


@pytest.mark.parametrize("activation", ["silu", "situ"])
def test_functional_sse_by_request_matches_reference(cuda_device, activation):
    source, candidates, x, gates, steps = _case(cuda_device)
    planes = linalg.split_tf32(x)
    teacher = scoring.expert_output(planes, scoring.ExpertOperands(*source), activation)
    for name, triplet in candidates.items():
        student = scoring.expert_output(planes, scoring.ExpertOperands(*triplet), activation)
        sse, energy, counts = scoring.functional_sse_by_request(teacher, student, gates, steps, helpers.SCORING_REQUESTS)
        want = GOLDEN[f"{activation}_{name}"]
        assert counts.tolist() == want["counts"]
        _close(sse, want["sse"], 1e-4)
        _close(energy, want["energy"], 2e-5)
        # the one-call form used by the encoder pipeline: the same numbers summed over the requests
        total, total_energy = scoring.routed_output_sse(x, gates, source, triplet, activation)
        _close(float(total), sum(want["sse"]), 1e-4)
        _close(float(total_energy), sum(want["energy"]), 2e-5)
    with pytest.raises(ValueError):
        scoring.functional_sse_by_request(teacher, teacher[:, :8], gates, steps, helpers.SCORING_REQUESTS)
    with pytest.raises(ValueError):
        scoring.functional_sse_by_request(teacher, teacher, gates, steps, {3: "a", 7: "b"})


@pytest.mark.parametrize("dtype_name", ["float64", "float32"])
def test_pooled_statistics_match_reference(cuda_device, dtype_name):
    source, candidates, x, gates, _ = _case(cuda_device)
    dtype = getattr(torch, dtype_name)
    source_middle = scoring.gated_middle(x, source[0], source[1], "situ")
    candidate_middle = scoring.gated_middle(x, candidates["coarse"][0], candidates["coarse"][1], "situ")
    stats = scoring.CandidateHiddenStatistics.zeros(256, device=cuda_device, dtype=dtype)
    stats.update(candidate_middle[:40], source_middle[:40], gates[:40])
    other = scoring.CandidateHiddenStatistics.zeros(256, device=cuda_device, dtype=dtype)
    other.update(candidate_middle[40:], source_middle[40:], gates[40:])
    stats.merge_(other)
    want = GOLDEN[f"statistics_{dtype_name}"]
    assert stats.rows == want["rows"]
    _close(stats.weight_sum, want["weight_sum"], 1e-6)
    _close(stats.weight_square_sum, want["weight_square_sum"], 1e-6)
    _close(stats.effective_sample_size, want["effective_sample_size"], 1e-6)
    probe = torch.linspace(-1.0, 1.0, 256, dtype=torch.float64, device=cuda_device)
    _close(float(stats.candidate_gram.trace()), want["candidate_gram_trace"], 2e-5)
    _close(float(probe @ stats.candidate_gram.double() @ probe), want["candidate_gram_probe"], 2e-5)
    _close(float(probe @ stats.candidate_source_cross.double() @ probe.flip(0)), want["candidate_source_cross_probe"], 1e-4)
    _close(float(stats.hidden_residual_gram.trace()), want["hidden_residual_gram_trace"], 1e-4)
    down_sse = scoring.decoded_down_sse(stats, candidates["coarse"][2].T, source[2].T)
    _close(float(down_sse), want["decoded_down_sse"], 2e-4 if dtype_name == "float32" else 1e-4)
    difference = scoring.decoded_down_sse_difference(stats, candidates["coarse"][2].T, candidates["fine"][2].T, source[2].T)
    _close(float(difference), want["decoded_down_sse_difference"], 2e-4 if dtype_name == "float32" else 1e-4)
    h2, evidence = scoring.candidate_h2(stats, max_local_alpha=0.75)
    _close(float(h2.trace()), want["h2_trace"], 2e-5)
    _close(float(probe @ h2.double() @ probe), want["h2_probe"], 2e-5)
    for key, value in want["h2_evidence"].items():
        _close(evidence[key], value, 2e-5)
    # the pooled form and the explicit routed error are the same quantity
    explicit, _ = scoring.routed_output_sse(x, gates, source, candidates["coarse"], "situ")
    _close(float(down_sse), float(explicit), 5e-4)
    with pytest.raises(ValueError):
        stats.update(candidate_middle[:, :8], source_middle[:, :8], gates)
    with pytest.raises(TypeError):
        scoring.CandidateHiddenStatistics.zeros(8, dtype=torch.float16)


def test_coupled_portfolio_matches_reference(cuda_device):
    source, candidates, x, gates, _ = _case(cuda_device)
    coordinates, executions = {}, {}
    for index, (name, triplet) in enumerate(candidates.items()):
        spec = coupled.CoupledHadamardSpec(intermediate_draw=index)
        executions[name] = coupled.CoupledHadamardExecution(hidden=512, intermediate=256, spec=spec)
        coordinates[name] = coupled.encode_coupled_weights(triplet, spec)
    batches = [{"input": x[:50], "route_weight": gates[:50], "row_index": torch.arange(0, 50)},
               {"input": x[50:], "route_weight": gates[50:], "row_index": torch.arange(50, x.shape[0])}]
    result = scoring.evaluate_coupled_candidate_portfolio_batches(
        batches, source=source, candidate_coordinates=coordinates, executions=executions)
    want = GOLDEN["portfolio"]
    assert result.routed_occurrences == want["routed_occurrences"]
    _close(result.source_energy, want["source_energy"], 2e-5)
    for name, value in want["candidate_sse"].items():
        _close(result.candidate_sse[name], value, 1e-4)
    with pytest.raises(ValueError):
        scoring.evaluate_coupled_candidate_portfolio_batches(
            [{"input": x[:4], "route_weight": gates[:4], "row_index": torch.tensor([3, 2, 1, 0])}],
            source=source, candidate_coordinates=coordinates, executions=executions)


def test_pipeline_routed_sse_matches_oracle_decode(cuda_device):
    """``encode_expert_batch(score=True)``: the stored payloads are decoded by the CPU restatement
    of the reference's decoder (pinned to its golden vectors) and scored in float64 with the
    formula of ``functional_sse_by_request``; the pipeline's device figure must agree to 1e-4."""

    g = torch.Generator().manual_seed(4321)
    hidden, inter, rows = 256, 128, 160
    experts = []
    for e in range(2):
        w1, w3 = torch.randn((inter, hidden), generator=g) * 0.05, torch.randn((inter, hidden), generator=g) * 0.05
        w2 = torch.randn((hidden, inter), generator=g) * 0.05
        x = torch.randn((rows, hidden), generator=g) * torch.exp(0.3 * torch.randn(hidden, generator=g))
        gates = torch.rand(rows, generator=g) * 0.5 + 0.05
        experts.append(pipeline.ExpertSource(w1.to(cuda_device), w3.to(cuda_device), w2.to(cuda_device),
                                             x.to(cuda_device), gates.to(cuda_device), e))
    payloads = pipeline.encode_expert_batch(experts, bits=3, device=cuda_device, layer_seed=2, score=True)
    lut = tables.sqg_xor_cheb_t12_bytes(3).numpy()
    for ex, payload in zip(experts, payloads):
        decoded = []
        for m in (payload.w1, payload.w3, payload.w2):
            states = oracle.unpack_trellis_states(m.trellis.cpu().numpy().reshape(-1, 16 * 3), 3).reshape(
                m.trellis.shape[0], m.trellis.shape[1], 256)
            decoded.append(torch.from_numpy(oracle.decode_weight(states, m.suh.cpu().numpy(), m.svh.cpu().numpy(), lut)).double().T)
        x, w = ex.rows.cpu().double(), ex.gates.cpu().double().square()

        def forward(w1, w3, w2):
            return (torch.nn.functional.silu(x @ w1.T) * (x @ w3.T)) @ w2.T

        teacher = forward(ex.w1.cpu().double(), ex.w3.cpu().double(), ex.w2.cpu().double())
        student = forward(*decoded)
        want_sse = float(((student - teacher).square().sum(dim=1) * w).sum())
        want_energy = float((teacher.square().sum(dim=1) * w).sum())
        _close(payload.routed_sse, want_sse, 1e-4)
        _close(payload.routed_energy, want_energy, 2e-5)
        assert 0.0 < payload.routed_sse < 0.2 * payload.routed_energy
