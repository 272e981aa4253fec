"""Generate tests/golden/scoring_golden.json from the reference's own scoring code (CPU).

    PYTHONPATH=<reference checkout> python tests/golden/make_scoring_golden.py

The seeded case of tests.helpers.scoring_inputs goes through

* qsrt.qsrt_candidates.functional_sse_by_request on explicit expert outputs (SiLU and SiTU experts),
* qsrt.pooled_calibration.CandidateHiddenStatistics.update / decoded_down_sse /
  decoded_down_sse_difference / candidate_h2,
* qsrt.pooled_calibration.evaluate_coupled_candidate_portfolio_batches with two candidates that use
  different intermediate draws of the coupled coordinates.

Every stored figure is a plain float64 number (sums, traces, probes of the matrices); the tests
compare at the tolerance of a float32 product summed in another order.
"""

import json
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

from qsrt.coupled_expert_study import CoupledTriplet
from qsrt.pooled_calibration import (CandidateHiddenStatistics, candidate_h2, decoded_down_sse,
                                     decoded_down_sse_difference, evaluate_coupled_candidate_portfolio_batches)
from qsrt.qsrt_candidates import functional_sse_by_request
from qsrt.qsrt_coupled import CoupledHadamardExecution, CoupledHadamardSpec, encode_coupled_weights
from qsrt.tp_simulator import situ

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from tests.helpers import SCORING_REQUESTS, scoring_inputs  # noqa: E402


def expert_output(x, triplet, activation):
    gate, up = F.linear(x, triplet[0]), F.linear(x, triplet[1])
    middle = F.silu(gate) * up if activation == "silu" else situ(gate, up)
    return middle, F.linear(middle, triplet[2])


def main() -> None:
    source, candidates, x, gates, steps = scoring_inputs()
    out = {}
    for activation in ("silu", "situ"):
        _, teacher = expert_output(x, source, activation)
        for name, triplet in candidates.items():
            _, student = expert_output(x, triplet, activation)
            sse, energy, counts = functional_sse_by_request(teacher, student, gates, steps, SCORING_REQUESTS)
            out[f"{activation}_{name}"] = {"sse": sse.tolist(), "energy": energy.tolist(), "counts": counts.tolist()}

    # pooled sufficient statistics of the "coarse" candidate (SiTU middle rows), in two row chunks
    source_middle, _ = expert_output(x, source, "situ")
    candidate_middle, _ = expert_output(x, candidates["coarse"], "situ")
    for dtype_name, dtype in (("float64", torch.float64), ("float32", torch.float32)):
        stats = CandidateHiddenStatistics.zeros(source_middle.shape[1], dtype=dtype)
        stats.update(candidate_middle[:40], source_middle[:40], gates[:40])
        other = CandidateHiddenStatistics.zeros(source_middle.shape[1], dtype=dtype)
        other.update(candidate_middle[40:], source_middle[40:], gates[40:])
        stats.merge_(other)
        down_sse = decoded_down_sse(stats, candidates["coarse"][2].T, source[2].T)
        difference = decoded_down_sse_difference(stats, candidates["coarse"][2].T, candidates["fine"][2].T, source[2].T)
        h2, evidence = candidate_h2(stats, max_local_alpha=0.75)
        probe = torch.linspace(-1.0, 1.0, h2.shape[0], dtype=h2.dtype)
        out[f"statistics_{dtype_name}"] = {
            "weight_sum": stats.weight_sum, "weight_square_sum": stats.weight_square_sum, "rows": stats.rows,
            "effective_sample_size": stats.effective_sample_size,
            "candidate_gram_trace": float(stats.candidate_gram.trace()),
            "candidate_gram_probe": float(probe @ stats.candidate_gram.to(h2.dtype) @ probe),
            "candidate_source_cross_probe": float(probe @ stats.candidate_source_cross.to(h2.dtype) @ probe.flip(0)),
            "candidate_residual_cross_probe": float(probe @ stats.candidate_residual_cross.to(h2.dtype) @ probe.flip(0)),
            "hidden_residual_gram_trace": float(stats.hidden_residual_gram.trace()),
            "decoded_down_sse": float(down_sse), "decoded_down_sse_difference": float(difference),
            "h2_probe": float(probe @ h2 @ probe), "h2_trace": float(h2.trace()),
            "h2_evidence": {k: float(v) for k, v in evidence.items()},
        }

    # coupled portfolio: one shared source forward, candidates with their own intermediate draw
    reference = CoupledTriplet(*source)
    coordinates, executions = {}, {}
    for index, (name, triplet) in enumerate(candidates.items()):
        spec = CoupledHadamardSpec(intermediate_draw=index)
        executions[name] = CoupledHadamardExecution(hidden=reference.hidden, intermediate=reference.intermediate, spec=spec)
        coordinates[name] = CoupledTriplet(*encode_coupled_weights(triplet, spec))
    batches = [{"input": x[:50], "route_weight": gates[:50], "row_index": torch.arange(0, 50)},
               {"input": x[50:], "route_weight": gates[50:], "row_index": torch.arange(50, x.shape[0])}]
    portfolio = evaluate_coupled_candidate_portfolio_batches(batches, source=reference, candidate_coordinates=coordinates,
                                                             executions=executions)
    out["portfolio"] = {"candidate_sse": dict(portfolio.candidate_sse), "source_energy": portfolio.source_energy,
                        "routed_occurrences": portfolio.routed_occurrences}
    path = ROOT / "tests" / "golden" / "scoring_golden.json"
    path.write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
    print("wrote", path)


if __name__ == "__main__":
    main()
