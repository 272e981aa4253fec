"""Generate tests/golden/refine_golden.npz from the reference's own refinement code.

    PYTHONPATH=<reference checkout> python tests/golden/make_refine_golden.py

qsrt.h2_viterbi_refine.refine_h2_viterbi_paths runs on the CPU; its ``quantize_tiles`` callback is
the C restatement of the reference's tile search (bit-exact with the reference CUDA kernel on the
pinned fixtures).  The starting point of every case is the independent tile-by-tile encoding of
the seeded weight.  Stored: initial and refined state grids, refined reconstruction and the sweep
statistics.
"""

import sys
from pathlib import Path

import numpy as np
import torch

from qsrt.gradient_guided_viterbi import ViterbiGradientGuidance
from qsrt.h2_viterbi_refine import H2ViterbiRefineConfig, refine_h2_viterbi_paths

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import qsrt_oracle  # noqa: E402
from tests.helpers import REFINE_CASES, matrix_to_tc_tiles, refine_case_inputs, tc_tiles_to_matrix  # noqa: E402

STAT_KEYS = ("objective_before", "objective_after", "quadratic_before", "quadratic_after", "linear_before",
             "linear_after", "accepted_tiles", "proposed_tiles", "unique_candidate_paths")


def main() -> None:
    order = torch.from_numpy(qsrt_oracle.tensor_core_perm().astype(np.int64))
    inverse = torch.argsort(order)
    out = {}
    for name, (bits, rows, columns, _, sweeps, _, strength, fp64) in REFINE_CASES.items():
        weight, hessian, column_weights, gradient = refine_case_inputs(name)
        table = qsrt_oracle.sqg_xor_cheb_t12_bytes(bits)

        def quantize(tiles: torch.Tensor):
            recon, states = qsrt_oracle.quantize_tiles(tiles.numpy(), table, bits)
            return torch.from_numpy(recon), torch.from_numpy(states)

        recon, states = quantize(matrix_to_tc_tiles(weight, order).contiguous())
        initial_q = tc_tiles_to_matrix(recon, inverse, rows, columns).contiguous()
        initial_states = states.reshape(rows // 16, columns // 16, 256)
        guidance = None
        if strength:
            guidance = ViterbiGradientGuidance(gradient=gradient, anchor=initial_q.clone(), anchor_id="initial",
                                               objective_id="seeded", strength=strength)
        config = H2ViterbiRefineConfig(sweeps=sweeps, score_dtype=torch.float64 if fp64 else torch.float32)
        result = refine_h2_viterbi_paths(weight, hessian, initial_q, initial_states, quantize, config,
                                         column_weights=column_weights, guidance=guidance)
        out[f"{name}_initial_states"] = initial_states.numpy()
        out[f"{name}_states"] = result.encoded.numpy()
        out[f"{name}_weight_q"] = result.weight_q.numpy()
        for key in STAT_KEYS:
            out[f"{name}_{key}"] = np.asarray([getattr(s, key) for s in result.sweep_stats], dtype=np.float64)
        print(name, [(s.accepted_tiles, s.objective_before, s.objective_after, s.unique_candidate_paths)
                     for s in result.sweep_stats])
    path = ROOT / "tests" / "golden" / "refine_golden.npz"
    np.savez_compressed(path, **out)
    print("wrote", path)


if __name__ == "__main__":
    main()
