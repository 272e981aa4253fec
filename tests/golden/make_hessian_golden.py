"""Generate tests/golden/hessian_golden.npz from the reference's own CPU code.

    PYTHONPATH=<reference checkout> python tests/golden/make_hessian_golden.py

The seeded case of tests.helpers.expert_hessian_inputs goes through
qsrt.qsrt_candidates.build_expert_hessians (global H13, blended H13, OAS H2 and fixed-alpha H2) and
qsrt.glm52_routed_input_curvature.routed_input_hessian on the CPU; matrices are stored as float32
and the evidence numbers as float64.
"""

import sys
from pathlib import Path

import numpy as np
import torch

from qsrt.glm52_routed_input_curvature import routed_input_hessian
from qsrt.qsrt_candidates import build_expert_hessians

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from tests.helpers import expert_hessian_inputs  # noqa: E402

EVIDENCE_KEYS = ("gate_square_sum", "h13_local_alpha", "h2_local_alpha", "h2_local_alpha_cap",
                 "h2_effective_sample_size", "h2_oas_shrinkage", "h2_identity_scale")


def main() -> None:
    inputs, gates, middle, global_h13, global_h2, route_weights = expert_hessian_inputs()
    cpu = torch.device("cpu")
    out = {}
    for name, kwargs in (("default", {}), ("blend", {"h13_alpha": 0.25}), ("fixed", {"h13_alpha": 0.25, "h2_alpha": 0.4})):
        h13, h2, evidence = build_expert_hessians(inputs, gates, middle, global_h13=global_h13,
                                                  global_h2=global_h2, device=cpu, **kwargs)
        if name == "blend":   # "default" returns the global matrix itself, "fixed" repeats the blend
            out["blend_h13"] = h13.numpy()
        out[f"{name}_h2"] = h2.numpy()
        out[f"{name}_policy"] = np.array(evidence["h2_shrinkage_policy"])
        for key in EVIDENCE_KEYS:
            if key in evidence:
                out[f"{name}_{key}"] = np.float64(evidence[key])
    for name, shrinkage in (("routed_010", 0.10), ("routed_100", 1.0)):
        hessian, stats = routed_input_hessian(inputs, route_weights, identity_shrinkage=shrinkage)
        if shrinkage < 1.0:
            out[f"{name}_hessian"] = hessian.float().numpy()
        else:                  # full shrinkage leaves a scaled identity
            assert torch.count_nonzero(hessian - torch.diag(hessian.diagonal())) == 0
            out[f"{name}_diagonal"] = hessian.diagonal().float().numpy()
        for key, value in stats.items():
            out[f"{name}_{key}"] = np.float64(value)
    path = ROOT / "tests" / "golden" / "hessian_golden.npz"
    np.savez_compressed(path, **out)
    print("wrote", path, {k: getattr(v, "shape", None) for k, v in out.items()})


if __name__ == "__main__":
    main()
