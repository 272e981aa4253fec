"""Test infrastructure only: float64 numpy restatement of the per-expert Hessian constructors.

Only tests, the smoke check and the benchmark's CPU baseline may import this module; the product
path never does.  Pinned against matrices the reference itself produced on the CPU
(tests/golden/hessian_golden.npz, written by tests/golden/make_hessian_golden.py).

  weighted_covariance          qsrt/candidate_hessian.py:70-112
  shrink_covariance            qsrt/candidate_hessian.py:115-140
  adaptive_identity_shrinkage  qsrt/candidate_hessian.py:143-216
  build_expert_hessians        qsrt/qsrt_candidates.py:534-618
  routed_input_hessian         qsrt/glm52_routed_input_curvature.py:76-109
"""

from __future__ import annotations

import numpy as np


def weighted_covariance(rows: np.ndarray, weights: np.ndarray) -> tuple[np.ndarray, float]:
    rows = np.asarray(rows, dtype=np.float64)
    weights = np.asarray(weights, dtype=np.float64)
    total = float(weights.sum())
    covariance = (rows.T * weights) @ rows / total
    return (covariance + covariance.T) * 0.5, total


def shrink_covariance(prior: np.ndarray, local: np.ndarray, alpha: float) -> np.ndarray:
    blended = prior + alpha * (np.asarray(local, dtype=np.float64) - prior)
    return (blended + blended.T) * 0.5


def adaptive_identity_shrinkage(local: np.ndarray, weights: np.ndarray, max_local_alpha: float = 0.75):
    weights = np.asarray(weights, dtype=np.float64)
    n_eff = float(weights.sum() ** 2 / np.square(weights).sum())
    dimension = local.shape[0]
    mu = np.trace(local) / dimension
    mean_square = np.square(local).mean()
    denominator = (n_eff + 1.0) * (mean_square - mu * mu / dimension)
    rho = 1.0 if denominator <= 0 else min(1.0, max(0.0, float((mean_square + mu * mu) / denominator)))
    alpha = min(max_local_alpha, 1.0 - rho)
    blended = shrink_covariance(np.eye(dimension) * mu, local, alpha)
    return blended, {"effective_sample_size": n_eff, "oas_shrinkage": rho, "local_alpha": alpha,
                     "max_local_alpha": max_local_alpha, "identity_scale": float(mu)}


def build_expert_hessians(inputs, gates, source_middle, global_h13, h13_alpha: float = 0.0,
                          h2_alpha: float | None = None):
    weights = np.square(np.asarray(gates, dtype=np.float64))
    if h13_alpha == 0.0:
        h13 = np.asarray(global_h13, dtype=np.float64)
    else:
        h13 = shrink_covariance(np.asarray(global_h13, dtype=np.float64), weighted_covariance(inputs, weights)[0], h13_alpha)
    local_h2, total = weighted_covariance(source_middle, weights)
    if h2_alpha is None:
        h2, info = adaptive_identity_shrinkage(local_h2, weights)
        evidence = {"h2_local_alpha": info["local_alpha"], "h2_local_alpha_cap": info["max_local_alpha"],
                    "h2_effective_sample_size": info["effective_sample_size"],
                    "h2_oas_shrinkage": info["oas_shrinkage"], "h2_identity_scale": info["identity_scale"]}
    else:
        scale = float(np.trace(local_h2) / local_h2.shape[0])
        h2 = shrink_covariance(np.eye(local_h2.shape[0]) * scale, local_h2, h2_alpha)
        evidence = {"h2_local_alpha": float(h2_alpha), "h2_local_alpha_cap": float(h2_alpha), "h2_identity_scale": scale}
    return h13, h2, {"gate_square_sum": total, "h13_local_alpha": float(h13_alpha), **evidence}


def routed_input_hessian(values, route_weights, identity_shrinkage: float):
    weights = np.maximum(np.asarray(route_weights, dtype=np.float64), 0.0)
    mass = float(np.square(weights).sum())
    weighted = np.asarray(values, dtype=np.float64) * weights[:, None]
    hessian = weighted.T @ weighted / mass
    diagonal_mean = float(np.diagonal(hessian).mean())
    hessian = hessian * (1.0 - identity_shrinkage)
    hessian[np.diag_indices_from(hessian)] += identity_shrinkage * diagonal_mean
    return hessian, {"row_count": int(weights.shape[0]), "squared_route_mass": mass,
                     "unshrunk_diagonal_mean": diagonal_mean, "identity_shrinkage": float(identity_shrinkage)}
