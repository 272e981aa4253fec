"""Calibration Hessians from routed activation rows.

Mirrors ``qsrt/candidate_hessian.py`` (``weighted_covariance``, ``shrink_covariance``,
``weighted_effective_sample_size``, ``adaptive_identity_shrinkage``) and the accumulator of
``qsrt/capture.py:714-731``.  The contraction runs on the tensor cores
(``qsrtb_hessian_accumulate_tc``: TMA-fed tcgen05 3xTF32 with float32 partial sums, within 1e-5
of FP64) when the feature count is a multiple of 128, otherwise in ``qsrtb_hessian_accumulate``
(weighted lower-triangular SYRK on the float32 FMA units); the scalar shrinkage statistics stay
on the host in float64 exactly as in the reference.
"""

from __future__ import annotations

import math

import torch

from . import _lib
from .tiles import _stream_ptr


# Rows handed to one tensor-core launch (its split operands take 16 bytes per row and feature).
TENSOR_CORE_CHUNK_ROWS = 2048
# Default for ``weighted_covariance(tensor_cores=None)``.
USE_TENSOR_CORES = True
_tc_workspace: dict[tuple[str, int], torch.Tensor] = {}   # per device and stream: launches on different streams must not share planes
_tc_built: list[bool] = []


def tensor_cores_available() -> bool:
    """True when the library was built with the tcgen05 Hessian kernel (CuTe headers present)."""

    import ctypes

    if not _tc_built:
        wanted = ctypes.c_size_t(0)
        _tc_built.append(_lib.lib().qsrtb_hessian_tc_workspace_bytes(32, 128, ctypes.byref(wanted)) == 0)
    return _tc_built[0]


def tensor_core_wait_probe(device: torch.device) -> int:
    """Run the tensor-core kernel's bounded wait on a barrier that is never satisfied and return the
    status word it leaves (``0x06000000 | lane``).  Takes about 20 ms; nothing faults or hangs."""

    status = torch.zeros(1, dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        _lib.check(_lib.lib().qsrtb_hessian_tc_wait_probe(status.data_ptr(), _stream_ptr(device)),
                   "qsrtb_hessian_tc_wait_probe")
    return int(status.item())


def accumulate_hessian_tensor_cores(lower: torch.Tensor, rows: torch.Tensor, weights: torch.Tensor | None, *,
                                    accumulate: bool = True) -> None:
    """``lower (+)= sum_r w_r x_r x_r^T`` with tcgen05 TF32 MMAs (split operands, float32
    accumulation in tensor memory).  The feature count must be a multiple of 128."""

    import ctypes

    d = lower.shape[0]
    if lower.ndim != 2 or lower.shape[1] != d or lower.dtype != torch.float32 or not lower.is_cuda or not lower.is_contiguous():
        raise ValueError("the accumulator must be a contiguous square CUDA float32 matrix")
    if d % 128:
        raise ValueError("the tensor-core Hessian needs a feature count that is a multiple of 128")
    rows = rows.to(device=lower.device, dtype=torch.float32).contiguous()
    if rows.ndim != 2 or rows.shape[1] != d:
        raise ValueError("invalid covariance sample shapes")
    if weights is not None:
        weights = weights.to(device=lower.device, dtype=torch.float32).contiguous()
    device = lower.device
    wanted = ctypes.c_size_t(0)
    _lib.check(_lib.lib().qsrtb_hessian_tc_workspace_bytes(TENSOR_CORE_CHUNK_ROWS, d, ctypes.byref(wanted)),
               "qsrtb_hessian_tc_workspace_bytes")
    key = (str(device), torch.cuda.current_stream(device).cuda_stream)
    work = _tc_workspace.get(key)
    if work is None or work.numel() < wanted.value:
        work = torch.empty(wanted.value, dtype=torch.uint8, device=device)
        _tc_workspace[key] = work
    status = torch.zeros(1, dtype=torch.int32, device=device)
    first = not accumulate
    with torch.cuda.device(device):
        for begin in range(0, rows.shape[0], TENSOR_CORE_CHUNK_ROWS):
            chunk = rows[begin:begin + TENSOR_CORE_CHUNK_ROWS]
            w = weights[begin:begin + TENSOR_CORE_CHUNK_ROWS] if weights is not None else None
            _lib.check(
                _lib.lib().qsrtb_hessian_accumulate_tc(
                    chunk.data_ptr(), w.data_ptr() if w is not None else None, chunk.shape[0], d, d,
                    lower.data_ptr(), d, 0 if first else 1, work.data_ptr(), work.numel(), status.data_ptr(),
                    _stream_ptr(device),
                ),
                "qsrtb_hessian_accumulate_tc",
            )
            first = False
    code = int(status.item())
    if code != 0:
        roles = {1: "producer waiting for a free stage", 2: "producer waiting for the last commits",
                 3: "MMA issuer waiting for a drained accumulator", 4: "MMA issuer waiting for a loaded stage",
                 5: "epilogue waiting for a finished segment"}
        raise RuntimeError(
            f"tensor-core Hessian kernel gave up: {roles.get(code >> 24, 'unknown wait')} "
            f"(sequence {code & 0xFFFFFF}, status 0x{code:08x})"
        )


def accumulate_hessian(lower: torch.Tensor, rows: torch.Tensor, weights: torch.Tensor | None, *, accumulate: bool = True) -> None:
    """``lower (+)= sum_r w_r x_r x_r^T`` on the lower triangle of a CUDA float32 matrix."""

    if lower.ndim != 2 or lower.shape[0] != lower.shape[1] or lower.dtype != torch.float32 or not lower.is_cuda:
        raise ValueError("the accumulator must be a square CUDA float32 matrix")
    if not lower.is_contiguous():
        raise ValueError("the accumulator must be contiguous")
    if rows.ndim != 2 or rows.shape[1] != lower.shape[0]:
        raise ValueError("invalid covariance sample shapes")
    rows = rows.to(device=lower.device, dtype=torch.float32).contiguous()
    if weights is not None:
        if weights.ndim != 1 or weights.shape[0] != rows.shape[0]:
            raise ValueError("invalid covariance sample shapes")
        weights = weights.to(device=lower.device, dtype=torch.float32).contiguous()
    d = lower.shape[0]
    with torch.cuda.device(lower.device):
        _lib.check(
            _lib.lib().qsrtb_hessian_accumulate(
                rows.data_ptr(), weights.data_ptr() if weights is not None else None, rows.shape[0], d, d,
                lower.data_ptr(), d, int(accumulate), _stream_ptr(lower.device),
            ),
            "qsrtb_hessian_accumulate",
        )


def finish_hessian(lower: torch.Tensor, weight_sum: float) -> torch.Tensor:
    """Divide by the weight sum and mirror the triangle (in place); returns ``lower``."""

    d = lower.shape[0]
    with torch.cuda.device(lower.device):
        _lib.check(
            _lib.lib().qsrtb_hessian_finish(lower.data_ptr(), d, d, float(weight_sum), _stream_ptr(lower.device)),
            "qsrtb_hessian_finish",
        )
    return lower


def weighted_covariance(rows: torch.Tensor, weights: torch.Tensor, *, device: torch.device,
                        chunk_rows: int = 65536, return_cpu: bool = True,
                        tensor_cores: bool | None = None) -> tuple[torch.Tensor, float]:
    """Return ``sum(w * x xT) / sum(w)`` as symmetric FP32 (qsrt/candidate_hessian.py:70-112).

    ``chunk_rows`` only bounds the staging copy of host-resident rows; the kernel streams any
    number of rows in one launch.  ``tensor_cores``: ``None`` follows ``USE_TENSOR_CORES``,
    ``False`` forces the float32 FMA kernel, ``True`` insists on the tensor-core kernel (and raises
    when the feature count is not a multiple of 128).
    """

    if rows.ndim != 2 or weights.ndim != 1 or rows.shape[0] != weights.shape[0]:
        raise ValueError("invalid covariance sample shapes")
    if not rows.shape[0] or not rows.shape[1]:
        raise ValueError("covariance samples must be nonempty")
    if chunk_rows <= 0:
        raise ValueError("chunk_rows must be positive")
    if not torch.all(torch.isfinite(rows)) or not torch.all(torch.isfinite(weights)):
        raise ValueError("covariance samples must be finite")
    if torch.any(weights < 0):
        raise ValueError("covariance weights must be nonnegative")
    device = torch.device(device)
    if device.type != "cuda":
        raise ValueError("the B200 Hessian path requires a CUDA device")
    dimension = int(rows.shape[1])
    denominator = float(weights.double().sum())
    if not math.isfinite(denominator) or denominator <= 0:
        raise ValueError("covariance weights must have a positive finite sum")
    accumulator = torch.empty((dimension, dimension), dtype=torch.float32, device=device)
    first = True
    if tensor_cores is None:
        use_tc = USE_TENSOR_CORES and dimension % 128 == 0 and tensor_cores_available()
    else:
        use_tc = bool(tensor_cores)
        if use_tc and dimension % 128:
            raise ValueError("tensor_cores=True needs a feature count that is a multiple of 128")
    for begin in range(0, int(rows.shape[0]), chunk_rows):
        step = accumulate_hessian_tensor_cores if use_tc else accumulate_hessian
        step(accumulator, rows[begin:begin + chunk_rows], weights[begin:begin + chunk_rows], accumulate=not first)
        first = False
    covariance = finish_hessian(accumulator, denominator)
    if return_cpu:
        covariance = covariance.cpu()
    if not torch.all(torch.isfinite(covariance)):
        raise ValueError("weighted covariance is non-finite")
    return covariance, denominator


def shrink_covariance(global_covariance: torch.Tensor, local_covariance: torch.Tensor, alpha: float) -> torch.Tensor:
    """Convex blend toward a global covariance (qsrt/candidate_hessian.py:115-140)."""

    alpha = float(alpha)
    if not math.isfinite(alpha) or not 0.0 <= alpha <= 1.0:
        raise ValueError("alpha must be finite and in [0, 1]")
    if (global_covariance.ndim != 2 or global_covariance.shape[0] != global_covariance.shape[1]
            or local_covariance.shape != global_covariance.shape):
        raise ValueError("global and local covariances must be equal-size squares")
    if not torch.all(torch.isfinite(global_covariance)) or not torch.all(torch.isfinite(local_covariance)):
        raise ValueError("covariances must be finite")
    blended = torch.lerp(global_covariance.float(), local_covariance.float(), alpha)
    return ((blended + blended.T) * 0.5).contiguous()


def weighted_effective_sample_size(weights: torch.Tensor) -> float:
    """Kish effective sample size (qsrt/candidate_hessian.py:143-153)."""

    if weights.ndim != 1 or not weights.numel():
        raise ValueError("weights must be a nonempty vector")
    if not torch.all(torch.isfinite(weights)) or torch.any(weights < 0):
        raise ValueError("weights must be finite and nonnegative")
    weights64 = weights.double()
    total = weights64.sum()
    squared_total = weights64.square().sum()
    if total <= 0 or squared_total <= 0:
        raise ValueError("weights must have positive effective support")
    return float(total.square() / squared_total)


def adaptive_identity_shrinkage(local_covariance: torch.Tensor, weights: torch.Tensor, *,
                                max_local_alpha: float = 0.75) -> tuple[torch.Tensor, dict[str, float]]:
    """OAS shrinkage toward the scaled identity with Kish n_eff (qsrt/candidate_hessian.py:156-216)."""

    max_local_alpha = float(max_local_alpha)
    if not math.isfinite(max_local_alpha) or not 0.0 <= max_local_alpha <= 1.0:
        raise ValueError("max_local_alpha must be finite and in [0, 1]")
    if local_covariance.ndim != 2 or local_covariance.shape[0] != local_covariance.shape[1]:
        raise ValueError("local covariance must be square")
    if not torch.all(torch.isfinite(local_covariance)):
        raise ValueError("local covariance must be finite")
    effective_rows = weighted_effective_sample_size(weights)
    dimension = int(local_covariance.shape[0])
    local64 = local_covariance.double()
    local_trace = torch.trace(local64)
    if local_trace <= 0:
        raise ValueError("local covariance trace must be positive")
    mu = local_trace / dimension
    mean_square = local64.square().mean()
    denominator = (effective_rows + 1.0) * (mean_square - mu.square() / dimension)
    if denominator <= 0:
        oas_shrinkage = 1.0
    else:
        oas_shrinkage = min(1.0, max(0.0, float((mean_square + mu.square()) / denominator)))
    local_alpha = min(max_local_alpha, 1.0 - oas_shrinkage)
    identity_scale = float(mu)
    scaled_identity = torch.eye(dimension, dtype=torch.float32, device=local_covariance.device).mul_(identity_scale)
    blended = shrink_covariance(scaled_identity, local_covariance, local_alpha)
    return blended, {
        "effective_sample_size": effective_rows,
        "oas_shrinkage": oas_shrinkage,
        "local_alpha": local_alpha,
        "max_local_alpha": max_local_alpha,
        "identity_scale": identity_scale,
    }


PHASE1_H13_EXPERT_LOCAL_ALPHA = 0.0
PHASE1_H2_EXPERT_LOCAL_ALPHA = 0.75
PHASE1_H2_SHRINKAGE_POLICY = "weighted_oas_scaled_identity"


def routed_input_hessian(values: torch.Tensor, route_weights: torch.Tensor, *, identity_shrinkage: float,
                         device: torch.device | None = None) -> tuple[torch.Tensor, dict[str, float]]:
    """Route-weighted covariance ``Σ w² x xᵀ / Σ w²`` blended with ``identity_shrinkage`` of its mean
    diagonal (qsrt/glm52_routed_input_curvature.py:76-109).  The contraction is the same weighted
    SYRK kernel as ``weighted_covariance`` with ``w²`` as row weights."""

    if values.ndim != 2 or route_weights.ndim != 1:
        raise ValueError("curvature values must be a matrix with one weight per row")
    if route_weights.numel() != values.shape[0]:
        raise ValueError("curvature route weights do not match the row count")
    if not math.isfinite(identity_shrinkage) or not 0.0 < identity_shrinkage <= 1.0:
        raise ValueError("identity_shrinkage must be in (0, 1]")
    device = torch.device(device) if device is not None else values.device
    if device.type != "cuda":
        raise ValueError("the B200 Hessian path requires a CUDA device")
    weights = route_weights.to(device=device, dtype=torch.float32).clamp_min(0.0)
    squared = weights.square()
    mass = float(squared.sum().item())
    if mass <= 0.0:
        raise ValueError("curvature route weights have zero squared mass")
    dimension = int(values.shape[1])
    accumulator = torch.empty((dimension, dimension), dtype=torch.float32, device=device)
    step = accumulate_hessian_tensor_cores if (
        USE_TENSOR_CORES and dimension % 128 == 0 and tensor_cores_available()) else accumulate_hessian
    step(accumulator, values.to(device=device, dtype=torch.float32), squared, accumulate=False)
    hessian = finish_hessian(accumulator, mass)
    diagonal_mean = float(hessian.diagonal().mean().item())
    if not math.isfinite(diagonal_mean) or diagonal_mean <= 0.0:
        raise ValueError("curvature covariance has a nonpositive mean diagonal")
    hessian.mul_(1.0 - identity_shrinkage)
    hessian.diagonal().add_(identity_shrinkage * diagonal_mean)
    return hessian.contiguous(), {
        "row_count": int(values.shape[0]),
        "squared_route_mass": mass,
        "unshrunk_diagonal_mean": diagonal_mean,
        "identity_shrinkage": float(identity_shrinkage),
    }


def build_expert_hessians(inputs: torch.Tensor, gates: torch.Tensor, source_middle: torch.Tensor, *,
                          global_h13: torch.Tensor, global_h2: torch.Tensor, device: torch.device,
                          h13_alpha: float = PHASE1_H13_EXPERT_LOCAL_ALPHA, h2_alpha: float | None = None,
                          chunk_rows: int = 256) -> tuple[torch.Tensor, torch.Tensor, dict]:
    """H13 and a support-aware post-activation H2 for one expert (qsrt/qsrt_candidates.py:534-618).

    Row weights are ``gate²``.  H13 is the global covariance, optionally blended with the expert's
    own; H2 is the expert's covariance of ``source_middle`` shrunk toward its trace-scaled identity,
    by weighted OAS (capped at 0.75) unless a fixed ``h2_alpha`` is given.  ``global_h2`` only fixes
    the dimension.  ``chunk_rows`` is accepted for compatibility: the kernels stream all rows.
    """

    if inputs.ndim != 2 or inputs.shape[0] != gates.shape[0]:
        raise ValueError("invalid expert input covariance samples")
    if source_middle.ndim != 2 or source_middle.shape[0] != inputs.shape[0]:
        raise ValueError("source middle rows do not match expert inputs")
    device = torch.device(device)
    global_h13 = global_h13.to(device=device, dtype=torch.float32)
    if global_h2.shape != (source_middle.shape[1], source_middle.shape[1]):
        raise ValueError("global H2 dimension does not match source middle rows")
    weights = gates.float().square()
    if h13_alpha == 0.0:
        h13, h13_weight = global_h13, float(weights.double().sum())
    else:
        local_h13, h13_weight = weighted_covariance(inputs, weights, device=device, return_cpu=False)
        h13 = shrink_covariance(global_h13, local_h13, h13_alpha)
    local_h2, h2_weight = weighted_covariance(source_middle, weights, device=device, return_cpu=False)
    if not math.isclose(h13_weight, h2_weight, rel_tol=1e-9, abs_tol=1e-12):
        raise ValueError("H13 and H2 expert covariance weights differ")
    if h2_alpha is None:
        h2, info = adaptive_identity_shrinkage(local_h2, weights, max_local_alpha=PHASE1_H2_EXPERT_LOCAL_ALPHA)
        evidence = {
            "h2_shrinkage_policy": PHASE1_H2_SHRINKAGE_POLICY,
            "h2_local_alpha": info["local_alpha"],
            "h2_local_alpha_cap": info["max_local_alpha"],
            "h2_effective_sample_size": info["effective_sample_size"],
            "h2_oas_shrinkage": info["oas_shrinkage"],
            "h2_identity_scale": info["identity_scale"],
        }
    else:
        identity_scale = float(torch.trace(local_h2) / local_h2.shape[0])
        prior = torch.eye(local_h2.shape[0], dtype=torch.float32, device=device).mul_(identity_scale)
        h2 = shrink_covariance(prior, local_h2, h2_alpha)
        evidence = {
            "h2_shrinkage_policy": "fixed_alpha_scaled_identity",
            "h2_local_alpha": float(h2_alpha),
            "h2_local_alpha_cap": float(h2_alpha),
            "h2_identity_scale": identity_scale,
        }
    return h13, h2, {"gate_square_sum": h13_weight, "h13_local_alpha": float(h13_alpha), **evidence}


# --------------------------------------------------------------------------------------
# capture -> Hessian streaming reducer
# --------------------------------------------------------------------------------------

def request_step_mask(observations: torch.Tensor, *, request_step_min: int, request_step_max: int | None,
                      request_steps: list[int] | None) -> torch.Tensor:
    """Request-epoch mask of captured observations: the epoch is ``observation_id >> 32``
    (qsrt/capture.py:734-750)."""

    steps = torch.bitwise_right_shift(observations.to(torch.int64), 32)
    selected = steps >= request_step_min
    if request_step_max is not None:
        selected &= steps <= request_step_max
    if request_steps is not None:
        selected &= torch.isin(steps, torch.tensor(request_steps, dtype=steps.dtype, device=steps.device))
    return selected


class StreamingHessianReducer:
    """All requested per-layer ``H13`` matrices in one pass over a capture's sample parts.

    The arithmetic of ``_build_h13_identity_h2_streaming`` (qsrt/capture.py:753-908) without its
    file handling: the caller reads each sample part (layer ids, split labels, observation ids,
    gate-square weights, input rows) however it stores them and hands the tensors to ``add_part``;
    rows are selected per layer by split and request epoch, moved to the device and accumulated
    into that layer's ``sum_r w_r x_r x_r^T`` by the Hessian kernels of this library (tensor
    cores when the input size is a multiple of 128).  ``finish`` divides by the weight sums,
    symmetrises and returns the matrices with the per-layer evidence the reference writes into its
    manifest (``w13_rows``, ``w13_total_rows``, ``w13_validation_rows``, ``w13_weight_sum``).
    The ``H2`` prior of this flow is the identity and is built nowhere, as in the reference."""

    SPLITS = {"train": 0, "validation": 1, "all": None}

    def __init__(self, input_size: int, selected: list[int], *, device: torch.device, sample_split: str = "train",
                 request_step_min: int = 0, request_step_max: int | None = None,
                 request_steps: list[int] | None = None, tensor_cores: bool | None = None) -> None:
        if sample_split not in self.SPLITS:
            raise ValueError("sample_split must be 'train', 'validation' or 'all'")
        device = torch.device(device)
        if device.type != "cuda":
            raise ValueError("the B200 Hessian path requires a CUDA device")
        self.input_size, self.selected, self.device = int(input_size), list(selected), device
        self.split_value = self.SPLITS[sample_split]
        self.sample_split = sample_split
        self.request = dict(request_step_min=request_step_min, request_step_max=request_step_max,
                            request_steps=request_steps)
        if tensor_cores is None:
            tensor_cores = USE_TENSOR_CORES and self.input_size % 128 == 0 and tensor_cores_available()
        elif tensor_cores and self.input_size % 128:
            raise ValueError("tensor_cores=True needs an input size that is a multiple of 128")
        self._step = accumulate_hessian_tensor_cores if tensor_cores else accumulate_hessian
        self._accumulators = {layer: torch.zeros((self.input_size, self.input_size), dtype=torch.float32, device=device)
                              for layer in self.selected}
        self.denominators = {layer: 0.0 for layer in self.selected}
        self.rows = {layer: 0 for layer in self.selected}
        self.total_rows = {layer: 0 for layer in self.selected}
        self.validation_rows = {layer: 0 for layer in self.selected}

    def add_part(self, layers: torch.Tensor, split: torch.Tensor, observations: torch.Tensor, weights: torch.Tensor,
                 values: torch.Tensor) -> None:
        """One sample part: ``layers`` / ``split`` / ``observations`` / ``weights`` are ``[rows]``,
        ``values`` is ``[rows, input_size]`` (any float dtype, host or device)."""

        layers = layers.to(torch.int64)
        split = split.to(torch.int8)
        observations = observations.to(torch.int64)
        weights = weights.to(torch.float32)
        if not (layers.ndim == split.ndim == observations.ndim == weights.ndim == 1
                and layers.numel() == split.numel() == observations.numel() == weights.numel()):
            raise ValueError("sample part has invalid input metadata")
        if tuple(values.shape) != (layers.numel(), self.input_size):
            raise ValueError("sample part has invalid input.values shape")
        if not bool(torch.all((split == 0) | (split == 1))):
            raise ValueError("sample part has invalid input split labels")
        epoch_mask = request_step_mask(observations, **self.request)
        chosen = set(self.selected)
        for raw_layer in torch.unique(layers).tolist():
            layer = int(raw_layer)
            if layer not in chosen:
                continue
            layer_mask = layers == layer
            self.total_rows[layer] += int(layer_mask.sum())
            self.validation_rows[layer] += int((layer_mask & (split == 1)).sum())
            mask = layer_mask & epoch_mask
            if self.split_value is not None:
                mask &= split == self.split_value
            indices = torch.nonzero(mask, as_tuple=False).flatten()
            if not indices.numel():
                continue
            x = values.index_select(0, indices.to(values.device)).to(device=self.device, dtype=torch.float32)
            w = weights.index_select(0, indices.to(weights.device)).to(device=self.device, dtype=torch.float32)
            self._step(self._accumulators[layer], x, w, accumulate=True)
            self.denominators[layer] += float(w.double().sum())
            self.rows[layer] += int(indices.numel())

    def finish(self, *, min_rows: int = 0, return_cpu: bool = True) -> dict[int, tuple[torch.Tensor, dict]]:
        """``{layer: (H13, evidence)}``; the accumulators are consumed."""

        out = {}
        for layer in self.selected:
            if self.rows[layer] < min_rows:
                raise ValueError(f"layer {layer} has too few H13 rows: {self.rows[layer]}, minimum={min_rows}")
            if self.denominators[layer] <= 0:
                raise ValueError(f"layer {layer} has a non-positive H13 denominator")
            h13 = finish_hessian(self._accumulators.pop(layer), self.denominators[layer])
            if return_cpu:
                h13 = h13.cpu().contiguous()
            out[layer] = (h13, {"row": layer, "w13_rows": self.rows[layer], "w13_total_rows": self.total_rows[layer],
                                "w13_validation_rows": self.validation_rows[layer],
                                "w13_weight_sum": self.denominators[layer], "w2_prior": "identity", "w2_rows": 0})
        return out
