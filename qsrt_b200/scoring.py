"""Routed-error scoring of encoded expert candidates (the C1 row of the hot path).

Mirrors, by name and argument meaning, the reference's evaluators:

* ``functional_sse_by_request`` (qsrt/qsrt_candidates.py:621-654) and the deferred row form
  ``row_sse`` (``_defer_functional_row_sse``, qsrt/pack/qsrt_candidates.py:318-349);
* ``CandidateHiddenStatistics``, ``decoded_down_sse``, ``decoded_down_sse_difference``,
  ``candidate_h2`` (qsrt/pooled_calibration.py:25-222, 774-924);
* ``PooledPortfolioEvaluation`` / ``evaluate_coupled_candidate_portfolio_batches``
  (qsrt/pooled_calibration.py:197-214, 661-771).

The dense products run on the tensor cores in float32 accuracy (``linalg.gemm_nt``: tcgen05 TF32
head / tail products), the gated activation is fused with the split of the middle rows into the
operand planes of the down product (``qsrtb_gated_activation``) and the per-row error sums are one
float64 pass (``qsrtb_routed_row_sse``).  Per candidate the work is ``2 R (2 Hd I + I Hd)`` flops.
"""

from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Iterable, Mapping

import torch

from . import _lib, linalg

ACTIVATIONS = {"silu": 0, "situ": 1}


def _stream_ptr(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


# --------------------------------------------------------------------------------------
# kernels
# --------------------------------------------------------------------------------------

def gated_activation(gate_up: torch.Tensor, activation: str = "silu", *, planes: bool = True, rows: bool = False):
    """``act(gate) * up`` of ``[R, 2 I]`` pre-activations (gate columns first).  Returns
    ``(planes or None, float32 rows or None)``."""

    if activation not in ACTIVATIONS:
        raise ValueError(f"unknown activation {activation!r}")
    if gate_up.dtype != torch.float32 or not gate_up.is_cuda or gate_up.ndim != 2 or gate_up.stride(1) != 1:
        raise TypeError("pre-activations must be a CUDA float32 matrix with contiguous rows")
    r, two_i = gate_up.shape
    inter = two_i // 2
    device = gate_up.device
    out_planes = out_rows = None
    if planes:
        out_planes = linalg.Planes(torch.empty((r, inter), dtype=torch.float32, device=device),
                                   torch.empty((r, inter), dtype=torch.float32, device=device))
    if rows:
        out_rows = torch.empty((r, inter), dtype=torch.float32, device=device)
    with torch.cuda.device(device):
        _lib.check(
            _lib.lib().qsrtb_gated_activation(
                gate_up.data_ptr(), r, inter, gate_up.stride(0), ACTIVATIONS[activation],
                out_planes.hi.data_ptr() if planes else None, out_planes.lo.data_ptr() if planes else None, inter,
                out_rows.data_ptr() if rows else None, inter, _stream_ptr(device)),
            "qsrtb_gated_activation")
    return out_planes, out_rows


def row_sse(reference: torch.Tensor, candidate: torch.Tensor, *, energy: bool = False):
    """Float64 ``sum_j (candidate - reference)^2`` per row (and ``sum_j reference^2`` with
    ``energy``), device tensors; nothing synchronises."""

    if reference.shape != candidate.shape or reference.ndim != 2:
        raise ValueError("reference and candidate outputs must be equal 2-D shapes")
    if not (reference.is_cuda and candidate.is_cuda):
        raise TypeError("routed-error rows are reduced on the device")
    reference = reference.float() if reference.dtype != torch.float32 else reference
    candidate = candidate.float() if candidate.dtype != torch.float32 else candidate
    if reference.stride(1) != 1 or reference.stride(0) % 4:
        reference = reference.contiguous()
    if candidate.stride(1) != 1 or candidate.stride(0) % 4:
        candidate = candidate.contiguous()
    rows, d = reference.shape
    device = reference.device
    out = torch.empty(rows, dtype=torch.float64, device=device)
    out_energy = torch.empty(rows, dtype=torch.float64, device=device) if energy else None
    if d % 4:   # rows of odd width are not 16-byte aligned: pad a copy
        pad = 4 - d % 4
        reference = torch.nn.functional.pad(reference, (0, pad))
        candidate = torch.nn.functional.pad(candidate, (0, pad))
    with torch.cuda.device(device):
        _lib.check(
            _lib.lib().qsrtb_routed_row_sse(
                reference.data_ptr(), candidate.data_ptr(), rows, d, reference.stride(0), candidate.stride(0),
                out.data_ptr(), out_energy.data_ptr() if energy else None, _stream_ptr(device)),
            "qsrtb_routed_row_sse")
    return (out, out_energy) if energy else out


# --------------------------------------------------------------------------------------
# expert forward on the tensor cores
# --------------------------------------------------------------------------------------

class ExpertOperands:
    """Operand planes of one gated expert: the stacked gate and up matrices ``[2 I, Hd]`` and the
    down matrix ``[Hd, I]``, split once and reused for every row batch."""

    def __init__(self, w1: torch.Tensor, w3: torch.Tensor, w2: torch.Tensor) -> None:
        if w1.shape != w3.shape or tuple(w2.shape) != (w1.shape[1], w1.shape[0]):
            raise ValueError("expert weights must be gate/up [I, Hd] and down [Hd, I]")
        self.intermediate, self.hidden = int(w1.shape[0]), int(w1.shape[1])
        stacked = torch.cat((w1.float(), w3.float()), dim=0)
        self.gate_up = linalg.split_tf32(stacked)
        self.down = linalg.split_tf32(w2.float().contiguous())


def expert_middle(row_planes: linalg.Planes, operands: ExpertOperands, activation: str = "silu", *,
                  planes: bool = True, rows: bool = False):
    """Middle activation of routed rows given as planes: one product against the stacked gate / up
    matrices, then the fused activation."""

    r = row_planes.hi.shape[0]
    pre = torch.empty((r, 2 * operands.intermediate), dtype=torch.float32, device=row_planes.hi.device)
    linalg.gemm_nt(row_planes, operands.gate_up, pre)
    return gated_activation(pre, activation, planes=planes, rows=rows)


def expert_output(row_planes: linalg.Planes, operands: ExpertOperands, activation: str = "silu") -> torch.Tensor:
    """``act(x W1^T, x W3^T) W2^T`` for routed rows given as planes -> float32 ``[R, Hd]``."""

    middle, _ = expert_middle(row_planes, operands, activation)
    out = torch.empty((row_planes.hi.shape[0], operands.hidden), dtype=torch.float32, device=row_planes.hi.device)
    return linalg.gemm_nt(middle, operands.down, out)


def gated_middle(rows: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    """Float32 middle rows ``act(x W1^T) * (x W3^T)`` (the input of the down-projection covariance)."""

    stacked = linalg.split_tf32(torch.cat((w1.float(), w3.float()), dim=0))
    pre = torch.empty((rows.shape[0], 2 * w1.shape[0]), dtype=torch.float32, device=rows.device)
    linalg.gemm_nt(linalg.split_tf32(rows.float().contiguous()), stacked, pre)
    return gated_activation(pre, activation, planes=False, rows=True)[1]


def routed_output_sse(rows: torch.Tensor, gates: torch.Tensor, source, candidate, activation: str = "silu"):
    """Routed functional error of a complete-expert candidate on its routed rows:
    ``sum_r gate_r^2 ||student_r - teacher_r||^2`` and the teacher energy, as 0-d float64 device
    tensors.  ``source`` / ``candidate`` are ``(w1, w3, w2)`` triplets or ``ExpertOperands``."""

    planes = linalg.split_tf32(rows.float().contiguous())
    source = source if isinstance(source, ExpertOperands) else ExpertOperands(*source)
    candidate = candidate if isinstance(candidate, ExpertOperands) else ExpertOperands(*candidate)
    teacher = expert_output(planes, source, activation)
    student = expert_output(planes, candidate, activation)
    sse, energy = row_sse(teacher, student, energy=True)
    w = gates.double().square()
    return (sse * w).sum(), (energy * w).sum()


# --------------------------------------------------------------------------------------
# functional_sse_by_request
# --------------------------------------------------------------------------------------

def functional_sse_by_request(reference: torch.Tensor, candidate: torch.Tensor, gates: torch.Tensor,
                              request_steps: torch.Tensor, requests: Mapping[int, str]):
    """Routed SSE, reference energy and row counts by request epoch
    (qsrt/qsrt_candidates.py:621-654).  Returns CPU tensors like the reference."""

    if reference.shape != candidate.shape or reference.ndim != 2:
        raise ValueError("reference and candidate outputs must be equal 2-D shapes")
    rows = reference.shape[0]
    if gates.ndim != 1 or request_steps.ndim != 1 or gates.numel() != rows or request_steps.numel() != rows:
        raise ValueError("functional metric metadata has the wrong shape")
    ordered_steps = sorted(map(int, requests))
    positions = {step: index for index, step in enumerate(ordered_steps)}
    try:
        indices = torch.tensor([positions[int(step)] for step in request_steps.cpu().tolist()], dtype=torch.long)
    except KeyError as exc:
        raise ValueError(f"metric row has unmapped request epoch {exc.args[0]}") from exc
    route_weights = gates.double().square().cpu()
    per_row, per_row_energy = row_sse(reference, candidate, energy=True)
    weighted_sse = per_row.cpu() * route_weights
    weighted_energy = per_row_energy.cpu() * route_weights
    sse = torch.zeros(len(ordered_steps), dtype=torch.float64)
    energy = torch.zeros_like(sse)
    counts = torch.zeros(len(ordered_steps), dtype=torch.int64)
    sse.scatter_add_(0, indices, weighted_sse)
    energy.scatter_add_(0, indices, weighted_energy)
    counts.scatter_add_(0, indices, torch.ones_like(indices, dtype=torch.int64))
    return sse, energy, counts


# --------------------------------------------------------------------------------------
# pooled sufficient statistics
# --------------------------------------------------------------------------------------

def _cross(left: torch.Tensor, right: torch.Tensor) -> torch.Tensor:
    """``left.T @ right`` for row blocks ``[R, w]``: tensor cores for float32, float64 as is."""

    if left.dtype == torch.float32 and left.is_cuda:
        rows = left.shape[0]
        pitch = (rows + 3) // 4 * 4   # plane rows must stay 16-byte aligned

        def turned(x):
            hi = torch.zeros((x.shape[1], pitch), dtype=torch.float32, device=x.device)
            lo = torch.zeros_like(hi)
            return linalg.split_tf32(x.contiguous(), transpose=True, out=linalg.Planes(hi[:, :rows], lo[:, :rows]))

        out = torch.empty((left.shape[1], right.shape[1]), dtype=torch.float32, device=left.device)
        return linalg.gemm_nt(turned(left), turned(right), out)
    return left.T @ right


@dataclass
class CandidateHiddenStatistics:
    """Weighted source / candidate post-activation cross-products (qsrt/pooled_calibration.py:25-222)."""

    candidate_gram: torch.Tensor
    candidate_source_cross: torch.Tensor
    source_gram: torch.Tensor | None
    candidate_residual_cross: torch.Tensor
    hidden_residual_gram: torch.Tensor | None
    weight_sum: float
    weight_square_sum: float
    rows: int

    @classmethod
    def zeros(cls, width: int, *, device="cpu", dtype: torch.dtype = torch.float64,
              retain_source_gram: bool = True) -> "CandidateHiddenStatistics":
        if width <= 0:
            raise ValueError("hidden width must be positive")
        if dtype not in (torch.float32, torch.float64):
            raise TypeError("sufficient statistics require FP32 or FP64")
        shape = (width, width)

        def zero():
            return torch.zeros(shape, device=device, dtype=dtype)

        return cls(zero(), zero(), zero() if retain_source_gram else None, zero(),
                   zero() if retain_source_gram else None, 0.0, 0.0, 0)

    @property
    def width(self) -> int:
        return int(self.candidate_gram.shape[0])

    @property
    def effective_sample_size(self) -> float:
        if self.weight_sum <= 0 or self.weight_square_sum <= 0:
            return 0.0
        return self.weight_sum ** 2 / self.weight_square_sum

    def _tensors(self):
        return tuple(t for t in (self.candidate_gram, self.candidate_source_cross, self.source_gram,
                                 self.candidate_residual_cross, self.hidden_residual_gram) if t is not None)

    def _validate(self) -> None:
        shape = self.candidate_gram.shape
        if (self.candidate_gram.ndim != 2 or shape[0] != shape[1] or any(t.shape != shape for t in self._tensors())
                or (self.source_gram is None) != (self.hidden_residual_gram is None)):
            raise ValueError("candidate statistics must contain equal-size squares")
        if not all(bool(torch.all(torch.isfinite(t))) for t in self._tensors()):
            raise ValueError("candidate statistics must be finite")
        if (not math.isfinite(self.weight_sum) or not math.isfinite(self.weight_square_sum)
                or self.weight_sum < 0 or self.weight_square_sum < 0 or self.rows < 0):
            raise ValueError("candidate statistics have invalid support")

    def update(self, candidate_hidden: torch.Tensor, source_hidden: torch.Tensor, route_weights: torch.Tensor) -> None:
        """Accumulate one row chunk using ``route_weights.square()``."""

        self._validate()
        if (candidate_hidden.ndim != 2 or source_hidden.shape != candidate_hidden.shape
                or candidate_hidden.shape[1] != self.width):
            raise ValueError("source and candidate hidden rows do not align")
        if route_weights.ndim != 1 or route_weights.numel() != candidate_hidden.shape[0]:
            raise ValueError("route weights must contain one value per hidden row")
        if not all(bool(torch.all(torch.isfinite(v))) for v in (candidate_hidden, source_hidden, route_weights)):
            raise ValueError("candidate rows and route weights must be finite")
        device, dtype = self.candidate_gram.device, self.candidate_gram.dtype
        candidate = candidate_hidden.to(device=device, dtype=dtype)
        source = source_hidden.to(device=device, dtype=dtype)
        weights = route_weights.to(device=device, dtype=dtype).square()
        if bool(torch.any(weights < 0)):
            raise ValueError("squared route weights must be nonnegative")
        weighted_candidate = candidate * weights[:, None]
        self.candidate_gram.add_(_cross(candidate, weighted_candidate))
        self.candidate_source_cross.add_(_cross(candidate, source * weights[:, None]))
        residual = candidate - source
        weighted_residual = residual * weights[:, None]
        self.candidate_residual_cross.add_(_cross(candidate, weighted_residual))
        if self.source_gram is not None:
            self.source_gram.add_(_cross(source, source * weights[:, None]))
            if self.hidden_residual_gram is None:
                raise AssertionError("retained source statistics are incomplete")
            self.hidden_residual_gram.add_(_cross(residual, weighted_residual))
        weights64 = weights.double()
        self.weight_sum += float(weights64.sum())
        self.weight_square_sum += float(weights64.square().sum())
        self.rows += int(candidate.shape[0])

    def merge_(self, other: "CandidateHiddenStatistics") -> None:
        """Merge a disjoint row partition."""

        self._validate()
        other._validate()
        if other.width != self.width:
            raise ValueError("candidate statistics widths differ")
        if (self.source_gram is None) != (other.source_gram is None):
            raise ValueError("candidate statistics disagree on source-Gram retention")
        self.candidate_gram.add_(other.candidate_gram.to(self.candidate_gram))
        self.candidate_source_cross.add_(other.candidate_source_cross.to(self.candidate_source_cross))
        self.candidate_residual_cross.add_(other.candidate_residual_cross.to(self.candidate_residual_cross))
        if self.source_gram is not None:
            self.source_gram.add_(other.source_gram.to(self.source_gram))
            self.hidden_residual_gram.add_(other.hidden_residual_gram.to(self.hidden_residual_gram))
        self.weight_sum += other.weight_sum
        self.weight_square_sum += other.weight_square_sum
        self.rows += other.rows

    def to(self, *, device, dtype: torch.dtype | None = None) -> "CandidateHiddenStatistics":
        """Copy tensor statistics while preserving scalar support evidence."""

        target = self.candidate_gram.dtype if dtype is None else dtype
        if target not in (torch.float32, torch.float64):
            raise TypeError("sufficient statistics require FP32 or FP64")

        def move(t):
            return None if t is None else t.to(device=device, dtype=target)

        return CandidateHiddenStatistics(move(self.candidate_gram), move(self.candidate_source_cross),
                                         move(self.source_gram), move(self.candidate_residual_cross),
                                         move(self.hidden_residual_gram), self.weight_sum, self.weight_square_sum,
                                         self.rows)


def decoded_down_sse(statistics: CandidateHiddenStatistics, candidate_down_t: torch.Tensor,
                     source_down_t: torch.Tensor) -> torch.Tensor:
    """Exact pooled SSE from cross-products, evaluated around the source down projection
    (qsrt/pooled_calibration.py:774-827); ``*_down_t`` are ``[intermediate, output]``."""

    statistics._validate()
    if statistics.source_gram is None:
        raise ValueError("decoded down SSE requires retained source Gram statistics")
    if candidate_down_t.ndim != 2:
        raise ValueError("candidate down projection must be two-dimensional")
    if tuple(candidate_down_t.shape) != (statistics.width, candidate_down_t.shape[1]):
        raise ValueError("candidate down projection has the wrong shape")
    if source_down_t.shape != candidate_down_t.shape:
        raise ValueError("source and candidate down projections do not align")
    dtype, device = statistics.candidate_gram.dtype, statistics.candidate_gram.device
    candidate = candidate_down_t.to(device=device, dtype=dtype)
    source = source_down_t.to(device=device, dtype=dtype)
    delta = candidate - source
    delta_term = torch.sum(delta * (statistics.candidate_gram @ delta))
    cross_term = torch.sum(delta * (statistics.candidate_residual_cross @ source))
    source_residual_term = torch.sum(source * (statistics.hidden_residual_gram @ source))
    value = delta_term + 2.0 * cross_term + source_residual_term
    tolerance = 64 * torch.finfo(dtype).eps * max(float(delta_term.abs()), float((2.0 * cross_term).abs()),
                                                  float(source_residual_term.abs()), 1.0)
    if float(value) < -tolerance:
        raise ArithmeticError(f"pooled SSE is negative beyond roundoff: {float(value):.9g}")
    return value.clamp_min(0)


def decoded_down_sse_difference(statistics: CandidateHiddenStatistics, candidate_down_t: torch.Tensor,
                                baseline_down_t: torch.Tensor, source_down_t: torch.Tensor) -> torch.Tensor:
    """Candidate-minus-baseline SSE without a source Gram matrix (qsrt/pooled_calibration.py:830-861)."""

    statistics._validate()
    if candidate_down_t.ndim != 2:
        raise ValueError("candidate down projection must be two-dimensional")
    if (tuple(candidate_down_t.shape) != (statistics.width, candidate_down_t.shape[1])
            or baseline_down_t.shape != candidate_down_t.shape or source_down_t.shape != candidate_down_t.shape):
        raise ValueError("down projections do not share the expected shape")
    dtype, device = statistics.candidate_gram.dtype, statistics.candidate_gram.device
    candidate = candidate_down_t.to(device=device, dtype=dtype)
    baseline = baseline_down_t.to(device=device, dtype=dtype)
    source = source_down_t.to(device=device, dtype=dtype)
    delta = candidate - baseline
    baseline_gradient = statistics.candidate_gram @ (baseline - source) + statistics.candidate_residual_cross @ source
    return 2.0 * torch.sum(delta * baseline_gradient) + torch.sum(delta * (statistics.candidate_gram @ delta))


def candidate_h2(statistics: CandidateHiddenStatistics, *, max_local_alpha: float = 0.75):
    """OAS-shrunk candidate-local covariance with the prior ``trace(H) / dimension * I``
    (qsrt/pooled_calibration.py:864-924)."""

    statistics._validate()
    max_local_alpha = float(max_local_alpha)
    if not math.isfinite(max_local_alpha) or not 0 <= max_local_alpha <= 1:
        raise ValueError("max_local_alpha must be finite and in [0, 1]")
    if statistics.weight_sum <= 0 or statistics.effective_sample_size <= 0:
        raise ValueError("candidate H2 requires positive weighted support")
    covariance = statistics.candidate_gram / statistics.weight_sum
    covariance = (covariance + covariance.T) * 0.5
    dimension = statistics.width
    trace = torch.trace(covariance)
    if float(trace) <= 0:
        raise ValueError("candidate covariance must have positive trace")
    identity_scale = trace / dimension
    trace_square = trace.square()
    frobenius_square = covariance.square().sum()
    denominator = (statistics.effective_sample_size + 1.0 - 2.0 / dimension) * (frobenius_square - trace_square / dimension)
    if float(denominator) <= 0:
        shrinkage = 1.0
    else:
        shrinkage = min(1.0, max(0.0, float(((1.0 - 2.0 / dimension) * frobenius_square + trace_square) / denominator)))
    local_alpha = min(max_local_alpha, 1.0 - shrinkage)
    identity = torch.eye(dimension, dtype=covariance.dtype, device=covariance.device).mul_(identity_scale)
    result = torch.lerp(identity, covariance, local_alpha)
    return result.contiguous(), {
        "rows": float(statistics.rows),
        "weight_sum": statistics.weight_sum,
        "effective_sample_size": statistics.effective_sample_size,
        "oas_shrinkage": shrinkage,
        "local_alpha": local_alpha,
        "max_local_alpha": max_local_alpha,
        "identity_scale": float(identity_scale),
    }


# --------------------------------------------------------------------------------------
# coupled candidate portfolio
# --------------------------------------------------------------------------------------

@dataclass(frozen=True)
class PooledPortfolioEvaluation:
    """Exact routed-function scores for candidates sharing one source expert
    (qsrt/pooled_calibration.py:197-214)."""

    candidate_sse: Mapping[str, float]
    source_energy: float
    routed_occurrences: int

    def __post_init__(self) -> None:
        if (not self.candidate_sse
                or any(not math.isfinite(v) or v < 0 for v in self.candidate_sse.values())
                or not math.isfinite(self.source_energy) or self.source_energy <= 0 or self.routed_occurrences <= 0):
            raise ValueError("pooled portfolio evaluation is invalid")


def _triplet(value):
    """(gate, up, down) from a tuple or from an object with those attributes."""

    if isinstance(value, (tuple, list)):
        return tuple(value)
    return value.gate, value.up, value.down


def evaluate_coupled_candidate_portfolio_batches(batches: Iterable[Mapping[str, torch.Tensor]], *, source,
                                                 candidate_coordinates: Mapping[str, object],
                                                 executions: Mapping[str, object]) -> PooledPortfolioEvaluation:
    """Score a coupled candidate portfolio with one shared source forward
    (qsrt/pooled_calibration.py:661-771).  ``source`` and the candidates are ``(gate, up, down)``
    triplets (tuples or objects with those attributes); every candidate is stored in the coupled
    coordinates of its own ``CoupledHadamardExecution``, all of which share the residual transform.
    The teacher is the ordinary-coordinate source expert under the bounded gated activation."""

    names = tuple(candidate_coordinates)
    if not names or set(executions) != set(names):
        raise ValueError("candidate coordinates and executions must share identities")
    src = tuple(t.float() for t in _triplet(source))
    candidates = {name: tuple(t.float() for t in _triplet(candidate_coordinates[name])) for name in names}
    devices = {t.device for triplet in candidates.values() for t in triplet}
    if len(devices) != 1:
        raise ValueError("pooled portfolio candidates must share one device")
    device = devices.pop()
    src = tuple(t.to(device) for t in src)
    inter, hidden = src[0].shape
    first = executions[names[0]]
    if first.hidden != hidden or first.intermediate != inter:
        raise ValueError("pooled portfolio execution geometry differs from the source")
    contract = (first.spec.residual_block_size, first.spec.residual_draw)
    for name in names:
        triplet, execution = candidates[name], executions[name]
        if (tuple(triplet[0].shape) != (inter, hidden) or execution.hidden != hidden or execution.intermediate != inter
                or (execution.spec.residual_block_size, execution.spec.residual_draw) != contract):
            raise ValueError("pooled portfolio candidates do not share residual geometry")

    source_operands = ExpertOperands(*src)
    sse = {name: torch.zeros((), dtype=torch.float64, device=device) for name in names}
    source_energy = torch.zeros((), dtype=torch.float64, device=device)
    occurrences, previous_row = 0, -1
    for batch in batches:
        if not {"input", "route_weight", "row_index"}.issubset(batch):
            raise ValueError("pooled expert batch lacks input, route weight, or row index")
        rows, route_weights, row_indices = batch["input"], batch["route_weight"], batch["row_index"]
        if (rows.ndim != 2 or rows.shape[1] != hidden or route_weights.ndim != 1 or row_indices.ndim != 1
                or route_weights.numel() != rows.shape[0] or row_indices.numel() != rows.shape[0]):
            raise ValueError("pooled portfolio batch tensors do not align")
        if rows.shape[0] == 0:
            continue
        if row_indices.dtype != torch.int64:
            raise TypeError("global row indices must be int64")
        if int(row_indices[0]) <= previous_row or bool(torch.any(row_indices[1:] <= row_indices[:-1])):
            raise ValueError("pooled expert rows must be globally increasing")
        previous_row = int(row_indices[-1])
        rows = rows.to(device=device, dtype=torch.float32).contiguous()
        weights = route_weights.to(device=device, dtype=torch.float32).double().square()
        source_output = expert_output(linalg.split_tf32(rows), source_operands, "situ")
        transformed = first.transform_inputs(rows)
        energy = (source_output.double().square().sum(dim=1) * weights).sum()
        source_energy += energy
        for name in names:
            gate, up, down = candidates[name]
            execution = executions[name]
            hidden_rows = execution.decode_middle(transformed, gate, up)
            output = execution.decode_output(linalg.matmul_nt(hidden_rows.float().contiguous(), down.contiguous()))
            sse[name] += (row_sse(source_output, output) * weights).sum()
        occurrences += int(rows.shape[0])
    return PooledPortfolioEvaluation({name: float(value) for name, value in sse.items()}, float(source_energy), occurrences)
