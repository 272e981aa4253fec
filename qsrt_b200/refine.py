"""Dense-H block-coordinate refinement of legal trellis paths on the B200 kernels.

Host mirror of ``qsrt/h2_viterbi_refine.py`` (``refine_h2_viterbi_paths`` :334-560, objectives
:71-139, ``config_from_quant_args`` :563-590), of the guidance containers of
``qsrt/gradient_guided_viterbi.py:17-207`` (target shifts included) and of ``refine_uniform_h2_candidate``
(``qsrt/exl3_encoder_backend.py:840-895``).

After BlockLDLQ every 16-row block is revisited with all quantisation errors known: the exact
conditional target of the block under the dense input Hessian is re-encoded by the tile search and
a tile switches path only if that strictly lowers the same objective.

Device flow per row block (no host synchronisation inside a sweep):

1. target = W_b + H_bb^-1 (H E)_b - E_b  from the LU factors of all diagonal blocks (one batched
   factorisation per call) and the running ``H E`` product;
2. the fused row kernel (``qsrtb_ldlq_quantize_rows``) searches the target and its dithered
   variants straight from row-major memory - no tile gather, no permutation tensors;
3. ``qsrtb_refine_select`` scores stored and proposed tiles, applies the acceptance rule and
   rewrites reconstruction, payload, error rows and the error change;
4. ``H E += H[:, b] @ delta`` (a plain library GEMM).

A caller-supplied ``quantize_tiles`` callable is honoured as in the reference (tiles are gathered in
tensor-core order for it); passing the encoder's ``quant_args`` dict instead selects step 2.
"""

from __future__ import annotations

import math
from dataclasses import asdict, dataclass
from typing import Callable

import torch

from . import _lib
from .tiles import _stream_ptr

QuantizeTiles = Callable[[torch.Tensor], tuple[torch.Tensor, torch.Tensor]]


# ---- guidance containers ---------------------------------------------------------------------------
def _require_floating(*tensors: torch.Tensor) -> None:
    if not all(t.is_floating_point() for t in tensors):
        raise TypeError("gradient guidance tensors must be floating point")


@dataclass(frozen=True)
class ViterbiGradientGuidance:
    """Objective gradient measured at ``anchor`` (``gradient_guided_viterbi.py:17-41``)."""

    gradient: torch.Tensor
    anchor: torch.Tensor
    anchor_id: str
    objective_id: str
    strength: float = 1.0

    def validate(self, shape) -> None:
        shape = tuple(shape)
        if tuple(self.gradient.shape) != shape or tuple(self.anchor.shape) != shape:
            raise ValueError("gradient guidance tensors do not match the encoded matrix")
        _require_floating(self.gradient, self.anchor)
        if not bool(torch.isfinite(self.gradient).all()):
            raise ValueError("objective gradient must be finite")
        if not bool(torch.isfinite(self.anchor).all()):
            raise ValueError("gradient anchor must be finite")
        if not self.anchor_id or not self.objective_id:
            raise ValueError("gradient guidance requires anchor and objective identities")
        if not math.isfinite(self.strength) or self.strength < 0.0:
            raise ValueError("gradient strength must be finite and nonnegative")


@dataclass(frozen=True)
class LowRankViterbiGradientGuidance:
    """``left @ right`` stands for the dense gradient (``gradient_guided_viterbi.py:43-120``)."""

    left: torch.Tensor
    right: torch.Tensor
    anchor: torch.Tensor
    anchor_id: str
    objective_id: str
    strength: float = 1.0

    def validate(self, shape) -> None:
        shape = tuple(shape)
        if len(shape) != 2:
            raise ValueError("low-rank gradient guidance requires a matrix")
        if self.left.ndim != 2 or self.right.ndim != 2:
            raise ValueError("low-rank gradient factors must be matrices")
        rank = self.left.shape[1]
        if self.left.shape[0] != shape[0] or tuple(self.right.shape) != (rank, shape[1]) \
                or tuple(self.anchor.shape) != shape:
            raise ValueError("low-rank gradient guidance has incompatible geometry")
        if rank <= 0:
            raise ValueError("low-rank gradient guidance must have positive rank")
        _require_floating(self.left, self.right, self.anchor)
        if not all(bool(torch.isfinite(t).all()) for t in (self.left, self.right, self.anchor)):
            raise ValueError("gradient guidance tensors must be finite")
        if not self.anchor_id or not self.objective_id:
            raise ValueError("gradient guidance requires anchor and objective identities")
        if not math.isfinite(self.strength) or self.strength < 0.0:
            raise ValueError("gradient strength must be finite and nonnegative")

    def rows(self, row_slice: slice, *, device, dtype) -> torch.Tensor:
        return self.left[row_slice].to(device=device, dtype=dtype) @ self.right.to(device=device, dtype=dtype)

    def linear_term(self, candidate: torch.Tensor, *, dtype) -> float:
        delta = candidate.to(dtype=dtype) - self.anchor.to(device=candidate.device, dtype=dtype)
        left = self.left.to(device=candidate.device, dtype=dtype)
        right = self.right.to(device=candidate.device, dtype=dtype)
        return float(self.strength) * float(((left.T @ delta) * right).sum().item())


GradientGuidance = ViterbiGradientGuidance | LowRankViterbiGradientGuidance


def shift_elementwise_target(target: torch.Tensor, gradient: torch.Tensor, *, strength: float,
                             quadratic_weight: torch.Tensor | float = 1.0) -> torch.Tensor:
    """Target with the minimiser of ``a (q - target)^2 + strength * gradient * q``
    (``gradient_guided_viterbi.py:123-152``): the tile search then optimises the guided objective
    unchanged."""

    if target.shape != gradient.shape:
        raise ValueError("target and gradient must have matching shapes")
    if not (target.is_floating_point() and gradient.is_floating_point()):
        raise TypeError("target and gradient must be floating point")
    if not math.isfinite(strength) or strength < 0.0:
        raise ValueError("gradient strength must be finite and nonnegative")
    weight = torch.as_tensor(quadratic_weight, device=target.device, dtype=torch.float32)
    if weight.ndim and weight.shape != target.shape:
        raise ValueError("quadratic weights must be scalar or match the target")
    if not bool(torch.isfinite(weight).all()) or not bool((weight > 0).all()):
        raise ValueError("quadratic weights must be finite and positive")
    return target.float() - 0.5 * float(strength) * gradient.float() / weight


def shift_two_sided_target(target: torch.Tensor, gradient: torch.Tensor, row_hessian: torch.Tensor,
                           column_hessian: torch.Tensor, *, strength: float) -> torch.Tensor:
    """Completed square under ``tr(E^T H_row E H_column)`` (``gradient_guided_viterbi.py:155-187``):
    ``target - strength/2 * H_row^-1 G H_column^-1`` by two solves."""

    if target.ndim != 2 or gradient.shape != target.shape:
        raise ValueError("two-sided target and gradient must be matching matrices")
    rows, columns = target.shape
    if tuple(row_hessian.shape) != (rows, rows):
        raise ValueError("row Hessian has incompatible geometry")
    if tuple(column_hessian.shape) != (columns, columns):
        raise ValueError("column Hessian has incompatible geometry")
    if not math.isfinite(strength) or strength < 0.0:
        raise ValueError("gradient strength must be finite and nonnegative")
    dtype = torch.float64 if target.dtype == torch.float64 else torch.float32
    move = dict(device=target.device, dtype=dtype)
    left = torch.linalg.solve(row_hessian.to(**move), gradient.to(**move))
    correction = torch.linalg.solve(column_hessian.to(**move).T, left.T).T
    if not bool(torch.isfinite(correction).all()):
        raise FloatingPointError("two-sided gradient target shift is non-finite")
    return target.to(dtype=dtype) - 0.5 * float(strength) * correction


def two_sided_guided_objective(target, candidate, anchor, gradient, row_hessian, column_hessian, *, strength: float):
    """Quadratic, linear and combined objectives as 0-d tensors (``gradient_guided_viterbi.py:190-207``)."""

    if not (target.shape == candidate.shape == anchor.shape == gradient.shape):
        raise ValueError("guided objective matrices must have matching shapes")
    error = candidate - target
    quadratic = torch.sum(error * (row_hessian @ error @ column_hessian))
    linear = float(strength) * torch.sum(gradient * (candidate - anchor))
    return quadratic, linear, quadratic + linear


# ---- configuration and results ---------------------------------------------------------------------
@dataclass(frozen=True)
class H2ViterbiRefineConfig:
    """Search controls (``h2_viterbi_refine.py:31-44``).  ``max_quantizer_batch`` only chunks calls
    of a caller-supplied ``quantize_tiles``; the fused row kernel takes a whole block at once."""

    sweeps: int = 1
    alternate_sweep_order: bool = True
    dither_scales: tuple[float, ...] = ()
    num_dither_patterns: int = 0
    seed: int = 0x48325643
    max_quantizer_batch: int = 256
    acceptance_abs_tol: float = 1.0e-8
    acceptance_rel_tol: float = 1.0e-8
    score_dtype: torch.dtype = torch.float32
    stop_on_no_change: bool = True


@dataclass(frozen=True)
class H2ViterbiSweepStats:
    sweep: int
    objective_before: float
    objective_after: float
    quadratic_before: float
    quadratic_after: float
    linear_before: float
    linear_after: float
    relative_improvement: float
    accepted_tiles: int
    proposed_tiles: int
    unique_candidate_paths: int


@dataclass
class H2ViterbiRefineResult:
    weight_q: torch.Tensor
    encoded: torch.Tensor
    sweep_stats: list[H2ViterbiSweepStats]

    def stats_dict(self) -> dict[str, object]:
        return {"sweeps": [asdict(stats) for stats in self.sweep_stats]}


def config_from_quant_args(quant_args: dict) -> H2ViterbiRefineConfig:
    """Refinement controls from the private encoder arguments (``h2_viterbi_refine.py:563-590``)."""

    get = quant_args.get
    return H2ViterbiRefineConfig(
        sweeps=int(get("h2_viterbi_refine_sweeps", 1)),
        alternate_sweep_order=bool(get("h2_viterbi_refine_alternate_order", True)),
        dither_scales=tuple(float(v) for v in get("h2_viterbi_refine_dither_scales", ())),
        num_dither_patterns=int(get("h2_viterbi_refine_patterns", 0)),
        seed=int(get("h2_viterbi_refine_seed", 0x48325643)),
        max_quantizer_batch=int(get("h2_viterbi_refine_max_batch", 256)),
        score_dtype=torch.float64 if get("h2_viterbi_refine_fp64_score", False) else torch.float32,
    )


# ---- objectives --------------------------------------------------------------------------------------
def _column_weights(column_weights, columns: int, device, dtype) -> torch.Tensor:
    if column_weights is None:
        return torch.ones(columns, dtype=dtype, device=device)
    if column_weights.numel() != columns:
        raise ValueError("column weights do not match the output dimension")
    weights = column_weights.reshape(-1).to(device=device, dtype=dtype)
    if bool(torch.any(weights < 0)):
        raise ValueError("column weights must be nonnegative")
    return weights


def dense_h_objective(weight: torch.Tensor, weight_q: torch.Tensor, hessian: torch.Tensor, *,
                      column_weights: torch.Tensor | None = None, chunk_columns: int = 512,
                      dtype: torch.dtype = torch.float64) -> float:
    """``sum_c a[c] * (W-Q)[:, c]^T H (W-Q)[:, c]`` (``h2_viterbi_refine.py:71-103``)."""

    if weight.shape != weight_q.shape or weight.ndim != 2:
        raise ValueError("weight and reconstruction must have one rank-2 shape")
    if hessian.shape != (weight.shape[0], weight.shape[0]):
        raise ValueError("Hessian shape does not match the input dimension")
    if chunk_columns <= 0:
        raise ValueError("chunk_columns must be positive")
    weights = _column_weights(column_weights, weight.shape[1], weight.device, dtype)
    hessian_work = hessian.to(device=weight.device, dtype=dtype)
    total = torch.zeros((), dtype=dtype, device=weight.device)
    for begin in range(0, weight.shape[1], chunk_columns):
        columns = slice(begin, begin + chunk_columns)
        error = (weight[:, columns] - weight_q[:, columns]).to(dtype)
        total += torch.sum(error * (hessian_work @ error) * weights[columns].unsqueeze(0))
    return float(total.item())


def _linear_term(guidance, candidate: torch.Tensor, dtype) -> float:
    if guidance is None:
        return 0.0
    if isinstance(guidance, LowRankViterbiGradientGuidance) or hasattr(guidance, "linear_term"):
        return guidance.linear_term(candidate, dtype=dtype)
    gradient = guidance.gradient.to(device=candidate.device, dtype=dtype)
    anchor = guidance.anchor.to(device=candidate.device, dtype=dtype)
    return float(float(guidance.strength) * torch.sum(gradient * (candidate.to(dtype) - anchor)).item())


def dense_h_guided_objective(weight: torch.Tensor, weight_q: torch.Tensor, hessian: torch.Tensor, guidance, *,
                             column_weights: torch.Tensor | None = None, chunk_columns: int = 512,
                             dtype: torch.dtype = torch.float64) -> tuple[float, float, float]:
    """Quadratic, anchor-relative linear and combined objectives (``h2_viterbi_refine.py:106-139``)."""

    guidance.validate(weight.shape)
    quadratic = dense_h_objective(weight, weight_q, hessian, column_weights=column_weights,
                                  chunk_columns=chunk_columns, dtype=dtype)
    linear = _linear_term(guidance, weight_q, dtype)
    return quadratic, linear, quadratic + linear


# ---- proposals ---------------------------------------------------------------------------------------
def _encoder():
    from . import encoder  # late: encoder imports the candidate schedules at its end

    return encoder


class _RowKernelProposer:
    """Tile search of ``[V, 16, n]`` row-major targets by the fused row kernel."""

    def __init__(self, quant_args: dict, device: torch.device, columns: int, variants: int) -> None:
        self.quant_args = quant_args
        self.bits = int(quant_args["K"])
        self.columns = columns
        self.recon = torch.empty((variants, 16, columns), dtype=torch.float32, device=device)
        self.states = torch.empty((variants, columns // 16, 256), dtype=torch.int16, device=device)

    def __call__(self, stacked: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        n = self.columns
        _encoder()._quantize_rows(
            stacked, None, 0.0, self.recon, None, self.states, self.quant_args, self.bits,
            batch=stacked.shape[0], n=n, ld=n, w_stride=16 * n, comp_ld=n, comp_stride=0,
            state_stride=(n // 16) * 256,
        )
        return self.recon, self.states


class _CallbackProposer:
    """The reference's callback contract: flattened tiles in tensor-core order, chunked calls."""

    def __init__(self, quantize_tiles: QuantizeTiles, device: torch.device, max_batch: int) -> None:
        if max_batch <= 0:
            raise ValueError("max_quantizer_batch must be positive")
        self.quantize_tiles, self.max_batch = quantize_tiles, max_batch
        self.order = _encoder().tensor_core_perm(device)
        self.inverse = torch.argsort(self.order)

    def __call__(self, stacked: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        variants, _, n = stacked.shape
        tiles = stacked.reshape(variants, 16, n // 16, 16).permute(0, 2, 1, 3).reshape(-1, 256)[:, self.order]
        recon, payload = [], []
        for begin in range(0, tiles.shape[0], self.max_batch):
            source = tiles[begin:begin + self.max_batch].contiguous()
            r, p = self.quantize_tiles(source)
            if r.shape != source.shape:
                raise ValueError("tile quantizer returned the wrong reconstruction shape")
            if p.ndim < 1 or p.shape[0] != source.shape[0]:
                raise ValueError("tile quantizer returned the wrong payload batch")
            recon.append(r)
            payload.append(p)
        payload = torch.cat(payload)
        if payload.shape[1:] != (256,) or payload.dtype != torch.int16:
            raise ValueError("stored and proposed trellis payload shapes differ")
        rows = torch.cat(recon)[:, self.inverse].reshape(variants, n // 16, 16, 16).permute(0, 2, 1, 3)
        return rows.reshape(variants, 16, n).contiguous().float(), payload.reshape(variants, n // 16, 256).contiguous()


def _whitened_patterns(hessian_block: torch.Tensor, count: int, seed: int, dtype) -> torch.Tensor:
    """``count`` sign patterns whitened by the block's Cholesky factor and scaled to H-energy 256
    (``h2_viterbi_refine.py:182-219``); the sign draw uses the device generator as the reference does."""

    device = hessian_block.device
    if count <= 0:
        return torch.empty((0, 16, 16), dtype=dtype, device=device)
    generator = torch.Generator(device=device)
    generator.manual_seed(seed)
    signs = torch.randint(0, 2, (count, 16, 16), generator=generator, device=device, dtype=torch.int64)
    signs = (signs * 2 - 1).to(dtype)
    work = hessian_block.to(dtype)
    upper = torch.linalg.cholesky(work).transpose(0, 1)
    columns = torch.linalg.solve_triangular(upper, signs.permute(1, 0, 2).reshape(16, count * 16), upper=True)
    patterns = columns.reshape(16, count, 16).permute(1, 0, 2)
    energy = torch.sum(patterns * torch.einsum("ij,pjc->pic", work, patterns), dim=(1, 2), keepdim=True)
    return patterns * torch.sqrt(256.0 / energy.clamp_min(1.0e-20))


# ---- the refinement ------------------------------------------------------------------------------------
@torch.no_grad()
def refine_h2_viterbi_paths(weight: torch.Tensor, hessian: torch.Tensor, initial_weight_q: torch.Tensor,
                            initial_encoded: torch.Tensor, quantize_tiles,
                            config: H2ViterbiRefineConfig = H2ViterbiRefineConfig(), *,
                            column_weights: torch.Tensor | None = None, guidance=None) -> H2ViterbiRefineResult:
    """Refine legal paths under dense-H plus an optional linear objective
    (``h2_viterbi_refine.py:334-560``).

    ``quantize_tiles`` is either the encoder's ``quant_args`` dict (the fused row kernel searches
    the targets) or a callable with the reference's contract.  The payload is the tile search's
    ``[rows/16, columns/16, 256]`` int16 state grid.
    """

    if weight.ndim != 2 or initial_weight_q.shape != weight.shape:
        raise ValueError("weight and reconstruction must have one rank-2 shape")
    rows, columns = weight.shape
    if rows % 16 or columns % 16:
        raise ValueError("weight dimensions must be multiples of 16")
    if hessian.shape != (rows, rows):
        raise ValueError("Hessian shape does not match the input dimension")
    row_blocks, column_blocks = rows // 16, columns // 16
    if initial_encoded.ndim < 3 or tuple(initial_encoded.shape[:2]) != (row_blocks, column_blocks):
        raise ValueError("stored trellis payload has the wrong tile grid")
    if config.sweeps <= 0:
        raise ValueError("sweeps must be positive")
    if guidance is not None:
        guidance.validate(weight.shape)
    device = weight.device
    if device.type != "cuda":
        raise ValueError("the B200 refinement requires CUDA tensors")
    if tuple(initial_encoded.shape[2:]) != (256,) or initial_encoded.dtype != torch.int16:
        raise ValueError("stored and proposed trellis payload shapes differ")
    dtype = config.score_dtype
    if dtype not in (torch.float32, torch.float64):
        raise ValueError("score_dtype must be float32 or float64")

    hessian_work = hessian.to(device=device, dtype=dtype).contiguous()
    weights_work = _column_weights(column_weights, columns, device, dtype).contiguous()
    strength = 0.0 if guidance is None else float(guidance.strength)
    low_rank = guidance is not None and hasattr(guidance, "rows")
    dense_gradient = None if guidance is None or low_rank else guidance.gradient.to(device=device, dtype=dtype)
    if guidance is not None and strength != 0.0 and bool(torch.any(weights_work <= 0)):
        raise ValueError("gradient-guided refinement requires positive column weights")

    weight_work = weight.to(device=device, dtype=torch.float32).contiguous()
    reconstruction = initial_weight_q.to(device=device, dtype=torch.float32).clone().contiguous()
    encoded = initial_encoded.to(device).clone().contiguous()
    error = (weight_work - reconstruction).to(dtype)
    hessian_error = hessian_work @ error

    def objectives() -> tuple[float, float]:
        quadratic = float(torch.sum(error * hessian_error * weights_work.unsqueeze(0)).item())
        return quadratic, _linear_term(guidance, reconstruction, dtype)

    quadratic, linear = objectives()
    objective = quadratic + linear

    # LU factors of every diagonal block, once
    diagonal = torch.arange(row_blocks, device=device)
    blocks = hessian_work.view(row_blocks, 16, row_blocks, 16).permute(0, 2, 1, 3)[diagonal, diagonal].contiguous()
    factors, pivots = torch.linalg.lu_factor(blocks)

    patterns_per_block = config.num_dither_patterns if config.dither_scales else 0
    variants = 1 + 2 * len(config.dither_scales) * max(patterns_per_block, 0)
    if isinstance(quantize_tiles, dict):
        propose = _RowKernelProposer(quantize_tiles, device, columns, variants)
    elif callable(quantize_tiles):
        propose = _CallbackProposer(quantize_tiles, device, config.max_quantizer_batch)
    else:
        raise TypeError("quantize_tiles must be the encoder's quant_args or a callable")
    stacked = torch.empty((variants, 16, columns), dtype=torch.float32, device=device)
    delta = torch.empty((16, columns), dtype=dtype, device=device)
    counters = torch.zeros(2, dtype=torch.int64, device=device)
    library, stream = _lib.lib(), _stream_ptr(device)

    sweep_stats: list[H2ViterbiSweepStats] = []
    for sweep in range(config.sweeps):
        before, quadratic_before, linear_before = objective, quadratic, linear
        counters.zero_()
        reverse = not config.alternate_sweep_order or sweep % 2 == 0
        for row_block in (range(row_blocks - 1, -1, -1) if reverse else range(row_blocks)):
            span = slice(row_block * 16, row_block * 16 + 16)
            block = blocks[row_block]
            cross = hessian_error[span] - block @ error[span]
            target = weight_work[span].to(dtype) + torch.linalg.lu_solve(factors[row_block], pivots[row_block], cross)
            if guidance is not None and strength != 0.0:
                gradient = guidance.rows(span, device=device, dtype=dtype) if low_rank else dense_gradient[span]
                correction = torch.linalg.lu_solve(factors[row_block], pivots[row_block],
                                                   gradient / weights_work.unsqueeze(0))
                target = target - 0.5 * strength * correction
            stacked[0] = target
            if variants > 1:
                patterns = _whitened_patterns(block, patterns_per_block,
                                              config.seed + 1009 * sweep + 9176 * row_block, torch.float32)
                tiles = stacked[0].view(16, column_blocks, 16)
                rms = tiles.square().mean(dim=(0, 2), keepdim=True).sqrt().clamp_min(1.0e-8)
                slot = 1
                for scale in config.dither_scales:
                    for pattern in patterns:
                        shift = (float(scale) * rms * pattern.unsqueeze(1)).reshape(16, columns)
                        stacked[slot] = stacked[0] + shift
                        stacked[slot + 1] = stacked[0] - shift
                        slot += 2
            candidates, candidate_states = propose(stacked)
            with torch.cuda.device(device):
                _lib.check(
                    library.qsrtb_refine_select(
                        weight_work[span].data_ptr(), columns, stacked.data_ptr(), columns,
                        reconstruction[span].data_ptr(), columns, columns,
                        candidates.data_ptr(), columns, 16 * columns, variants,
                        candidate_states.data_ptr(), column_blocks * 256, encoded[row_block].data_ptr(),
                        block.data_ptr(), 16, weights_work.data_ptr(), error[span].data_ptr(), columns,
                        delta.data_ptr(), columns, float(config.acceptance_abs_tol),
                        float(config.acceptance_rel_tol), int(dtype == torch.float64),
                        counters.data_ptr(), stream,
                    ),
                    "qsrtb_refine_select",
                )
            hessian_error.addmm_(hessian_work[:, span], delta)

        hessian_error = hessian_work @ error
        quadratic, linear = objectives()
        objective = quadratic + linear
        if objective > before + max(1.0e-5, 1.0e-6 * abs(before)):
            raise RuntimeError("dense-H objective increased; quantizer coordinates are inconsistent")
        accepted, unique = (int(v) for v in counters.tolist())
        sweep_stats.append(H2ViterbiSweepStats(
            sweep=sweep, objective_before=before, objective_after=objective,
            quadratic_before=quadratic_before, quadratic_after=quadratic,
            linear_before=linear_before, linear_after=linear,
            relative_improvement=(before - objective) / max(abs(before), 1.0e-30),
            accepted_tiles=accepted, proposed_tiles=row_blocks * column_blocks, unique_candidate_paths=unique,
        ))
        if config.stop_on_no_change and accepted == 0:
            break
    return H2ViterbiRefineResult(reconstruction, encoded, sweep_stats)


def refine_uniform_h2_candidate(weight: torch.Tensor, hessian: torch.Tensor, weight_q: torch.Tensor,
                                encoded: torch.Tensor, quant_args: dict, *, guidance=None):
    """Revisit a uniform-rate candidate under its dense-H proxy with the candidate's own rate, table
    and tail-biting search (``exl3_encoder_backend.py:840-895``).  Off unless
    ``h2_viterbi_refine_sweeps`` is positive."""

    sweeps = int(quant_args.get("h2_viterbi_refine_sweeps", 0))
    if sweeps <= 0:
        return weight_q, encoded, {"enabled": False, "sweeps": []}
    if quant_args.get("periodic_rate_schedules") is not None:
        raise ValueError("dense-H path refinement requires one fixed tile rate")
    if len(quant_args["devices"]) != 1:
        raise ValueError("dense-H path refinement requires one quantizer device")
    local_args = dict(quant_args)
    if "mixed_rate_axis" in quant_args or "mixed_tile_bits" in quant_args:
        _, tile_bits = _encoder().mixed_rate_spec(weight.shape[0], weight.shape[1], quant_args)
        distinct = set(tile_bits)
        if len(distinct) != 1:
            raise ValueError("dense-H path refinement requires a uniform rate map")
        local_args["K"] = distinct.pop()
    if quant_args.get("mixed_tile_codebook_ids") is not None:
        raise ValueError("dense-H path refinement does not support tile-local codebook selectors")
    result = refine_h2_viterbi_paths(weight, hessian.to(device=weight.device), weight_q, encoded, local_args,
                                     config_from_quant_args(local_args), guidance=guidance)
    return result.weight_q, result.encoded, {"enabled": True, "rate_bits": int(local_args["K"]),
                                             **result.stats_dict()}
