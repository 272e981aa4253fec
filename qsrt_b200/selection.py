"""Host-side candidate selection and expert sharding.

Scores are a few scalars per expert; as in the reference this logic stays on the host.

* ``select_pooled_candidate`` mirrors ``qsrt/pooled_selection.py:54-99`` (minimum SSE with a
  source-energy tie tolerance, then fewer metadata bytes, fewer transfers, stable name).
* ``assign_experts`` shards the experts of a layer over ranks (longest-processing-time first on
  the routed-row counts, ties to the lower expert id), the expert-wise partition the
  reference's driver performs with one worker process per GPU
  (``scripts/pack_qsrt_candidates.py:2025-2125``).
* ``gather_candidate_table`` is the path's only collective: an all-gather of the
  ``[experts_local, candidates, 2]`` float64 (SSE, bytes) table.
* ``equal_byte_exchange`` is the greedy K2<->K4 exchange around a K3 baseline: every rank runs
  it on the identical gathered table, so every rank selects the same rates without another
  exchange.  It follows the reference's exchange rule (one K2 donor funds one K4 recipient,
  accepted while ``c2[donor] + c4[recipient] - c3[donor] - c3[recipient] < 0``,
  ``qsrt/high_rate_allocation.py:229-330``) at expert granularity.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Iterable, Sequence

import torch


@dataclass(frozen=True)
class PooledCandidateScore:
    name: str
    sse: float
    source_energy: float
    metadata_bytes: int
    n13: int = 0
    n2: int = 0

    def validate(self) -> None:
        if not self.name:
            raise ValueError("candidate name must be nonempty")
        if not math.isfinite(self.sse) or self.sse < 0:
            raise ValueError(f"candidate {self.name!r} has invalid SSE")
        if not math.isfinite(self.source_energy) or self.source_energy <= 0:
            raise ValueError(f"candidate {self.name!r} has invalid source energy")
        if self.metadata_bytes < 0:
            raise ValueError(f"candidate {self.name!r} has invalid metadata size")
        if self.n13 < 0 or self.n2 < 0:
            raise ValueError(f"candidate {self.name!r} has invalid transfer count")

    @property
    def transfer_count(self) -> int:
        return self.n13 + self.n2


@dataclass(frozen=True)
class PooledSelection:
    selected: PooledCandidateScore
    minimum_sse: float
    tie_tolerance: float
    tied_names: tuple[str, ...]


def select_pooled_candidate(candidates: Iterable[PooledCandidateScore], *,
                            tie_relative_to_source_energy: float = 1e-10) -> PooledSelection:
    scores = tuple(candidates)
    if not scores:
        raise ValueError("pooled selection requires at least one candidate")
    for score in scores:
        score.validate()
    if len({score.name for score in scores}) != len(scores):
        raise ValueError("pooled candidate names must be unique")
    source_energy = scores[0].source_energy
    energy_tolerance = max(64 * math.ulp(source_energy), 1e-12 * source_energy)
    if any(abs(score.source_energy - source_energy) > energy_tolerance for score in scores):
        raise ValueError("pooled candidates do not share one source-energy reference")
    relative_tolerance = float(tie_relative_to_source_energy)
    if not math.isfinite(relative_tolerance) or relative_tolerance < 0:
        raise ValueError("tie tolerance must be finite and nonnegative")
    minimum = min(score.sse for score in scores)
    tolerance = relative_tolerance * source_energy
    tied = tuple(score for score in scores if score.sse <= minimum + tolerance)
    selected = min(tied, key=lambda s: (s.metadata_bytes, s.transfer_count, s.n13, s.n2, s.name))
    return PooledSelection(selected, minimum, tolerance, tuple(sorted(s.name for s in tied)))


def assign_experts(row_counts: Sequence[int], world_size: int, *, fixed_cost: float = 4096.0) -> list[list[int]]:
    """Experts -> ranks.  Encode cost is nearly constant per expert (``fixed_cost`` rows'
    worth) and Hessian / scoring cost grows with the routed rows; heaviest experts are placed
    first on the least-loaded rank.  Deterministic: ties go to the lower expert id / rank."""

    if world_size <= 0:
        raise ValueError("world_size must be positive")
    order = sorted(range(len(row_counts)), key=lambda e: (-(row_counts[e] + fixed_cost), e))
    loads = [0.0] * world_size
    counts = [0] * world_size
    shards: list[list[int]] = [[] for _ in range(world_size)]
    cap = math.ceil(len(row_counts) / world_size)
    for expert in order:
        open_ranks = [r for r in range(world_size) if counts[r] < cap]
        rank = min(open_ranks, key=lambda r: (loads[r], r))
        shards[rank].append(expert)
        loads[rank] += row_counts[expert] + fixed_cost
        counts[rank] += 1
    return [sorted(s) for s in shards]


def gather_candidate_table(local_table: torch.Tensor, local_experts: Sequence[int], num_experts: int,
                           group=None) -> torch.Tensor:
    """All-gather ``[experts_local, candidates, 2]`` float64 tables into the layer table
    ``[num_experts, candidates, 2]`` (rows of experts nobody owns stay NaN)."""

    import torch.distributed as dist

    if local_table.ndim != 3 or local_table.shape[0] != len(local_experts) or local_table.dtype != torch.float64:
        raise ValueError("local table must be float64 [experts_local, candidates, 2]")
    full = torch.full((num_experts, *local_table.shape[1:]), float("nan"), dtype=torch.float64, device=local_table.device)
    if not (dist.is_available() and dist.is_initialized()):
        full[torch.as_tensor(list(local_experts), dtype=torch.long, device=local_table.device)] = local_table
        return full
    world = dist.get_world_size(group)
    cap = torch.tensor([len(local_experts)], dtype=torch.int64, device=local_table.device)
    caps = [torch.zeros_like(cap) for _ in range(world)]
    dist.all_gather(caps, cap, group=group)
    width = int(max(int(c.item()) for c in caps))
    padded = torch.full((width, *local_table.shape[1:]), float("nan"), dtype=torch.float64, device=local_table.device)
    padded[: len(local_experts)] = local_table
    ids = torch.full((width,), -1, dtype=torch.int64, device=local_table.device)
    ids[: len(local_experts)] = torch.as_tensor(list(local_experts), dtype=torch.int64, device=local_table.device)
    tables = [torch.empty_like(padded) for _ in range(world)]
    id_lists = [torch.empty_like(ids) for _ in range(world)]
    dist.all_gather(tables, padded, group=group)
    dist.all_gather(id_lists, ids, group=group)
    for table, idl in zip(tables, id_lists):
        keep = idl >= 0
        full[idl[keep]] = table[keep]
    return full


@dataclass(frozen=True)
class RateAllocation:
    bits: tuple[int, ...]          # selected rate per expert
    total_sse: float
    total_bytes: float
    exchanges: int
    baseline_sse: float


def equal_byte_exchange(table: torch.Tensor, *, rates: Sequence[int] = (2, 3, 4), free_upgrades: int = 0) -> RateAllocation:
    """Greedy equal-byte K2<->K4 exchanges around the K3 baseline.

    ``table[e, c] = (sse, bytes)`` for candidate rate ``rates[c]`` of expert ``e``.  Starting
    from all-K3 (plus ``free_upgrades`` experts moved to K4 by largest gain when the byte budget
    exceeds 3 bits per weight), the pair (donor, recipient) with the most negative
    ``c2[donor] + c4[recipient] - c3[donor] - c3[recipient]`` is exchanged until no exchange
    lowers the total error.  A K2 donor releases exactly the bytes a K4 recipient consumes when
    experts have equal sizes, so the byte total is unchanged.  Ties: lower expert id.
    """

    if tuple(rates) != (2, 3, 4) or table.ndim != 3 or table.shape[1:] != (3, 2):
        raise ValueError("table must be [experts, 3, 2] for rates (2, 3, 4)")
    sse = table[:, :, 0].double().cpu()
    size = table[:, :, 1].double().cpu()
    if not bool(torch.isfinite(sse).all()):
        raise ValueError("candidate table has missing or non-finite errors")
    experts = sse.shape[0]
    bits = [3] * experts
    gain4 = (sse[:, 1] - sse[:, 2]).tolist()   # error saved by K3 -> K4
    loss2 = (sse[:, 0] - sse[:, 1]).tolist()   # error added by K3 -> K2
    for e in sorted(range(experts), key=lambda e: (-gain4[e], e))[: max(0, int(free_upgrades))]:
        bits[e] = 4
    baseline = float(sum(sse[e, bits[e] - 2] for e in range(experts)))
    exchanges = 0
    while True:
        donors = [e for e in range(experts) if bits[e] == 3]
        if len(donors) < 2:
            break
        donor = min(donors, key=lambda e: (loss2[e], e))
        recipients = [e for e in donors if e != donor]
        recipient = min(recipients, key=lambda e: (-gain4[e], e))
        delta = loss2[donor] - gain4[recipient]
        if not delta < 0:
            break
        bits[donor], bits[recipient] = 2, 4
        exchanges += 1
    total_sse = float(sum(sse[e, bits[e] - 2] for e in range(experts)))
    total_bytes = float(sum(size[e, bits[e] - 2] for e in range(experts)))
    return RateAllocation(tuple(bits), total_sse, total_bytes, exchanges, baseline)


# ---- phase-1 rate selection with a bootstrap gate (qsrt/qsrt_candidates.py:657-898) -------------

PHASE1_MODE_IDS = (0, 1, 2)
PHASE1_MIN_FIT_DOCUMENTS = 6
PHASE1_MIN_CONFIRMATION_DOCUMENTS = 4
PHASE1_BOOTSTRAP_REPLICATES = 2_000
PHASE1_SELECTION_SEED = 20_260_801


@dataclass(frozen=True)
class ModeSelection:
    """A mode proposed on the fit documents and gated on the confirmation documents."""

    proposed_r: int
    selected_r: int
    accepted: bool
    reason: str
    fit_documents: int
    confirmation_documents: int
    confirmation_relative_improvement: float | None
    confirmation_ci95: tuple[float | None, float | None]
    bootstrap_replicates_valid: int


@dataclass(frozen=True)
class RatePairSelection:
    """An ``(r13, r2)`` pair ranked and gated on the confirmation documents."""

    proposed_r13: int
    proposed_r2: int
    selected_r13: int
    selected_r2: int
    accepted: bool
    reason: str
    fit_documents: int
    confirmation_documents: int
    confirmation_relative_improvement: float | None
    confirmation_ci95: tuple[float | None, float | None]
    bootstrap_replicates_valid: int

    @property
    def proposed(self) -> tuple[int, int]:
        return self.proposed_r13, self.proposed_r2

    @property
    def selected(self) -> tuple[int, int]:
        return self.selected_r13, self.selected_r2


def bootstrap_improvement(baseline: torch.Tensor, candidate: torch.Tensor, support: torch.Tensor, *,
                          replicates: int, seed: int):
    """Relative SSE improvement ``1 - sum(candidate) / sum(baseline)`` over the supported documents
    and its 95 % bootstrap interval (qsrt/qsrt_candidates.py:657-696).

    Documents are resampled with replacement by ``numpy.random.default_rng(seed)`` in batches of
    at most 512 replicates, exactly as in the reference, so the interval is reproducible bit for
    bit.  Returns ``(observed, (low, high), valid_replicates)``; ``None`` where undefined.
    """

    import numpy as np

    if replicates < 100:
        raise ValueError("bootstrap replicates must be at least 100")
    if baseline.shape != candidate.shape or baseline.ndim != 1:
        raise ValueError("bootstrap SSE vectors must be equal one-dimensional shapes")
    if support.dtype != torch.bool or support.shape != baseline.shape:
        raise ValueError("bootstrap support mask has the wrong shape")
    base = baseline[support].double().cpu().numpy()
    trial = candidate[support].double().cpu().numpy()
    if base.size == 0 or not np.isfinite(base).all() or not np.isfinite(trial).all():
        return None, (None, None), 0
    total = float(base.sum())
    if total <= 0:
        return None, (None, None), 0
    observed = 1.0 - float(trial.sum()) / total
    rng = np.random.default_rng(int(seed))
    kept = []
    left = int(replicates)
    while left:
        count = min(left, 512)
        draw = rng.integers(0, base.size, size=(count, base.size))
        drawn_base, drawn_trial = base[draw].sum(axis=1), trial[draw].sum(axis=1)
        usable = drawn_base > 0
        if np.any(usable):
            kept.append(1.0 - drawn_trial[usable] / drawn_base[usable])
        left -= count
    if not kept:
        return observed, (None, None), 0
    samples = np.concatenate(kept)
    low, high = np.quantile(samples, (0.025, 0.975)).tolist()
    return observed, (float(low), float(high)), int(samples.size)


def _gate_reason(interval, minimum_improvement: float) -> tuple[bool, str]:
    if interval[0] is None:
        return False, "confirmation bootstrap has no valid baseline samples"
    if interval[0] <= minimum_improvement:
        return False, "confirmation lower confidence bound did not clear the margin"
    return True, "confirmation lower confidence bound cleared the margin"


def select_phase1_mode(fit_sse, confirmation_sse, *, fit_counts: torch.Tensor, confirmation_counts: torch.Tensor,
                       mode_ids: Sequence[int] = PHASE1_MODE_IDS, min_fit_documents: int = PHASE1_MIN_FIT_DOCUMENTS,
                       min_confirmation_documents: int = PHASE1_MIN_CONFIRMATION_DOCUMENTS,
                       minimum_improvement: float = 0.0, bootstrap_replicates: int = PHASE1_BOOTSTRAP_REPLICATES,
                       seed: int = PHASE1_SELECTION_SEED) -> ModeSelection:
    """Propose the fit-document argmin and accept it only if the lower end of the confirmation
    documents' bootstrap interval clears the margin (qsrt/qsrt_candidates.py:699-790)."""

    modes = tuple(int(m) for m in mode_ids)
    if not modes or modes[0] != 0 or len(set(modes)) != len(modes):
        raise ValueError("mode_ids must be unique and begin with R0")
    if set(fit_sse) != set(modes) or set(confirmation_sse) != set(modes):
        raise ValueError("SSE tables must contain every requested mode")
    fit_support, confirmation_support = fit_counts > 0, confirmation_counts > 0
    fit_documents, confirmation_documents = int(fit_support.sum()), int(confirmation_support.sum())

    def decision(proposed, selected, accepted, reason, improvement=None, interval=(None, None), valid=0):
        return ModeSelection(proposed, selected, accepted, reason, fit_documents, confirmation_documents,
                             improvement, interval, valid)

    if fit_documents < min_fit_documents:
        return decision(0, 0, False, "insufficient fit-document support")
    proposed = min(modes, key=lambda m: (float(fit_sse[m][fit_support].double().sum()), m))
    if proposed == 0:
        return decision(0, 0, False, "R0 is the fit-document argmin")
    improvement, interval, valid = bootstrap_improvement(
        confirmation_sse[0], confirmation_sse[proposed], confirmation_support,
        replicates=bootstrap_replicates, seed=seed)
    cleared, reason = _gate_reason(interval, minimum_improvement)
    if confirmation_documents < min_confirmation_documents:
        cleared, reason = False, "insufficient confirmation-document support"
    return decision(proposed, proposed if cleared else 0, cleared, reason, improvement, interval, valid)


def select_phase1_rate_pair(fit_sse, confirmation_sse, *, fit_counts: torch.Tensor, confirmation_counts: torch.Tensor,
                            modes: Sequence[tuple[int, int]], min_fit_documents: int = PHASE1_MIN_FIT_DOCUMENTS,
                            min_confirmation_documents: int = PHASE1_MIN_CONFIRMATION_DOCUMENTS,
                            minimum_improvement: float = 0.0, bootstrap_replicates: int = PHASE1_BOOTSTRAP_REPLICATES,
                            seed: int = PHASE1_SELECTION_SEED) -> RatePairSelection:
    """Rank the ``(r13, r2)`` grid on the confirmation documents (the fit documents built the
    encoder's Hessians and only have to exist) and bootstrap-gate the winner against R0/R0
    (qsrt/qsrt_candidates.py:793-898).  Ties go to fewer transfers, then the smaller r13, r2."""

    candidates = tuple((int(a), int(b)) for a, b in modes)
    if not candidates or candidates[0] != (0, 0) or len(set(candidates)) != len(candidates):
        raise ValueError("rate-pair candidates must be unique and begin with R0/R0")
    if set(fit_sse) != set(candidates) or set(confirmation_sse) != set(candidates):
        raise ValueError("rate-pair SSE tables must contain every requested candidate")
    fit_support, confirmation_support = fit_counts > 0, confirmation_counts > 0
    fit_documents, confirmation_documents = int(fit_support.sum()), int(confirmation_support.sum())

    def decision(proposed, selected, accepted, reason, improvement=None, interval=(None, None), valid=0):
        return RatePairSelection(proposed[0], proposed[1], selected[0], selected[1], accepted, reason,
                                 fit_documents, confirmation_documents, improvement, interval, valid)

    if fit_documents < min_fit_documents:
        return decision((0, 0), (0, 0), False, "insufficient fit-document support")
    if confirmation_documents < min_confirmation_documents:
        return decision((0, 0), (0, 0), False, "insufficient confirmation-document support")
    proposed = min(candidates, key=lambda p: (float(confirmation_sse[p][confirmation_support].double().sum()),
                                               p[0] + p[1], p[0], p[1]))
    if proposed == (0, 0):
        return decision(proposed, proposed, False, "R0/R0 is the confirmation-document argmin")
    improvement, interval, valid = bootstrap_improvement(
        confirmation_sse[(0, 0)], confirmation_sse[proposed], confirmation_support,
        replicates=bootstrap_replicates, seed=seed)
    cleared, reason = _gate_reason(interval, minimum_improvement)
    return decision(proposed, proposed if cleared else (0, 0), cleared, reason, improvement, interval, valid)


def select_coupled_modes(matrix_sse, families) -> dict:
    """Minimum total SSE per coupled matrix family, ties to the lower mode
    (qsrt/qsrt_codec_pilot.py:760-798).  ``matrix_sse[matrix][mode]`` are per-matrix errors and
    ``families[name]`` the matrices that must share one mode; the families must partition the
    matrices exactly."""

    if not matrix_sse or not families:
        raise ValueError("mode selection requires matrices and families")
    covered: list[str] = []
    out: dict[str, dict] = {}
    for family, matrices in families.items():
        members = tuple(matrices)
        if not members:
            raise ValueError(f"rate family {family!r} is empty")
        covered.extend(members)
        if members[0] not in matrix_sse:
            raise KeyError(f"unknown matrix in rate family {family!r}")
        ladder = set(matrix_sse[members[0]])
        for matrix in members[1:]:
            if matrix not in matrix_sse:
                raise KeyError(f"unknown matrix {matrix!r}")
            if set(matrix_sse[matrix]) != ladder:
                raise ValueError("coupled matrices do not share one mode ladder")
        totals = {int(mode): sum(float(matrix_sse[m][mode]) for m in members) for mode in ladder}
        if not totals or any(not math.isfinite(v) or v < 0.0 for v in totals.values()):
            raise ValueError("mode SSE must be finite and nonnegative")
        best = min(totals, key=lambda mode: (totals[mode], mode))
        out[str(family)] = {"matrices": list(members), "selected_mode": int(best),
                            "sse_by_mode": {f"R{mode}": totals[mode] for mode in sorted(totals)}}
    if len(covered) != len(set(covered)) or set(covered) != set(matrix_sse):
        raise ValueError("rate families must partition the codec matrices exactly")
    return out
