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
