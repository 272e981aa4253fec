"""Host logic of sharding and selection, including the world_size-2 gather on gloo."""

import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from qsrt_b200 import selection
from qsrt_b200.selection import PooledCandidateScore


def test_pooled_selection_tie_breaks():
    """Tie-break order of the reference (tests/test_pooled_selection.py): bytes, transfers, name."""

    a = PooledCandidateScore("r0", 10.0, 1e3, 64, 0, 0)
    b = PooledCandidateScore("r1", 10.0 + 1e-9, 1e3, 32, 1, 0)
    c = PooledCandidateScore("r2", 11.0, 1e3, 0, 0, 0)
    picked = selection.select_pooled_candidate([a, b, c])
    assert picked.selected.name == "r1" and picked.tied_names == ("r0", "r1")
    assert selection.select_pooled_candidate([a, b, c], tie_relative_to_source_energy=0.0).selected.name == "r0"
    same = [PooledCandidateScore("z", 1.0, 5.0, 8, 1, 1), PooledCandidateScore("y", 1.0, 5.0, 8, 2, 0),
            PooledCandidateScore("x", 1.0, 5.0, 8, 1, 1)]
    assert selection.select_pooled_candidate(same).selected.name == "x"
    with pytest.raises(ValueError):
        selection.select_pooled_candidate([])
    with pytest.raises(ValueError):
        selection.select_pooled_candidate([a, PooledCandidateScore("r0", 1.0, 1e3, 0)])
    with pytest.raises(ValueError):
        selection.select_pooled_candidate([a, PooledCandidateScore("q", 1.0, 2e3, 0)])
    with pytest.raises(ValueError):
        selection.select_pooled_candidate([PooledCandidateScore("n", -1.0, 1.0, 0)])


def test_assign_experts_is_balanced_and_deterministic():
    g = torch.Generator().manual_seed(0)
    rows = (1.0 / torch.arange(1, 385) ** 1.1 * 65536 * 8 / 4.6).long().tolist()
    shards = selection.assign_experts(rows, 8)
    assert sorted(e for s in shards for e in s) == list(range(384))
    assert all(len(s) == 48 for s in shards)
    loads = [sum(rows[e] + 4096 for e in s) for s in shards]
    assert max(loads) / min(loads) < 1.3  # the single hottest expert alone outweighs the rest
    assert shards == selection.assign_experts(rows, 8)
    assert selection.assign_experts([5, 5, 5], 2) == [[0, 2], [1]]
    with pytest.raises(ValueError):
        selection.assign_experts(rows, 0)


def test_equal_byte_exchange_keeps_bytes_and_never_raises_error():
    g = torch.Generator().manual_seed(3)
    experts = 48
    base = torch.rand(experts, generator=g).double() + 0.5
    sse = torch.stack([base * 4.0, base, base * 0.25 * (1 + torch.rand(experts, generator=g).double())], dim=1)
    sse[5, 0] = sse[5, 1] * 1.01          # an expert that barely notices K2
    sse[7, 2] = sse[7, 1] * 0.01          # an expert that gains a lot from K4
    size = torch.tensor([2.0, 3.0, 4.0]).double().expand(experts, 3) * 1000
    table = torch.stack([sse, size], dim=2)
    result = selection.equal_byte_exchange(table)
    assert result.total_bytes == 3000.0 * experts
    assert result.total_sse <= result.baseline_sse
    assert result.bits.count(2) == result.bits.count(4) == result.exchanges
    assert result.bits[5] == 2 and result.bits[7] == 4
    upgraded = selection.equal_byte_exchange(table, free_upgrades=4)
    assert upgraded.bits.count(4) - upgraded.bits.count(2) == 4
    with pytest.raises(ValueError):
        bad = table.clone()
        bad[0, 0, 0] = float("nan")
        selection.equal_byte_exchange(bad)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gather_worker(rank: int, world: int, port: int, out_dir: str) -> None:
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rows = [100, 5, 40, 7, 60]
    shards = selection.assign_experts(rows, world)
    mine = shards[rank]
    local = torch.zeros((len(mine), 3, 2), dtype=torch.float64)
    for i, e in enumerate(mine):
        local[i, :, 0] = torch.tensor([4.0, 1.0, 0.25]) * (e + 1)
        local[i, :, 1] = torch.tensor([2.0, 3.0, 4.0])
    table = selection.gather_candidate_table(local, mine, len(rows))
    allocation = selection.equal_byte_exchange(table)
    torch.save({"table": table, "bits": allocation.bits, "shard": mine}, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.destroy_process_group()


def test_two_rank_gather_gives_identical_selection_on_every_rank(tmp_path):
    port = _free_port()
    mp.spawn(_gather_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0 = torch.load(tmp_path / "rank0.pt")
    r1 = torch.load(tmp_path / "rank1.pt")
    assert torch.equal(r0["table"], r1["table"]) and bool(torch.isfinite(r0["table"]).all())
    assert r0["bits"] == r1["bits"]
    assert sorted(r0["shard"] + r1["shard"]) == [0, 1, 2, 3, 4]
    for e in range(5):
        assert r0["table"][e, 1, 0].item() == float(e + 1)


def test_single_process_gather_needs_no_process_group():
    local = torch.ones((2, 3, 2), dtype=torch.float64)
    full = selection.gather_candidate_table(local, [1, 3], 4)
    assert bool(torch.isnan(full[0]).all()) and bool((full[1] == 1).all()) and bool((full[3] == 1).all())


# ---- phase-1 selection with the bootstrap gate, coupled-mode selection -----------------------------

def _selection_golden():
    import json
    from pathlib import Path

    return json.loads((Path(__file__).parent / "golden" / "selection_golden.json").read_text())


def test_phase1_selection_matches_reference_decisions_and_intervals():
    """Decisions, reasons and bootstrap intervals equal the reference's own
    (tests/golden/selection_golden.json, made by tests/golden/make_selection_golden.py)."""

    from dataclasses import asdict

    from tests.helpers import COUPLED_MODE_CASE, phase1_case

    gold = _selection_golden()

    def same(got: dict, want: dict) -> None:
        got = dict(got)
        got["confirmation_ci95"] = list(got["confirmation_ci95"])
        assert got == want

    for trial in range(8):
        case = phase1_case(trial)
        pair = selection.select_phase1_rate_pair(
            case["fit"], case["confirmation"], fit_counts=case["fit_counts"],
            confirmation_counts=case["confirmation_counts"], modes=case["pairs"],
            bootstrap_replicates=case["replicates"], seed=trial)
        same(asdict(pair), gold["pair"][trial])
        fit = {m: case["fit"][(m, 0)] for m in (0, 1, 2)}
        confirmation = {m: case["confirmation"][(m, 0)] for m in (0, 1, 2)}
        mode = selection.select_phase1_mode(
            fit, confirmation, fit_counts=case["fit_counts"], confirmation_counts=case["confirmation_counts"],
            bootstrap_replicates=case["replicates"], seed=trial)
        same(asdict(mode), gold["mode"][trial])
    assert selection.select_coupled_modes(*COUPLED_MODE_CASE) == gold["coupled"]


def test_phase1_rate_pair_gate_and_support_rules():
    """The scenarios of the reference's tests/test_qsrt_candidates.py:500-612."""

    pairs = tuple((a, b) for a in (0, 1, 2) for b in (0, 1, 2))
    ones = torch.ones(8, dtype=torch.int64)
    fit = {p: torch.full((8,), 10.0 + p[0] + p[1]) for p in pairs}       # the fit fold prefers R0/R0 ...
    confirmation = {p: torch.full((8,), 10.0) for p in pairs}
    confirmation[(2, 1)] = torch.full((8,), 7.0)                         # ... the confirmation fold does not
    chosen = selection.select_phase1_rate_pair(fit, confirmation, fit_counts=ones, confirmation_counts=ones,
                                               modes=pairs, bootstrap_replicates=200, seed=7)
    assert chosen.proposed == (2, 1) and chosen.selected == (2, 1) and chosen.accepted
    assert chosen.confirmation_ci95[0] > 0

    two = ((0, 0), (0, 1))
    flat = {p: torch.ones(6) for p in two}
    weak = selection.select_phase1_rate_pair(flat, flat, fit_counts=torch.ones(6, dtype=torch.int64),
                                             confirmation_counts=torch.ones(3, dtype=torch.int64), modes=two,
                                             min_fit_documents=4, min_confirmation_documents=4,
                                             bootstrap_replicates=200)
    assert weak.selected == (0, 0) and weak.reason == "insufficient confirmation-document support"

    fit_m = {0: torch.full((8,), 10.0), 1: torch.full((8,), 10.5), 2: torch.full((8,), 8.0)}
    conf_m = {0: torch.full((6,), 10.0), 1: torch.full((6,), 10.5), 2: torch.full((6,), 8.0)}
    kwargs = dict(fit_counts=ones, confirmation_counts=torch.ones(6, dtype=torch.int64), mode_ids=(0, 1, 2),
                  bootstrap_replicates=200, seed=7)
    assert selection.select_phase1_mode(fit_m, conf_m, **kwargs).selected_r == 2
    conf_m[2] = torch.full((6,), 12.0)
    rejected = selection.select_phase1_mode(fit_m, conf_m, **kwargs)
    assert rejected.proposed_r == 2 and rejected.selected_r == 0 and not rejected.accepted
    few = selection.select_phase1_mode({m: torch.ones(5) for m in (0, 1)}, {m: torch.ones(5) for m in (0, 1)},
                                       fit_counts=torch.ones(5, dtype=torch.int64),
                                       confirmation_counts=torch.ones(5, dtype=torch.int64), mode_ids=(0, 1),
                                       bootstrap_replicates=200)
    assert few.selected_r == 0 and few.reason == "insufficient fit-document support"

    with pytest.raises(ValueError, match="begin with R0/R0"):
        selection.select_phase1_rate_pair(flat, flat, fit_counts=ones[:6], confirmation_counts=ones[:6],
                                          modes=((0, 1), (0, 0)))
    with pytest.raises(ValueError, match="at least 100"):
        selection.bootstrap_improvement(torch.ones(4), torch.ones(4), torch.ones(4, dtype=torch.bool),
                                        replicates=10, seed=0)
    assert selection.bootstrap_improvement(torch.zeros(4), torch.ones(4), torch.ones(4, dtype=torch.bool),
                                           replicates=100, seed=0) == (None, (None, None), 0)


def test_coupled_mode_selection_rules():
    sse = {"w1": {0: 3.0, 1: 2.0}, "w3": {0: 3.0, 1: 2.5}, "w2": {0: 1.0, 1: 1.0}}
    picked = selection.select_coupled_modes(sse, {"r13": ("w1", "w3"), "r2": ("w2",)})
    assert picked["r13"]["selected_mode"] == 1 and picked["r2"]["selected_mode"] == 0   # tie -> lower mode
    assert picked["r13"]["sse_by_mode"] == {"R0": 6.0, "R1": 4.5}
    with pytest.raises(ValueError, match="partition"):
        selection.select_coupled_modes(sse, {"r13": ("w1", "w3")})
    with pytest.raises(ValueError, match="share one mode ladder"):
        selection.select_coupled_modes({"w1": {0: 1.0}, "w3": {0: 1.0, 1: 2.0}}, {"r13": ("w1", "w3")})
    with pytest.raises(KeyError):
        selection.select_coupled_modes(sse, {"r13": ("w1", "w9"), "r2": ("w2",)})
    with pytest.raises(ValueError, match="finite and nonnegative"):
        selection.select_coupled_modes({"w2": {0: -1.0}}, {"r2": ("w2",)})
