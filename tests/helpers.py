"""Shared test inputs and the loader of the prebuilt reference extension."""

from __future__ import annotations

import math
from pathlib import Path

import numpy as np
import torch

from oracle import ref_kernel

ROOT = Path(__file__).resolve().parents[1]
REF_EXT = ref_kernel.REF_EXT
FAMILIES = ("normal", "scaled", "heavy", "spike")


def make_tiles(family: str, tiles: int, seed: int) -> torch.Tensor:
    """Seeded tile families with the distributions of the reference's kernel A/B harness
    (scripts/benchmark_sqg_tile_encoder.py:98-116): unit normal; normal times a cycling scale
    in {1/4 .. 4}; Student-t(3); normal with 1 % of entries multiplied by 100."""

    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn((tiles, 256), generator=g, dtype=torch.float32)
    if family == "normal":
        return x
    if family == "scaled":
        cycle = torch.tensor([0.25, 0.5, 1.0, 2.0, 4.0])
        return x * cycle[torch.arange(tiles) % 5][:, None]
    if family == "heavy":
        chi2 = torch.randn((tiles, 256, 3), generator=g).square().sum(-1)
        return x * torch.rsqrt(chi2 / 3.0).clamp(max=1e3)
    if family == "spike":
        hit = torch.rand((tiles, 256), generator=g) < 0.01
        return torch.where(hit, x * 100.0, x)
    raise ValueError(family)


def mixed_tiles(per_family: int, seed: int) -> torch.Tensor:
    """All four families plus the reference's structural rows (tests/test_sqg_quantizer.py:
    176-179: a row x100, a zero row, a row x-40) and two saturated rows of 1000.0."""

    parts = [make_tiles(f, per_family, seed + i) for i, f in enumerate(FAMILIES)]
    extra = make_tiles("normal", 5, seed + 99)
    extra[0] *= 100.0
    extra[1] = 0.0
    extra[2] *= -40.0
    extra[3] = 1000.0
    extra[4] = -1000.0
    return torch.cat(parts + [extra]).contiguous()


def reference_extension():
    """The UNMODIFIED reference CUDA extension built by oracle/build_ref.py, or None."""

    return ref_kernel.reference_extension()


_reference_searches: dict = {}


def reference_quantize_tiles(tiles: torch.Tensor, lut_state: torch.Tensor, bits: int, context: int):
    """Drive the reference kernel exactly as qsrt/sqg_quantizer.py:607-651 does."""

    key = (str(tiles.device), bits, context, lut_state.data_ptr())
    if key not in _reference_searches:
        _reference_searches[key] = (lut_state, ref_kernel.ReferenceTileSearch(lut_state, bits, context, tiles.device))
    out, idx = _reference_searches[key][1](tiles)
    torch.cuda.synchronize(tiles.device)
    return out, idx


def coupled_inputs(hidden: int = 512, inter: int = 128, rows: int = 48, seed: int = 77):
    """Seeded expert triplet, routed rows and Hessians for the coupled-coordinate fixtures."""

    g = torch.Generator(device="cpu").manual_seed(seed)
    w1 = torch.randn((inter, hidden), generator=g) * 0.02
    w3 = torch.randn((inter, hidden), generator=g) * 0.02
    w2 = torch.randn((hidden, inter), generator=g) * 0.02
    x = torch.randn((rows, hidden), generator=g)
    h13 = (x.T @ x / rows).float()
    m = torch.randn((rows, inter), generator=g)
    h2 = (m.T @ m / rows).float()
    return w1, w3, w2, x, h13, h2


# ---- mixed-rate record container / atom storage cases (Kimi-K3 geometry, the only one the
# reference container accepts) ----------------------------------------------------------------
RECORD_CASES = tuple((mode, axis) for mode in ("R0", "R1", "R2", "H308", "K2") for axis in ("k", "n"))
EXPERT_CASE = (9, 77, 1, 2)  # layer, expert, r13 (w1/w3 mode), r2 (w2 mode)
_MODE_IDS = {"R0": 0, "R1": 1, "R2": 2, "H308": 3, "K2": 4}


def record_shape(axis: str) -> tuple[int, int, int]:
    return (192, 224, 256) if axis == "k" else (224, 192, 256)


def record_case_seed(mode: str, axis: str) -> int:
    return 200 + 10 * _MODE_IDS[mode] + (axis == "n")


def expert_case_inputs():
    """Seeded numpy states, local (3072) and shared (3584) float16 scales of one expert."""

    import numpy as np

    from oracle.records_oracle import legal_states

    _, _, r13, r2 = EXPERT_CASE
    bits_of = {0: (3,) * 24, 1: (2, 4) + (3,) * 22, 2: (2, 4, 2, 4) + (3,) * 20}
    rng = np.random.default_rng(4242)
    states, local, shared = {}, {}, {}
    for index, matrix in enumerate(("w1", "w3", "w2")):
        axis = "k" if matrix == "w2" else "n"
        bits = bits_of[r2 if matrix == "w2" else r13]
        states[matrix] = legal_states(record_shape(axis), bits, axis, 900 + index)
        local[matrix] = (rng.standard_normal(3072) * 0.1).astype(np.float16)
        shared[matrix] = (rng.standard_normal(3584) * 0.1).astype(np.float16)
    return states, local, shared


# ---- phase-1 selection cases (seeded per-document SSE tables) ------------------------------------
COUPLED_MODE_CASE = (
    {"w1": {0: 3.0, 1: 2.0, 2: 2.5}, "w3": {0: 3.0, 1: 2.6, 2: 2.0}, "w2": {0: 1.0, 1: 1.0, 2: 4.0}},
    {"r13": ("w1", "w3"), "r2": ("w2",)},
)


def phase1_case(trial: int) -> dict:
    """Per-document SSE of the nine ``(r13, r2)`` candidates on a fit and a confirmation fold."""

    g = torch.Generator().manual_seed(6000 + trial)
    documents = 8 + 2 * trial
    pairs = tuple((a, b) for a in (0, 1, 2) for b in (0, 1, 2))
    fit = {p: torch.rand(documents, generator=g) * 10 + 5 for p in pairs}
    spread = 10.0 if trial % 3 == 0 else 8.5   # every third case gives the transfers no edge
    confirmation = {p: torch.rand(documents, generator=g) * (10.0 if p == (0, 0) else spread) + 5 for p in pairs}
    fit_counts = (torch.rand(documents, generator=g) > 0.1).long()
    confirmation_counts = (torch.rand(documents, generator=g) > (0.7 if trial == 5 else 0.2)).long()
    return {"pairs": pairs, "fit": fit, "confirmation": confirmation, "fit_counts": fit_counts,
            "confirmation_counts": confirmation_counts, "replicates": 300 + 100 * trial}


# ---- tile error surfaces / high-rate allocation cases ---------------------------------------------
def allocation_inputs(seed: int = 515, k: int = 256, n: int = 384):
    """Seeded regularised reference / reconstruction, dense covariance and scale vectors (CPU)."""

    g = torch.Generator().manual_seed(seed)
    reference = torch.randn((k, n), generator=g)
    reconstruction = reference + 0.05 * torch.randn((k, n), generator=g)
    x = torch.randn((4 * k, k), generator=g) * torch.exp(0.5 * torch.randn(k, generator=g))
    hessian = (x.T @ x / (4 * k)).float()
    suh = (torch.rand(k, generator=g) + 0.5) * torch.sign(torch.randn(k, generator=g))
    svh = (torch.rand(n, generator=g) + 0.5) * torch.sign(torch.randn(n, generator=g))
    return reference, reconstruction, hessian, suh, svh


def allocation_cost_surfaces(axis: str, seed: int = 99):
    """Two K2/K3/K4 cost surfaces on the Kimi-K3 tile grid (float64, CPU)."""

    g = torch.Generator().manual_seed(seed + (axis == "n"))
    grid = (192, 224) if axis == "k" else (224, 192)
    gain = {2: 1.3, 3: 1.0, 4: 0.8}
    return [{b: torch.rand(grid, generator=g, dtype=torch.float64) * gain[b] for b in (2, 3, 4)} for _ in range(2)]


# ---- per-expert Hessian construction cases --------------------------------------------------------
def expert_hessian_inputs(seed: int = 2718, tokens: int = 640, hidden: int = 256, middle: int = 128):
    """Seeded routed inputs, gates, post-activation rows and global covariances (CPU float32)."""

    g = torch.Generator().manual_seed(seed)
    scale = torch.exp(0.4 * torch.randn(hidden, generator=g))
    inputs = torch.randn((tokens, hidden), generator=g) * scale
    gates = torch.rand(tokens, generator=g) * 0.6 + 0.02
    gates[::17] = 0.0
    source_middle = torch.randn((tokens, middle), generator=g) * torch.exp(0.3 * torch.randn(middle, generator=g))
    base = torch.randn((4 * hidden, hidden), generator=g) * scale
    global_h13 = (base.T @ base / (4 * hidden)).float()
    global_h2 = torch.eye(middle)
    route_weights = gates.clone()
    route_weights[5::29] = -0.3   # negative route weights are clamped to zero
    return inputs, gates, source_middle, global_h13, global_h2, route_weights


# ---- dense-H path refinement cases ----------------------------------------------------------------
def spd_hessian(size: int, condition: float, seed: int) -> torch.Tensor:
    """Seeded SPD matrix with log-spaced spectrum, unit mean diagonal (float32, CPU)."""

    g = torch.Generator().manual_seed(seed)
    basis, _ = torch.linalg.qr(torch.randn((size, size), generator=g, dtype=torch.float64))
    half = 0.5 * math.log(condition)
    spectrum = torch.exp(torch.linspace(-half, half, size, dtype=torch.float64))
    h = (basis * spectrum) @ basis.T + 0.025 * torch.eye(size, dtype=torch.float64)
    return (h / h.diagonal().mean()).float()


REFINE_CASES = {
    # name: (bits, rows, columns, condition, sweeps, column weights?, guidance strength, fp64 score?)
    "k3_plain": (3, 64, 96, 30.0, 2, False, 0.0, False),
    "k2_weighted_guided_fp64": (2, 48, 64, 12.0, 2, True, 0.5, True),
}


def refine_case_inputs(name: str):
    """Seeded weight, Hessian, column weights and guidance tensors of one refinement case (CPU)."""

    bits, rows, columns, condition, sweeps, weighted, strength, fp64 = REFINE_CASES[name]
    seed = 1000 + 17 * bits + rows
    g = torch.Generator().manual_seed(seed)
    weight = 1.2 * torch.randn((rows, columns), generator=g)
    hessian = spd_hessian(rows, condition, seed + 1)
    column_weights = (0.5 + torch.rand(columns, generator=g)) if weighted else None
    gradient = 0.05 * torch.randn((rows, columns), generator=g) if strength else None
    return weight, hessian, column_weights, gradient


def matrix_to_tc_tiles(matrix: torch.Tensor, order: torch.Tensor) -> torch.Tensor:
    rows, columns = matrix.shape
    return matrix.reshape(rows // 16, 16, columns // 16, 16).permute(0, 2, 1, 3).reshape(-1, 256)[:, order]


def tc_tiles_to_matrix(tiles: torch.Tensor, inverse: torch.Tensor, rows: int, columns: int) -> torch.Tensor:
    return tiles[:, inverse].reshape(rows // 16, columns // 16, 16, 16).permute(0, 2, 1, 3).reshape(rows, columns)


# ---- quantize_qsrt cases pinned by the reference's own encoder code ---------------------------------
ENCODER_CASES = {
    # name: (bits, in, out, g_scale_override, apply_out_scales, sigma_reg)
    "k3_override": (3, 256, 128, 0.9, False, 1e-2),
    "k2_override_auto_scales": (2, 256, 128, 1.15, None, 0.025),
    "k4_override_out_scales": (4, 128, 256, 0.8, True, 0.025),
    "k2_scale_search": (2, 128, 128, None, False, 1e-2),
    "k3_no_hessian_fallback": (3, 128, 128, 0.9, True, 1e-2),
    "k3_refine_sweep": (3, 128, 128, 0.9, False, 1e-2),
    "k3_1024_tiles_scale_search": (3, 512, 512, None, None, 0.025),
}
# extra quant_args and the sample count of the capture (0 = no Hessian: the fallback path)
ENCODER_EXTRA_ARGS = {"k3_refine_sweep": {"h2_viterbi_refine_sweeps": 1}}
ENCODER_CAPTURE_COUNT = {"k3_no_hessian_fallback": 0}


def encoder_case_inputs(name: str):
    """Seeded weight [in, out] and capture Hessian of one encoder case (CPU float32)."""

    bits, k, n, _, _, _ = ENCODER_CASES[name]
    g = torch.Generator().manual_seed(4000 + 13 * bits + k + n)
    x = torch.randn((4 * k, k), generator=g) * torch.exp(0.5 * torch.randn(k, generator=g))
    hessian = (x.T @ x / x.shape[0]).float()
    weight = 0.02 * torch.randn((k, n), generator=g) * torch.exp(0.3 * torch.randn(n, generator=g))
    return weight, hessian


def encoder_case_args(name: str, device: str, table: torch.Tensor) -> dict:
    bits, _, _, override, out_scales, sigma = ENCODER_CASES[name]
    args = {"K": bits, "seed": 11, "sv_seed": 12, "sigma_reg": sigma, "devices": [device], "device_ratios": None,
            "apply_out_scales": out_scales, "ldlq_tf32": False, "tailbite_context": 128, "sqg_e4m3_lut": table}
    if override is not None:
        args["g_scale_override"] = override
    args.update(ENCODER_EXTRA_ARGS.get(name, {}))
    return args


# ---- quantize_qsrt_batch cases (candidate grids) pinned the same way -------------------------------
BATCH_SHAPE = (256, 256)
BATCH_CASES = {
    # name: (rate axis, rate maps per source; the first map is the all-K3 base)
    "n_axis_reuse": ("n", ([3] * 16, [2] * 4 + [3] * 8 + [4] * 4, [2] * 8 + [4] * 8)),
    "k_axis_prefix": ("k", ([3] * 16, [2] * 4 + [4] * 4 + [3] * 8, [3] * 4 + [4] * 4 + [3] * 8)),
}


def batch_case_inputs(name: str, sources: int = 2):
    """Seeded weights [in, out] and capture Hessians of one candidate-grid case (CPU float32)."""

    k, n = BATCH_SHAPE
    out = []
    for index in range(sources):
        g = torch.Generator().manual_seed(7000 + 31 * index + (name == "k_axis_prefix"))
        x = torch.randn((4 * k, k), generator=g) * torch.exp(0.5 * torch.randn(k, generator=g))
        out.append((0.02 * torch.randn((k, n), generator=g), (x.T @ x / x.shape[0]).float()))
    return out


def batch_case_args(name: str, device: str, tables_by_bits: dict) -> list[dict]:
    axis, maps = BATCH_CASES[name]
    return [{"K": 3, "seed": 11, "sv_seed": 12, "sigma_reg": 0.025, "devices": [device], "device_ratios": None,
             "apply_out_scales": False, "ldlq_tf32": False, "tailbite_context": 128, "buf_size_k": 128,
             "g_scale_override": 0.95, "sqg_e4m3_luts_by_bits": tables_by_bits, "mixed_rate_axis": axis,
             "mixed_tile_bits": tuple(m)} for m in maps]


def tile_digests(states) -> np.ndarray:
    """64-bit digest of every tile's 256 states ([..., 256] int16 -> [...] uint64)."""

    import hashlib

    flat = np.ascontiguousarray(np.asarray(states).reshape(-1, 256).astype(np.int16))
    return np.array([int.from_bytes(hashlib.blake2b(row.tobytes(), digest_size=8).digest(), "little") for row in flat],
                    dtype=np.uint64)


# ---- teacher-forced replay of the reference's BlockLDLQ recursion on the device ---------------------
def teacher_forced_replay(weight_r: torch.Tensor, factor: torch.Tensor, forced_weight_q: torch.Tensor, *,
                          tile_search, order: torch.Tensor, buf_size_k: int = 128):
    """Walk the reverse block recursion of ``ldlq`` (qsrt/exl3_encoder_backend.py:470-539) with the
    reference's own call shapes - ``addmm_`` of the in-span factor slice per 16-row block, one
    ``addmm_`` of the whole span afterwards - but with the history taken from ``forced_weight_q``
    (the regularised-domain reconstruction somebody else produced), so that a differing tile does
    not compound.  ``tile_search(tiles [n, 256] in tensor-core order) -> states [n, 256] int16``.
    Returns ``(states [k/16, n/16, 256] int16, targets [k, n] float32)``: what the reference's
    loop would have encoded at every step, and the encoder inputs it would have seen."""

    size_k, size_n = weight_r.shape
    tiles_n = size_n // 16
    device = weight_r.device
    prod_cache = torch.zeros((size_k, size_n), dtype=torch.float32, device=device)
    states = torch.zeros((size_k // 16, tiles_n, 256), dtype=torch.int16, device=device)
    targets = torch.empty_like(weight_r)
    allow = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        for j in range(size_k, 0, -buf_size_k):
            i = j - buf_size_k
            b_weight, b_weight_q = weight_r[i:j], forced_weight_q[i:j]
            b_factor = factor[i:j]
            for bj in range(buf_size_k, 0, -16):
                bi = bj - 16
                compensation = prod_cache[i + bi:i + bj]
                compensation.addmm_(b_factor[bj:, i + bi:i + bj].T, b_weight[bj:] - b_weight_q[bj:])
                rows = b_weight[bi:bj] + compensation
                targets[i + bi:i + bj] = rows
                tiles = rows.reshape(16, tiles_n, 16).permute(1, 0, 2).reshape(tiles_n, 256)[:, order].contiguous()
                states[(i + bi) // 16] = tile_search(tiles)
            prod_cache.addmm_(b_factor.T, b_weight - b_weight_q)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = allow
    return states, targets


# ---- routed-error scoring cases -------------------------------------------------------------------
SCORING_REQUESTS = {3: "doc-a", 7: "doc-b", 8: "doc-c"}


def scoring_inputs(seed: int = 1618, rows: int = 96, hidden: int = 512, inter: int = 256):
    """Seeded expert triplet, a perturbed candidate triplet, routed rows, gates and request epochs
    (CPU float32).  Hidden 512 and intermediate 256 admit the coupled 512 / 128 / 128 blocks."""

    g = torch.Generator().manual_seed(seed)
    source = (torch.randn((inter, hidden), generator=g) * 0.05, torch.randn((inter, hidden), generator=g) * 0.05,
              torch.randn((hidden, inter), generator=g) * 0.05)
    candidates = {}
    for name, noise in (("fine", 0.002), ("coarse", 0.01)):
        candidates[name] = tuple(w + noise * torch.randn(w.shape, generator=g) for w in source)
    x = torch.randn((rows, hidden), generator=g) * torch.exp(0.3 * torch.randn(hidden, generator=g))
    gates = torch.rand(rows, generator=g) * 0.5 + 0.05
    steps = torch.tensor([sorted(SCORING_REQUESTS)[i % 3] for i in range(rows)], dtype=torch.int64)
    return source, candidates, x, gates, steps


# ---- capture -> Hessian streaming reducer case ------------------------------------------------------
CAPTURE_CASE = {
    "layers": 4, "input_size": 128, "selected": [1, 3],
    "runs": {
        "train_epochs_2_to_9": dict(sample_split="train", request_step_min=2, request_step_max=9, request_steps=None),
        "all_listed_epochs": dict(sample_split="all", request_step_min=0, request_step_max=None, request_steps=[1, 4, 11]),
    },
}


def capture_parts(seed: int = 2024, parts: int = 3, rows: int = 160):
    """Seeded sample parts of a small capture: per part layer ids, split labels, observation ids
    (request epoch in the high 32 bits), gate-square weights and bf16 input rows (CPU tensors)."""

    g = torch.Generator().manual_seed(seed)
    out = []
    for part in range(parts):
        layer = torch.randint(0, CAPTURE_CASE["layers"], (rows,), generator=g, dtype=torch.int32)
        split = (torch.rand(rows, generator=g) < 0.25).to(torch.int8)
        epoch = torch.randint(0, 13, (rows,), generator=g, dtype=torch.int64)
        observation = (epoch << 32) | (torch.arange(rows, dtype=torch.int64) + part * rows)
        weight = torch.rand(rows, generator=g) ** 2
        values = (torch.randn((rows, CAPTURE_CASE["input_size"]), generator=g)
                  * torch.exp(0.4 * torch.randn(CAPTURE_CASE["input_size"], generator=g))).to(torch.bfloat16)
        out.append({"layer": layer, "split": split, "observation": observation, "weight": weight, "values": values})
    return out
