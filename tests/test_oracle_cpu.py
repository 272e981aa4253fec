"""CPU tests: the oracle against the reference's golden vectors and GPU-generated fixtures."""

import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import qsrt_oracle as oracle
from qsrt_b200 import tables
from tests import helpers

GOLDEN = Path(__file__).resolve().parent / "golden"

# SHA-256 pins held by the reference's tests (tests/test_sqg_e4m3.py:30-38).
SQG_XOR_CHEB_T12_SHA256 = {
    "t12": "cca11fe5744c9c93a34f4217f342fbc0f74ecc8a007c076582424a505fc9da5e",
    1: "12d404e5a107582a8b4e38f80ac51117e8519c65e8b18f59f463aa1f8442c5ee",
    2: "62027916386245a84c86156a0a08b6cf07e41548871af0e56fb40780558f6293",
    3: "afe7b3633e7d243b00b379b18ec4dca573722b3727cafef47fcb6470d7e7e6c9",
    4: "5a9620f0c4d8f0a60d0b6fbea921dcecbd193e6febf31043aaa6403c20389c2f",
    5: "a1caf5572c67d4face423478f423e1ed6149a8c920be5c28d4702946c93cae2f",
    6: "8e0edc92e20eb92f5287dbdadc8e870fc500fc03c5eed996cae0781d197ebcb0",
}


def _sha(array) -> str:
    return hashlib.sha256(np.ascontiguousarray(array).tobytes()).hexdigest()


def test_t12_staircase_matches_reference_hash():
    assert _sha(oracle.sqg_xor_cheb_t12_rank_lut_bytes()) == SQG_XOR_CHEB_T12_SHA256["t12"]
    assert _sha(tables.sqg_xor_cheb_t12_rank_lut_bytes().numpy()) == SQG_XOR_CHEB_T12_SHA256["t12"]


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6])
def test_state_tables_match_reference_hashes(bits):
    assert _sha(oracle.sqg_xor_cheb_t12_bytes(bits)) == SQG_XOR_CHEB_T12_SHA256[bits]
    assert _sha(tables.sqg_xor_cheb_t12_bytes(bits).numpy()) == SQG_XOR_CHEB_T12_SHA256[bits]
    ranks = oracle.sqg_xor_rank_permutation(bits)
    assert np.array_equal(np.sort(ranks), np.arange(1 << 16))
    assert np.array_equal(ranks, tables.sqg_xor_rank_permutation(bits).numpy())


@pytest.mark.parametrize(
    ("bits", "expected_prefix"),
    [
        (2, [6939] * 6),
        (3, [30469, 1337, 1337, 14711, 14711, 30469]),
        (4, [17767, 291, -12817, -30293, 17767, 291]),
    ],
)
def test_packer_word_order_matches_reference_prefix(bits, expected_prefix):
    """Golden words of tests/test_qsrt.py:242-259."""

    indices = (np.arange(256) % (1 << bits)).astype(np.int16)[None]
    packed = oracle.pack_trellis_edges(indices, bits)
    assert packed.shape == (1, 16 * bits)
    assert packed[0, : len(expected_prefix)].tolist() == expected_prefix
    assert np.array_equal(oracle.unpack_trellis_edges(packed, bits), indices)


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_cyclic_states_match_scalar_recurrence(bits):
    """tests/test_qsrt.py:281-298."""

    rng = np.random.default_rng(175 + bits)
    edges = rng.integers(0, 1 << bits, (3, 5, 256))
    state = np.zeros(edges.shape[:-1], dtype=np.int64)
    lags = (16 + bits - 1) // bits
    for i in range(256 - lags, 256):
        state = ((state << bits) | edges[..., i]) & 0xFFFF
    expected = []
    for i in range(256):
        state = ((state << bits) | edges[..., i]) & 0xFFFF
        expected.append(state)
    expected = np.stack(expected, axis=-1).astype(np.uint16).view(np.int16)
    got = oracle.reconstruct_trellis_states(edges, bits)
    assert np.array_equal(got, expected)
    packed = oracle.pack_trellis_edges(got, bits)
    assert np.array_equal(oracle.unpack_trellis_states(packed, bits), got)


def test_half_rounding_matches_numpy():
    rng = np.random.default_rng(1)
    lib = oracle._lib()
    values = np.concatenate(
        [rng.standard_normal(2000) * 10.0 ** rng.integers(-9, 6, 2000), [0.0, 65504.0, 65519.9, 65520.0, 2.0 ** -25, 2.0 ** -25 * 1.0000001, 2.0 ** -24]]
    )
    for v in values:
        expect = np.float64(v).astype(np.float16).view(np.uint16)
        assert lib.qsrt_oracle_d2h(float(v)) == int(expect), v
    for bits in range(0, 65536, 97):
        d = lib.qsrt_oracle_h2d(bits)
        ref = np.array([bits], dtype=np.uint16).view(np.float16)[0]
        assert (np.isnan(d) and np.isnan(ref)) or d == float(ref)
    ref8 = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    mine = oracle.e4m3_to_float(np.arange(256, dtype=np.uint8))
    assert np.array_equal(np.nan_to_num(mine, nan=-1), np.nan_to_num(ref8.astype(np.float64), nan=-1))


@pytest.mark.parametrize("bits,context", [(2, 1), (2, 32), (3, 1), (3, 32), (4, 1), (4, 32)])
def test_cpu_restatement_reproduces_reference_kernel_states(bits, context):
    """States emitted by the unmodified reference CUDA kernel on a B200 (fixture made by
    tests/golden/make_viterbi_golden.py); the inputs are regenerated from the stored seed."""

    golden = np.load(GOLDEN / "viterbi_golden.npz")
    tiles = helpers.mixed_tiles(int(golden["per_family"]), int(golden["seed"])).numpy()
    expected = golden[f"states_k{bits}_c{context}"]
    pick = np.r_[0:3, 8:10, 16:18, 24:26, 32:37]  # some of each family + all structural rows
    _, states = oracle.quantize_tiles(tiles[pick], oracle.sqg_xor_cheb_t12_bytes(bits), bits, context)
    assert np.array_equal(states, expected[pick])
    assert oracle.states_close(states, bits)


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_cpu_restatement_full_context_rows(bits):
    golden = np.load(GOLDEN / "viterbi_golden.npz")
    tiles = helpers.mixed_tiles(int(golden["per_family"]), int(golden["seed"])).numpy()
    pick = np.r_[1, 9, 17, 25, 32, 33, 35]
    _, states = oracle.quantize_tiles(tiles[pick], oracle.sqg_xor_cheb_t12_bytes(bits), bits, 128)
    assert np.array_equal(states, golden[f"states_k{bits}_c128"][pick])


# ---- Hessian constructors: float64 restatement vs matrices the reference produced ------------------
def _rel_fro(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))


@pytest.mark.parametrize("name,kwargs", [("default", {}), ("blend", {"h13_alpha": 0.25}),
                                         ("fixed", {"h13_alpha": 0.25, "h2_alpha": 0.4})])
def test_hessian_oracle_matches_reference_made_golden(name, kwargs):
    from oracle import hessian_oracle

    golden = np.load(Path(__file__).parent / "golden" / "hessian_golden.npz")
    inputs, gates, middle, global_h13, _, _ = helpers.expert_hessian_inputs()
    h13, h2, evidence = hessian_oracle.build_expert_hessians(
        inputs.numpy(), gates.numpy(), middle.numpy(), global_h13.numpy(), **kwargs)
    if name != "default":
        assert _rel_fro(h13, golden["blend_h13"]) < 1e-5
    assert _rel_fro(h2, golden[f"{name}_h2"]) < 1e-5
    for key, value in evidence.items():
        want = float(golden[f"{name}_{key}"])
        assert abs(value - want) <= 2e-6 * max(1.0, abs(want)), key


def test_routed_hessian_oracle_matches_reference_made_golden():
    from oracle import hessian_oracle

    golden = np.load(Path(__file__).parent / "golden" / "hessian_golden.npz")
    inputs, _, _, _, _, route_weights = helpers.expert_hessian_inputs()
    hessian, stats = hessian_oracle.routed_input_hessian(inputs.numpy(), route_weights.numpy(), 0.10)
    assert _rel_fro(hessian, golden["routed_010_hessian"]) < 1e-5
    for key, value in stats.items():
        want = float(golden[f"routed_010_{key}"])
        assert abs(value - want) <= 2e-6 * abs(want), key
    full, _ = hessian_oracle.routed_input_hessian(inputs.numpy(), route_weights.numpy(), 1.0)
    assert _rel_fro(np.diagonal(full), golden["routed_100_diagonal"]) < 2e-6
