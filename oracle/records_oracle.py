"""CPU restatement (numpy) of the mixed-rate record container and the atom-major storage
image.  TEST INFRASTRUCTURE ONLY: nothing in the product imports this file.

Follows qsrt/qsrt.py:1042-1172 (`_record_tiles`, `pack_qsrt_trellis`,
`unpack_qsrt_trellis_edges`, `unpack_qsrt_trellis_states`) and qsrt/qsrt_storage.py:194-231,
292-315, 347-362, 441-462 (`pack_matrix_atoms`, `pack_local_scale_atoms`, `rotate_expert_atoms`,
`QSRTLayerLayout.atom_bundle_offset`).

Pinned: tests/golden/records_golden.json holds SHA-256 digests of the reference's own outputs
(generator: tests/golden/make_records_golden.py, which imports qsrt.qsrt and
qsrt.qsrt_storage) for seeded inputs that the tests regenerate.
"""

from __future__ import annotations

import numpy as np

from .qsrt_oracle import pack_trellis_edges, reconstruct_trellis_states, unpack_trellis_edges

STRIPES = 8  # tile rows (columns) per 128-channel record


def legal_states(shape: tuple[int, int, int], record_bits, rate_axis: str, seed: int) -> np.ndarray:
    """Seeded closed cyclic paths: random K-bit edges per record, states from the recurrence."""

    rng = np.random.default_rng(seed)
    states = np.empty(shape, dtype=np.int16)
    for record, bits in enumerate(record_bits):
        begin = record * STRIPES
        if rate_axis == "k":
            edges = rng.integers(0, 1 << bits, size=(STRIPES, shape[1], 256)).astype(np.int16)
            states[begin : begin + STRIPES] = reconstruct_trellis_states(edges, bits)
        else:
            edges = rng.integers(0, 1 << bits, size=(shape[0], STRIPES, 256)).astype(np.int16)
            states[:, begin : begin + STRIPES] = reconstruct_trellis_states(edges, bits)
    return states


def _record_tiles(states: np.ndarray, record: int, rate_axis: str) -> np.ndarray:
    begin = record * STRIPES
    part = states[begin : begin + STRIPES] if rate_axis == "k" else states[:, begin : begin + STRIPES]
    return np.ascontiguousarray(part).reshape(-1, 256)


def pack_records(states: np.ndarray, record_bits, rate_axis: str) -> np.ndarray:
    """qsrt/qsrt.py:1051-1082: per-record packed tiles, concatenated."""

    pieces = [
        pack_trellis_edges(_record_tiles(states, record, rate_axis), bits).reshape(-1)
        for record, bits in enumerate(record_bits)
    ]
    return np.concatenate(pieces).astype(np.int16)


def unpack_records(payload: np.ndarray, shape: tuple[int, int, int], record_bits, rate_axis: str,
                   want_states: bool) -> np.ndarray:
    """qsrt/qsrt.py:1085-1172."""

    out = np.empty(shape, dtype=np.int16)
    orth = shape[1] if rate_axis == "k" else shape[0]
    cursor = 0
    for record, bits in enumerate(record_bits):
        count = STRIPES * orth * 16 * bits
        edges = unpack_trellis_edges(payload[cursor : cursor + count].reshape(STRIPES * orth, 16 * bits), bits)
        tiles = reconstruct_trellis_states(edges, bits) if want_states else edges
        begin = record * STRIPES
        if rate_axis == "k":
            out[begin : begin + STRIPES] = tiles.reshape(STRIPES, orth, 256)
        else:
            out[:, begin : begin + STRIPES] = tiles.reshape(orth, STRIPES, 256)
        cursor += count
    assert cursor == payload.size
    return out


def matrix_atoms(payload: np.ndarray, record_bits, rate_axis: str, orth: int) -> np.ndarray:
    """qsrt/qsrt_storage.py:194-231: ``[pairs * 8, words]`` logical atoms from the payload."""

    offsets = np.concatenate([[0], np.cumsum([STRIPES * orth * 16 * b for b in record_bits])])
    pairs = len(record_bits) // 2
    atoms = []
    for pair in range(pairs):
        for stripe in range(STRIPES):
            pieces = []
            for record in (2 * pair, 2 * pair + 1):
                bits = record_bits[record]
                source = payload[offsets[record] : offsets[record + 1]]
                if rate_axis == "k":
                    source = source.reshape(STRIPES, orth, 16 * bits)[stripe]
                else:
                    source = source.reshape(orth, STRIPES, 16 * bits)[:, stripe]
                pieces.append(np.ascontiguousarray(source).reshape(-1))
            atoms.append(np.concatenate(pieces))
    return np.stack(atoms).astype(np.int16)


def scale_atoms(scale: np.ndarray) -> np.ndarray:
    """qsrt/qsrt_storage.py:292-315 for a float16 vector of pairs*256 values."""

    pairs = scale.size // 256
    out = np.empty((pairs * STRIPES, 32), dtype=scale.dtype)
    for pair in range(pairs):
        for stripe in range(STRIPES):
            for side, record in enumerate((2 * pair, 2 * pair + 1)):
                begin = record * 128 + stripe * 16
                out[pair * STRIPES + stripe, side * 16 : side * 16 + 16] = scale[begin : begin + 16]
    return out


def rotate_atoms(atoms: np.ndarray, rotation: int) -> np.ndarray:
    """qsrt/qsrt_storage.py:347-362: slot s holds logical atom (s - rotation) mod n."""

    n = atoms.shape[0]
    return atoms[(np.arange(n) - rotation) % n]


def expert_slab(slab: np.ndarray, pitch: int, bundle_bytes: int, compressed_slot: int, rotation: int,
                matrix_atoms_by_name: dict[str, np.ndarray], scale_atoms_by_name: dict[str, np.ndarray]) -> None:
    """Write one expert's bundles into ``slab`` (uint8 ``[slots, pitch]``): w1, w3, w2 trellis atoms
    then their scale atoms, per qsrt/qsrt_storage.py:61-75,441-462."""

    cursor = compressed_slot * bundle_bytes
    for group in (matrix_atoms_by_name, scale_atoms_by_name):
        for name in ("w1", "w3", "w2"):
            raw = rotate_atoms(group[name], rotation).view(np.uint8).reshape(slab.shape[0], -1)
            slab[:, cursor : cursor + raw.shape[1]] = raw
            cursor += raw.shape[1]
    assert cursor == (compressed_slot + 1) * bundle_bytes
