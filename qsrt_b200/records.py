"""Mixed-rate record container for one complete expert matrix (device resident).

Mirrors the reference's candidate payload with the same names, argument meaning and error
behaviour (``qsrt/qsrt.py``): rate-transfer modes ``R0/R1/R2``, the fixed ``H308`` profile and
uniform ``K2`` (``:144-255``), ``record_bits`` / ``pair_bits`` / ``pair_kinds`` (``:516-561``),
``repack_encoded_records`` (``:824-853``), ``QSRTTrellisDescriptor`` / ``PackedQSRTTrellis``
(``:916-1027``), ``pack_qsrt_trellis`` / ``unpack_qsrt_trellis_edges`` /
``unpack_qsrt_trellis_states`` (``:1051-1172``).

The reference loops over the 24 records in Python and packs each with int64 bit twiddling;
here one kernel (``qsrtb_pack_records``) reads the states once and writes the whole payload,
checking that every tile is a closed cyclic path in the same pass.  As in the reference the
container accepts the Kimi-K3 geometry only (3072-channel rate axis, 3584-channel orthogonal
axis); the kernel itself takes any record description.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Literal, Sequence

import torch

from . import _lib
from .tiles import _stream_ptr

INTERMEDIATE_CHANNELS = 3072
LATENT_CHANNELS = 3584
TILE_CHANNELS = 16
TILE_VALUES = TILE_CHANNELS * TILE_CHANNELS
RECORD_CHANNELS = 128
PAIR_CHANNELS = 2 * RECORD_CHANNELS
RECORDS_PER_EXPERT = INTERMEDIATE_CHANNELS // RECORD_CHANNELS
PAIRS_PER_EXPERT = RECORDS_PER_EXPERT // 2
TILES_PER_RECORD_AXIS = RECORD_CHANNELS // TILE_CHANNELS
SCHEMA = "qsrt_kimi_k3_qsrt_candidate_v1"
LOGICAL_CANDIDATE_SCHEMAS = (SCHEMA,)
FIXED_HIGH_RATE_RECORD_BITS = (3,) * 22 + (4,) * 2
FIXED_HIGH_RATE_TRELLIS_BYTES = (
    INTERMEDIATE_CHANNELS * LATENT_CHANNELS * sum(FIXED_HIGH_RATE_RECORD_BITS) // (RECORDS_PER_EXPERT * 8)
)
RateAxis = Literal["k", "n"]
MATRIX_RATE_AXIS: dict[str, str] = {"w1": "n", "w3": "n", "w2": "k"}


@dataclass(frozen=True)
class ModeSpec:
    """One rate schedule, contexts ordered from low to high importance (qsrt/qsrt.py:144-201)."""

    mode_id: int
    name: str
    context_bits: tuple[int, ...]

    def __post_init__(self) -> None:
        if isinstance(self.mode_id, bool) or not isinstance(self.mode_id, int):
            raise TypeError("mode_id must be an integer")
        if not 0 <= self.mode_id <= 4:
            raise ValueError("QSRT mode_id must identify R0, R1, R2, H308, or K2")
        if not self.name:
            raise ValueError("mode name must not be empty")
        uniform_k2 = self.mode_id == 4
        fixed_high = self.mode_id == 3
        bits = self.context_bits
        if not bits or (len(bits) % 2 and not uniform_k2):
            raise ValueError("a mode must contain an even, nonzero context count")
        if any(b not in (2, 3, 4) for b in bits):
            raise ValueError("Kimi-K3 QSRT supports only K2, K3, and K4")
        if fixed_high:
            if self.name != "H308" or bits != FIXED_HIGH_RATE_RECORD_BITS:
                raise ValueError("H308 must contain exactly 22 K3 and 2 K4 records")
        elif uniform_k2:
            if self.name != "K2" or bits != (2,):
                raise ValueError("K2 must contain one uniform two-bit context")
        elif sum(bits) != 3 * len(bits):
            raise ValueError("a rate-transfer mode must average exactly three bits")
        if INTERMEDIATE_CHANNELS % len(bits):
            raise ValueError("contexts must divide the 3072-channel axis")
        if (INTERMEDIATE_CHANNELS // len(bits)) % RECORD_CHANNELS:
            raise ValueError("each context must contain whole 128-channel records")
        if tuple(sorted(bits)) != bits:
            raise ValueError("context rates must be monotone from K2 through K4")
        if fixed_high or uniform_k2:
            return
        per_context = RECORDS_PER_EXPERT // len(bits)
        donors = bits.count(2) * per_context
        if donors != bits.count(4) * per_context:
            raise ValueError("K2 and K4 record counts must match")
        if self.mode_id != donors:
            raise ValueError(f"mode_id must equal the rate-transfer count {donors}")

    @property
    def context_count(self) -> int:
        return len(self.context_bits)

    @property
    def records_per_context(self) -> int:
        return RECORDS_PER_EXPERT // self.context_count


RATE_TRANSFER_MODES = tuple(
    ModeSpec(r, f"R{r}", (2,) * r + (3,) * (RECORDS_PER_EXPERT - 2 * r) + (4,) * r) for r in range(3)
)
R0, R1, R2 = RATE_TRANSFER_MODES
H308 = ModeSpec(3, "H308", FIXED_HIGH_RATE_RECORD_BITS)
K2 = ModeSpec(4, "K2", (2,))
_ALL_MODES = (*RATE_TRANSFER_MODES, H308, K2)
_MODES_BY_NAME = {m.name: m for m in _ALL_MODES}
_MODES_BY_ID = {m.mode_id: m for m in _ALL_MODES}


def resolve_mode(mode: ModeSpec | str | int) -> ModeSpec:
    if isinstance(mode, ModeSpec):
        return mode
    if isinstance(mode, str):
        try:
            return _MODES_BY_NAME[mode.upper()]
        except KeyError as exc:
            raise ValueError(f"unknown QSRT mode: {mode}") from exc
    if isinstance(mode, int) and not isinstance(mode, bool):
        try:
            return _MODES_BY_ID[mode]
        except KeyError as exc:
            raise ValueError(f"unknown QSRT mode ID: {mode}") from exc
    raise TypeError("mode must be a ModeSpec, name, or integer ID")


def mode_from_context_bits(context_bits: Sequence[int]) -> ModeSpec:
    """Canonical mode of a record-rate allocation (qsrt/qsrt.py:239-253)."""

    bits = tuple(context_bits)
    if bits == FIXED_HIGH_RATE_RECORD_BITS:
        return H308
    if bits == (2,):
        return K2
    if not bits or RECORDS_PER_EXPERT % len(bits):
        raise ValueError("allocation contexts must divide the 24 records")
    r = bits.count(2) * (RECORDS_PER_EXPERT // len(bits))
    ModeSpec(r, "candidate", bits)  # validates monotonicity, rate and donor balance
    return RATE_TRANSFER_MODES[r]


def matrix_rate_axis(matrix: str) -> str:
    try:
        return MATRIX_RATE_AXIS[matrix]
    except KeyError as exc:
        raise ValueError(f"unknown expert matrix: {matrix}") from exc


def record_contexts(mode: ModeSpec | str | int) -> tuple[int, ...]:
    """Context of each stored record, low/high contexts interleaved (qsrt/qsrt.py:516-531)."""

    spec = resolve_mode(mode)
    if spec.mode_id == H308.mode_id:
        return tuple(range(RECORDS_PER_EXPERT))
    if spec.mode_id == K2.mode_id:
        return (0,) * RECORDS_PER_EXPERT
    out: list[int] = []
    for low in range(spec.context_count // 2):
        high = spec.context_count - 1 - low
        out.extend((low, high) * spec.records_per_context)
    if len(out) != RECORDS_PER_EXPERT:
        raise AssertionError("mode construction did not cover 24 records")
    return tuple(out)


def record_bits(mode: ModeSpec | str | int) -> tuple[int, ...]:
    spec = resolve_mode(mode)
    return tuple(spec.context_bits[c] for c in record_contexts(spec))


def pair_bits(mode: ModeSpec | str | int) -> tuple[tuple[int, int], ...]:
    bits = record_bits(mode)
    pairs = tuple(zip(bits[0::2], bits[1::2]))
    want = 4 if resolve_mode(mode).mode_id == K2.mode_id else 6
    if len(pairs) != PAIRS_PER_EXPERT or any(sum(p) != want for p in pairs):
        raise ValueError("QSRT record pairs do not match the mode rate sum")
    return pairs


def pair_kinds(mode: ModeSpec | str | int) -> tuple[str, ...]:
    names = {(2, 2): "P22", (2, 4): "P24", (3, 3): "P33"}
    kinds = []
    for pair in pair_bits(mode):
        if pair not in names:
            raise ValueError(f"unsupported QSRT pair schedule: {pair}")
        kinds.append(names[pair])
    return tuple(kinds)


def _validate_permutation(order: torch.Tensor, size: int, name: str) -> None:
    if order.ndim != 1 or order.numel() != size:
        raise ValueError(f"{name} must contain exactly {size} entries")
    if order.dtype == torch.bool or order.is_floating_point():
        raise TypeError(f"{name} must use an integer dtype")
    if sorted(order.cpu().tolist()) != list(range(size)):
        raise ValueError(f"{name} must be a permutation of 0..{size - 1}")


def _validate_encoded_shape(encoded: torch.Tensor, rate_axis: str) -> None:
    if encoded.ndim != 3 or encoded.shape[-1] != TILE_VALUES:
        raise ValueError("encoded states must have shape [K/16, N/16, 256]")
    if encoded.dtype == torch.bool or encoded.is_floating_point():
        raise TypeError("encoded states must use an integer dtype")
    if rate_axis not in ("k", "n"):
        raise ValueError("rate_axis must be 'k' or 'n'")
    rate_tiles = encoded.shape[0] if rate_axis == "k" else encoded.shape[1]
    if rate_tiles * TILE_CHANNELS != INTERMEDIATE_CHANNELS:
        raise ValueError("encoded rate axis must contain exactly 3072 channels")


def repack_encoded_records(encoded: torch.Tensor, record_order: torch.Tensor, rate_axis: str) -> torch.Tensor:
    """Reorder whole 128-channel records of ``[K/16, N/16, 256]`` states (qsrt/qsrt.py:824-853).

    ``record_order[d]`` is the source record that lands in destination record ``d``.
    """

    _validate_encoded_shape(encoded, rate_axis)
    _validate_permutation(record_order, RECORDS_PER_EXPERT, "record_order")
    order = record_order.to(device=encoded.device, dtype=torch.long)
    tiles = (order[:, None] * TILES_PER_RECORD_AXIS + torch.arange(TILES_PER_RECORD_AXIS, device=encoded.device)).flatten()
    return encoded.index_select(0 if rate_axis == "k" else 1, tiles).contiguous()


@dataclass(frozen=True)
class QSRTTrellisDescriptor:
    """Description of one packed expert matrix, free of tensor-parallel geometry (qsrt/qsrt.py:916-1012)."""

    mode_id: int
    rate_axis: str
    k_tiles: int
    n_tiles: int
    schema: str = SCHEMA
    intermediate_channels: int = INTERMEDIATE_CHANNELS
    record_channels: int = RECORD_CHANNELS

    def __post_init__(self) -> None:
        if self.schema not in LOGICAL_CANDIDATE_SCHEMAS:
            raise ValueError(f"unsupported QSRT schema: {self.schema}")
        if self.intermediate_channels != INTERMEDIATE_CHANNELS:
            raise ValueError("Kimi-K3 QSRT requires a 3072-channel intermediate axis")
        if self.record_channels != RECORD_CHANNELS:
            raise ValueError("Kimi-K3 QSRT requires 128-channel records")
        resolve_mode(self.mode_id)
        if self.rate_axis not in ("k", "n"):
            raise ValueError("rate_axis must be 'k' or 'n'")
        if self.k_tiles <= 0 or self.n_tiles <= 0:
            raise ValueError("tile dimensions must be positive")
        rate_tiles = self.k_tiles if self.rate_axis == "k" else self.n_tiles
        if rate_tiles * TILE_CHANNELS != INTERMEDIATE_CHANNELS:
            raise ValueError("rate axis must contain exactly 3072 channels")
        if self.orthogonal_tiles * TILE_CHANNELS != LATENT_CHANNELS:
            raise ValueError("orthogonal axis must contain exactly 3584 channels")

    @property
    def mode(self) -> ModeSpec:
        return resolve_mode(self.mode_id)

    @property
    def orthogonal_tiles(self) -> int:
        return self.n_tiles if self.rate_axis == "k" else self.k_tiles

    @property
    def tiles_per_record(self) -> int:
        return TILES_PER_RECORD_AXIS * self.orthogonal_tiles

    @property
    def words_per_pair(self) -> int:
        if self.mode.mode_id == H308.mode_id:
            raise ValueError("H308 has no fixed six-bit record-pair contract")
        return self.tiles_per_record * TILE_CHANNELS * sum(pair_bits(self.mode)[0])

    @property
    def words_per_record(self) -> tuple[int, ...]:
        unit = self.tiles_per_record * TILE_CHANNELS
        return tuple(unit * b for b in record_bits(self.mode))

    @property
    def payload_words(self) -> int:
        return sum(self.words_per_record)

    @property
    def payload_bytes(self) -> int:
        return 2 * self.payload_words

    @property
    def weight_count(self) -> int:
        return self.k_tiles * self.n_tiles * TILE_VALUES

    def to_manifest(self) -> dict[str, object]:
        fixed_pairs = self.mode.mode_id != H308.mode_id
        return {
            "schema": self.schema,
            "mode_id": self.mode_id,
            "mode": self.mode.name,
            "rate_axis": self.rate_axis,
            "k_tiles": self.k_tiles,
            "n_tiles": self.n_tiles,
            "intermediate_channels": self.intermediate_channels,
            "record_channels": self.record_channels,
            "pair_channels": PAIR_CHANNELS,
            "record_bits": list(record_bits(self.mode)),
            "pair_kinds": list(pair_kinds(self.mode)) if fixed_pairs else None,
            "words_per_pair": self.words_per_pair if fixed_pairs else None,
            "words_per_record": list(self.words_per_record),
            "payload_words": self.payload_words,
            "payload_bytes": self.payload_bytes,
        }


@dataclass(frozen=True)
class PackedQSRTTrellis:
    descriptor: QSRTTrellisDescriptor
    payload: torch.Tensor

    def validate(self) -> None:
        if self.payload.dtype != torch.int16:
            raise TypeError("QSRT trellis payload must use torch.int16")
        if self.payload.ndim != 1:
            raise ValueError("QSRT trellis payload must be one-dimensional")
        if self.payload.numel() != self.descriptor.payload_words:
            raise ValueError("QSRT trellis payload length does not match its descriptor")


def _bits_array(bits: Sequence[int]):
    import ctypes

    return (ctypes.c_uint8 * len(bits))(*bits)


def pack_qsrt_trellis(
    encoded: torch.Tensor,
    mode: ModeSpec | str | int,
    *,
    rate_axis: str,
    schema: str = SCHEMA,
    validate_states: bool = True,
) -> PackedQSRTTrellis:
    """Pack a complete matrix into its per-record payload (qsrt/qsrt.py:1051-1082)."""

    _validate_encoded_shape(encoded, rate_axis)
    spec = resolve_mode(mode)
    descriptor = QSRTTrellisDescriptor(
        mode_id=spec.mode_id, rate_axis=rate_axis, k_tiles=encoded.shape[0], n_tiles=encoded.shape[1], schema=schema
    )
    if not encoded.is_cuda:
        raise ValueError("encoded states must be on a CUDA device (there is no CPU path)")
    states = encoded.to(torch.int16).contiguous()
    payload = torch.empty(descriptor.payload_words, dtype=torch.int16, device=states.device)
    open_paths = torch.zeros(1, dtype=torch.int32, device=states.device) if validate_states else None
    bits = record_bits(spec)
    with torch.cuda.device(states.device):
        _lib.check(
            _lib.lib().qsrtb_pack_records(
                states.data_ptr(), descriptor.k_tiles, descriptor.n_tiles, 0 if rate_axis == "k" else 1,
                len(bits), TILES_PER_RECORD_AXIS, _bits_array(bits), 0, 0, 0, payload.data_ptr(),
                descriptor.payload_bytes, open_paths.data_ptr() if open_paths is not None else None,
                _stream_ptr(states.device),
            ),
            "qsrtb_pack_records",
        )
    if open_paths is not None and int(open_paths.item()) != 0:
        raise ValueError("encoded input is not a closed cyclic trellis path")
    packed = PackedQSRTTrellis(descriptor, payload)
    packed.validate()
    return packed


def _unpack(packed: PackedQSRTTrellis, want_states: bool) -> torch.Tensor:
    packed.validate()
    d = packed.descriptor
    payload = packed.payload
    if not payload.is_cuda:
        raise ValueError("payload must be on a CUDA device (there is no CPU path)")
    payload = payload.contiguous()
    out = torch.empty((d.k_tiles, d.n_tiles, TILE_VALUES), dtype=torch.int16, device=payload.device)
    bits = record_bits(d.mode)
    with torch.cuda.device(payload.device):
        _lib.check(
            _lib.lib().qsrtb_unpack_records(
                payload.data_ptr(), d.payload_bytes, d.k_tiles, d.n_tiles, 0 if d.rate_axis == "k" else 1,
                len(bits), TILES_PER_RECORD_AXIS, _bits_array(bits), 0, 0, 0,
                out.data_ptr() if want_states else None, None if want_states else out.data_ptr(),
                _stream_ptr(payload.device),
            ),
            "qsrtb_unpack_records",
        )
    return out


def unpack_qsrt_trellis_edges(packed: PackedQSRTTrellis) -> torch.Tensor:
    """Payload -> stored K-bit edge symbols in ``[K/16, N/16, 256]`` (qsrt/qsrt.py:1085-1118)."""

    return _unpack(packed, want_states=False)


def unpack_qsrt_trellis_states(packed: PackedQSRTTrellis) -> torch.Tensor:
    """Payload -> cyclic 16-bit states in ``[K/16, N/16, 256]`` (qsrt/qsrt.py:1121-1172)."""

    return _unpack(packed, want_states=True)
