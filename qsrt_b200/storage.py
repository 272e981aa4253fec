"""Atom-major storage image of a compressed MoE layer (device resident).

Mirrors the reference's storage geometry with the same names and argument meaning
(``qsrt/qsrt_storage.py``): a 32-channel atom holds matching 16-channel stripes of the low and
high record of one record pair (always six trellis bits per coefficient pair), plus the local
scale fragments of w1, w3 and w2; an expert's 96 atoms are rotated by whole record pairs and
stored in 96 slot rows shared by all compressed experts of the layer.

* atom arithmetic: ``balanced_atom_partition``, ``logical_atom_index``, ``atom_components``,
  ``atom_record_indices``, ``atom_rates``, ``physical_atom_rotation``, ``physical_atom_slot``,
  ``logical_atom_for_slot`` (``:92-174``);
* ``pack_matrix_atoms`` / ``unpack_matrix_atoms`` (``:194-289``): here one kernel
  (``qsrtb_records_atoms``) moving whole packed tile paths, where the reference runs
  96 x 2 slice copies in Python;
* ``pack_local_scale_atoms`` / ``unpack_local_scale_atoms`` (``:292-344``),
  ``rotate_expert_atoms`` / ``unrotate_expert_atoms`` (``:347-381``);
* ``QSRTShardExtent``, ``QSRTLayerLayout``, ``QSRTLayerHeader`` (``:384-632``);
* ``write_expert_atoms`` / ``read_expert_atoms`` (no reference counterpart as one call): trellis
  states of the three matrices -> their bundles inside the layer image in one pass per matrix
  (``qsrtb_pack_records`` with the atom layout), skipping the record payload, the logical atom
  tensor and the rotated copy the reference materialises on the way.
"""

from __future__ import annotations

import json
import struct
from dataclasses import dataclass

import torch

from . import _lib
from .records import (
    INTERMEDIATE_CHANNELS,
    LATENT_CHANNELS,
    PAIRS_PER_EXPERT,
    RECORDS_PER_EXPERT,
    TILE_CHANNELS,
    TILE_VALUES,
    TILES_PER_RECORD_AXIS,
    ModeSpec,
    PackedQSRTTrellis,
    QSRTTrellisDescriptor,
    _bits_array,
    matrix_rate_axis,
    pair_bits,
    record_bits,
    resolve_mode,
)
from .tiles import _stream_ptr

EXPERTS_PER_LAYER = 896
STORAGE_ALIGNMENT = 4096
PAIR_ROTATION_EXPERT_MULTIPLIER = 5
SCALE_BYTES = 2
LOCAL_SCALE_VECTORS = 3
LAYER_HEADER_BYTES = STORAGE_ALIGNMENT
FORMAT_SECTION_BYTES = STORAGE_ALIGNMENT
SHARED_SCALE_SECTION_BYTES = 6 * STORAGE_ALIGNMENT
PAIR_BYTES = 256 * LATENT_CHANNELS * 3 // 8
MATRIX_TRELLIS_BYTES = PAIRS_PER_EXPERT * PAIR_BYTES
EXPERT_TRELLIS_BYTES = 3 * MATRIX_TRELLIS_BYTES

SCHEMA = "qsrt_kimi_k3_qsrt_atoms_v1"
VERSION = 1
ENCODING_QSRT_SQG_E4M3 = "qsrt_sqg_e4m3"
PROFILE_ID_QSRT_SQG_E4M3 = 1
_HEADER_LENGTH = struct.Struct("<Q")
_FORMAT_TENSOR_NAME = "_qsrt_format_section"
_SHARED_SCALE_TENSOR_NAME = "_qsrt_shared_scale_section"
_ATOM_TENSOR_NAME = "qsrt_atoms"

ATOM_SIDE_CHANNELS = TILE_CHANNELS
ATOM_CHANNELS = 2 * ATOM_SIDE_CHANNELS
ATOMS_PER_RECORD_PAIR = 128 // ATOM_SIDE_CHANNELS
ATOMS_PER_EXPERT = PAIRS_PER_EXPERT * ATOMS_PER_RECORD_PAIR
K2_STRIPE_BYTES = ATOM_SIDE_CHANNELS * LATENT_CHANNELS * 2 // 8
K3_STRIPE_BYTES = ATOM_SIDE_CHANNELS * LATENT_CHANNELS * 3 // 8
K4_STRIPE_BYTES = ATOM_SIDE_CHANNELS * LATENT_CHANNELS * 4 // 8
MATRIX_ATOM_TRELLIS_BYTES = ATOM_CHANNELS * LATENT_CHANNELS * 3 // 8
MATRIX_ATOM_SCALE_BYTES = ATOM_CHANNELS * SCALE_BYTES
ATOM_TRELLIS_BYTES = 3 * MATRIX_ATOM_TRELLIS_BYTES
ATOM_SCALE_BYTES = LOCAL_SCALE_VECTORS * MATRIX_ATOM_SCALE_BYTES
ATOM_BUNDLE_BYTES = ATOM_TRELLIS_BYTES + ATOM_SCALE_BYTES
MATRIX_ORDER = ("w1", "w3", "w2")
MATRIX_ATOM_TRELLIS_OFFSETS = {m: i * MATRIX_ATOM_TRELLIS_BYTES for i, m in enumerate(MATRIX_ORDER)}
MATRIX_ATOM_SCALE_OFFSETS = {m: ATOM_TRELLIS_BYTES + i * MATRIX_ATOM_SCALE_BYTES for i, m in enumerate(MATRIX_ORDER)}
ATOM_SLAB_OFFSET = LAYER_HEADER_BYTES + FORMAT_SECTION_BYTES + SHARED_SCALE_SECTION_BYTES
EQUAL_SHARD_COUNTS = tuple(n for n in range(1, ATOMS_PER_EXPERT + 1) if ATOMS_PER_EXPERT % n == 0)


def align_up(value: int, alignment: int = STORAGE_ALIGNMENT) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value < 0:
        raise ValueError("value must be a non-negative integer")
    if isinstance(alignment, bool) or not isinstance(alignment, int) or alignment <= 0 or alignment & (alignment - 1):
        raise ValueError("alignment must be a positive power of two")
    return (value + alignment - 1) & -alignment


def _index(value: int, upper: int, name: str) -> None:
    if isinstance(value, bool) or not isinstance(value, int):
        raise TypeError(f"{name} must be an integer")
    if not 0 <= value < upper:
        raise ValueError(f"{name} must be in 0..{upper - 1}")


def pair_rotation(layer: int, expert: int) -> int:
    """Cyclic logical-pair placement that balances P24 work (qsrt/qsrt.py:101-116)."""

    if isinstance(layer, bool) or not isinstance(layer, int) or layer not in range(1, 93):
        raise ValueError("K3 MoE layer must be in 1..92")
    if isinstance(expert, bool) or not isinstance(expert, int) or not 0 <= expert < EXPERTS_PER_LAYER:
        raise ValueError(f"expert must be in 0..{EXPERTS_PER_LAYER - 1}")
    return (PAIR_ROTATION_EXPERT_MULTIPLIER * expert + layer) % PAIRS_PER_EXPERT


def balanced_atom_partition(shard_count: int, shard_index: int) -> tuple[int, int]:
    """``(first_atom, atom_count)`` of a whole-atom partition (qsrt/qsrt_storage.py:92-112)."""

    if isinstance(shard_count, bool) or not isinstance(shard_count, int):
        raise TypeError("shard_count must be an integer")
    if not 1 <= shard_count <= ATOMS_PER_EXPERT:
        raise ValueError(f"shard_count must be in 1..{ATOMS_PER_EXPERT}")
    _index(shard_index, shard_count, "shard_index")
    quotient, remainder = divmod(ATOMS_PER_EXPERT, shard_count)
    return shard_index * quotient + min(shard_index, remainder), quotient + int(shard_index < remainder)


def logical_atom_index(record_pair: int, stripe: int) -> int:
    _index(record_pair, PAIRS_PER_EXPERT, "record_pair")
    _index(stripe, ATOMS_PER_RECORD_PAIR, "stripe")
    return record_pair * ATOMS_PER_RECORD_PAIR + stripe


def atom_components(logical_atom: int) -> tuple[int, int]:
    _index(logical_atom, ATOMS_PER_EXPERT, "logical_atom")
    return divmod(logical_atom, ATOMS_PER_RECORD_PAIR)


def atom_record_indices(logical_atom: int) -> tuple[int, int]:
    pair, _ = atom_components(logical_atom)
    return 2 * pair, 2 * pair + 1


def atom_rates(mode: ModeSpec | str | int, logical_atom: int) -> tuple[int, int]:
    pair, _ = atom_components(logical_atom)
    return (2, 4) if pair < resolve_mode(mode).mode_id else (3, 3)


def physical_atom_rotation(layer: int, expert: int) -> int:
    return ATOMS_PER_RECORD_PAIR * pair_rotation(layer, expert)


def physical_atom_slot(layer: int, expert: int, logical_atom: int) -> int:
    atom_components(logical_atom)
    return (logical_atom + physical_atom_rotation(layer, expert)) % ATOMS_PER_EXPERT


def logical_atom_for_slot(layer: int, expert: int, physical_slot: int) -> int:
    _index(physical_slot, ATOMS_PER_EXPERT, "physical_slot")
    return (physical_slot - physical_atom_rotation(layer, expert)) % ATOMS_PER_EXPERT


def _require_six_bit_pairs(mode: ModeSpec) -> tuple[int, ...]:
    bits = record_bits(mode)
    if any(bits[2 * p] + bits[2 * p + 1] != 6 for p in range(PAIRS_PER_EXPERT)):
        raise AssertionError("balanced atom did not contain six rate bits")
    return bits


def _records_atoms(records: torch.Tensor, atoms: torch.Tensor, descriptor: QSRTTrellisDescriptor,
                   bits: tuple[int, ...], to_records: bool) -> None:
    with torch.cuda.device(records.device):
        _lib.check(
            _lib.lib().qsrtb_records_atoms(
                records.data_ptr(), records.numel() * 2, descriptor.k_tiles, descriptor.n_tiles,
                0 if descriptor.rate_axis == "k" else 1, len(bits), TILES_PER_RECORD_AXIS, _bits_array(bits), 0,
                MATRIX_ATOM_TRELLIS_BYTES, atoms.data_ptr(), atoms.numel() * 2, int(to_records),
                _stream_ptr(records.device),
            ),
            "qsrtb_records_atoms",
        )


def pack_matrix_atoms(packed: PackedQSRTTrellis) -> torch.Tensor:
    """Record payload -> ``[96, 21504]`` int16 logical atoms, bits untouched (qsrt/qsrt_storage.py:194-231)."""

    packed.validate()
    bits = _require_six_bit_pairs(packed.descriptor.mode)
    payload = packed.payload
    if not payload.is_cuda:
        raise ValueError("payload must be on a CUDA device (there is no CPU path)")
    payload = payload.contiguous()
    atoms = torch.empty((ATOMS_PER_EXPERT, MATRIX_ATOM_TRELLIS_BYTES // 2), dtype=torch.int16, device=payload.device)
    _records_atoms(payload, atoms, packed.descriptor, bits, to_records=False)
    return atoms


def unpack_matrix_atoms(atoms: torch.Tensor, descriptor: QSRTTrellisDescriptor) -> PackedQSRTTrellis:
    """Inverse of :func:`pack_matrix_atoms` (qsrt/qsrt_storage.py:234-289)."""

    words = MATRIX_ATOM_TRELLIS_BYTES // 2
    if atoms.dtype != torch.int16 or tuple(atoms.shape) != (ATOMS_PER_EXPERT, words) or not atoms.is_contiguous():
        raise ValueError(f"matrix atoms must be contiguous int16 [{ATOMS_PER_EXPERT}, {words}]")
    if not atoms.is_cuda:
        raise ValueError("atoms must be on a CUDA device (there is no CPU path)")
    bits = _require_six_bit_pairs(descriptor.mode)
    payload = torch.empty(descriptor.payload_words, dtype=torch.int16, device=atoms.device)
    _records_atoms(payload, atoms, descriptor, bits, to_records=True)
    packed = PackedQSRTTrellis(descriptor, payload)
    packed.validate()
    return packed


def pack_local_scale_atoms(scale: torch.Tensor) -> torch.Tensor:
    """3072 local FP16 scales -> ``[96, 32]``: low-record stripe then high-record stripe
    (qsrt/qsrt_storage.py:292-315)."""

    if scale.dtype != torch.float16 or tuple(scale.shape) != (INTERMEDIATE_CHANNELS,) or not scale.is_contiguous():
        raise ValueError(f"local scale must be contiguous float16 [{INTERMEDIATE_CHANNELS}]")
    # [pair, side, stripe, 16] -> [pair, stripe, side, 16]
    return (
        scale.view(PAIRS_PER_EXPERT, 2, ATOMS_PER_RECORD_PAIR, ATOM_SIDE_CHANNELS)
        .permute(0, 2, 1, 3)
        .reshape(ATOMS_PER_EXPERT, ATOM_CHANNELS)
        .contiguous()
    )


def unpack_local_scale_atoms(atoms: torch.Tensor) -> torch.Tensor:
    if atoms.dtype != torch.float16 or tuple(atoms.shape) != (ATOMS_PER_EXPERT, ATOM_CHANNELS) or not atoms.is_contiguous():
        raise ValueError(f"scale atoms must be contiguous float16 [{ATOMS_PER_EXPERT}, {ATOM_CHANNELS}]")
    return (
        atoms.view(PAIRS_PER_EXPERT, ATOMS_PER_RECORD_PAIR, 2, ATOM_SIDE_CHANNELS)
        .permute(0, 2, 1, 3)
        .reshape(INTERMEDIATE_CHANNELS)
        .contiguous()
    )


def rotate_expert_atoms(logical_atoms: torch.Tensor, layer: int, expert: int) -> torch.Tensor:
    """Logical atoms -> global physical-slot order (qsrt/qsrt_storage.py:347-362)."""

    if logical_atoms.ndim < 1 or logical_atoms.shape[0] != ATOMS_PER_EXPERT:
        raise ValueError(f"logical_atoms must have leading dimension {ATOMS_PER_EXPERT}")
    return torch.roll(logical_atoms, physical_atom_rotation(layer, expert), dims=0).contiguous()


def unrotate_expert_atoms(physical_atoms: torch.Tensor, layer: int, expert: int) -> torch.Tensor:
    if physical_atoms.ndim < 1 or physical_atoms.shape[0] != ATOMS_PER_EXPERT:
        raise ValueError(f"physical_atoms must have leading dimension {ATOMS_PER_EXPERT}")
    return torch.roll(physical_atoms, -physical_atom_rotation(layer, expert), dims=0).contiguous()


@dataclass(frozen=True)
class QSRTShardExtent:
    """One shard's single contiguous read of the atom slab."""

    shard_count: int
    shard_index: int
    first_atom_slot: int
    atom_slots: int
    intermediate_channels: int
    offset_bytes: int
    extent_bytes: int
    payload_bytes: int
    padding_bytes: int


@dataclass(frozen=True)
class QSRTLayerLayout:
    """Atom-major layer layout: 96 slot rows of ``compressed_experts`` bundles, each row padded
    to 4 KiB (qsrt/qsrt_storage.py:399-519)."""

    compressed_experts: int
    x4t_experts: int

    def __post_init__(self) -> None:
        for name, value in (("compressed_experts", self.compressed_experts), ("x4t_experts", self.x4t_experts)):
            if isinstance(value, bool) or not isinstance(value, int) or value < 0:
                raise ValueError(f"{name} must be a non-negative integer")
        if self.compressed_experts + self.x4t_experts != EXPERTS_PER_LAYER:
            raise ValueError(f"a layer must account for exactly {EXPERTS_PER_LAYER} experts")

    @property
    def atom_slot_payload_bytes(self) -> int:
        return self.compressed_experts * ATOM_BUNDLE_BYTES

    @property
    def atom_slot_stride_bytes(self) -> int:
        return align_up(self.atom_slot_payload_bytes, STORAGE_ALIGNMENT)

    @property
    def atom_slot_padding_bytes(self) -> int:
        return self.atom_slot_stride_bytes - self.atom_slot_payload_bytes

    @property
    def compressed_payload_bytes(self) -> int:
        return self.compressed_experts * (
            EXPERT_TRELLIS_BYTES + LOCAL_SCALE_VECTORS * INTERMEDIATE_CHANNELS * SCALE_BYTES
        )

    @property
    def disk_bytes(self) -> int:
        return ATOM_SLAB_OFFSET + ATOMS_PER_EXPERT * self.atom_slot_stride_bytes

    def atom_bundle_offset(self, physical_slot: int, compressed_slot: int) -> int:
        """Absolute file offset of one expert's bundle in one slot row."""

        if isinstance(physical_slot, bool) or not isinstance(physical_slot, int) or not 0 <= physical_slot < ATOMS_PER_EXPERT:
            raise ValueError(f"physical_slot must be in 0..{ATOMS_PER_EXPERT - 1}")
        if (
            isinstance(compressed_slot, bool)
            or not isinstance(compressed_slot, int)
            or not 0 <= compressed_slot < self.compressed_experts
        ):
            raise ValueError(f"compressed_slot must be in 0..{self.compressed_experts - 1}")
        return ATOM_SLAB_OFFSET + physical_slot * self.atom_slot_stride_bytes + compressed_slot * ATOM_BUNDLE_BYTES

    def shard_extent(self, shard_count: int, shard_index: int, *, require_equal: bool = False) -> QSRTShardExtent:
        first, atom_slots = balanced_atom_partition(shard_count, shard_index)
        if require_equal and shard_count not in EQUAL_SHARD_COUNTS:
            raise ValueError(
                f"{shard_count} shards do not divide the QSRT atom axis; equal partitions are {EQUAL_SHARD_COUNTS}"
            )
        extent = atom_slots * self.atom_slot_stride_bytes
        payload = atom_slots * self.atom_slot_payload_bytes
        return QSRTShardExtent(
            shard_count=shard_count,
            shard_index=shard_index,
            first_atom_slot=first,
            atom_slots=atom_slots,
            intermediate_channels=atom_slots * ATOM_CHANNELS,
            offset_bytes=ATOM_SLAB_OFFSET + first * self.atom_slot_stride_bytes,
            extent_bytes=extent,
            payload_bytes=payload,
            padding_bytes=extent - payload,
        )

    def to_manifest(self) -> dict[str, int | str | list[int]]:
        return {
            "schema": SCHEMA,
            "alignment_bytes": STORAGE_ALIGNMENT,
            "compressed_experts": self.compressed_experts,
            "x4t_experts": self.x4t_experts,
            "atom_channels": ATOM_CHANNELS,
            "atom_slots": ATOMS_PER_EXPERT,
            "atom_bundle_bytes": ATOM_BUNDLE_BYTES,
            "atom_slot_payload_bytes": self.atom_slot_payload_bytes,
            "atom_slot_stride_bytes": self.atom_slot_stride_bytes,
            "atom_slot_padding_bytes": self.atom_slot_padding_bytes,
            "compressed_payload_bytes": self.compressed_payload_bytes,
            "atom_slab_offset": ATOM_SLAB_OFFSET,
            "disk_bytes": self.disk_bytes,
            "equal_shard_counts": list(EQUAL_SHARD_COUNTS),
        }


@dataclass(frozen=True)
class QSRTLayerHeader:
    """Canonical 4 KiB safetensors header of one atom-major layer (qsrt/qsrt_storage.py:523-632)."""

    layer: int
    layout: QSRTLayerLayout
    profile_id: int = PROFILE_ID_QSRT_SQG_E4M3

    def __post_init__(self) -> None:
        if isinstance(self.layer, bool) or not isinstance(self.layer, int):
            raise TypeError("layer must be an integer")
        if not 1 <= self.layer <= 92:
            raise ValueError("K3 MoE layer must be in 1..92")
        if self.profile_id != PROFILE_ID_QSRT_SQG_E4M3:
            raise ValueError("unsupported QSRT reconstruction profile")

    def _document(self) -> dict[str, object]:
        stride = self.layout.atom_slot_stride_bytes
        sections = FORMAT_SECTION_BYTES + SHARED_SCALE_SECTION_BYTES
        metadata = {
            "format": "pt",
            "schema": SCHEMA,
            "version": VERSION,
            "encoding": ENCODING_QSRT_SQG_E4M3,
            "layer": self.layer,
            "profile_id": self.profile_id,
            "experts": EXPERTS_PER_LAYER,
            "compressed_experts": self.layout.compressed_experts,
            "x4t_experts": self.layout.x4t_experts,
            "intermediate_channels": INTERMEDIATE_CHANNELS,
            "latent_channels": LATENT_CHANNELS,
            "atom_channels": ATOM_CHANNELS,
            "atom_slots": ATOMS_PER_EXPERT,
            "atom_bundle_bytes": ATOM_BUNDLE_BYTES,
            "atom_slot_payload_bytes": self.layout.atom_slot_payload_bytes,
            "atom_slot_stride_bytes": stride,
            "alignment_bytes": STORAGE_ALIGNMENT,
        }
        return {
            "__metadata__": {key: str(value) for key, value in metadata.items()},
            _FORMAT_TENSOR_NAME: {"dtype": "U8", "shape": [FORMAT_SECTION_BYTES], "data_offsets": [0, FORMAT_SECTION_BYTES]},
            _SHARED_SCALE_TENSOR_NAME: {
                "dtype": "U8",
                "shape": [SHARED_SCALE_SECTION_BYTES],
                "data_offsets": [FORMAT_SECTION_BYTES, sections],
            },
            _ATOM_TENSOR_NAME: {
                "dtype": "U8",
                "shape": [ATOMS_PER_EXPERT, stride],
                "data_offsets": [sections, sections + ATOMS_PER_EXPERT * stride],
            },
        }

    def to_bytes(self) -> bytes:
        capacity = LAYER_HEADER_BYTES - _HEADER_LENGTH.size
        document = json.dumps(self._document(), sort_keys=True, separators=(",", ":")).encode("utf-8")
        if len(document) > capacity:
            raise AssertionError("QSRT safetensors header exceeds its 4 KiB budget")
        return _HEADER_LENGTH.pack(capacity) + document + b" " * (capacity - len(document))

    @classmethod
    def from_bytes(cls, payload: bytes) -> "QSRTLayerHeader":
        if len(payload) != LAYER_HEADER_BYTES:
            raise ValueError(f"QSRT layer header must contain {LAYER_HEADER_BYTES} bytes")
        if _HEADER_LENGTH.unpack_from(payload)[0] != LAYER_HEADER_BYTES - _HEADER_LENGTH.size:
            raise ValueError("QSRT safetensors header must occupy exactly 4 KiB")
        try:
            document = json.loads(payload[_HEADER_LENGTH.size:].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise ValueError("QSRT safetensors header is invalid JSON") from exc
        if not isinstance(document, dict):
            raise ValueError("QSRT safetensors header must be a JSON object")
        metadata = document.get("__metadata__")
        if not isinstance(metadata, dict):
            raise ValueError("QSRT safetensors header omits metadata")
        try:
            result = cls(
                layer=int(metadata["layer"]),
                layout=QSRTLayerLayout(int(metadata["compressed_experts"]), int(metadata["x4t_experts"])),
                profile_id=int(metadata["profile_id"]),
            )
        except (KeyError, TypeError, ValueError) as exc:
            raise ValueError("QSRT safetensors metadata is malformed") from exc
        if document != result._document():
            raise ValueError("QSRT safetensors header is noncanonical")
        return result


def _image_view(image: torch.Tensor, layout: QSRTLayerLayout) -> None:
    if image.dtype != torch.uint8 or image.ndim != 1 or not image.is_contiguous():
        raise ValueError("layer image must be a contiguous one-dimensional uint8 tensor")
    if image.numel() != layout.disk_bytes:
        raise ValueError(f"layer image must contain exactly {layout.disk_bytes} bytes")
    if not image.is_cuda:
        raise ValueError("layer image must be on a CUDA device (there is no CPU path)")


def _matrix_geometry(matrix: str, states: torch.Tensor) -> tuple[int, int, int]:
    axis = matrix_rate_axis(matrix)
    want = (
        (INTERMEDIATE_CHANNELS // TILE_CHANNELS, LATENT_CHANNELS // TILE_CHANNELS)
        if axis == "k"
        else (LATENT_CHANNELS // TILE_CHANNELS, INTERMEDIATE_CHANNELS // TILE_CHANNELS)
    )
    if states.ndim != 3 or tuple(states.shape) != (*want, TILE_VALUES):
        raise ValueError(f"{matrix} states must have shape [{want[0]}, {want[1]}, 256]")
    return want[0], want[1], 0 if axis == "k" else 1


def write_expert_atoms(
    image: torch.Tensor,
    layout: QSRTLayerLayout,
    layer: int,
    expert: int,
    compressed_slot: int,
    states: dict[str, torch.Tensor],
    modes: dict[str, ModeSpec | str | int],
    local_scales: dict[str, torch.Tensor],
    *,
    validate_states: bool = True,
) -> None:
    """Write one expert's 96 bundles into the layer image, straight from trellis states.

    ``states[m]`` are the ``[K/16, N/16, 256]`` states of ``m`` in ("w1", "w3", "w2"),
    ``modes[m]`` a six-bit-pair schedule (R0/R1/R2), ``local_scales[m]`` the 3072 intermediate-side
    FP16 scales (w1.svh, w3.svh, w2.suh).  Equals, byte for byte, packing each matrix, cutting
    it into logical atoms, rotating them and copying every atom to
    ``layout.atom_bundle_offset(slot, compressed_slot) + MATRIX_ATOM_TRELLIS_OFFSETS[m]``.

    The closed-path check runs inside the packing pass, so a ``ValueError`` for states that are
    not closed cyclic paths is raised after the expert's bundles have been written: the contents
    of that compressed slot are then undefined and the caller must rewrite or discard the slot
    (the reference validates before it produces a payload, ``qsrt/qsrt.py:916-1024``).
    """

    _image_view(image, layout)
    _index(compressed_slot, layout.compressed_experts, "compressed_slot")
    rotation = physical_atom_rotation(layer, expert)
    pitch = layout.atom_slot_stride_bytes
    open_paths = torch.zeros(1, dtype=torch.int32, device=image.device) if validate_states else None
    base = ATOM_SLAB_OFFSET + compressed_slot * ATOM_BUNDLE_BYTES
    span = (ATOMS_PER_EXPERT - 1) * pitch + MATRIX_ATOM_TRELLIS_BYTES
    with torch.cuda.device(image.device):
        for matrix in MATRIX_ORDER:
            st = states[matrix]
            if st.dtype == torch.bool or st.is_floating_point():
                raise TypeError("encoded states must use an integer dtype")
            k_tiles, n_tiles, axis = _matrix_geometry(matrix, st)
            if st.dtype in (torch.int32, torch.int64) and st.numel():
                low, high = int(st.min()), int(st.max())
                if low < -32768 or high > 65535:
                    raise ValueError("encoded states do not fit 16 bits")
            st = st.to(device=image.device, dtype=torch.int16).contiguous()
            bits = _require_six_bit_pairs(resolve_mode(modes[matrix]))
            offset = base + MATRIX_ATOM_TRELLIS_OFFSETS[matrix]
            _lib.check(
                _lib.lib().qsrtb_pack_records(
                    st.data_ptr(), k_tiles, n_tiles, axis, len(bits), TILES_PER_RECORD_AXIS, _bits_array(bits), 1,
                    rotation, pitch, image.data_ptr() + offset, span,
                    open_paths.data_ptr() if open_paths is not None else None, _stream_ptr(image.device),
                ),
                "qsrtb_pack_records",
            )
    slab = image[ATOM_SLAB_OFFSET:].view(ATOMS_PER_EXPERT, pitch)
    for matrix in MATRIX_ORDER:
        atoms = rotate_expert_atoms(pack_local_scale_atoms(local_scales[matrix].to(image.device)), layer, expert)
        begin = compressed_slot * ATOM_BUNDLE_BYTES + MATRIX_ATOM_SCALE_OFFSETS[matrix]
        slab[:, begin : begin + MATRIX_ATOM_SCALE_BYTES].copy_(atoms.view(torch.uint8))
    if open_paths is not None and int(open_paths.item()) != 0:
        raise ValueError("encoded input is not a closed cyclic trellis path")


def read_expert_atoms(
    image: torch.Tensor,
    layout: QSRTLayerLayout,
    layer: int,
    expert: int,
    compressed_slot: int,
    modes: dict[str, ModeSpec | str | int],
) -> tuple[dict[str, torch.Tensor], dict[str, torch.Tensor]]:
    """Inverse of :func:`write_expert_atoms`: ``(states, local_scales)`` of the three matrices."""

    _image_view(image, layout)
    _index(compressed_slot, layout.compressed_experts, "compressed_slot")
    rotation = physical_atom_rotation(layer, expert)
    pitch = layout.atom_slot_stride_bytes
    base = ATOM_SLAB_OFFSET + compressed_slot * ATOM_BUNDLE_BYTES
    span = (ATOMS_PER_EXPERT - 1) * pitch + MATRIX_ATOM_TRELLIS_BYTES
    states: dict[str, torch.Tensor] = {}
    scales: dict[str, torch.Tensor] = {}
    slab = image[ATOM_SLAB_OFFSET:].view(ATOMS_PER_EXPERT, pitch)
    with torch.cuda.device(image.device):
        for matrix in MATRIX_ORDER:
            axis_name = matrix_rate_axis(matrix)
            k_tiles = (INTERMEDIATE_CHANNELS if axis_name == "k" else LATENT_CHANNELS) // TILE_CHANNELS
            n_tiles = (LATENT_CHANNELS if axis_name == "k" else INTERMEDIATE_CHANNELS) // TILE_CHANNELS
            bits = _require_six_bit_pairs(resolve_mode(modes[matrix]))
            out = torch.empty((k_tiles, n_tiles, TILE_VALUES), dtype=torch.int16, device=image.device)
            _lib.check(
                _lib.lib().qsrtb_unpack_records(
                    image.data_ptr() + base + MATRIX_ATOM_TRELLIS_OFFSETS[matrix], span, k_tiles, n_tiles,
                    0 if axis_name == "k" else 1, len(bits), TILES_PER_RECORD_AXIS, _bits_array(bits), 1, rotation,
                    pitch, out.data_ptr(), None, _stream_ptr(image.device),
                ),
                "qsrtb_unpack_records",
            )
            states[matrix] = out
            begin = compressed_slot * ATOM_BUNDLE_BYTES + MATRIX_ATOM_SCALE_OFFSETS[matrix]
            raw = slab[:, begin : begin + MATRIX_ATOM_SCALE_BYTES].contiguous().view(torch.float16)
            scales[matrix] = unpack_local_scale_atoms(unrotate_expert_atoms(raw, layer, expert))
    return states, scales
