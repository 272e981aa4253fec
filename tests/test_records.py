"""Mixed-rate record container (pack_qsrt_trellis family) and atom-major storage image.

CPU part: the numpy restatement against SHA-256 digests of the reference's own outputs
(tests/golden/records_golden.json), and the host-side mirror (modes, descriptor, layout, header).
GPU part: the CUDA kernels against the same digests, round trips and rejections, following
the reference's tests/test_qsrt.py:342-412 and tests/test_qsrt_storage.py.
"""

import hashlib
import json
from dataclasses import replace
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import records_oracle as ro
from qsrt_b200 import records as rec
from qsrt_b200 import storage as st
from tests.helpers import EXPERT_CASE, RECORD_CASES, expert_case_inputs, record_case_seed, record_shape

GOLDEN = json.loads((Path(__file__).parent / "golden" / "records_golden.json").read_text())


def sha(a) -> str:
    if isinstance(a, torch.Tensor):
        a = a.detach().cpu().contiguous().numpy()
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def case_states(mode: str, axis: str) -> np.ndarray:
    return ro.legal_states(record_shape(axis), rec.record_bits(mode), axis, record_case_seed(mode, axis))


# ---------------------------------------------------------------------------- CPU: oracle pins

@pytest.mark.parametrize(("mode", "axis"), [("R2", "k"), ("H308", "n"), ("K2", "k"), ("R1", "n")])
def test_oracle_payload_matches_reference_digests(mode, axis):
    gold = GOLDEN["payload"][f"{mode}/{axis}"]
    states = case_states(mode, axis)
    assert sha(states) == gold["states"]
    bits = rec.record_bits(mode)
    payload = ro.pack_records(states, bits, axis)
    assert payload.size == gold["words"]
    assert sha(payload) == gold["payload"]
    assert sha(ro.unpack_records(payload, states.shape, bits, axis, want_states=False)) == gold["edges"]
    assert np.array_equal(ro.unpack_records(payload, states.shape, bits, axis, want_states=True), states)


def test_oracle_atoms_match_reference_digests():
    for mode, axis in (("R1", "k"), ("R2", "n")):
        states = case_states(mode, axis)
        bits = rec.record_bits(mode)
        atoms = ro.matrix_atoms(ro.pack_records(states, bits, axis), bits, axis, 224)
        assert atoms.shape == (96, st.MATRIX_ATOM_TRELLIS_BYTES // 2)
        assert sha(atoms) == GOLDEN["atoms"][f"{mode}/{axis}"]


def oracle_expert_bundles() -> np.ndarray:
    layer, expert, r13, r2 = EXPERT_CASE
    states, local, _ = expert_case_inputs()
    trellis, scales = {}, {}
    for matrix in st.MATRIX_ORDER:
        axis = rec.matrix_rate_axis(matrix)
        bits = rec.record_bits(r2 if matrix == "w2" else r13)
        trellis[matrix] = ro.matrix_atoms(ro.pack_records(states[matrix], bits, axis), bits, axis, 224)
        scales[matrix] = ro.scale_atoms(local[matrix])
    slab = np.zeros((96, st.ATOM_BUNDLE_BYTES), dtype=np.uint8)
    ro.expert_slab(slab, st.ATOM_BUNDLE_BYTES, st.ATOM_BUNDLE_BYTES, 0, st.physical_atom_rotation(layer, expert),
                   trellis, scales)
    return slab


def test_oracle_expert_bundles_match_reference_digest():
    slab = oracle_expert_bundles()
    assert list(slab.shape) == GOLDEN["expert"]["shape"]
    assert sha(slab) == GOLDEN["expert"]["physical_atoms"]


# ---------------------------------------------------------------------------- CPU: host mirror

def test_mode_schedules_and_pairs():
    assert rec.record_bits("R0") == (3,) * 24
    assert rec.record_bits("R1") == (2, 4) + (3,) * 22
    assert rec.record_bits("R2") == (2, 4, 2, 4) + (3,) * 20
    assert rec.record_bits("H308") == (3,) * 22 + (4,) * 2
    assert rec.record_bits("K2") == (2,) * 24
    assert rec.pair_kinds("R2") == ("P24", "P24") + ("P33",) * 10
    assert rec.pair_kinds("K2") == ("P22",) * 12
    with pytest.raises(ValueError):
        rec.pair_bits("H308")
    assert rec.mode_from_context_bits((2,) + (3,) * 22 + (4,)) is rec.R1
    with pytest.raises(ValueError):
        rec.mode_from_context_bits((2, 3, 4))  # eight K2 donors: beyond the R0..R2 ladder
    with pytest.raises(ValueError):
        rec.ModeSpec(1, "R1", (2, 3, 3, 4) * 3)  # not monotone
    with pytest.raises(ValueError, match="unknown QSRT mode"):
        rec.resolve_mode("R9")
    with pytest.raises(TypeError):
        rec.resolve_mode(True)
    assert rec.matrix_rate_axis("w2") == "k" and rec.matrix_rate_axis("w1") == "n"


def test_descriptor_contract():
    d = rec.QSRTTrellisDescriptor(2, "k", 192, 224)
    assert d.payload_words == 192 * 224 * 256 * 3 // 16
    assert d.words_per_pair * rec.PAIRS_PER_EXPERT == d.payload_words
    assert d.to_manifest()["pair_kinds"] == list(rec.pair_kinds("R2"))
    h = rec.QSRTTrellisDescriptor(3, "n", 224, 192)
    assert h.payload_bytes == rec.FIXED_HIGH_RATE_TRELLIS_BYTES
    assert h.to_manifest()["pair_kinds"] is None
    with pytest.raises(ValueError, match="rate_axis"):
        replace(d, rate_axis="x")
    with pytest.raises(ValueError, match="3072"):
        rec.QSRTTrellisDescriptor(2, "k", 184, 224)
    with pytest.raises(ValueError, match="3584"):
        rec.QSRTTrellisDescriptor(2, "k", 192, 200)
    packed = rec.PackedQSRTTrellis(d, torch.zeros(d.payload_words - 1, dtype=torch.int16))
    with pytest.raises(ValueError, match="length"):
        packed.validate()
    with pytest.raises(TypeError, match="torch.int16"):
        rec.PackedQSRTTrellis(d, torch.zeros(d.payload_words, dtype=torch.int32)).validate()


def test_atom_arithmetic_and_layout():
    atoms = [st.logical_atom_index(p, s) for p in range(12) for s in range(8)]
    assert atoms == list(range(96))
    assert st.atom_record_indices(17) == (4, 5)
    assert st.atom_rates("R2", 15) == (2, 4) and st.atom_rates("R2", 16) == (3, 3)
    for layer, expert in ((1, 0), (92, 895), (9, 77)):
        slots = [st.physical_atom_slot(layer, expert, a) for a in range(96)]
        assert sorted(slots) == list(range(96))
        assert [st.logical_atom_for_slot(layer, expert, s) for s in slots] == list(range(96))
    covered = []
    for index in range(7):
        first, count = st.balanced_atom_partition(7, index)
        covered.extend(range(first, first + count))
    assert covered == list(range(96))
    layout = st.QSRTLayerLayout(800, 96)
    assert layout.atom_slot_stride_bytes % st.STORAGE_ALIGNMENT == 0
    assert layout.disk_bytes == st.ATOM_SLAB_OFFSET + 96 * layout.atom_slot_stride_bytes
    assert 96 * st.ATOM_BUNDLE_BYTES == st.EXPERT_TRELLIS_BYTES + 3 * 3072 * 2
    extent = layout.shard_extent(8, 3, require_equal=True)
    assert extent.atom_slots == 12 and extent.offset_bytes == st.ATOM_SLAB_OFFSET + 36 * layout.atom_slot_stride_bytes
    with pytest.raises(ValueError, match="do not divide"):
        layout.shard_extent(7, 0, require_equal=True)
    with pytest.raises(ValueError):
        st.QSRTLayerLayout(800, 95)


def test_layer_header_round_trip_and_canonical_form():
    layout = st.QSRTLayerLayout(800, 96)
    header = st.QSRTLayerHeader(7, layout)
    raw = header.to_bytes()
    assert len(raw) == st.LAYER_HEADER_BYTES
    assert st.QSRTLayerHeader.from_bytes(raw) == header
    document = json.loads(raw[8:].decode())
    assert document["qsrt_atoms"]["shape"] == [96, layout.atom_slot_stride_bytes]
    assert document["__metadata__"]["schema"] == st.SCHEMA
    tampered = raw.replace(b'"layer":"7"', b'"layer":"8"')
    assert st.QSRTLayerHeader.from_bytes(tampered).layer == 8
    with pytest.raises(ValueError, match="noncanonical"):
        st.QSRTLayerHeader.from_bytes(raw.replace(b'"experts":"896"', b'"experts":"897"'))
    with pytest.raises(ValueError):
        st.QSRTLayerHeader.from_bytes(raw[:-1])
    with pytest.raises(ValueError):
        st.QSRTLayerHeader(93, layout)


def test_scale_atoms_and_rotation_are_exact_inverses():
    scale = (torch.arange(3072, dtype=torch.float32) / 64).half()
    atoms = st.pack_local_scale_atoms(scale)
    assert np.array_equal(atoms.numpy(), ro.scale_atoms(scale.numpy()))
    assert torch.equal(st.unpack_local_scale_atoms(atoms), scale)
    rotated = st.rotate_expert_atoms(atoms, 9, 77)
    assert np.array_equal(rotated.numpy(), ro.rotate_atoms(atoms.numpy(), st.physical_atom_rotation(9, 77)))
    assert torch.equal(st.unrotate_expert_atoms(rotated, 9, 77), atoms)
    with pytest.raises(ValueError):
        st.pack_local_scale_atoms(scale[:-1])


def test_product_refuses_cpu_tensors():
    states = torch.zeros((192, 224, 256), dtype=torch.int16)
    with pytest.raises(ValueError, match="CUDA"):
        rec.pack_qsrt_trellis(states, "R2", rate_axis="k")


# ---------------------------------------------------------------------------- GPU: kernels

def _dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a).cuda()


@pytest.mark.gpu
@pytest.mark.parametrize(("mode", "axis"), RECORD_CASES)
def test_payload_matches_reference_digest_and_closes(mode, axis):
    gold = GOLDEN["payload"][f"{mode}/{axis}"]
    states = case_states(mode, axis)
    packed = rec.pack_qsrt_trellis(_dev(states), mode, rate_axis=axis)
    assert packed.descriptor.schema == rec.SCHEMA
    assert packed.payload.numel() == gold["words"] == packed.descriptor.payload_words
    assert sha(packed.payload) == gold["payload"]
    assert sha(rec.unpack_qsrt_trellis_edges(packed)) == gold["edges"]
    assert torch.equal(rec.unpack_qsrt_trellis_states(packed).cpu(), torch.from_numpy(states))


@pytest.mark.gpu
def test_packer_rejects_noncyclic_states_and_bad_shapes():
    malformed = torch.zeros((192, 224, 256), dtype=torch.int16, device="cuda")
    malformed[..., 0] = 1
    with pytest.raises(ValueError, match="closed cyclic trellis path"):
        rec.pack_qsrt_trellis(malformed, "R2", rate_axis="k")
    # the same input is accepted when the caller waives the check, as in the reference
    rec.pack_qsrt_trellis(malformed, "R2", rate_axis="k", validate_states=False)
    good = torch.zeros((192, 224, 256), dtype=torch.int16, device="cuda")
    with pytest.raises(ValueError, match="3072"):
        rec.pack_qsrt_trellis(good[:184], "R2", rate_axis="k")
    with pytest.raises(ValueError, match="3584"):
        rec.pack_qsrt_trellis(good[:, :200], "R2", rate_axis="k")
    with pytest.raises(TypeError):
        rec.pack_qsrt_trellis(good.float(), "R2", rate_axis="k")
    with pytest.raises(ValueError, match="rate_axis"):
        rec.pack_qsrt_trellis(good, "R2", rate_axis="x")


@pytest.mark.gpu
def test_repack_encoded_records_moves_whole_records():
    states = _dev(case_states("R1", "n"))
    order = torch.randperm(24, generator=torch.Generator().manual_seed(5))
    moved = rec.repack_encoded_records(states, order, "n")
    for dst in (0, 7, 23):
        src = int(order[dst])
        assert torch.equal(moved[:, dst * 8 : dst * 8 + 8], states[:, src * 8 : src * 8 + 8])
    with pytest.raises(ValueError):
        rec.repack_encoded_records(states, torch.zeros(24, dtype=torch.long), "n")


@pytest.mark.gpu
@pytest.mark.parametrize(("mode", "axis"), [(m, a) for m, a in RECORD_CASES if m in ("R0", "R1", "R2")])
def test_matrix_atoms_match_reference_digest_and_invert(mode, axis):
    packed = rec.pack_qsrt_trellis(_dev(case_states(mode, axis)), mode, rate_axis=axis)
    atoms = st.pack_matrix_atoms(packed)
    assert tuple(atoms.shape) == (96, st.MATRIX_ATOM_TRELLIS_BYTES // 2)
    assert sha(atoms) == GOLDEN["atoms"][f"{mode}/{axis}"]
    back = st.unpack_matrix_atoms(atoms, packed.descriptor)
    assert torch.equal(back.payload, packed.payload)
    with pytest.raises(ValueError):
        st.unpack_matrix_atoms(atoms[:, :-1], packed.descriptor)


@pytest.mark.gpu
def test_matrix_atoms_refuse_unbalanced_pairs():
    packed = rec.pack_qsrt_trellis(_dev(case_states("H308", "k")), "H308", rate_axis="k")
    with pytest.raises(AssertionError, match="six rate bits"):
        st.pack_matrix_atoms(packed)


@pytest.mark.gpu
def test_expert_written_straight_into_layer_image_matches_reference_bundles():
    layer, expert, r13, r2 = EXPERT_CASE
    states, local, _ = expert_case_inputs()
    layout = st.QSRTLayerLayout(3, 893)
    slot = 1
    image = torch.zeros(layout.disk_bytes, dtype=torch.uint8, device="cuda")
    modes = {"w1": r13, "w3": r13, "w2": r2}
    st.write_expert_atoms(
        image, layout, layer, expert, slot,
        {m: _dev(states[m]) for m in st.MATRIX_ORDER}, modes, {m: _dev(local[m]) for m in st.MATRIX_ORDER},
    )
    slab = image[st.ATOM_SLAB_OFFSET:].view(96, layout.atom_slot_stride_bytes).cpu()
    mine = slab[:, slot * st.ATOM_BUNDLE_BYTES : (slot + 1) * st.ATOM_BUNDLE_BYTES]
    assert sha(mine) == GOLDEN["expert"]["physical_atoms"]
    # neighbours, row padding and the sections before the slab stay untouched
    assert int(slab[:, : slot * st.ATOM_BUNDLE_BYTES].count_nonzero()) == 0
    assert int(slab[:, (slot + 1) * st.ATOM_BUNDLE_BYTES :].count_nonzero()) == 0
    assert int(image[: st.ATOM_SLAB_OFFSET].count_nonzero()) == 0
    # every bundle sits where the layout says
    probe = layout.atom_bundle_offset(5, slot)
    assert torch.equal(image[probe : probe + 64].cpu(), mine[5, :64])
    got_states, got_scales = st.read_expert_atoms(image, layout, layer, expert, slot, modes)
    for m in st.MATRIX_ORDER:
        assert torch.equal(got_states[m].cpu(), torch.from_numpy(states[m]))
        assert torch.equal(got_scales[m].cpu(), torch.from_numpy(local[m]))
    bad = {m: _dev(states[m]).clone() for m in st.MATRIX_ORDER}
    bad["w3"][3, 4, 9] ^= 0x100
    with pytest.raises(ValueError, match="closed cyclic trellis path"):
        st.write_expert_atoms(image, layout, layer, expert, slot, bad, modes,
                              {m: _dev(local[m]) for m in st.MATRIX_ORDER})


@pytest.mark.gpu
def test_record_kernels_reject_bad_descriptions():
    from qsrt_b200 import _lib

    states = torch.zeros((16, 4, 256), dtype=torch.int16, device="cuda")
    out = torch.zeros(16 * 4 * 64, dtype=torch.int16, device="cuda")
    lib = _lib.lib()
    bits = rec._bits_array((3, 5))
    assert lib.qsrtb_pack_records(states.data_ptr(), 16, 4, 0, 2, 8, bits, 0, 0, 0, out.data_ptr(), out.numel() * 2,
                                  None, None) != 0
    bits = rec._bits_array((2, 4))
    # records do not cover the axis
    assert lib.qsrtb_pack_records(states.data_ptr(), 16, 4, 0, 2, 4, bits, 0, 0, 0, out.data_ptr(), out.numel() * 2,
                                  None, None) != 0
    # destination too small
    assert lib.qsrtb_pack_records(states.data_ptr(), 16, 4, 0, 2, 8, bits, 0, 0, 0, out.data_ptr(), 64, None, None) != 0
    # atom pitch smaller than an atom
    assert lib.qsrtb_pack_records(states.data_ptr(), 16, 4, 0, 2, 8, bits, 1, 0, 64, out.data_ptr(), out.numel() * 2,
                                  None, None) != 0
    # a small general geometry (2 records x 8 stripes, 4 orthogonal tiles) round-trips in both layouts
    rng = np.random.default_rng(3)
    legal = np.empty((16, 4, 256), dtype=np.int16)
    from oracle.qsrt_oracle import reconstruct_trellis_states
    for r, b in enumerate((2, 4)):
        legal[r * 8 : r * 8 + 8] = reconstruct_trellis_states(rng.integers(0, 1 << b, size=(8, 4, 256)), b)
    dev = torch.from_numpy(legal).cuda()
    for layout_id, pitch in ((0, 0), (1, 4 * 32 * 6 + 64)):
        out.zero_()
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        _lib.check(lib.qsrtb_pack_records(dev.data_ptr(), 16, 4, 0, 2, 8, bits, layout_id, 3 if layout_id else 0, pitch,
                                          out.data_ptr(), out.numel() * 2, flag.data_ptr(), None), "pack")
        assert int(flag.item()) == 0
        back = torch.empty_like(dev)
        _lib.check(lib.qsrtb_unpack_records(out.data_ptr(), out.numel() * 2, 16, 4, 0, 2, 8, bits, layout_id,
                                            3 if layout_id else 0, pitch, back.data_ptr(), None, None), "unpack")
        assert torch.equal(back, dev)
        if layout_id == 0:
            assert np.array_equal(out[: 16 * 4 * 48].cpu().numpy(), ro.pack_records(legal, (2, 4), "k"))
