"""GPU parity of the tile encoder: CUDA kernel vs the CPU restatement vs the reference kernel."""

import numpy as np
import pytest
import torch

from oracle import qsrt_oracle as oracle
from qsrt_b200 import tables, tiles as tile_api
from tests import helpers

pytestmark = pytest.mark.gpu


def _lut(bits):
    return tables.sqg_xor_cheb_t12_bytes(bits)


@pytest.mark.parametrize("context", [1, 32, 128])
@pytest.mark.parametrize("bits", [2, 3, 4])
def test_kernel_matches_cpu_oracle_bit_for_bit(cuda_device, bits, context):
    tiles = helpers.mixed_tiles(6, seed=100 * bits + context)
    lut = _lut(bits)
    out, idx = tile_api.encode_tiles(tiles.to(cuda_device), lut, bits, context)
    ref_out, ref_idx = oracle.quantize_tiles(tiles.numpy(), lut.numpy(), bits, context)
    assert np.array_equal(idx.cpu().numpy(), ref_idx)
    assert np.array_equal(out.cpu().numpy(), ref_out)


@pytest.mark.parametrize("context", [1, 128])
def test_generic_k2_arithmetic_matches_cpu_oracle(cuda_device, context):
    """K2 tables with |label| > 16 use the saturating generic arithmetic (sqg_quantize.cu:735-748)."""

    tiles = helpers.mixed_tiles(4, seed=77 + context)
    lut = _lut(2)
    out, idx = tile_api.encode_tiles(tiles.to(cuda_device), lut, 2, context, force_generic=True)
    ref_out, ref_idx = oracle.quantize_tiles(
        tiles.numpy(), lut.numpy(), 2, context, variant=oracle.VARIANT_GENERIC
    )
    assert np.array_equal(idx.cpu().numpy(), ref_idx)
    assert np.array_equal(out.cpu().numpy(), ref_out)


@pytest.mark.parametrize("context", [1, 32, 128])
@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("family", helpers.FAMILIES)
def test_kernel_matches_reference_kernel(cuda_device, family, bits, context):
    """512 tiles per family through the unmodified reference CUDA kernel (prebuilt)."""

    if helpers.reference_extension() is None:
        pytest.skip("oracle/_ref was not built")
    tiles = helpers.make_tiles(family, 512, seed=20260816).to(cuda_device)
    lut = _lut(bits)
    out, idx = tile_api.encode_tiles(tiles, lut, bits, context)
    ref_out, ref_idx = helpers.reference_quantize_tiles(tiles, lut, bits, context)
    same = (idx == ref_idx).all(dim=1)
    assert bool(same.all()), f"{int((~same).sum())} of 512 tiles differ"
    assert torch.equal(out, ref_out)


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_structural_rows_match_reference_kernel(cuda_device, bits):
    if helpers.reference_extension() is None:
        pytest.skip("oracle/_ref was not built")
    tiles = helpers.mixed_tiles(2, seed=5).to(cuda_device)
    lut = _lut(bits)
    out, idx = tile_api.encode_tiles(tiles, lut, bits, 128)
    ref_out, ref_idx = helpers.reference_quantize_tiles(tiles, lut, bits, 128)
    assert torch.equal(idx, ref_idx)
    assert torch.equal(out, ref_out)


@pytest.mark.parametrize("context", [1, 32, 128])
def test_k2_closes_trellis_and_decodes_states(cuda_device, context):
    """Mirror of tests/test_sqg_quantizer.py:169-207 of the reference."""

    g = torch.Generator(device="cpu").manual_seed(7)
    tiles = torch.randn((64, 256), generator=g, dtype=torch.float32)
    tiles[3] *= 100.0
    tiles[11] = 0.0
    tiles[17] *= -40.0
    lut = _lut(2)
    output, states = tile_api.quantize_tiles(
        tiles.to(cuda_device),
        {"K": 2, "devices": ["cuda:0"], "sqg_e4m3_lut": lut, "tailbite_context": context},
    )
    assert oracle.states_close(states.cpu().numpy(), 2)
    decoded = lut.view(torch.float8_e4m3fn).float()[states.cpu().long() & 0xFFFF]
    assert torch.equal(decoded, output.cpu())


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_saturated_cost_paths_stay_closed(cuda_device, bits):
    """Mirror of tests/test_sqg_quantizer.py:210-231 (K1 is outside this encoder)."""

    tiles = torch.full((2, 256), 1000.0, dtype=torch.float32, device=cuda_device)
    _out, states = tile_api.quantize_tiles(
        tiles, {"K": bits, "devices": ["cuda:0"], "sqg_e4m3_luts_by_bits": {bits: _lut(bits)}}
    )
    assert oracle.states_close(states.cpu().numpy(), bits)


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_thread_layouts_agree(cuda_device, bits):
    """1024 threads with fp8 labels and 512 threads with half2 labels give the same bits."""

    tiles = helpers.mixed_tiles(5, seed=31 + bits).to(cuda_device)
    lut = _lut(bits)
    out1, idx1 = tile_api.encode_tiles(tiles, lut, bits, 128, units_per_thread=1)
    gen1 = tile_api.encode_tiles(tiles, lut, bits, 32, force_generic=True, units_per_thread=1)
    out2, idx2 = tile_api.encode_tiles(tiles, lut, bits, 128, units_per_thread=2)
    gen2 = tile_api.encode_tiles(tiles, lut, bits, 32, force_generic=True, units_per_thread=2)
    assert torch.equal(idx1, idx2) and torch.equal(out1, out2)
    assert torch.equal(gen1[1], gen2[1])
    ref_out, ref_idx = oracle.quantize_tiles(tiles.cpu().numpy()[:8], lut.numpy(), bits, 128)
    assert np.array_equal(idx2.cpu().numpy()[:8], ref_idx)


@pytest.mark.parametrize("context", [1, 32, 128])
@pytest.mark.parametrize("bits,generic", [(2, False), (2, True), (3, False), (4, False)])
def test_traceback_organisations_agree(cuda_device, bits, generic, context):
    """Survivor decisions for every step, or path costs for the constrained pass with the one
    decision per step recomputed by the traceback chain: same states, same reconstruction.  The
    batch gives every CTA several tiles (chains overlapping the next tile), includes rows that
    meet the fp16 clamp (re-encoded with the literal arithmetic while a chain is in flight) and
    contexts whose primer is too short to hide a chain (the rest is walked at the end)."""

    tiles = helpers.mixed_tiles(160, seed=11 * bits + context).to(cuda_device)
    tiles[5::37] *= 60.0
    lut = _lut(bits)
    for units in (1, 2):
        kept = tile_api.encode_tiles(tiles, lut, bits, context, force_generic=generic,
                                     units_per_thread=units, traceback=1)
        lazy = tile_api.encode_tiles(tiles, lut, bits, context, force_generic=generic,
                                     units_per_thread=units, traceback=2)
        same = (kept[1] == lazy[1]).all(dim=1)
        assert bool(same.all()), f"units {units}: {int((~same).sum())} of {tiles.shape[0]} tiles differ"
        assert torch.equal(kept[0], lazy[0])
    chosen = tile_api.encode_tiles(tiles, lut, bits, context, force_generic=generic)
    assert torch.equal(chosen[1], kept[1])


@pytest.mark.parametrize("extra", [1, 147, 148, 149, 296, 300])
def test_interleaved_passes_at_every_tile_count(cuda_device, extra):
    """The path-cost organisation interleaves the passes of a CTA's tiles (primer of the next
    tile before the constrained pass of this one); CTAs with one, two, three and four tiles, and
    launches where the CTAs differ in their count, all give the states of the decisions kernel."""

    sms = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    tiles = helpers.make_tiles("heavy", sms + extra, seed=extra).to(cuda_device)
    for bits in (3, 4):
        lut = _lut(bits)
        kept = tile_api.encode_tiles(tiles, lut, bits, 128, traceback=1)
        lazy = tile_api.encode_tiles(tiles, lut, bits, 128, traceback=2)
        assert torch.equal(kept[1], lazy[1]) and torch.equal(kept[0], lazy[0])


def test_lazy_traceback_matches_reference_kernel(cuda_device):
    """The path-cost organisation against the unmodified reference kernel, every family."""

    if helpers.reference_extension() is None:
        pytest.skip("oracle/_ref was not built")
    for bits in (2, 3, 4):
        lut = _lut(bits)
        tiles = torch.cat([helpers.make_tiles(f, 400, seed=41 + bits) for f in helpers.FAMILIES]).to(cuda_device)
        out, idx = tile_api.encode_tiles(tiles, lut, bits, 128, traceback=2)
        ref_out, ref_idx = helpers.reference_quantize_tiles(tiles, lut, bits, 128)
        same = (idx == ref_idx).all(dim=1)
        assert bool(same.all()), f"K{bits}: {int((~same).sum())} of {tiles.shape[0]} tiles differ"
        assert torch.equal(out, ref_out)


def test_empty_and_ragged_batches(cuda_device):
    lut = _lut(3)
    out, idx = tile_api.encode_tiles(torch.empty((0, 256), device=cuda_device), lut, 3)
    assert out.shape == (0, 256) and idx.shape == (0, 256)
    tiles = helpers.make_tiles("normal", 301, seed=3).to(cuda_device)  # more tiles than CTAs, odd count
    out_all, idx_all = tile_api.encode_tiles(tiles, lut, 3)
    out_head, idx_head = tile_api.encode_tiles(tiles[:7].contiguous(), lut, 3)
    assert torch.equal(idx_all[:7], idx_head) and torch.equal(out_all[:7], out_head)


def test_argument_errors(cuda_device):
    lut = _lut(2)
    good = torch.zeros((1, 256), device=cuda_device)
    with pytest.raises(ValueError):
        tile_api.encode_tiles(torch.zeros((1, 255), device=cuda_device), lut, 2)
    with pytest.raises(ValueError):
        tile_api.encode_tiles(good, lut, 2, 129)
    with pytest.raises(ValueError):
        tile_api.encode_tiles(good, lut, 5)
    with pytest.raises(ValueError):
        tile_api.quantize_tiles(good, {"K": 2, "devices": ["cuda:0"]})
    with pytest.raises(ValueError):
        tile_api.quantize_tiles(good, {"K": 2, "devices": ["cuda:0", "cuda:1"], "sqg_e4m3_lut": lut})
