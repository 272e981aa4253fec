"""CPU checks of the C ABI: the library loads and exports every declared symbol."""

import ctypes
import re
from pathlib import Path

from qsrt_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    header = (ROOT / "include" / "qsrt_b200.h").read_text()
    return sorted(set(re.findall(r"\b(qsrtb_[a-z0-9_]+)\s*\(", header)))


def test_library_exports_every_declared_symbol():
    handle = ctypes.CDLL(str(_lib.LIBRARY))
    names = declared_symbols()
    assert len(names) >= 14
    for name in names:
        assert hasattr(handle, name), f"{name} is declared in include/qsrt_b200.h but not exported"


def test_binding_covers_the_header():
    assert sorted(_lib.exported_symbols()) == declared_symbols()


def test_host_only_entry_points_work_without_a_gpu():
    handle = _lib.lib()
    assert handle.qsrtb_abi_version() == 1
    # argument validation happens before any CUDA call
    status = handle.qsrtb_quantize_tiles(None, 4, None, None, 7, 128, 0, None, None, None, 0, None)
    assert status == _lib.EINVAL
    assert b"bits" in handle.qsrtb_last_error()
    status = handle.qsrtb_pack_trellis(None, -1, 3, None, None)
    assert status == _lib.EINVAL


def test_variant_word_of_the_search_entry_points():
    """Host-side assembly of ``variant``: bit 0 dedicated K2, bits 4-5 layout, bits 6-7 traceback."""

    import pytest

    from qsrt_b200 import tiles

    assert tiles.search_variant(False) == (0, False)
    assert tiles.search_variant(True, {"tile_search_traceback": 1}) == (1 | (1 << 6), False)
    assert tiles.search_variant(False, {"tile_search_traceback": 2}, units_per_thread=2) == ((2 << 4) | (2 << 6), True)
    assert tiles.search_variant(True, {"tile_search_traceback": 2}, traceback=0) == (1, False)
    with pytest.raises(ValueError):
        tiles.search_variant(False, {"tile_search_traceback": 3})
    handle = _lib.lib()
    # a variant with unknown bits, or traceback organisation 3, is refused before any CUDA call
    for bad in (1 << 8, 3 << 6, 3 << 4):
        status = handle.qsrtb_quantize_tiles(None, 4, None, None, 3, 128, bad, None, None, None, 0, None)
        assert status == _lib.EINVAL and b"variant" in handle.qsrtb_last_error()

