"""Loader and driver of the UNMODIFIED reference tile-encoder extension (test infrastructure).

``oracle/build_ref.py`` compiles the reference's own CUDA sources into ``oracle/_ref``; this
module loads that prebuilt extension and drives it the way the reference's hook does
(qsrt/sqg_quantizer.py:607-651).  It is used by the ``gpu`` parity tests as ground truth and by
``bench.py`` for its "reference GPU" column; the product never loads it.
"""

from __future__ import annotations

import importlib.util
import sys
from functools import lru_cache
from pathlib import Path

REF_EXT = Path(__file__).resolve().parent / "_ref" / "qsrt_ref_sqg_ext.so"


@lru_cache(maxsize=1)
def reference_extension():
    """The prebuilt reference extension, or None when it has not been built."""

    if not REF_EXT.exists():
        return None
    import torch  # noqa: F401  (the extension links against libtorch)

    spec = importlib.util.spec_from_file_location("qsrt_ref_sqg_ext", REF_EXT)
    module = importlib.util.module_from_spec(spec)
    sys.modules["qsrt_ref_sqg_ext"] = module
    spec.loader.exec_module(module)
    return module


class ReferenceTileSearch:
    """Scratch buffers and table layout of one rate, prepared once
    (qsrt/sqg_quantizer.py:410-427, 611-640), then ``__call__(tiles) -> (reconstruction, states)``."""

    def __init__(self, lut_state, bits: int, context: int, device) -> None:
        import torch

        self.ext = reference_extension()
        if self.ext is None:
            raise RuntimeError("the reference extension has not been built (oracle/build_ref.py)")
        self.bits, self.context = int(bits), int(context)
        edges = 65536 >> bits
        decisions = edges // 4 if bits == 2 else edges // 2 if bits <= 4 else edges
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        max_batch = max(256, 3 * sms)
        self.costs = torch.zeros((max_batch, 2, edges), dtype=torch.float16, device=device)
        self.trace = torch.empty((max_batch, 256, decisions), dtype=torch.uint8, device=device)
        lut = lut_state.to(device=device, dtype=torch.uint8).contiguous()
        self.abs_max = float(lut.view(torch.float8_e4m3fn).float().abs().amax())
        if bits in (2, 3, 4):
            lut = lut.reshape(1 << bits, edges // 2, 2).permute(1, 0, 2).contiguous().reshape(-1)
        self.lut = lut

    def __call__(self, tiles):
        import torch

        tiles = tiles.contiguous()
        out = torch.empty_like(tiles)
        idx = torch.empty_like(tiles, dtype=torch.int16)
        self.ext.quantize_tiles_sqg(tiles, out, idx, self.costs, self.trace, self.lut, self.bits, self.context,
                                    self.abs_max)
        return out, idx
