"""Tile quantizer hook: ``quantize_tiles(tiles, quant_args)``.

Host-side mirror of the function the reference installs on its encoder module
(``qsrt/sqg_quantizer.py:478-654``): same arguments, same ``quant_args`` keys, same error
behaviour, same outputs (freshly allocated, enqueued on the current stream, no host sync
after the first use of a table).  The work is done by ``qsrtb_quantize_tiles`` in
``libqsrt_b200.so``.
"""

from __future__ import annotations

import ctypes
from collections.abc import Mapping

import torch

from . import _lib

# Largest |label| the dedicated K2 arithmetic admits (qsrt/csrc/sqg_quantize.cu:735-737).
K2_DEDICATED_MAX_LABEL = 16.0

_UNSUPPORTED_KEYS = {
    "periodic_rate_schedules": "periodic (within-tile variable) rates",
    "sqg_fp16_lut": "experimental FP16 tables",
}

# (device, bits, source key) -> (source tensor, state-indexed device table, predecessor-major
# device table, max |label|)
# When a list, every tile-search launch appends (start_event, end_event, n_tiles, bits); the
# benchmark uses it to time the dominant kernel on the launching stream.
search_timings: list | None = None


class timed_search:
    """Context manager recording CUDA events around one tile-search launch."""

    def __init__(self, device: torch.device, n_tiles: int, bits: int) -> None:
        self.active = search_timings is not None
        self.device, self.n_tiles, self.bits = device, n_tiles, bits

    def __enter__(self):
        if self.active:
            self.start = torch.cuda.Event(enable_timing=True)
            self.end = torch.cuda.Event(enable_timing=True)
            self.start.record(torch.cuda.current_stream(self.device))
        return self

    def __exit__(self, *exc):
        if self.active:
            self.end.record(torch.cuda.current_stream(self.device))
            search_timings.append((self.start, self.end, self.n_tiles, self.bits))
        return False


_tables: dict[tuple[str, int, int], tuple[torch.Tensor, torch.Tensor, torch.Tensor, float]] = {}
_scratch: dict[tuple[str, int, int], torch.Tensor] = {}


def _stream_ptr(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def prepared_table(codebook: torch.Tensor, bits: int, device: torch.device):
    """Device copies of a state-indexed table: (state order, predecessor-major order, amax)."""

    source_key = codebook.data_ptr() if codebook.is_cuda else id(codebook)
    key = (str(device), bits, source_key)
    cached = _tables.get(key)
    if cached is not None and cached[0] is codebook:
        return cached[1], cached[2], cached[3]
    lut = codebook.to(device=device, dtype=torch.uint8).contiguous()
    if lut.numel() != 65536:
        raise ValueError("codebook must contain 65,536 uint8 E4M3 values")
    lut = lut.reshape(-1)
    lut_pm = torch.empty_like(lut)
    amax = torch.empty(1, dtype=torch.float32, device=device)
    with torch.cuda.device(device):
        _lib.check(
            _lib.lib().qsrtb_lut_prepare(
                lut.data_ptr(), bits, lut_pm.data_ptr(), amax.data_ptr(), _stream_ptr(device)
            ),
            "qsrtb_lut_prepare",
        )
    abs_max = float(amax.item())  # one host sync per table, as in the reference
    _tables[key] = (codebook, lut, lut_pm, abs_max)
    return lut, lut_pm, abs_max


def traceback_scratch(device: torch.device, bits: int, cost_rows: bool = False) -> torch.Tensor:
    """Traceback scratch of the current stream: one slice per resident CTA of the persistent
    grid.  Keyed by stream so that searches enqueued on different streams never share rows.
    ``cost_rows`` asks for the path-cost rows per CTA that an explicit ``traceback=2`` needs at
    every rate (the default size already has them at 3 and 4 bits)."""

    key = (str(device), bits, torch.cuda.current_stream(device).cuda_stream, bool(cost_rows))
    buffer = _scratch.get(key)
    if buffer is None:
        wanted = ctypes.c_size_t(0)
        with torch.cuda.device(device):
            _lib.check(
                _lib.lib().qsrtb_viterbi_scratch_bytes(bits, 1 << 30, ctypes.byref(wanted)),
                "qsrtb_viterbi_scratch_bytes",
            )
        size = wanted.value
        if cost_rows:
            with torch.cuda.device(device):
                _lib.check(
                    _lib.lib().qsrtb_viterbi_cost_scratch_bytes(bits, 1 << 30, ctypes.byref(wanted)),
                    "qsrtb_viterbi_cost_scratch_bytes",
                )
            size = max(size, wanted.value)
        buffer = torch.empty(size, dtype=torch.uint8, device=device)
        _scratch[key] = buffer
    return buffer


def search_variant(dedicated: bool, quant_args: dict | None = None, units_per_thread: int = 0,
                   traceback: int | None = None) -> tuple[int, bool]:
    """The ``variant`` word of the search entry points and whether the launch needs the
    path-cost scratch at every rate.  ``quant_args["tile_search_traceback"]`` (0 the kernel's
    choice, 1 survivor decisions, 2 path costs) is this library's own tuning key; the results do
    not depend on it."""

    if traceback is None:
        traceback = int((quant_args or {}).get("tile_search_traceback", 0))
    if traceback not in (0, 1, 2):
        raise ValueError("traceback must be 0 (kernel's choice), 1 (decisions) or 2 (path costs)")
    return (1 if dedicated else 0) | (int(units_per_thread) << 4) | (traceback << 6), traceback == 2


def encode_tiles(
    tiles: torch.Tensor,
    codebook: torch.Tensor,
    bits: int,
    tailbite_context: int = 128,
    *,
    force_generic: bool = False,
    units_per_thread: int = 0,
    traceback: int = 0,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Encode ``[N, 256]`` float32 CUDA tiles with a state-indexed E4M3 table.

    ``units_per_thread`` picks the search kernel's thread layout for this call (0 = per-rate
    default, 1 = 1024 threads with fp8 labels, 2 = 512 threads with half2 labels) and
    ``traceback`` what the kernel keeps for its traceback (0 = the kernel's choice, 1 = survivor
    decisions, 2 = path costs with the decisions recomputed lazily); the results do not depend
    on either."""

    if not tiles.is_cuda:
        raise ValueError("input_tiles must be CUDA")
    if tiles.dtype != torch.float32 or tiles.ndim != 2 or tiles.shape[1] != 256:
        raise ValueError("SQG tiles must be contiguous FP32 [N, 256]")
    if bits not in (2, 3, 4):
        raise ValueError("the B200 tile encoder supports K2, K3 and K4")
    if not 1 <= int(tailbite_context) <= 128:
        raise ValueError("tailbite_context must be in 1..128")
    if units_per_thread not in (0, 1, 2):
        raise ValueError("units_per_thread must be 0 (per-rate default), 1 or 2")
    variant, cost_rows = search_variant(False, None, units_per_thread, traceback)
    tiles = tiles.contiguous()
    device = tiles.device
    lut, lut_pm, abs_max = prepared_table(codebook, bits, device)
    dedicated = (
        bits == 2
        and not force_generic
        and abs_max == abs_max
        and 0.0 < abs_max <= K2_DEDICATED_MAX_LABEL
    )
    output = torch.empty_like(tiles)
    indices = torch.empty_like(tiles, dtype=torch.int16)
    if tiles.shape[0] == 0:
        return output, indices
    scratch = traceback_scratch(device, bits, cost_rows=cost_rows)
    with torch.cuda.device(device), timed_search(device, tiles.shape[0], bits):
        _lib.check(
            _lib.lib().qsrtb_quantize_tiles(
                tiles.data_ptr(), tiles.shape[0], lut.data_ptr(), lut_pm.data_ptr(), bits,
                int(tailbite_context), variant | (1 if dedicated else 0), output.data_ptr(),
                indices.data_ptr(), scratch.data_ptr(), scratch.numel(), _stream_ptr(device),
            ),
            "qsrtb_quantize_tiles",
        )
    return output, indices


def quantize_tiles(tiles: torch.Tensor, quant_args: dict):
    """Drop-in for the reference's patched ``quantize_tiles`` (sqg_quantizer.py:478-654)."""

    for key, what in _UNSUPPORTED_KEYS.items():
        if quant_args.get(key) is not None:
            raise NotImplementedError(f"{what} are outside the B200 encoder hot path")
    codebook = quant_args.get("sqg_e4m3_lut")
    rate_codebooks = quant_args.get("sqg_e4m3_luts_by_bits")
    mode = quant_args.get("sqg_e4m3_mode")
    if codebook is None and rate_codebooks is None and mode is None:
        raise ValueError(
            "quantize_tiles needs a QSRT table (sqg_e4m3_lut or sqg_e4m3_luts_by_bits); "
            "the upstream procedural codebooks are not part of this encoder"
        )
    if mode is not None:
        raise NotImplementedError("the R44 'normal' research law is outside the B200 hot path")
    if len(quant_args["devices"]) != 1:
        raise ValueError("the SQG validation hook currently requires one CUDA device")
    if tiles.dtype != torch.float32 or tiles.ndim != 2 or tiles.shape[1] != 256:
        raise ValueError("SQG tiles must be contiguous FP32 [N, 256]")
    bits = int(quant_args["K"])
    if rate_codebooks is not None:
        if codebook is not None:
            raise ValueError("rate-specific SQG LUTs cannot be combined with another SQG law")
        if not isinstance(rate_codebooks, Mapping):
            raise TypeError("sqg_e4m3_luts_by_bits must be a mapping")
        if set(rate_codebooks) - {1, 2, 3, 4}:
            raise ValueError("rate-specific SQG LUT keys must be K1 through K4")
        try:
            codebook = rate_codebooks[bits]
        except KeyError as exc:
            raise ValueError(f"missing rate-specific SQG K{bits} LUT") from exc
        if codebook is None:
            raise NotImplementedError("procedural (MCG) rate entries are outside the B200 hot path")
    return encode_tiles(tiles, codebook, bits, int(quant_args.get("tailbite_context", 128)))
