"""B200-native offline trellis encoder hot path (drop-in for the QSRT ``quantizer_module``)."""

from .tiles import encode_tiles, quantize_tiles  # noqa: F401

__all__ = ["encode_tiles", "quantize_tiles"]
