"""CPU oracle for the offline trellis-encoder hot path (numpy + the C restatement).

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module; it is the
checker used by ``tests/``, by the smoke test, and as the timed CPU baseline of the benchmark.

Every function names the reference code it restates (paths are relative to the reference
checkout).  Integer and byte results are meant to be bit-exact with the reference.
"""

from __future__ import annotations

import ctypes
import math
import os
import subprocess
from functools import lru_cache
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libqsrt_oracle.so"
_SRC_PATH = _HERE / "viterbi_oracle.c"


def build_c_oracle(force: bool = False) -> Path:
    """Compile ``viterbi_oracle.c`` (gcc, OpenMP) next to its source."""

    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < _SRC_PATH.stat().st_mtime:
        subprocess.run(
            [
                "gcc", "-O3", "-fopenmp", "-shared", "-fPIC",
                "-o", str(_LIB_PATH), str(_SRC_PATH), "-lm",
            ],
            check=True,
        )
    return _LIB_PATH


@lru_cache(maxsize=1)
def _lib() -> ctypes.CDLL:
    if not _LIB_PATH.exists():
        build_c_oracle()
    lib = ctypes.CDLL(str(_LIB_PATH))
    lib.qsrt_oracle_quantize_tiles.restype = ctypes.c_int
    lib.qsrt_oracle_quantize_tiles.argtypes = [
        ctypes.c_void_p, ctypes.c_long, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
        ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
    ]
    lib.qsrt_oracle_lut_abs_max.restype = ctypes.c_double
    lib.qsrt_oracle_lut_abs_max.argtypes = [ctypes.c_void_p]
    lib.qsrt_oracle_d2h.restype = ctypes.c_uint16
    lib.qsrt_oracle_d2h.argtypes = [ctypes.c_double]
    lib.qsrt_oracle_h2d.restype = ctypes.c_double
    lib.qsrt_oracle_h2d.argtypes = [ctypes.c_uint16]
    lib.qsrt_oracle_e4m3.restype = ctypes.c_double
    lib.qsrt_oracle_e4m3.argtypes = [ctypes.c_uint8]
    return lib


# --------------------------------------------------------------------------------------
# T1: reconstruction tables (qsrt/sqg_e4m3.py:196-301)
# --------------------------------------------------------------------------------------

def e4m3_to_float(raw: np.ndarray) -> np.ndarray:
    """Decode raw E4M3 (finite, "fn" flavour) bytes to float64."""

    raw = np.asarray(raw, dtype=np.uint8).astype(np.int64)
    sign = np.where(raw >> 7, -1.0, 1.0)
    exponent = (raw >> 3) & 15
    mantissa = raw & 7
    value = np.where(
        exponent == 0,
        mantissa * 2.0 ** -9,
        (8 + mantissa) * np.exp2(exponent.astype(np.float64) - 10.0),
    )
    value = np.where((exponent == 15) & (mantissa == 7), np.nan, value)
    return sign * value


def float_to_e4m3(values: np.ndarray) -> np.ndarray:
    """Round float32 values to E4M3 bytes, round-to-nearest-even (torch ``float8_e4m3fn``)."""

    x = np.asarray(values, dtype=np.float32).astype(np.float64)
    sign = np.signbit(x)
    a = np.abs(x)
    _, exponent = np.frexp(np.where(a == 0, 1.0, a))  # a = m * 2**exponent, m in [0.5, 1)
    e = exponent - 1
    e = np.maximum(e, -6)  # subnormal spacing below 2**-6
    step = np.exp2((e - 3).astype(np.float64))
    q = np.rint(a / step)  # ties to even
    overflow = q >= 16
    e = np.where(overflow, e + 1, e)
    q = np.where(overflow, 8, q)
    biased = e + 7
    normal = q >= 8
    byte = np.where(normal, (biased << 3) | (q.astype(np.int64) - 8), q.astype(np.int64))
    byte = np.where(a == 0, 0, byte)
    if np.any(byte > 0x7E):
        raise ValueError("value out of the finite E4M3 range")
    return (byte | (sign.astype(np.int64) << 7)).astype(np.uint8)


def _reverse_low_bits(values: np.ndarray, bits: int) -> np.ndarray:
    result = np.zeros_like(values)
    for index in range(bits):
        result |= ((values >> index) & 1) << (bits - 1 - index)
    return result


@lru_cache(maxsize=None)
def sqg_xor_rank_permutation(bits: int) -> np.ndarray:
    """qsrt/sqg_e4m3.py:259-284: carry-mixed rank of every 16-bit codeword."""

    if bits not in range(1, 7):
        raise ValueError("SQG supports integer K1 through K6")
    width = 16 - bits
    history_mask = (1 << width) - 1
    codeword = np.arange(1 << 16, dtype=np.int64)
    history = codeword >> bits
    branch = codeword & ((1 << bits) - 1)
    mixed = history ^ (history >> 11)
    mixed = mixed ^ ((mixed << 11) & history_mask)
    product = (0x3FA7D929 * mixed + 0xC928FD8E) & 0xFFFFFFFF
    phase = product & history_mask
    syndrome = product >> (32 - bits)
    stratum = _reverse_low_bits(branch, bits) ^ syndrome
    return (stratum << width) | phase


@lru_cache(maxsize=1)
def sqg_cheb_normal_rank_e4m3_bytes() -> np.ndarray:
    """qsrt/sqg_e4m3.py:196-229: the exact normal-quantile staircase rounded to E4M3."""

    from scipy.special import ndtri

    ranks = np.arange(1 << 16, dtype=np.float64)
    values = 1.5 * ndtri((ranks + 0.5) / (1 << 16))
    raw = float_to_e4m3(values.astype(np.float32))
    raw = raw.copy()
    raw[(raw & 0x7F) == 0] = 0
    decoded = e4m3_to_float(raw)
    if not np.all(decoded[1:] >= decoded[:-1]):
        raise RuntimeError("rank law is not monotone after E4M3 rounding")
    return raw


@lru_cache(maxsize=1)
def sqg_xor_cheb_t12_rank_lut_bytes() -> np.ndarray:
    """qsrt/sqg_e4m3.py:241-256: modal byte of each block of 16 ranks (ties: lower byte)."""

    exact = sqg_cheb_normal_rank_e4m3_bytes().reshape(1 << 12, 16)
    result = np.empty(1 << 12, dtype=np.uint8)
    for index, block in enumerate(exact):
        labels, counts = np.unique(block, return_counts=True)
        result[index] = labels[counts == counts.max()].min()
    return result


@lru_cache(maxsize=None)
def sqg_xor_cheb_t12_bytes(bits: int) -> np.ndarray:
    """qsrt/sqg_e4m3.py:287-301: state-indexed E4M3 labels of the primary codebook."""

    return sqg_xor_cheb_t12_rank_lut_bytes()[sqg_xor_rank_permutation(bits) >> 4].copy()


# --------------------------------------------------------------------------------------
# X1: tensor-core element order (qsrt/exl3_encoder_backend.py:35-57)
# --------------------------------------------------------------------------------------

@lru_cache(maxsize=1)
def tensor_core_perm() -> np.ndarray:
    perm = np.zeros(256, dtype=np.int64)
    for t in range(32):
        r0 = (t % 4) * 2
        rows = (r0, r0 + 1, r0 + 8, r0 + 9)
        c0 = t // 4
        for j, row in enumerate(rows):
            perm[t * 8 + j] = row * 16 + c0
            perm[t * 8 + 4 + j] = row * 16 + c0 + 8
    return perm


@lru_cache(maxsize=1)
def tensor_core_perm_inverse() -> np.ndarray:
    return np.argsort(tensor_core_perm())


def matrix_to_tiles(weight: np.ndarray) -> np.ndarray:
    """[K, N] -> [K/16, N/16, 256] in tensor-core order (exl3_encoder_backend.py:506-509)."""

    k, n = weight.shape
    tiles = weight.reshape(k // 16, 16, n // 16, 16).transpose(0, 2, 1, 3).reshape(k // 16, n // 16, 256)
    return tiles[..., tensor_core_perm()]


def tiles_to_matrix(tiles: np.ndarray) -> np.ndarray:
    """Inverse of :func:`matrix_to_tiles` (exl3_reference.py:132-140)."""

    kt, nt, _ = tiles.shape
    rowmajor = tiles[..., tensor_core_perm_inverse()]
    return rowmajor.reshape(kt, nt, 16, 16).transpose(0, 2, 1, 3).reshape(kt * 16, nt * 16)


# --------------------------------------------------------------------------------------
# V1-V5: tile encoder (C restatement)
# --------------------------------------------------------------------------------------

VARIANT_AUTO, VARIANT_GENERIC, VARIANT_K2 = 0, 1, 2

# OpenMP threads used when a call does not say (0 = the OpenMP default, which launchers such
# as torchrun pin to 1 through OMP_NUM_THREADS).
DEFAULT_THREADS = 0


def quantize_tiles(
    tiles: np.ndarray,
    lut: np.ndarray,
    bits: int,
    tailbite_context: int = 128,
    *,
    variant: int = VARIANT_AUTO,
    threads: int = 0,
) -> tuple[np.ndarray, np.ndarray]:
    """Encode ``[N, 256]`` float32 tiles; returns (reconstruction float32, states int16).

    ``lut`` is the state-indexed 65,536-byte E4M3 table, exactly what callers put into
    ``quant_args["sqg_e4m3_lut"]`` (qsrt/sqg_quantizer.py:478-654).
    """

    tiles = np.ascontiguousarray(tiles, dtype=np.float32)
    lut = np.ascontiguousarray(lut, dtype=np.uint8)
    if tiles.ndim != 2 or tiles.shape[1] != 256:
        raise ValueError("tiles must be [N, 256]")
    if lut.size != 65536:
        raise ValueError("lut must hold 65,536 bytes")
    out = np.empty_like(tiles)
    idx = np.empty(tiles.shape, dtype=np.uint16)
    status = _lib().qsrt_oracle_quantize_tiles(
        tiles.ctypes.data, tiles.shape[0], lut.ctypes.data, int(bits), int(tailbite_context),
        int(variant), out.ctypes.data, idx.ctypes.data, int(threads or DEFAULT_THREADS),
    )
    if status != 0:
        raise ValueError(f"oracle tile encoder rejected its arguments (status {status})")
    return out, idx.view(np.int16)


def lut_abs_max(lut: np.ndarray) -> float:
    lut = np.ascontiguousarray(lut, dtype=np.uint8)
    return float(_lib().qsrt_oracle_lut_abs_max(lut.ctypes.data))


def path_cost(tiles: np.ndarray, states: np.ndarray, lut: np.ndarray, clamp: float | None = None) -> np.ndarray:
    """Float64 squared error of each tile's decoded path against the half-rounded input."""

    w = np.asarray(tiles, dtype=np.float32)
    if clamp is not None:
        w = np.clip(w, -clamp, clamp)
    w = w.astype(np.float16).astype(np.float64)
    decoded = e4m3_to_float(np.asarray(lut, dtype=np.uint8)[states.view(np.uint16).astype(np.int64)])
    return ((decoded - w) ** 2).sum(axis=-1)


def states_close(states: np.ndarray, bits: int) -> bool:
    """Tail-biting closure: each state's low 16-K bits are the next state's high bits."""

    s = states.view(np.uint16).astype(np.int64)
    nxt = np.roll(s, -1, axis=-1)
    return bool(np.all((s & ((1 << (16 - bits)) - 1)) == (nxt >> bits)))


# --------------------------------------------------------------------------------------
# P1: bit packer (qsrt/qsrt.py:861-913, qsrt/qsrt_codec_pilot.py:220-280)
# --------------------------------------------------------------------------------------

def pack_trellis_edges(indices: np.ndarray, bits: int) -> np.ndarray:
    """Low K bits of each of 256 symbols, MSB first, as 16-bit words with pairs swapped."""

    values = np.asarray(indices).astype(np.int64) & ((1 << bits) - 1)
    lead = values.shape[:-1]
    symbol_shifts = np.arange(bits - 1, -1, -1)
    bitstream = ((values[..., None] >> symbol_shifts) & 1).reshape(*lead, 16 * bits, 16)
    words = (bitstream << np.arange(15, -1, -1)).sum(axis=-1)
    swapped = words.reshape(*lead, -1, 2)[..., ::-1].reshape(*lead, 16 * bits)
    return swapped.astype(np.uint16).view(np.int16)


def unpack_trellis_edges(packed: np.ndarray, bits: int) -> np.ndarray:
    words = np.asarray(packed).view(np.uint16).astype(np.int64)
    lead = words.shape[:-1]
    words = words.reshape(*lead, -1, 2)[..., ::-1].reshape(*lead, 16 * bits)
    bitstream = ((words[..., None] >> np.arange(15, -1, -1)) & 1).reshape(*lead, 256, bits)
    values = (bitstream << np.arange(bits - 1, -1, -1)).sum(axis=-1)
    return values.astype(np.int16)


# --------------------------------------------------------------------------------------
# D1: decoder (qsrt/exl3_reference.py:34-58, 108-140, 210-243, 280-302)
# --------------------------------------------------------------------------------------

def reconstruct_trellis_states(edges: np.ndarray, bits: int) -> np.ndarray:
    e = np.asarray(edges).astype(np.int64) & ((1 << bits) - 1)
    states = np.zeros_like(e)
    for lag in range(math.ceil(16 / bits)):
        states |= np.roll(e, lag, axis=-1) << (lag * bits)
    return (states & 0xFFFF).astype(np.uint16).view(np.int16)


def unpack_trellis_states(packed: np.ndarray, bits: int) -> np.ndarray:
    return reconstruct_trellis_states(unpack_trellis_edges(packed, bits), bits)


def decode_states_e4m3(states: np.ndarray, lut: np.ndarray) -> np.ndarray:
    """The FP8 decode target: one raw E4M3 byte per weight, in tile (tensor-core) order."""

    return np.asarray(lut, dtype=np.uint8)[np.asarray(states).view(np.uint16).astype(np.int64)]


def decode_regularized_weight(states: np.ndarray, lut: np.ndarray) -> np.ndarray:
    """[K/16, N/16, 256] states -> transformed [K, N] float32 weight."""

    decoded = e4m3_to_float(decode_states_e4m3(states, lut)).astype(np.float32)
    return tiles_to_matrix(decoded)


@lru_cache(maxsize=None)
def normalized_hadamard(size: int = 128) -> np.ndarray:
    matrix = np.ones((1, 1), dtype=np.float32)
    while matrix.shape[0] < size:
        matrix = np.block([[matrix, matrix], [matrix, -matrix]])
    return (matrix * np.float32(1.0 / math.sqrt(size))).astype(np.float32)


def hadamard_left(weight: np.ndarray, block: int = 128) -> np.ndarray:
    """had @ W per block of `block` rows (exl3_encoder_backend.py:295-306)."""

    k, n = weight.shape
    had = normalized_hadamard(block)
    return np.matmul(had, weight.reshape(k // block, block, n)).reshape(k, n).astype(np.float32)


def hadamard_right(weight: np.ndarray, block: int = 128) -> np.ndarray:
    """W @ had per block of `block` columns (exl3_encoder_backend.py:309-320)."""

    k, n = weight.shape
    had = normalized_hadamard(block)
    return np.matmul(weight.reshape(k, n // block, block), had).reshape(k, n).astype(np.float32)


def decode_weight(states: np.ndarray, suh: np.ndarray, svh: np.ndarray, lut: np.ndarray) -> np.ndarray:
    """qsrt/exl3_reference.py:280-302: states + fp16 scales -> [K, N] float32 weight."""

    weight = decode_regularized_weight(states, lut)
    weight = hadamard_left(weight)
    weight = weight * suh.astype(np.float32)[:, None]
    weight = hadamard_right(weight)
    weight = weight * svh.astype(np.float32)[None, :]
    return weight.astype(np.float32)
