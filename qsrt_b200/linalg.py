"""Dense float32 linear algebra of the encoder on the tensor cores.

Bindings of ``qsrtb_split_tf32``, ``qsrtb_gemm3x_tc`` and ``qsrtb_cholesky_blocked``
(``include/qsrt_b200.h``).  They stand in for the library calls the reference makes on this path:
``torch.linalg.cholesky`` inside ``block_ldl`` (qsrt/exl3_encoder_backend.py:335), the feedback
``addmm_`` / ``baddbmm`` of the BlockLDLQ recursion (:494-501, 533-534, 1170-1187) and the
``F.linear`` products of the routed scoring (qsrt/pooled_calibration.py:734-753).
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib


def _stream_ptr(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


class Planes:
    """TF32 head and tail of a stack of K-major matrices: ``hi + lo`` reproduces the float32
    source up to the tail's rounding (about 2^-22 relative)."""

    __slots__ = ("hi", "lo")

    def __init__(self, hi: torch.Tensor, lo: torch.Tensor) -> None:
        self.hi, self.lo = hi, lo

    @property
    def shape(self):
        return self.hi.shape


def _as_stack(x: torch.Tensor, what: str) -> torch.Tensor:
    if x.dtype != torch.float32 or not x.is_cuda:
        raise TypeError(f"{what} must be a CUDA float32 tensor")
    if x.ndim == 2:
        x = x.unsqueeze(0)
    if x.ndim != 3 or x.stride(2) != 1:
        raise ValueError(f"{what} must be a matrix or a stack of matrices with contiguous rows")
    return x


def split_tf32(x: torch.Tensor, *, transpose: bool = False, out: Planes | None = None) -> Planes:
    """Head / tail planes of ``x`` ([rows, cols] or a stack); with ``transpose`` the planes hold
    ``x^T``.  Rows may be strided (``x`` may be a slice of a wider matrix)."""

    squeeze = x.ndim == 2
    src = _as_stack(x, "split input")
    batch, rows, cols = src.shape
    shape = (batch, cols, rows) if transpose else (batch, rows, cols)
    if out is None:
        hi = torch.empty(shape, dtype=torch.float32, device=x.device)
        lo = torch.empty(shape, dtype=torch.float32, device=x.device)
    else:
        hi, lo = _as_stack(out.hi, "plane"), _as_stack(out.lo, "plane")
        if tuple(hi.shape) != shape or tuple(lo.shape) != shape:
            raise ValueError("output planes have the wrong shape")
        if hi.stride() != lo.stride():
            raise ValueError("head and tail planes must share their strides")
    with torch.cuda.device(x.device):
        _lib.check(
            _lib.lib().qsrtb_split_tf32(
                src.data_ptr(), batch, rows, cols, src.stride(1), src.stride(0) if batch > 1 else 0,
                hi.data_ptr(), lo.data_ptr(), hi.stride(1), hi.stride(0) if batch > 1 else 0,
                int(transpose), _stream_ptr(x.device)),
            "qsrtb_split_tf32")
    if out is not None:
        return out
    return Planes(hi[0], lo[0]) if squeeze else Planes(hi, lo)


_status: dict[tuple[str, int], torch.Tensor] = {}


def _status_word(device: torch.device) -> torch.Tensor:
    key = (str(device), torch.cuda.current_stream(device).cuda_stream)
    if key not in _status:
        _status[key] = torch.zeros(2, dtype=torch.int32, device=device)
    return _status[key]


def check_status(device: torch.device) -> None:
    """Host check (one synchronisation) of the bounded-wait status of the tensor-core products
    enqueued on the current stream of ``device`` since the last check."""

    word = _status_word(device)
    value = int(word[1].item())
    if value != 0:
        word.zero_()
        raise RuntimeError(f"a bounded wait inside a tensor-core kernel expired (status 0x{value & 0xffffffff:08x})")


def gemm_nt(a: Planes, b: Planes, out: torch.Tensor, *, alpha: float = 1.0, beta: float = 0.0,
            lower_only: bool = False, transposed_out: bool = False, k: int | None = None) -> torch.Tensor:
    """``out = alpha * A @ B^T + beta * out`` per matrix of the stack; ``A`` [m, k] and ``B`` [n, k]
    are given as planes, ``out`` is ``[m, n]`` (or ``[n, m]`` with ``transposed_out``).  Every
    operand may be a strided view as long as its rows are contiguous and 16-byte aligned."""

    a_hi, a_lo = _as_stack(a.hi, "A plane"), _as_stack(a.lo, "A plane")
    b_hi, b_lo = _as_stack(b.hi, "B plane"), _as_stack(b.lo, "B plane")
    d = _as_stack(out, "output")
    batch, m, ka = a_hi.shape
    _, n, kb = b_hi.shape
    k = min(ka, kb) if k is None else int(k)
    if b_hi.shape[0] != batch or d.shape[0] != batch:
        raise ValueError("operand stacks differ in length")
    if tuple(d.shape[1:]) != ((n, m) if transposed_out else (m, n)):
        raise ValueError("output shape does not match the product")
    if a_hi.stride() != a_lo.stride() or b_hi.stride() != b_lo.stride():
        raise ValueError("head and tail planes must share their strides")
    device = out.device
    status = _status_word(device)
    with torch.cuda.device(device):
        _lib.check(
            _lib.lib().qsrtb_gemm3x_tc(
                a_hi.data_ptr(), a_lo.data_ptr(), a_hi.stride(1), a_hi.stride(0) if batch > 1 else 0,
                b_hi.data_ptr(), b_lo.data_ptr(), b_hi.stride(1), b_hi.stride(0) if batch > 1 else 0,
                batch, m, n, k, d.data_ptr(), d.stride(1), d.stride(0) if batch > 1 else 0,
                float(alpha), float(beta), int(lower_only), int(transposed_out),
                None, status[1:].data_ptr(), _stream_ptr(device)),
            "qsrtb_gemm3x_tc")
    return out


def matmul_nt(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` in float32 accuracy on the tensor cores (the ``F.linear`` of the scoring path)."""

    out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
    return gemm_nt(split_tf32(x.contiguous()), split_tf32(w.contiguous()), out)


_chol_workspace: dict[tuple[str, int, int], torch.Tensor] = {}


def cholesky_(matrix: torch.Tensor) -> int:
    """In-place lower Cholesky factor of a symmetric float32 matrix (its lower triangle is read).

    Returns LAPACK's ``info``: 0, or the 1-based column of the first pivot that was not positive
    (the matrix contents are then undefined).  The strict upper triangle is scratch.  One host
    synchronisation (reading the status word), as ``torch.linalg.cholesky_ex(...).info.item()``."""

    if matrix.dtype != torch.float32 or not matrix.is_cuda or matrix.ndim != 2 or matrix.shape[0] != matrix.shape[1]:
        raise TypeError("Cholesky input must be a square CUDA float32 matrix")
    if matrix.stride(1) != 1:
        raise ValueError("Cholesky input must have contiguous rows")
    n = matrix.shape[0]
    if n == 0:
        return 0
    device = matrix.device
    key = (str(device), torch.cuda.current_stream(device).cuda_stream, n)
    work = _chol_workspace.get(key)
    if work is None:
        wanted = ctypes.c_size_t(0)
        _lib.check(_lib.lib().qsrtb_cholesky_workspace_bytes(n, ctypes.byref(wanted)), "qsrtb_cholesky_workspace_bytes")
        work = torch.empty(wanted.value, dtype=torch.uint8, device=device)
        _chol_workspace[key] = work
    status = torch.zeros(2, dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        _lib.check(
            _lib.lib().qsrtb_cholesky_blocked(matrix.data_ptr(), n, matrix.stride(0), work.data_ptr(), work.numel(),
                                              status.data_ptr(), _stream_ptr(device)),
            "qsrtb_cholesky_blocked")
    info, waited = status.tolist()
    if waited != 0:
        raise RuntimeError(f"a bounded wait inside the Cholesky update expired (status 0x{waited & 0xffffffff:08x})")
    return int(info)
