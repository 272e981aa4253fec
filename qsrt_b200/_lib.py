"""ctypes binding of ``libqsrt_b200.so`` (the C ABI declared in ``include/qsrt_b200.h``).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes
from functools import lru_cache
from pathlib import Path

LIBRARY = Path(__file__).resolve().parent / "libqsrt_b200.so"

OK = 0
EINVAL, ESCRATCH, ECUDA, ENOTPD = -1, -2, -3, -4

_c = ctypes
_PTR = _c.c_void_p
_SIGNATURES = {
    "qsrtb_abi_version": (_c.c_int, []),
    "qsrtb_last_error": (_c.c_char_p, []),
    "qsrtb_probe_half2_fma": (_c.c_int, [_c.c_int, _PTR, _c.POINTER(_c.c_double), _PTR]),
    "qsrtb_lut_prepare": (_c.c_int, [_PTR, _c.c_int, _PTR, _PTR, _PTR]),
    "qsrtb_viterbi_scratch_bytes": (_c.c_int, [_c.c_int, _c.c_int64, _c.POINTER(_c.c_size_t)]),
    "qsrtb_viterbi_cost_scratch_bytes": (_c.c_int, [_c.c_int, _c.c_int64, _c.POINTER(_c.c_size_t)]),
    "qsrtb_quantize_tiles": (
        _c.c_int,
        [_PTR, _c.c_int64, _PTR, _PTR, _c.c_int, _c.c_int, _c.c_int, _PTR, _PTR, _PTR, _c.c_size_t, _PTR],
    ),
    "qsrtb_quantize_tiles_static": (
        _c.c_int,
        [_PTR, _c.c_int64, _PTR, _PTR, _c.c_int, _c.c_int, _c.c_int, _PTR, _PTR, _PTR],
    ),
    "qsrtb_ldlq_quantize_rows": (
        _c.c_int,
        [_PTR, _PTR, _c.c_float, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int64, _c.c_int64,
         _PTR, _PTR, _c.c_int, _c.c_int, _c.c_int, _PTR, _PTR, _PTR, _c.c_int64, _PTR, _c.c_int,
         _PTR, _c.c_size_t, _PTR],
    ),
    "qsrtb_ldlq_quantize_members": (
        _c.c_int,
        [_PTR, _PTR, _c.c_float, _PTR, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int64, _c.c_int64,
         _PTR, _PTR, _c.c_int, _c.c_int, _c.c_int, _PTR, _PTR, _PTR, _c.c_int64, _PTR, _c.c_int,
         _PTR, _c.c_size_t, _PTR],
    ),
    "qsrtb_hessian_accumulate": (
        _c.c_int, [_PTR, _PTR, _c.c_int64, _c.c_int, _c.c_int, _PTR, _c.c_int, _c.c_int, _PTR]
    ),
    "qsrtb_hessian_tc_workspace_bytes": (_c.c_int, [_c.c_int64, _c.c_int, _c.POINTER(_c.c_size_t)]),
    "qsrtb_hessian_accumulate_tc": (
        _c.c_int,
        [_PTR, _PTR, _c.c_int64, _c.c_int, _c.c_int, _PTR, _c.c_int, _c.c_int, _PTR, _c.c_size_t, _PTR, _PTR],
    ),
    "qsrtb_hessian_tc_wait_probe": (_c.c_int, [_PTR, _PTR]),
    "qsrtb_gemm3x_tc": (
        _c.c_int,
        [_PTR, _PTR, _c.c_int, _c.c_int64, _PTR, _PTR, _c.c_int, _c.c_int64, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
         _PTR, _c.c_int, _c.c_int64, _c.c_float, _c.c_float, _c.c_int, _c.c_int, _PTR, _PTR, _PTR],
    ),
    "qsrtb_split_tf32": (
        _c.c_int,
        [_PTR, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int64, _PTR, _PTR, _c.c_int, _c.c_int64, _c.c_int, _PTR],
    ),
    "qsrtb_gated_activation": (
        _c.c_int, [_PTR, _c.c_int64, _c.c_int, _c.c_int, _c.c_int, _PTR, _PTR, _c.c_int, _PTR, _c.c_int, _PTR]),
    "qsrtb_routed_row_sse": (
        _c.c_int, [_PTR, _PTR, _c.c_int64, _c.c_int, _c.c_int, _c.c_int, _PTR, _PTR, _PTR]),
    "qsrtb_cholesky_workspace_bytes": (_c.c_int, [_c.c_int, _c.POINTER(_c.c_size_t)]),
    "qsrtb_cholesky_blocked": (_c.c_int, [_PTR, _c.c_int, _c.c_int, _PTR, _c.c_size_t, _PTR, _PTR]),
    "qsrtb_hessian_finish": (_c.c_int, [_PTR, _c.c_int, _c.c_int, _c.c_double, _PTR]),
    "qsrtb_hadamard128": (
        _c.c_int,
        [_PTR, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int64, _c.c_int, _PTR, _c.c_int64,
         _c.c_int, _c.c_int, _c.c_int, _PTR, _c.c_int64, _PTR],
    ),
    "qsrtb_signed_block_hadamard": (
        _c.c_int, [_PTR, _c.c_int64, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _PTR, _c.c_int, _PTR]
    ),
    "qsrtb_mxfp4_signed_block_hadamard": (
        _c.c_int, [_PTR, _PTR, _c.c_int64, _c.c_int, _PTR, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _PTR, _c.c_int, _PTR]
    ),
    "qsrtb_col_sumsq": (
        _c.c_int,
        [_PTR, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int64, _PTR, _c.c_int64, _PTR,
         _c.c_size_t, _PTR],
    ),
    "qsrtb_block_ldl_normalize": (_c.c_int, [_PTR, _c.c_int, _c.c_int, _PTR]),
    "qsrtb_pack_trellis": (_c.c_int, [_PTR, _c.c_int64, _c.c_int, _PTR, _PTR]),
    "qsrtb_mxfp4_dequant": (_c.c_int, [_PTR, _PTR, _c.c_int, _c.c_int, _PTR, _c.c_int, _c.c_int, _PTR]),
    "qsrtb_tile_reduce": (_c.c_int, [_PTR, _PTR, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _PTR, _PTR]),
    "qsrtb_refine_select": (
        _c.c_int,
        [_PTR, _c.c_int, _PTR, _c.c_int, _PTR, _c.c_int, _c.c_int, _PTR, _c.c_int, _c.c_int64, _c.c_int,
         _PTR, _c.c_int64, _PTR, _PTR, _c.c_int, _PTR, _PTR, _c.c_int, _PTR, _c.c_int, _c.c_double,
         _c.c_double, _c.c_int, _PTR, _PTR],
    ),
    "qsrtb_pack_records": (
        _c.c_int,
        [_PTR, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _PTR, _c.c_int, _c.c_int, _c.c_int64,
         _PTR, _c.c_int64, _PTR, _PTR],
    ),
    "qsrtb_unpack_records": (
        _c.c_int,
        [_PTR, _c.c_int64, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _PTR, _c.c_int, _c.c_int,
         _c.c_int64, _PTR, _PTR, _PTR],
    ),
    "qsrtb_records_atoms": (
        _c.c_int,
        [_PTR, _c.c_int64, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _PTR, _c.c_int, _c.c_int64,
         _PTR, _c.c_int64, _c.c_int, _PTR],
    ),
    "qsrtb_states_to_matrix": (_c.c_int, [_PTR, _c.c_int, _c.c_int, _PTR, _PTR, _c.c_int, _PTR]),
    "qsrtb_unpack_decode": (_c.c_int, [_PTR, _c.c_int64, _c.c_int, _PTR, _PTR, _PTR, _PTR]),
}


def exported_symbols() -> tuple[str, ...]:
    return tuple(_SIGNATURES)


# Kernel launches issued by one call of each entry point (0 = host only).
_KERNELS_PER_CALL = {
    "qsrtb_abi_version": 0,
    "qsrtb_last_error": 0,
    "qsrtb_viterbi_scratch_bytes": 0,
    "qsrtb_viterbi_cost_scratch_bytes": 0,
    "qsrtb_hessian_tc_workspace_bytes": 0,
    "qsrtb_cholesky_workspace_bytes": 0,
    # per 128-column panel: diagonal block, rows below it, trailing update (the last has only the first)
    "qsrtb_cholesky_blocked": lambda args: max(0, 3 * ((int(args[1]) + 127) // 128) - 2),
    "qsrtb_hessian_accumulate_tc": 2,
    "qsrtb_col_sumsq": 2,
    "qsrtb_block_ldl_normalize": 3,
    "qsrtb_signed_block_hadamard": 1,
}
launch_counts: dict[str, int] = {}


def kernel_launches() -> int:
    """Kernels of this library launched so far by this process."""

    return sum(launch_counts.values())


class _Counted:
    """The loaded library with per-entry-point launch accounting."""

    def __init__(self, handle: ctypes.CDLL) -> None:
        self._handle = handle
        for name in _SIGNATURES:
            setattr(self, name, self._wrap(name, getattr(handle, name)))

    @staticmethod
    def _wrap(name, fn):
        per_call = _KERNELS_PER_CALL.get(name, 1)
        if per_call == 0:
            return fn

        def counted(*args):
            launch_counts[name] = launch_counts.get(name, 0) + (per_call(args) if callable(per_call) else per_call)
            return fn(*args)

        return counted


@lru_cache(maxsize=1)
def lib() -> "_Counted":
    if not LIBRARY.exists():
        raise RuntimeError(
            f"{LIBRARY} is missing: build it with `python -m qsrt_b200.build` "
            "(there is no CPU or PyTorch fallback for the encoder kernels)"
        )
    handle = ctypes.CDLL(str(LIBRARY))
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(handle, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return _Counted(handle)


def check(status: int, what: str) -> None:
    if status == OK:
        return
    message = lib().qsrtb_last_error().decode("utf-8", "replace")
    text = f"{what} failed (status {status}): {message}"
    if status == EINVAL:
        raise ValueError(text)
    raise RuntimeError(text)
