"""CPU restatement (numpy) of the MXFP4 source dequantiser.  TEST INFRASTRUCTURE ONLY.

Follows qsrt/io/mxfp4.py:19-63 and the E2M1 table of qsrt/constants.py:68-74.  Pinned:
tests/golden/mxfp4_golden.json holds SHA-256 digests of the reference's own `dequant` outputs
for seeded inputs (generator: tests/golden/make_mxfp4_golden.py).
"""

from __future__ import annotations

import numpy as np

E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
                dtype=np.float32)


def seeded_source(rows: int, cols: int, seed: int, *, corner_cases: bool = False):
    """Codes uniform over 0..15; E8M0 byte = 127 + round(N(-6, 1)) per 32 inputs."""

    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 16, size=(rows, cols), dtype=np.uint8)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    scale = np.clip(127 + np.rint(rng.normal(-6.0, 1.0, size=(rows, cols // 32))), 0, 255).astype(np.uint8)
    if corner_cases:
        scale[0, 0] = 0      # 2^-127, a float32 subnormal
        scale[1, 0] = 255    # +inf: code 0 * inf = NaN
        scale[2, 0] = 254
        scale[3, 0] = 1
    return packed, scale


def dequant(packed: np.ndarray, scale: np.ndarray) -> np.ndarray:
    codes = np.empty((packed.shape[0], packed.shape[1] * 2), dtype=np.uint8)
    codes[:, 0::2] = packed & 0x0F
    codes[:, 1::2] = packed >> 4
    values = E2M1[codes]
    with np.errstate(over="ignore", invalid="ignore"):
        # exact powers of two (numpy's float32 exp2 is off by an ulp near 2^127)
        factors = np.ldexp(np.float32(1.0), scale.astype(np.int32) - 127).astype(np.float32)
        out = values.reshape(packed.shape[0], -1, 32) * factors[:, :, None]
    return out.reshape(packed.shape[0], -1).astype(np.float32)
