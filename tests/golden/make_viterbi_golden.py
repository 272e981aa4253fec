"""Generate tests/golden/viterbi_golden.npz ON A GPU BOX from the unmodified reference kernel.

Run (from the repository root, after `python oracle/build_ref.py` produced oracle/_ref):
    python tests/golden/make_viterbi_golden.py [output.npz]
The file holds, for K in {2,3,4} x tailbite context in {1,32,128}, the 16-bit states the
reference CUDA extension emits for 8 seeded tiles of each input family plus the structural
rows; inputs are regenerated from the seeds by tests/helpers.py, so only states are stored.
"""

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from qsrt_b200 import tables  # noqa: E402
from tests import helpers  # noqa: E402

SEED = 424242


def main(out_path: str) -> None:
    device = torch.device("cuda:0")
    tiles = helpers.mixed_tiles(8, SEED).to(device)
    arrays = {"seed": np.int64(SEED), "per_family": np.int64(8)}
    for bits in (2, 3, 4):
        lut = tables.sqg_xor_cheb_t12_bytes(bits)
        for context in (1, 32, 128):
            _, idx = helpers.reference_quantize_tiles(tiles, lut, bits, context)
            arrays[f"states_k{bits}_c{context}"] = idx.cpu().numpy()
    np.savez_compressed(out_path, **arrays)
    print("wrote", out_path, {k: getattr(v, "shape", None) for k, v in arrays.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else str(ROOT / "tests" / "golden" / "viterbi_golden.npz"))
