"""Tile-encoder microbenchmark (kernel only), the counterpart of the reference's A/B harness
``scripts/benchmark_sqg_tile_encoder.py``: seeded tile families, K in {2,3,4}, CUDA-event timing.

    python -m qsrt_b200.bench_tiles --tiles 1184 --bits 3 --context 128 --family normal --iters 5
"""

from __future__ import annotations

import argparse
import json

import torch

from . import tables, tiles as tile_api

METRICS_PER_STEP = 65536


def make_tiles(family: str, count: int, seed: int) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn((count, 256), generator=g, dtype=torch.float32)
    if family == "scaled":
        x = x * torch.tensor([0.25, 0.5, 1.0, 2.0, 4.0])[torch.arange(count) % 5][:, None]
    elif family == "heavy":
        chi2 = torch.randn((count, 256, 3), generator=g).square().sum(-1)
        x = x * torch.rsqrt(chi2 / 3.0).clamp(max=1e3)
    elif family == "spike":
        x = torch.where(torch.rand((count, 256), generator=g) < 0.01, x * 100.0, x)
    elif family != "normal":
        raise ValueError(f"unknown tile family {family!r}")
    return x


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--tiles", type=int, default=148 * 8)
    p.add_argument("--bits", type=int, default=3)
    p.add_argument("--context", type=int, default=128)
    p.add_argument("--family", default="normal")
    p.add_argument("--iters", type=int, default=5)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--seed", type=int, default=20260816)
    p.add_argument("--units", type=int, default=0, help="work units per thread of the search kernel (0 auto, 1 or 2)")
    p.add_argument("--traceback", type=int, default=0,
                   help="what the kernel keeps for its traceback (0 its own choice, 1 decisions, 2 path costs)")
    args = p.parse_args()
    device = torch.device("cuda:0")
    x = make_tiles(args.family, args.tiles, args.seed).to(device)
    lut = tables.sqg_xor_cheb_t12_bytes(args.bits)
    for _ in range(args.warmup):
        tile_api.encode_tiles(x, lut, args.bits, args.context, units_per_thread=args.units, traceback=args.traceback)
    torch.cuda.synchronize()
    times = []
    for _ in range(args.iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        tile_api.encode_tiles(x, lut, args.bits, args.context, units_per_thread=args.units, traceback=args.traceback)
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    ms = sorted(times)[len(times) // 2]
    metrics = args.tiles * (256 + 2 * args.context) * METRICS_PER_STEP
    print(json.dumps({
        "tiles": args.tiles, "bits": args.bits, "context": args.context, "family": args.family, "units": args.units,
        "traceback": args.traceback, "median_ms": ms, "ktiles_per_s": args.tiles / ms, "mweights_per_s": args.tiles * 256 / ms / 1e3,
        "g_branch_metrics_per_s": metrics / ms / 1e6,
    }))


if __name__ == "__main__":
    main()
