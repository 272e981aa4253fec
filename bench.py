"""Headline benchmark: MoE-layer trellis encode throughput (Mweights/s).

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched under torchrun)
    python bench.py --impl reference --steps K --warmup W  (CPU restatement of the same path)

One step = one pass of the whole hot path over a batch of synthetic experts of the full MoE
layer shape (hidden 7168, intermediate 2048, uniform K3): routed-row Hessians -> regularise /
Hadamard -> BlockLDLQ with the Viterbi tile search -> pack -> decode check -> routed error.
Every rank encodes its own experts (expert-wise sharding, weak scaling); with N > 1 the
per-expert (error, bytes) table is all-gathered each step, which is the path's only exchange.
Rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HIDDEN, INTER, EXPERTS, TOKENS, TOPK = 7168, 2048, 384, 65536, 8
BITS = 3
WEIGHTS_PER_EXPERT = 3 * HIDDEN * INTER
METRICS_PER_TILE = (256 + 2 * 128) * 65536  # branch metrics of one tile at tailbite context 128


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="b200", choices=["b200", "reference"])
    p.add_argument("--experts-per-step", type=int, default=4,
                   help="experts encoded together per GPU and step; 4 fills the 148-SM waves of every launch best")
    p.add_argument("--tokens", type=int, default=TOKENS)
    p.add_argument("--hidden", type=int, default=HIDDEN)
    p.add_argument("--inter", type=int, default=INTER)
    p.add_argument("--no-cpu-baseline", action="store_true")
    return p.parse_args()


# --------------------------------------------------------------------------------------
# reference arm: the CPU restatement, all host threads, bounded sample per step
# --------------------------------------------------------------------------------------

def cpu_sample_inputs(seed: int, k: int = 128, n: int = 128):
    import numpy as np

    rng = np.random.default_rng(seed)
    weight = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    x = (rng.standard_normal((1024, k)) * np.exp(0.5 * rng.standard_normal(k))).astype(np.float32)
    hessian = (x.T @ x / 1024).astype(np.float32)
    su = np.sign(rng.standard_normal(k)).astype(np.float32)
    sv = np.sign(rng.standard_normal(n)).astype(np.float32)
    return weight, hessian, su, sv


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import encoder_oracle as eo
    from oracle import qsrt_oracle as oracle

    oracle.build_c_oracle()
    cores = os.cpu_count() or 1
    oracle.DEFAULT_THREADS = cores  # torchrun exports OMP_NUM_THREADS=1
    lut = oracle.sqg_xor_cheb_t12_bytes(BITS)
    k, n = 128, 128
    times = []
    for step in range(args.warmup + args.steps):
        weight, hessian, su, sv = cpu_sample_inputs(9000 + step, k, n)
        t0 = time.perf_counter()
        eo.quantize_qsrt(weight, hessian, su, sv, lut=lut, bits=BITS, sigma_reg=0.025, context=128)
        dt = time.perf_counter() - t0
        if step >= args.warmup:
            times.append(dt)
    total = sum(times)
    value = args.steps * k * n / total / 1e6
    sample = (f"one [{k}x{n}] sub-block of a layer-shaped matrix per step through the full CPU restatement "
              "(Hessian factor, regularise, scale search, BlockLDLQ, Viterbi tiles, pack)")
    line = {
        "impl": "reference",
        "metric": "MoE-layer encode Mweights/s",
        "value": value,
        "unit": "Mweights/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f16",
        "data": "synthetic",
        "config": workload_config(args, args.experts_per_step),
        "cpu_baseline": {"value": value, "unit": "Mweights/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "Mweights/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, experts_per_gpu: int) -> dict:
    return {
        "workload": "full MoE layer shape, uniform K3 QSRT (BASELINE configs[2]), expert-wise shard: "
                    f"{experts_per_gpu} experts per GPU per step",
        "hidden": args.hidden,
        "intermediate": args.inter,
        "layer_experts": EXPERTS,
        "tokens": args.tokens,
        "routing": "top-8 Zipf(1.1)",
        "bits": BITS,
        "tailbite_context": 128,
        "sigma_reg": 0.025,
        "l2": "inputs larger than L2 (each expert streams > 1 GB of weights, Hessians and factors)",
        "parallelism": f"ep{args.gpus}",
    }


# --------------------------------------------------------------------------------------
# B200 arm
# --------------------------------------------------------------------------------------

class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        try:
            os.unlink(self.file.name)
        except OSError:
            pass
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(sm_max) if sm_max else None,
            "reasons": sorted(reasons),
            "samples": len(sm),
        }


def make_layer(args, device, expert_ids, seed=3000):
    """Synthetic stand-in for the MoE layer: tokens, Zipf(1.1) top-8 routing, expert weights."""

    import torch

    g = torch.Generator(device="cpu").manual_seed(seed + 1)
    gd = torch.Generator(device=device).manual_seed(seed + 1)
    tokens = torch.randn((args.tokens, args.hidden), generator=gd, dtype=torch.float32, device=device)
    freq = 1.0 / torch.arange(1, EXPERTS + 1, dtype=torch.float64) ** 1.1
    selected = torch.multinomial((freq / freq.sum()).float().expand(args.tokens, -1), TOPK, replacement=False, generator=g)
    gates = torch.softmax(torch.randn((args.tokens, TOPK), generator=g), dim=-1)
    experts = []
    for e in expert_ids:
        ge = torch.Generator(device="cpu").manual_seed(seed + e)
        w1 = torch.randn((args.inter, args.hidden), generator=ge) * 0.02
        w3 = torch.randn((args.inter, args.hidden), generator=ge) * 0.02
        w2 = torch.randn((args.hidden, args.inter), generator=ge) * 0.02
        hit = selected == e
        token_idx = hit.any(dim=1).nonzero().flatten()
        gate_e = (gates * hit).sum(dim=1)[token_idx].float()
        experts.append({"id": e, "w1": w1, "w3": w3, "w2": w2, "token_idx": token_idx, "gates": gate_e})
    return tokens, experts


def run_b200(args) -> None:
    import torch

    from qsrt_b200 import _lib, pipeline
    from qsrt_b200 import tiles as tile_api

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: there is no CPU fallback for the encoder kernels")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)

    per_gpu = args.experts_per_step
    stride = max(1, EXPERTS // (world * per_gpu))
    expert_ids = [(stride // 2 + (rank * per_gpu + i) * stride) % EXPERTS for i in range(per_gpu)]
    tokens, experts_cpu = make_layer(args, device, expert_ids)

    def to_sources(weights_on_device):
        out = []
        for meta, w in zip(experts_cpu, weights_on_device):
            idx = meta["token_idx"].to(device)
            out.append(pipeline.ExpertSource(w["w1"], w["w3"], w["w2"], tokens.index_select(0, idx),
                                             meta["gates"].to(device), meta["id"]))
        return out

    resident = [{k: m[k].to(device) for k in ("w1", "w3", "w2")} for m in experts_cpu]
    pinned = [{k: m[k].pin_memory() for k in ("w1", "w3", "w2")} for m in experts_cpu]

    def step(sources):
        payloads = pipeline.encode_expert_batch(sources, bits=BITS, device=device, layer_seed=1, score=True)
        for p in payloads:
            if not (pipeline.verify_payload_roundtrip(p.w1) and pipeline.verify_payload_roundtrip(p.w2)):
                raise RuntimeError("packed payload failed its decode round trip")
        table = torch.tensor([[p.routed_sse, float(p.payload_bytes)] for p in payloads], dtype=torch.float64, device=device)
        if dist is not None:
            gathered = [torch.empty_like(table) for _ in range(world)]
            dist.all_gather(gathered, table)
            table = torch.cat(gathered)
        return payloads, table

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    def timed(fn, steps):
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        end.record()
        barrier()
        ms = torch.tensor([start.elapsed_time(end)], dtype=torch.float64, device=device)
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    last = {}

    def resident_step():
        last["payloads"], last["table"] = step(to_sources(resident))

    d2h_bytes = [0]
    h2d_bytes = [0]

    def e2e_step():
        staged, nbytes = [], 0
        for w in pinned:
            dev = {k: v.to(device, non_blocking=True) for k, v in w.items()}
            nbytes += sum(v.numel() * 4 for v in w.values())
            staged.append(dev)
        sources = to_sources(staged)
        nbytes += sum(m["token_idx"].numel() * 8 + m["gates"].numel() * 4 for m in experts_cpu)
        payloads, table = step(sources)
        out_bytes = 0
        for p in payloads:
            for mp in (p.w1, p.w3, p.w2):
                for t in (mp.trellis, mp.suh, mp.svh):
                    host = t.to("cpu", non_blocking=False)
                    out_bytes += host.numel() * host.element_size()
        host_table = table.cpu()
        out_bytes += host_table.numel() * 8
        h2d_bytes[0], d2h_bytes[0] = nbytes, out_bytes

    for _ in range(max(args.warmup, 3)):
        resident_step()

    launches_before = _lib.kernel_launches()
    tile_api.search_timings = []
    base_event = torch.cuda.Event(enable_timing=True)
    base_event.record()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    total_ms = timed(resident_step, args.steps)
    clocks = sampler.stop() if rank == 0 else {}
    launches = _lib.kernel_launches() - launches_before
    torch.cuda.synchronize(device)
    # Search launches of independent recursions overlap on different streams: the kernel's
    # busy time is the union of the launch intervals, placed on one clock through a base event.
    intervals = sorted((base_event.elapsed_time(s), base_event.elapsed_time(e)) for s, e, _, _ in tile_api.search_timings)
    search_ms, cursor = 0.0, float("-inf")
    for begin, end in intervals:
        if end > cursor:
            search_ms += end - max(begin, cursor)
            cursor = end
    launch_ms_sum = sum(e - b for b, e in intervals)
    search_tiles = sum(n for _, _, n, _ in tile_api.search_timings)
    search_launches = len(tile_api.search_timings)
    tile_api.search_timings = None

    e2e_ms = timed(e2e_step, args.steps)

    # half2 FMA rate of this device, measured live (denominator of the Viterbi ALU roofline)
    sink = torch.zeros(1, device=device)
    import ctypes
    lanes = ctypes.c_double(0.0)
    best = None
    for _ in range(5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        _lib.check(_lib.lib().qsrtb_probe_half2_fma(200000, sink.data_ptr(), ctypes.byref(lanes),
                                                    ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)), "probe")
        b.record()
        torch.cuda.synchronize(device)
        ms = a.elapsed_time(b)
        best = ms if best is None else min(best, ms)
    fma_lanes_per_s = lanes.value / (best * 1e-3)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    weights_per_step = world * per_gpu * 3 * args.hidden * args.inter
    value = weights_per_step * args.steps / (total_ms * 1e-3) / 1e6
    e2e_value = weights_per_step * args.steps / (e2e_ms * 1e-3) / 1e6
    achieved = search_tiles * METRICS_PER_TILE / (search_ms * 1e-3) / 1e9 if search_ms > 0 else 0.0
    peak = fma_lanes_per_s / 3.0 / 1e9
    payload = last["payloads"][0]
    line = {
        "metric": "MoE-layer encode Mweights/s",
        "value": value,
        "unit": "Mweights/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": max(args.warmup, 3),
        "ms_per_step": total_ms / args.steps,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f16",
        "data": "synthetic",
        "config": workload_config(args, per_gpu),
        "e2e": {"value": e2e_value, "unit": "Mweights/s", "h2d_bytes_per_step": h2d_bytes[0],
                "d2h_bytes_per_step": d2h_bytes[0]},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {
            "bound": "alu",
            "kernel": "viterbi_kernel<3>",
            "achieved": achieved,
            "peak": peak,
            "unit": "G branch metrics/s",
            "frac": achieved / peak if peak > 0 else None,
            # DRAM bytes per launch: one ncu capture of this kernel on 592 tiles measured
            # 1 107.7 MB read + written = 1.871 MB per tile (the survivor rows); the traffic grows
            # in proportion to the tiles, so it is scaled to this run's average launch.
            "traffic": NCU_DRAM_BYTES_PER_TILE * search_tiles / max(search_launches, 1),
            "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of a 592-tile launch, scaled per tile",
            "algorithmic_dram_bytes_per_tile": 4 * 256 * 4 + 256 * 2,  # rows + compensation in, reconstruction + error + states out
            "peak_source": "live half2 FMA probe / 3 half ops per branch metric (MEASURED_PEAKS.json holds no ALU figure)",
            "launches": search_launches,
            "avg_launch_ms": launch_ms_sum / max(search_launches, 1),
            "busy_ms": search_ms,
            "tiles_per_s": search_tiles / (search_ms * 1e-3) if search_ms > 0 else 0.0,
            "share_of_step": search_ms / total_ms if total_ms > 0 else None,
        },
        "quality": {"expert": payload.expert_id, "proxy_w1": payload.w1.proxy, "proxy_w2": payload.w2.proxy,
                    "routed_rel_sse": payload.routed_sse / max(payload.routed_energy, 1e-30)},
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_tile_baseline(last["payloads"][0])
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def cpu_tile_baseline(payload) -> dict:
    """The C restatement of the tile search (OpenMP, all host cores) on a bounded sample of this
    workload's tiles: the regularised gate matrix's first rows of tiles, re-derived from the
    decoded payload so that the sample is shaped like real encoder input."""

    import numpy as np

    from oracle import qsrt_oracle as oracle
    from qsrt_b200 import codec, tables

    oracle.build_c_oracle()
    cores = os.cpu_count() or 1
    oracle.DEFAULT_THREADS = cores
    lut = tables.sqg_xor_cheb_t12_bytes(BITS)
    states = codec.unpack_trellis_states(payload.w1.trellis[:4], BITS)
    work = codec.decode_regularized_weight(states, lut=lut).cpu().numpy()
    rng = np.random.default_rng(5)
    tiles = oracle.matrix_to_tiles(work).reshape(-1, 256)
    tiles = (tiles + 0.25 * rng.standard_normal(tiles.shape)).astype(np.float32)  # undo quantisation roughly
    n = min(tiles.shape[0], 20 * cores)
    tiles = np.ascontiguousarray(tiles[:n])
    t0 = time.perf_counter()
    oracle.quantize_tiles(tiles, lut.numpy(), BITS, 128)
    dt = time.perf_counter() - t0
    return {
        "value": n * 256 / dt / 1e6,
        "unit": "Mweights/s",
        "cores": cores,
        "kind": "port",
        "sample": f"{n} K3 tiles (tailbite context 128) of this workload through the C restatement of the tile "
                  f"search only, OpenMP on {cores} threads, {dt:.1f} s",
    }


NCU_DRAM_BYTES_PER_TILE = (817.4e6 + 290.3e6) / 592


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
