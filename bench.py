"""Headline benchmark: MoE-layer trellis encode throughput (Mweights/s).

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched under torchrun)
    python bench.py --impl reference --steps K --warmup W  (CPU restatement of the same path)
    python bench.py --config c4|c5 [--layer-experts E]     (non-headline layer configurations)

One step = one pass of the whole hot path over a group of distinct experts of the synthetic MoE
layer (hidden 7168, intermediate 2048, uniform K3): routed-row Hessians -> regularise / Hadamard
-> BlockLDLQ with the Viterbi tile search -> pack -> decode check -> routed error.  The layer's
384 experts are sharded over the ranks by routed-row count (``selection.assign_experts``); step
``i`` encodes the ``i``-th group of this rank's shard with its own routed rows and Hessians, so
``ceil(shard / experts-per-step)`` consecutive steps are one pass over the layer, reported as
``full_layer_s`` when the timed steps cover it.  With N > 1 the per-expert (error, bytes) table is
all-gathered each step (the path's only exchange), overlapped with the next step.  Rank 0 prints
one JSON line.
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

TOPK = 8
METRICS_PER_TILE = (256 + 2 * 128) * 65536  # branch metrics of one tile at tailbite context 128
HALF_LANES_PER_SM_CLOCK = 128               # 64 HFMA2 threads per clock and SM, two half lanes each

CONFIGS = {
    # name: hidden, intermediate, experts, tokens, Zipf exponent, bits, what
    "c3": dict(hidden=7168, inter=2048, experts=384, tokens=65536, zipf=1.1, bits=3,
               what="full MoE layer, uniform K3 QSRT (third configuration of the baseline file)"),
    "c4": dict(hidden=6144, inter=2048, experts=256, tokens=32768, zipf=1.2, bits=2,
               what="coupled-Hadamard two-bit layer: gate/up encoded first, down against the covariance of the "
                    "reconstructed activations (fourth configuration of the baseline file)"),
    "c5": dict(hidden=7168, inter=2048, experts=384, tokens=65536, zipf=1.1, bits=3,
               what="mixed-rate candidate selection: every expert at K2, K3 and K4, all-gathered routed errors, "
                    "equal-byte K2<->K4 exchange under 3.083333 bpw, decode check (fifth configuration of the "
                    "baseline file)"),
}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=3,
                   help="timed steps; 0 = one full pass over this rank's shard of the layer")
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="b200", choices=["b200", "reference"])
    p.add_argument("--config", default="c3", choices=sorted(CONFIGS))
    p.add_argument("--experts-per-step", type=int, default=6,
                   help="experts encoded together per GPU and step: more tiles per search launch, so the two "
                        "decision passes per CTA and launch weigh less (4: 65.5, 6: 67.3, 8: 68.3 Mweights/s)")
    p.add_argument("--layer-experts", type=int, default=0, help="override the layer's expert count (0 = the configuration's)")
    p.add_argument("--tokens", type=int, default=0)
    p.add_argument("--hidden", type=int, default=0)
    p.add_argument("--inter", type=int, default=0)
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-reference-gpu", action="store_true")
    p.add_argument("--no-e2e", action="store_true",
                   help="skip the end-to-end leg (for long non-headline runs such as a full pass of --config c4)")
    args = p.parse_args()
    cfg = CONFIGS[args.config]
    args.hidden = args.hidden or cfg["hidden"]
    args.inter = args.inter or cfg["inter"]
    args.tokens = args.tokens or cfg["tokens"]
    args.layer_experts = args.layer_experts or cfg["experts"]
    args.bits = cfg["bits"]
    args.zipf = cfg["zipf"]
    return args


def workload_config(args, experts_per_gpu: int) -> dict:
    cfg = CONFIGS[args.config]
    return {
        "workload": f"{cfg['what']}; expert-wise shard, {experts_per_gpu} distinct experts per GPU per step",
        "name": args.config,
        "hidden": args.hidden,
        "intermediate": args.inter,
        "layer_experts": args.layer_experts,
        "tokens": args.tokens,
        "routing": f"top-{TOPK} Zipf({args.zipf})",
        "bits": args.bits if args.config != "c5" else [2, 3, 4],
        "tailbite_context": 128,
        "sigma_reg": 0.025,
        "l2": "inputs larger than L2 (each expert streams > 1 GB of weights, Hessians and factors)",
        "parallelism": f"ep{args.gpus}",
    }


# --------------------------------------------------------------------------------------
# CPU arm: the restatement of the whole path, all host threads, bounded sample per step
# --------------------------------------------------------------------------------------

CPU_BLOCK = (128, 128)   # [in, out] sub-block of a layer-shaped matrix encoded per CPU step
CPU_ROWS = 1024


def cpu_sample_inputs(seed: int, k: int, n: int):
    import numpy as np

    rng = np.random.default_rng(seed)
    weight = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    x = (rng.standard_normal((CPU_ROWS, k)) * np.exp(0.5 * rng.standard_normal(k))).astype(np.float32)
    hessian = (x.T @ x / CPU_ROWS).astype(np.float32)
    su = np.sign(rng.standard_normal(k)).astype(np.float32)
    sv = np.sign(rng.standard_normal(n)).astype(np.float32)
    return weight, hessian, su, sv


def cpu_end_to_end(steps: int, warmup: int, bits: int):
    """Times the CPU restatement of the path (Hessian factor, regularise, scale search, BlockLDLQ
    with the C tile search on every host thread, pack) on one sub-block per step."""

    from oracle import encoder_oracle as eo
    from oracle import qsrt_oracle as oracle

    oracle.build_c_oracle()
    cores = os.cpu_count() or 1
    oracle.DEFAULT_THREADS = cores  # torchrun exports OMP_NUM_THREADS=1
    lut = oracle.sqg_xor_cheb_t12_bytes(bits)
    k, n = CPU_BLOCK
    times = []
    for step in range(warmup + steps):
        weight, hessian, su, sv = cpu_sample_inputs(9000 + step, k, n)
        t0 = time.perf_counter()
        eo.quantize_qsrt(weight, hessian, su, sv, lut=lut, bits=bits, sigma_reg=0.025, context=128)
        dt = time.perf_counter() - t0
        if step >= warmup:
            times.append(dt)
    total = sum(times)
    sample = (f"one [{k}x{n}] sub-block (in x out) of a layer-shaped matrix with a {CPU_ROWS}-row synthetic Hessian per "
              f"step through the CPU restatement of the whole path (Hessian factor, regularise, scale search, BlockLDLQ, "
              f"Viterbi tiles in C on {cores} threads, pack); {steps} steps in {total:.1f} s; the layer figure is "
              f"this rate extrapolated, the sub-block's recursion being 56x shorter than a 7168-row matrix's")
    return steps * k * n / total / 1e6, total, cores, sample


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    value, total, cores, sample = cpu_end_to_end(args.steps or 1, args.warmup, args.bits)
    steps = args.steps or 1
    config = workload_config(args, args.experts_per_step)
    config["workload"] = (f"bounded CPU sample of: {config['workload']} -- measured: one {CPU_BLOCK[0]}x{CPU_BLOCK[1]} "
                          f"sub-block with a {CPU_ROWS}-row synthetic Hessian per step, CPU restatement")
    config["sample"] = {"block_in_out": list(CPU_BLOCK), "hessian_rows": CPU_ROWS, "extrapolated_to_layer": True}
    line = {
        "impl": "reference",
        "metric": "MoE-layer encode Mweights/s",
        "value": value,
        "unit": "Mweights/s",
        "n_gpus": args.gpus,
        "steps": steps,
        "warmup": args.warmup,
        "ms_per_step": 1e3 * total / steps,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f16",
        "data": "synthetic",
        "config": config,
        "cpu_baseline": {"value": value, "unit": "Mweights/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "Mweights/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


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


class Layer:
    """Synthetic stand-in for the MoE layer: resident tokens, Zipf top-8 routing, expert weights
    drawn on the device from a per-expert seed (kept resident once drawn)."""

    def __init__(self, args, device, seed: int = 3000) -> None:
        import torch

        self.args, self.device, self.seed = args, device, seed
        g = torch.Generator(device="cpu").manual_seed(seed + 1)
        gd = torch.Generator(device=device).manual_seed(seed + 1)
        self.tokens = torch.randn((args.tokens, args.hidden), generator=gd, dtype=torch.float32, device=device)
        freq = 1.0 / torch.arange(1, args.layer_experts + 1, dtype=torch.float64) ** args.zipf
        self.selected = torch.multinomial((freq / freq.sum()).float().expand(args.tokens, -1), TOPK, replacement=False,
                                          generator=g)
        self.gates = torch.softmax(torch.randn((args.tokens, TOPK), generator=g), dim=-1)
        self.row_counts = torch.bincount(self.selected.flatten(), minlength=args.layer_experts).tolist()
        self._weights: dict[int, dict] = {}
        self._routes: dict[int, tuple] = {}

    def weights(self, expert: int) -> dict:
        import torch

        if expert not in self._weights:
            a = self.args
            ge = torch.Generator(device=self.device).manual_seed(self.seed + 17 * expert + 5)

            def draw(shape):
                if a.config == "c4":
                    # Student-t(5) * 0.015, stored as bf16 like the checkpoint the configuration describes
                    z = torch.randn(shape, generator=ge, device=self.device)
                    chi = torch.randn((*shape, 5), generator=ge, device=self.device).square().sum(-1)
                    return (0.015 * z * torch.rsqrt(chi / 5.0)).to(torch.bfloat16).float()
                return torch.randn(shape, generator=ge, device=self.device) * 0.02

            self._weights[expert] = {"w1": draw((a.inter, a.hidden)), "w3": draw((a.inter, a.hidden)),
                                     "w2": draw((a.hidden, a.inter))}
        return self._weights[expert]

    def route(self, expert: int):
        if expert not in self._routes:
            hit = self.selected == expert
            token_idx = hit.any(dim=1).nonzero().flatten()
            gate_e = (self.gates * hit).sum(dim=1)[token_idx].float()
            self._routes[expert] = (token_idx.to(self.device), gate_e.to(self.device))
        return self._routes[expert]

    def source(self, expert: int, weights: dict | None = None):
        from qsrt_b200 import pipeline

        w = self.weights(expert) if weights is None else weights
        idx, gates = self.route(expert)
        return pipeline.ExpertSource(w["w1"], w["w3"], w["w2"], self.tokens.index_select(0, idx), gates, expert)


class LazySources:
    """Sequence of ``ExpertSource`` built on demand (only the slice in use holds its routed rows)."""

    def __init__(self, layer: Layer, experts: list[int]) -> None:
        self.layer, self.experts = layer, experts

    def __len__(self) -> int:
        return len(self.experts)

    def __getitem__(self, key):
        if isinstance(key, slice):
            return [self.layer.source(e) for e in self.experts[key]]
        return self.layer.source(self.experts[key])


def run_b200(args) -> None:
    import torch

    from qsrt_b200 import _lib, pipeline, selection
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

    layer = Layer(args, device)
    shard = selection.assign_experts(layer.row_counts, world)[rank]
    per_gpu = args.experts_per_step
    # Groups are dealt from the shard sorted by routed rows, so that every step holds experts from
    # each part of the Zipf-skewed row distribution and costs about the same (a few leading steps
    # are then representative of the whole pass).
    by_rows = sorted(shard, key=lambda e: (-layer.row_counts[e], e))
    count = (len(shard) + per_gpu - 1) // per_gpu
    chunks = [by_rows[q * count:(q + 1) * count] for q in range(per_gpu)]   # dealt back and forth
    groups = [sorted(c[g] if q % 2 == 0 else c[len(c) - 1 - g] for q, c in enumerate(chunks) if g < len(c))
              for g in range(count)]
    steps = args.steps if args.steps > 0 else len(groups)
    warmup = max(args.warmup, 3) if args.config == "c3" else max(args.warmup, 1)
    weights_per_expert = 3 * args.hidden * args.inter

    if args.config == "c5":
        run_mixed_layer(args, layer, shard, device, dist, world, rank)
        return

    encode_kwargs = dict(bits=args.bits, device=device, layer_seed=1, score=True)
    if args.config == "c4":
        from qsrt_b200 import coupled

        encode_kwargs.update(coupled_spec=coupled.CoupledHadamardSpec(), down_from_reconstruction=True)

    def group_of(step_index: int) -> list[int]:
        return groups[step_index % len(groups)]

    pending = {}

    def finish_gather():
        handle = pending.pop("handle", None)
        if handle is not None:
            handle.wait()

    def step(sources):
        payloads = pipeline.encode_expert_batch(sources, **encode_kwargs)
        for p in payloads:
            if not (pipeline.verify_payload_roundtrip(p.w1) and pipeline.verify_payload_roundtrip(p.w2)):
                raise RuntimeError("packed payload failed its decode round trip")
        table = torch.tensor([[p.routed_sse, float(p.payload_bytes)] for p in payloads], dtype=torch.float64, device=device)
        if dist is not None:
            # the exchange of step i is waited for at the start of step i + 1's exchange
            finish_gather()
            pending["out"] = [torch.empty_like(table) for _ in range(world)]
            pending["handle"] = dist.all_gather(pending["out"], table, async_op=True)
        return payloads, table

    def barrier():
        finish_gather()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    last = {}
    marks: list = []

    def timed(fn, count, first_index=0):
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        marks.clear()
        start.record()
        for i in range(count):
            fn(first_index + i)
            mark = torch.cuda.Event(enable_timing=True)
            mark.record()
            marks.append(mark)
        finish_gather()
        end.record()
        barrier()
        per_step = [start.elapsed_time(m) for m in marks]
        ms = torch.tensor([start.elapsed_time(end)], dtype=torch.float64, device=device)
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), per_step

    def resident_step(index):
        last["payloads"], last["table"] = step([layer.source(e) for e in group_of(index)])

    # warm-up on the groups at the end of the shard, so that the timed steps start at group 0;
    # every expert the timed region touches is drawn (resident in HBM) before the clock starts
    for i in range(warmup):
        resident_step(len(groups) - 1 - (i % len(groups)))
    for i in range(steps):
        for e in group_of(i):
            layer.weights(e)
            layer.route(e)

    launches_before = _lib.kernel_launches()
    tile_api.search_timings = []
    base_event = torch.cuda.Event(enable_timing=True)
    base_event.record()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    total_ms, per_step = timed(resident_step, steps)
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

    # one pass over the layer = the first len(groups) steps of the timed region
    pass_ms = per_step[len(groups) - 1] if steps >= len(groups) else None
    pass_info = torch.tensor([pass_ms if pass_ms is not None else -1.0, per_step[-1]], dtype=torch.float64, device=device)
    if dist is not None:
        gathered = [torch.empty_like(pass_info) for _ in range(world)]
        dist.all_gather(gathered, pass_info)
        pass_table = torch.stack(gathered).cpu()
    else:
        pass_table = pass_info.cpu().unsqueeze(0)

    # end to end: the step's expert weights come from pinned host memory, the payload goes back
    pool = 0 if args.no_e2e else min(steps, len(groups), 3)
    pinned = {e: {k: v.cpu().pin_memory() for k, v in layer.weights(e).items()} for g in range(pool) for e in groups[g]}
    d2h_bytes, h2d_bytes = [0], [0]

    def e2e_step(index):
        experts = groups[index % pool]
        sources, nbytes = [], 0
        for e in experts:
            staged = {k: v.to(device, non_blocking=True) for k, v in pinned[e].items()}
            nbytes += sum(v.numel() * 4 for v in pinned[e].values())
            idx, gates = layer.route(e)
            nbytes += idx.numel() * 8 + gates.numel() * 4
            sources.append(layer.source(e, staged))
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

    e2e_ms = float("nan") if args.no_e2e else timed(e2e_step, steps)[0]

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

    experts_done = sum(len(group_of(i)) for i in range(steps))
    weights_done = world * experts_done * weights_per_expert
    value = weights_done / (total_ms * 1e-3) / 1e6
    e2e_value = weights_done / (e2e_ms * 1e-3) / 1e6
    achieved = search_tiles * METRICS_PER_TILE / (search_ms * 1e-3) / 1e9 if search_ms > 0 else 0.0
    peak = fma_lanes_per_s / 3.0 / 1e9
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    sm_mhz = clocks.get("sm_mhz") or clocks.get("sm_max_mhz") or 0.0
    nominal = sms * sm_mhz * 1e6 * HALF_LANES_PER_SM_CLOCK / 3.0 / 1e9
    payload = last["payloads"][0]
    pass_values = [float(v) for v in pass_table[:, 0]]
    layer_pass = {
        "groups_per_rank": len(groups),
        "experts_per_rank": len(shard),
        "steps_timed": steps,
        "covers_layer": steps >= len(groups),
        "rank_pass_s": [v / 1e3 for v in pass_values] if steps >= len(groups) else None,
        "step_ms": [round(b - a, 1) for a, b in zip([0.0] + per_step[:-1], per_step)],
        "step_rows": [sum(layer.row_counts[e] for e in group_of(i)) for i in range(steps)],
    }
    line = {
        "metric": "MoE-layer encode Mweights/s",
        "value": value,
        "unit": "Mweights/s",
        "n_gpus": world,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": total_ms / steps,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f16",
        "data": "synthetic",
        "config": workload_config(args, per_gpu),
        "full_layer_s": max(pass_values) / 1e3 if steps >= len(groups) else None,
        "layer_pass": layer_pass,
        "e2e": None if args.no_e2e else {"value": e2e_value, "unit": "Mweights/s", "h2d_bytes_per_step": h2d_bytes[0],
                "d2h_bytes_per_step": d2h_bytes[0],
                "note": f"weights of {pool} distinct expert groups staged in pinned host memory, cycled over the steps"},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {
            "bound": "alu",
            "kernel": SEARCH_KERNEL[args.bits],
            "achieved": achieved,
            "peak": peak,
            "unit": "G branch metrics/s",
            "frac": achieved / peak if peak > 0 else None,
            # DRAM bytes per launch: one ncu capture of this kernel measured the bytes read + written
            # per tile below (survivor decisions and, at three and four bits, path-cost rows); the
            # traffic grows in proportion to the tiles, so it is scaled to this run's average launch.
            "traffic": (NCU_DRAM_BYTES_PER_TILE[args.bits] * search_tiles / max(search_launches, 1)
                        if NCU_DRAM_BYTES_PER_TILE[args.bits] else None),
            "traffic_source": NCU_DRAM_SOURCE[args.bits],
            "algorithmic_dram_bytes_per_tile": 4 * 256 * 4 + 256 * 2,  # rows + compensation in, reconstruction + error + states out
            "peak_source": "of live probe: half2 FMA lanes/s measured in this run / 3 half operations per branch metric "
                           "(the driver's measured-peaks file holds no ALU figure)",
            "peak_nominal": nominal,
            "peak_nominal_source": f"{sms} SMs x {sm_mhz:.0f} MHz (median sampled under load) x "
                                   f"{HALF_LANES_PER_SM_CLOCK} half lanes per SM and clock / 3",
            "frac_of_nominal": achieved / nominal if nominal > 0 else None,
            "launches": search_launches,
            "avg_launch_ms": launch_ms_sum / max(search_launches, 1),
            "busy_ms": search_ms,
            "tiles_per_s": search_tiles / (search_ms * 1e-3) if search_ms > 0 else 0.0,
            "share_of_step": search_ms / total_ms if total_ms > 0 else None,
        },
        "quality": {"expert": payload.expert_id, "proxy_w1": payload.w1.proxy, "proxy_w2": payload.w2.proxy,
                    "routed_rel_sse": payload.routed_sse / max(payload.routed_energy, 1e-30)},
    }
    if world == 1 and not args.no_reference_gpu:
        line["reference_gpu"] = reference_gpu_column(device)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(last["payloads"][0], args.bits)
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_mixed_layer(args, layer, shard, device, dist, world, rank) -> None:
    """``--config c5``: every expert of the shard at K2, K3 and K4, the gathered candidate table,
    the equal-byte exchange and the decode check of the selected payloads, timed once end to end."""

    import torch

    from qsrt_b200 import _lib, pipeline

    if dist is not None:
        dist.barrier()
    # one small warm-up batch (tables, scratch, cuBLAS handles), then the whole shard
    pipeline.encode_expert_batch(LazySources(layer, shard[:1])[0:1], bits=3, device=device, layer_seed=1, score=True)
    for e in shard:
        layer.weights(e)
        layer.route(e)
    torch.cuda.synchronize(device)
    if dist is not None:
        dist.barrier()
    launches_before = _lib.kernel_launches()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    result = pipeline.encode_layer_mixed(LazySources(layer, shard), layer_experts=args.layer_experts, device=device,
                                         experts_per_batch=args.experts_per_step, layer_seed=1)
    end.record()
    torch.cuda.synchronize(device)
    ms = torch.tensor([start.elapsed_time(end)], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        total_ms = float(ms.item())
        weights = 3 * args.layer_experts * 3 * args.hidden * args.inter   # three complete candidates per expert
        counts = {b: result.bits.count(b) for b in (2, 3, 4)}
        print(json.dumps({
            "metric": "MoE-layer encode Mweights/s",
            "value": weights / (total_ms * 1e-3) / 1e6,
            "unit": "Mweights/s",
            "n_gpus": world, "steps": 1, "warmup": 1, "ms_per_step": total_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(args, args.experts_per_step),
            "full_layer_s": total_ms / 1e3,
            "gpu_launches": _lib.kernel_launches() - launches_before,
            "selection": {"experts_at_rate": counts, "exchanges": result.exchanges, "trellis_bpw": result.trellis_bpw,
                          "total_sse": result.total_sse, "all_k3_sse": result.baseline_sse,
                          "selected_payloads_decode_bit_exact": True},
        }), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def reference_gpu_column(device) -> dict:
    """The unmodified reference tile kernel (built from the reference's own sources into
    ``oracle/_ref``) beside the product kernel on the same seeded tiles, timed like the reference's
    own A/B harness (scripts/benchmark_sqg_tile_encoder.py:203-214): CUDA events, alternating
    iterations, median."""

    import torch

    from oracle import ref_kernel
    from qsrt_b200 import tables
    from qsrt_b200 import tiles as tile_api

    if ref_kernel.reference_extension() is None:
        return {"unavailable": "oracle/_ref holds no prebuilt reference extension"}
    count = 8 * torch.cuda.get_device_properties(device).multi_processor_count
    g = torch.Generator(device="cpu").manual_seed(20260816)
    tiles = torch.randn((count, 256), generator=g, dtype=torch.float32).to(device)
    out = {"tiles": count, "family": "normal", "tailbite_context": 128,
           "timing": "CUDA events, 3 alternating iterations after one warm-up each, median"}
    for bits in (2, 3, 4):
        lut = tables.sqg_xor_cheb_t12_bytes(bits)
        reference = ref_kernel.ReferenceTileSearch(lut, bits, 128, device)
        arms = {"reference": lambda: reference(tiles), "product": lambda: tile_api.encode_tiles(tiles, lut, bits, 128)}
        results = {name: fn() for name, fn in arms.items()}     # warm-up and identity check
        torch.cuda.synchronize(device)
        identical = bool(torch.equal(results["reference"][1], results["product"][1]))
        times = {name: [] for name in arms}
        for _ in range(3):
            for name, fn in arms.items():
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                torch.cuda.synchronize(device)
                times[name].append(a.elapsed_time(b))
        ref_ms, own_ms = (statistics.median(times[name]) for name in ("reference", "product"))
        out[f"k{bits}"] = {"reference_tiles_per_s": count / ref_ms * 1e3, "product_tiles_per_s": count / own_ms * 1e3,
                           "speedup": ref_ms / own_ms, "states_identical": identical}
        del reference
    return out


def cpu_baseline(payload, bits: int) -> dict:
    """CPU figures beside the GPU line, on bounded samples: the restatement of the whole path on
    one sub-block (the headline CPU number), and the C restatement of the tile search alone on
    tiles of this workload."""

    import numpy as np

    from oracle import qsrt_oracle as oracle
    from qsrt_b200 import codec, tables

    value, total, cores, sample = cpu_end_to_end(1, 0, bits)
    lut = tables.sqg_xor_cheb_t12_bytes(bits)
    states = codec.unpack_trellis_states(payload.w1.trellis[:4], bits)
    work = codec.decode_regularized_weight(states, lut=lut).cpu().numpy()
    rng = np.random.default_rng(5)
    tiles = oracle.matrix_to_tiles(work).reshape(-1, 256)
    tiles = (tiles + 0.25 * rng.standard_normal(tiles.shape)).astype(np.float32)  # undo quantisation roughly
    n = min(tiles.shape[0], 20 * cores)
    tiles = np.ascontiguousarray(tiles[:n])
    t0 = time.perf_counter()
    oracle.quantize_tiles(tiles, lut.numpy(), bits, 128)
    dt = time.perf_counter() - t0
    return {
        "value": value,
        "unit": "Mweights/s",
        "cores": cores,
        "kind": "port",
        "sample": sample,
        "tile_search_only": {
            "value": n * 256 / dt / 1e6, "unit": "Mweights/s",
            "sample": f"{n} K{bits} tiles (tailbite context 128) of this workload through the C restatement of the tile "
                      f"search alone, OpenMP on {cores} threads, {dt:.1f} s"},
    }


# The search kernel a layer-sized launch gets at each rate, and its DRAM bytes per tile from the
# ncu captures summarised under profiles/ (dram__bytes_read.sum + dram__bytes_write.sum).
SEARCH_KERNEL = {
    2: "viterbi_lazy_kernel<2, dedicated, 2 units/thread> (every second path-cost row, decisions recomputed by the traceback chains)",
    3: "viterbi_lazy_kernel<3, generic, 2 units/thread> (path costs, decisions recomputed by the traceback chains)",
    4: "viterbi_lazy_kernel<4, generic, 2 units/thread> (path costs, decisions recomputed by the traceback chains)",
}
NCU_DRAM_BYTES_PER_TILE = {
    2: (6545.6e6 + 496.9e6) / 1184,
    3: (6528.9e6 + 500.5e6) / 1184,
    4: None,
}
NCU_DRAM_SOURCE = {
    2: "ncu capture of a 1184-tile launch (8 tiles per CTA), scaled per tile",
    3: "ncu capture of a 1184-tile launch (8 tiles per CTA), scaled per tile",
    4: "not captured (half of the three-bit figure by construction: rows of 4096 states)",
}


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
