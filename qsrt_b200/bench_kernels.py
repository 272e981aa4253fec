"""Microbenchmarks of the memory- and FLOP-bound helper kernels at the headline shapes.

    python -m qsrt_b200.bench_kernels [--only NAME] [--iters 5]

Prints one JSON line per kernel with its algorithmic bytes (or flops) per launch, the CUDA-event
time and the achieved GB/s (or TFLOP/s).  Shapes: gate/up in encoder orientation [7168, 2048],
Hessian 7168 x 7168; out-features default to 8192 (four matrices side by side) so that every
input exceeds the L2, which is also flushed between timed iterations.
"""

from __future__ import annotations

import argparse
import json

import torch

from . import allocation, codec, coupled, encoder, hessian, linalg, mxfp4, records, refine, scoring, storage, tables
from . import tiles as tile_search


_flush = None


def _time(fn, iters: int, warmup: int = 3) -> float:
    """Median CUDA-event time; a 512 MB write between iterations evicts the 126 MB L2."""

    global _flush
    if _flush is None:
        _flush = torch.empty(512 << 20, dtype=torch.uint8, device="cuda:0")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        _flush.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return sorted(times)[len(times) // 2]


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--only", default=None)
    p.add_argument("--iters", type=int, default=5)
    p.add_argument("--k", type=int, default=7168)
    p.add_argument("--n", type=int, default=8192, help="out-features; 8192 = four stacked 2048-wide matrices")
    p.add_argument("--rows", type=int, default=4096)
    args = p.parse_args()
    dev = torch.device("cuda:0")
    k, n = args.k, args.n
    g = torch.Generator(device=dev).manual_seed(1)
    w = torch.randn((k, n), device=dev, generator=g)
    sv = torch.rand(n, device=dev, generator=g) + 0.5
    su = torch.rand(k, device=dev, generator=g) + 0.5
    sums = torch.empty(k, device=dev)
    h = torch.randn((k, k), device=dev, generator=g)
    x = torch.randn((args.rows, k), device=dev, generator=g)
    wts = torch.rand(args.rows, device=dev, generator=g)
    acc = torch.empty((k, k), device=dev)
    bits = 3
    lut = tables.sqg_xor_cheb_t12_bytes(bits).to(dev)
    states = torch.randint(-32768, 32767, (k // 16, n // 16, 256), device=dev, dtype=torch.int16, generator=g)
    packed = codec.pack_trellis_edges(states, bits)
    tiles = states.shape[0] * states.shape[1]
    signs_n = torch.ones(n, device=dev)
    signs_k = torch.ones(k, device=dev)

    # record container / atom image: 16 Kimi-geometry matrices per timed call (350 MB of states)
    rec_states = [codec.reconstruct_trellis_states(
        torch.randint(0, 4, (192, 224, 256), device=dev, dtype=torch.int16, generator=g), 2) for _ in range(16)]
    rec_bytes = 16 * (192 * 224 * (512 + 96))
    layout = storage.QSRTLayerLayout(16, 880)
    image = torch.zeros(layout.disk_bytes, dtype=torch.uint8, device=dev)
    scale = torch.ones(3072, dtype=torch.float16, device=dev)
    rec_payloads = [records.pack_qsrt_trellis(s_, "K2", rate_axis="k") for s_ in rec_states]

    rec_states_n = [s_.reshape(224, 192, 256) for s_ in rec_states]   # same tiles, N-axis geometry

    def write_image():
        for slot in range(5):
            trio = {"w1": rec_states_n[3 * slot], "w3": rec_states_n[3 * slot + 1], "w2": rec_states[3 * slot + 2]}
            storage.write_expert_atoms(image, layout, 9, slot, slot, trio, {"w1": 0, "w3": 0, "w2": 0},
                                       {"w1": scale, "w3": scale, "w2": scale}, validate_states=False)

    # one large launch of the same kernels: 64 records x 32 stripes along K, 224 tiles across
    big_bits = records._bits_array(tuple((2, 4, 3, 3)[r % 4] for r in range(64)))
    big_k, big_n = 64 * 32, 224
    big_states = torch.randint(-32768, 32767, (big_k, big_n, 256), device=dev, dtype=torch.int16, generator=g)
    big_payload = torch.empty(big_k * big_n * 48, dtype=torch.int16, device=dev)
    big_pitch = 224 * 32 * 6
    lib = encoder._lib.lib()

    def big_pack(layout_id):
        encoder._lib.check(lib.qsrtb_pack_records(
            big_states.data_ptr(), big_k, big_n, 0, 64, 32, big_bits, layout_id, 5 if layout_id else 0,
            big_pitch if layout_id else 0, big_payload.data_ptr(), big_payload.numel() * 2, None, None), "pack")

    def big_unpack():
        encoder._lib.check(lib.qsrtb_unpack_records(
            big_payload.data_ptr(), big_payload.numel() * 2, big_k, big_n, 0, 64, 32, big_bits, 0, 0, 0,
            big_states.data_ptr(), None, None), "unpack")

    big_tiles = big_k * big_n
    mx_rows, mx_cols = 8192, 7168   # four gate-shaped source matrices
    mx_packed = torch.randint(0, 256, (mx_rows, mx_cols // 2), device=dev, dtype=torch.uint8, generator=g)
    mx_scale = torch.randint(110, 130, (mx_rows, mx_cols // 32), device=dev, dtype=torch.uint8, generator=g)
    mx_bytes = mx_rows * mx_cols * 4 + mx_packed.numel() + mx_scale.numel()
    w_other = torch.randn((k, n), device=dev, generator=g)
    # dense-H path refinement of one down projection in encoder orientation [2048, 7168], K3
    rf_rows, rf_cols = 2048, 7168
    rf_weight = torch.randn((rf_rows, rf_cols), device=dev, generator=g)
    rf_x = torch.randn((4 * rf_rows, rf_rows), device=dev, generator=g)
    rf_hessian = (rf_x.T @ rf_x) / rf_x.shape[0]
    rf_hessian.diagonal().add_(0.025)
    rf_args = {"K": 3, "devices": [str(dev)], "tailbite_context": 128, "sqg_e4m3_lut": tables.sqg_xor_cheb_t12_bytes(3)}
    rf_order = encoder.tensor_core_perm(dev)
    rf_tiles = rf_weight.reshape(rf_rows // 16, 16, rf_cols // 16, 16).permute(0, 2, 1, 3).reshape(-1, 256)
    rf_recon, rf_states = tile_search.quantize_tiles(rf_tiles[:, rf_order].contiguous(), rf_args)
    rf_q = rf_recon[:, torch.argsort(rf_order)].reshape(rf_rows // 16, rf_cols // 16, 16, 16).permute(0, 2, 1, 3)
    rf_q = rf_q.reshape(rf_rows, rf_cols).contiguous()
    rf_states = rf_states.reshape(rf_rows // 16, rf_cols // 16, 256)
    rf_config = refine.H2ViterbiRefineConfig(sweeps=1)
    del rf_x, rf_tiles, rf_recon
    # tensor-core products and scoring at the headline shapes: 4096 routed rows of one expert
    sc_rows = args.rows
    sc_x = linalg.split_tf32(x)                                            # [rows, 7168]
    sc_gate_up = linalg.split_tf32(torch.randn((4096, k), device=dev, generator=g) * 0.02)   # stacked gate / up
    sc_down = linalg.split_tf32(torch.randn((k, 2048), device=dev, generator=g) * 0.02)
    sc_pre = torch.empty((sc_rows, 4096), device=dev)
    sc_mid, _ = scoring.gated_activation(torch.randn((sc_rows, 4096), device=dev, generator=g))
    sc_out = torch.empty((sc_rows, k), device=dev)
    sc_ref = torch.randn((sc_rows, k), device=dev, generator=g)
    chol_x = torch.randn((k + 512, k), device=dev, generator=g)
    chol_h = chol_x.T @ chol_x / chol_x.shape[0]
    chol_h.diagonal().add_(0.025 * chol_h.diagonal().mean())
    chol_work = torch.empty_like(chol_h)
    del chol_x
    chol_copy_ms = _time(lambda: chol_work.copy_(chol_h), args.iters) if not args.only or "cholesky" in args.only else 0.0

    def factor():
        chol_work.copy_(chol_h)
        linalg.cholesky_(chol_work)

    syrk_panel = linalg.split_tf32(torch.randn((k - 128, 128), device=dev, generator=g))
    mx_out = torch.empty((mx_rows, mx_cols), device=dev)

    def fused_ingest():
        encoder._lib.check(lib.qsrtb_mxfp4_signed_block_hadamard(
            mx_packed.data_ptr(), mx_scale.data_ptr(), mx_rows, mx_cols, mx_out.data_ptr(), mx_cols, 1, 0, 512,
            signs_k.data_ptr(), 1, None), "fused ingest")

    cases = {
        f"gemm3x tcgen05 (gate|up pre-activations) [{sc_rows}, {k}] x [4096, {k}]^T":
            (lambda: linalg.gemm_nt(sc_x, sc_gate_up, sc_pre), 2 * sc_rows * 4096 * k, "F"),
        f"gemm3x tcgen05 (down product) [{sc_rows}, 2048] x [{k}, 2048]^T":
            (lambda: linalg.gemm_nt(sc_mid, sc_down, sc_out), 2 * sc_rows * 2048 * k, "F"),
        f"gemm3x tcgen05 (Cholesky trailing update, rank 128, lower tiles of {k - 128}^2)":
            (lambda: linalg.gemm_nt(syrk_panel, syrk_panel, h[:k - 128, :k - 128], alpha=-1.0, beta=1.0, lower_only=True),
             (k - 128) * (k - 128) * 128, "F"),
        f"cholesky_blocked {k} (copy of {chol_copy_ms:.2f} ms included)": (factor, k * k * k / 3, "F"),
        "split_tf32 (rows -> head / tail planes)": (lambda: linalg.split_tf32(x, out=sc_x), 12 * sc_rows * k, "B"),
        "gated_activation (SiLU, -> planes)":
            (lambda: scoring.gated_activation(sc_pre, "silu"), sc_rows * 4096 * 4 + 2 * sc_rows * 2048 * 4, "B"),
        "routed_row_sse": (lambda: scoring.row_sse(sc_ref, sc_out, energy=True), 8 * sc_rows * k, "B"),
        "mxfp4 -> signed_block_hadamard rows 512 (fused ingest)": (fused_ingest, mx_bytes, "B"),
        "refine_h2_viterbi_paths, one sweep [2048, 7168] K3 (128 row blocks of 448 tiles)":
            (lambda: refine.refine_h2_viterbi_paths(rf_weight, rf_hessian, rf_q, rf_states, rf_args, rf_config),
             (rf_rows // 16) * (rf_cols // 16), "T"),
        "tile_squared_error": (lambda: allocation.tile_squared_error(w, w_other), 8 * k * n + k * n // 32, "B"),
        "mxfp4_dequant [out, in]": (lambda: mxfp4.dequant(mx_packed, mx_scale), mx_bytes, "B"),
        "mxfp4_dequant -> encoder orientation [in, out]":
            (lambda: mxfp4.dequant_encoder_orientation(mx_packed, mx_scale), mx_bytes, "B"),
        "pack_records kernel, record layout (458k tiles, mixed K2/K3/K4)": (lambda: big_pack(0), big_tiles * (512 + 96), "B"),
        "pack_records kernel, atom layout (458k tiles)": (lambda: big_pack(1), big_tiles * (512 + 96), "B"),
        "unpack_records kernel -> states (458k tiles)": (big_unpack, big_tiles * (512 + 96), "B"),
        "pack_records R2 (16 matrices)":
            (lambda: [records.pack_qsrt_trellis(s_, "R2", rate_axis="k", validate_states=False) for s_ in rec_states],
             rec_bytes, "B"),
        "unpack_records K2 -> states (16 matrices)":
            (lambda: [records.unpack_qsrt_trellis_states(p_) for p_ in rec_payloads],
             16 * 192 * 224 * (64 + 512), "B"),
        "write_expert_atoms R0 (5 experts -> layer image)": (write_image, 15 * 192 * 224 * (512 + 96), "B"),
        "hadamard_rows (divide by sv + had_r + row sums)":
            (lambda: encoder._hadamard(w, 1, sv, per_col=True, divide=True, row_sumsq=sums), 8 * k * n, "B"),
        "hadamard_cols (divide by su + had_l)":
            (lambda: encoder._hadamard(w, 0, su, per_col=False, divide=True), 8 * k * n, "B"),
        "hadamard_rows 7168^2 (Hessian congruence)":
            (lambda: encoder._hadamard(h, 1, su, per_col=True), 8 * k * k, "B"),
        "hadamard_cols 7168^2 (Hessian congruence)":
            (lambda: encoder._hadamard(h, 0, su, per_col=False), 8 * k * k, "B"),
        "col_sumsq": (lambda: encoder._col_sumsq(w), 4 * k * n, "B"),
        "block_ldl_normalize 7168": (lambda: encoder._lib.lib().qsrtb_block_ldl_normalize(
            h.data_ptr(), k, k, None), 8 * k * k // 2, "B"),
        "pack_trellis K3": (lambda: codec.pack_trellis_edges(states, bits), tiles * (512 + 32 * bits), "B"),
        "unpack_decode K3 -> E4M3": (lambda: codec.decode_e4m3(packed, bits, lut), tiles * (32 * bits + 256), "B"),
        "unpack K3 -> states": (lambda: codec.unpack_trellis_states(packed, bits), tiles * (32 * bits + 512), "B"),
        "states_to_matrix": (lambda: codec.decode_regularized_weight(states, lut=lut), tiles * (512 + 1024), "B"),
        "signed_block_hadamard rows 512": (lambda: coupled._transform_(w, 1, 512, signs_n, False), 8 * k * n, "B"),
        "signed_block_hadamard cols 512": (lambda: coupled._transform_(w, 0, 512, signs_k, False), 16 * k * n, "B"),
        f"weighted_syrk {args.rows}x{k}": (lambda: hessian.accumulate_hessian(acc, x, wts, accumulate=False),
                                           args.rows * k * k, "F"),
        f"weighted_syrk tcgen05 3xTF32 {args.rows}x{k}": (
            lambda: hessian.accumulate_hessian_tensor_cores(acc, x, wts, accumulate=False), args.rows * k * k, "F"),
        "hessian_finish": (lambda: hessian.finish_hessian(acc, 1.0), 8 * k * k, "B"),
    }
    for name, (fn, work, kind) in cases.items():
        if args.only and args.only not in name:
            continue
        ms = _time(fn, args.iters)
        rate = work / (ms * 1e-3)
        line = {"kernel": name, "ms": ms, "work_per_launch": work}
        if kind == "T":
            # share of the call spent inside the tile-search launches (events on the launching stream)
            tile_search.search_timings = []
            fn()
            torch.cuda.synchronize()
            line["tile_search_ms"] = sum(a.elapsed_time(b) for a, b, _, _ in tile_search.search_timings)
            tile_search.search_timings = None
        if kind == "B":
            line["GB_per_s"] = rate / 1e9
        elif kind == "T":
            line["tiles_per_s"] = rate
        else:
            line["TFLOP_per_s"] = rate / 1e12
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
