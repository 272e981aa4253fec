"""Generate tests/golden/encoder_golden.npz by running the reference's own encoder code on the CPU.

    PYTHONPATH=<reference checkout> python tests/golden/make_encoder_golden.py

qsrt/exl3_encoder_backend.py is written to live inside an ExLlamaV3 checkout (relative imports of
its extension and utilities) and to run on CUDA tensors.  This script loads the unmodified file
under a stand-in package (one device-placement guard of ldlq_mixed_batched lifted, see
load_reference_encoder) and supplies only what lies outside the file:

  * ext.pack_trellis            -> the pinned packer restatement (oracle.qsrt_oracle);
  * quantize_tiles              -> the C restatement of the reference's tile search, bit-exact
                                   with the reference CUDA kernel on the pinned fixtures (what
                                   install_sqg_quantizer does with the CUDA extension);
  * util.hadamard.get_hadamard_dt -> the Sylvester matrix times the given scale, which is what
                                   the reference's own decoder uses (qsrt/exl3_reference.py:210-227);
  * progress / memory / image helpers -> no-ops;
  * torch.cuda stream, event and synchronize calls -> no-ops, and Tensor.cpu() of a CPU tensor
    -> a copy, as it is for the CUDA tensors the file expects (block_ldl overwrites the device
    matrix after taking that copy).

Everything else - Hessian preparation and congruence, block LDL, regularisation, scale search,
the BlockLDLQ recursion, proxy error, packing - is the reference's code.  Stored per case: the
initial sign vectors, suh, svh, the packed trellis, g_scale, proxy error and probes of L and the
work-coordinate Hessian.  Candidate grids go through the reference's quantize_qsrt_batch (mixed-rate
LDLQ with the output-axis reuse and the input-axis prefix trie); stored per candidate: a 64-bit
digest of every tile's states, proxy error, suh, svh.
"""

import contextlib
import importlib.util
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import qsrt_oracle  # noqa: E402
from tests.helpers import (  # noqa: E402
    BATCH_CASES, ENCODER_CAPTURE_COUNT, ENCODER_CASES, batch_case_args, batch_case_inputs, encoder_case_args, encoder_case_inputs,
    tile_digests,
)


def _module(name: str, **attrs):
    module = types.ModuleType(name)
    module.__path__ = []
    module.__dict__.update(attrs)
    sys.modules[name] = module
    return module


class _Quiet:
    """Stands in for progress bars, streams and events."""

    def __init__(self, *args, **kwargs):
        pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False

    def __getattr__(self, name):
        return lambda *args, **kwargs: None


def _sylvester(size, device, dtype, scale):
    h = torch.ones((1, 1), dtype=torch.float64)
    while h.shape[0] < size:
        h = torch.cat((torch.cat((h, h), 1), torch.cat((h, -h), 1)), 0)
    return (h * scale).to(device=device, dtype=dtype)


def _pack_trellis(packed, encoded, bits):
    words = qsrt_oracle.pack_trellis_edges(encoded.reshape(-1, 256).numpy(), bits)
    packed.copy_(torch.from_numpy(np.ascontiguousarray(words)).view(torch.int16).reshape(packed.shape))


def _quantize_tiles(tiles, quant_args):
    bits = int(quant_args["K"])
    table = quant_args.get("sqg_e4m3_lut")
    if table is None:
        table = quant_args["sqg_e4m3_luts_by_bits"][bits]
    recon, states = qsrt_oracle.quantize_tiles(tiles.contiguous().numpy(), table.numpy(), bits,
                                               int(quant_args.get("tailbite_context", 128)))
    return torch.from_numpy(recon), torch.from_numpy(states)


def load_reference_encoder():
    import qsrt

    source = Path(qsrt.__file__).parent / "exl3_encoder_backend.py"
    _module("xl3")
    _module("xl3.ext", exllamav3_ext=types.SimpleNamespace(pack_trellis=_pack_trellis))
    _module("xl3.util", cuda_sync_active=lambda: None)
    _module("xl3.util.progress", ProgressBar=_Quiet)
    _module("xl3.util.memory", free_mem=lambda: None, list_gpu_tensors=lambda *a, **k: None)
    _module("xl3.util.hadamard", get_hadamard_dt=_sylvester)
    _module("xl3.util.tensor", save_tensor_image=lambda *a, **k: None)
    for name in ("xl3.a", "xl3.a.b", "xl3.a.b.c"):
        _module(name)
    spec = importlib.util.spec_from_file_location("xl3.a.b.c.quantize", source)
    module = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = module
    torch.cuda.synchronize = lambda *a, **k: None
    torch.cuda.Stream = _Quiet
    torch.cuda.Event = _Quiet
    torch.cuda.stream = lambda stream: contextlib.nullcontext()
    to_host = torch.Tensor.cpu
    torch.Tensor.cpu = lambda self, *a, **k: self.clone() if self.device.type == "cpu" else to_host(self, *a, **k)
    # ldlq_mixed_batched refuses tensors that are not on a CUDA device; that one placement guard is
    # lifted so that the candidate-grid code can run here.  Nothing else of the file is touched.
    text = source.read_text()
    guard = 'if weights.device != Ls.device or weights.device.type != "cuda":'
    assert text.count(guard) == 1
    text = text.replace(guard, "if weights.device != Ls.device:")
    module.__file__ = str(source)
    exec(compile(text, str(source), "exec"), module.__dict__)
    module.quantize_tiles = _quantize_tiles
    return module


def main() -> None:
    """With case names as arguments only those cases are run and merged into the stored file."""

    from qsrt.ldlq import make_shared_h
    from qsrt.sqg_e4m3 import sqg_xor_cheb_t12_bytes

    encoder = load_reference_encoder()
    path = ROOT / "tests" / "golden" / "encoder_golden.npz"
    only = set(sys.argv[1:])
    out = dict(np.load(path)) if only else {}
    for name, (bits, k, n, _, _, _) in ENCODER_CASES.items():
        if only and name not in only:
            continue
        probe = torch.Generator().manual_seed(99 + k + n + bits)
        weight, hessian = encoder_case_inputs(name)
        args = encoder_case_args(name, "cpu", sqg_xor_cheb_t12_bytes(bits))
        h_data = make_shared_h(k, torch.device("cpu"), hessian)
        h_data["count"] = ENCODER_CAPTURE_COUNT.get(name, h_data["count"])
        weight_q, proxy, tensors = encoder.quantize_qsrt(weight.clone(), h_data, args, True)
        vector = torch.randn(k, generator=probe)
        out[f"{name}_su_sign"] = torch.sign(-tensors["suh"].float()).to(torch.int8).numpy()  # su = sign * rms / (-c)
        assert np.array_equal(out[f"{name}_su_sign"], torch.sign(h_data["su"].flatten()).to(torch.int8).numpy())
        out[f"{name}_sv_sign"] = torch.sign(encoder.output_signs(n, torch.device("cpu"), args)).flatten().to(torch.int8).numpy()
        out[f"{name}_suh"] = tensors["suh"].numpy()
        out[f"{name}_svh"] = tensors["svh"].numpy()
        out[f"{name}_trellis"] = tensors["trellis"].numpy()
        out[f"{name}_g_scale"] = np.float64(args["g_scale"])
        out[f"{name}_proxy"] = np.float64(proxy)
        out[f"{name}_apply_out_scales"] = np.bool_(args["apply_out_scales"])
        out[f"{name}_probe"] = vector.numpy()
        if h_data["L"] is not None:
            out[f"{name}_L_probe"] = (h_data["L"] @ vector).numpy()
            out[f"{name}_H_probe"] = (h_data["H"] @ vector).numpy()
        receipt = args.get("h2_viterbi_refine_receipt") or {}
        if receipt.get("enabled"):
            out[f"{name}_refine_accepted"] = np.int64(receipt["sweeps"][0]["accepted_tiles"])
            out[f"{name}_refine_objective"] = np.float64([receipt["sweeps"][0]["objective_before"],
                                                          receipt["sweeps"][0]["objective_after"]])
        out[f"{name}_weight_q_probe"] = (vector @ weight_q).numpy()
        print(name, "g_scale", args["g_scale"], "proxy", proxy, "apply_out_scales", args["apply_out_scales"])
    # candidate grids through the reference's quantize_qsrt_batch (reuse schedules included)
    tables_by_bits = {bits: sqg_xor_cheb_t12_bytes(bits) for bits in (2, 3, 4)}
    for name in BATCH_CASES:
        if only and name not in only:
            continue
        sources = batch_case_inputs(name)
        groups = [batch_case_args(name, "cpu", tables_by_bits) for _ in sources]
        h_datas = [make_shared_h(w.shape[0], torch.device("cpu"), h) for w, h in sources]
        results = encoder.quantize_qsrt_batch([w.clone() for w, _ in sources], h_datas, groups, return_weight_q=False)
        # su = sign * rms / (-c): the drawn sign is the opposite of the stored vector's
        out[f"{name}_su_sign"] = torch.sign(-results[0][0]["suh"].float()).to(torch.int8).numpy()
        out[f"{name}_sv_sign"] = torch.sign(encoder.output_signs(sources[0][0].shape[1], torch.device("cpu"),
                                                                 groups[0][0])).flatten().to(torch.int8).numpy()
        for s_index, group in enumerate(results):
            for c_index, result in enumerate(group):
                key = f"{name}_{s_index}_{c_index}"
                out[f"{key}_tiles"] = tile_digests(result["encoded"].numpy())
                out[f"{key}_proxy"] = np.float64(result["proxy"])
                out[f"{key}_suh"] = result["suh"].numpy()
                out[f"{key}_svh"] = result["svh"].numpy()
                print(key, "proxy", result["proxy"], "g_scale", result["g_scale"])
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
