"""Expert-level orchestration of the encoder hot path.

One gated expert is three matrices: ``w1`` (gate) and ``w3`` (up), both ``[intermediate,
hidden]``, and ``w2`` (down) ``[hidden, intermediate]``.  Following the reference's
whole-expert flow (``qsrt/pack/qsrt_candidates.py:1258-1375`` and, for the GLM variant,
``qsrt/glm52_down_construction.py:159-260``):

1. ``H13`` = gate^2-weighted covariance of the routed input rows (``build_expert_hessians``,
   ``qsrt/qsrt_candidates.py:534-618``);
2. ``w1`` and ``w3`` share ``H13`` and are encoded together (one LDLQ pass over their
   concatenated output channels, ``quantize_uniform_batch``);
3. the middle activation ``act(x w1^T) * (x w3^T)`` of the routed rows - from the source
   weights or from the just-encoded reconstructions - gives ``H2`` with OAS shrinkage;
4. ``w2`` is encoded against ``H2`` (experts of a batch stacked, one launch per 16-row step);
5. the routed functional error ``sum_rows gate^2 * ||y_hat - y||^2`` scores the candidate
   (``functional_sse_by_request``, ``qsrt/qsrt_candidates.py:621-654``);
6. payloads are packed; decoding them back to E4M3 must reproduce the encoder's states.

Everything stays on the device; the only host synchronisations are the ones the reference
also has (scale search, Cholesky status, proxy traces).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from . import codec, encoder, hessian, tables


@dataclass
class ExpertSource:
    """Source weights and routed calibration rows of one expert (device tensors)."""

    w1: torch.Tensor          # gate  [intermediate, hidden]
    w3: torch.Tensor          # up    [intermediate, hidden]
    w2: torch.Tensor          # down  [hidden, intermediate]
    rows: torch.Tensor        # routed inputs [R, hidden]
    gates: torch.Tensor       # routing weights [R]
    expert_id: int = 0


@dataclass
class MatrixPayload:
    trellis: torch.Tensor     # int16 [in/16, out/16, 16*bits]
    suh: torch.Tensor         # float16 [in]
    svh: torch.Tensor         # float16 [out]
    bits: int
    proxy: float
    g_scale: float


@dataclass
class ExpertPayload:
    expert_id: int
    bits: int
    w1: MatrixPayload
    w3: MatrixPayload
    w2: MatrixPayload
    routed_sse: float = float("nan")
    routed_energy: float = float("nan")
    payload_bytes: int = 0
    evidence: dict = field(default_factory=dict)


def situ(gate: torch.Tensor, up: torch.Tensor, *, beta: float = 4.0, linear_beta: float = 25.0) -> torch.Tensor:
    """Kimi's bounded gated activation (qsrt/tp_simulator.py:82-93)."""

    gate_value = beta * torch.tanh(gate.float() / beta) * torch.sigmoid(gate.float())
    up_value = linear_beta * torch.tanh(up.float() / linear_beta)
    return (gate_value * up_value).to(gate.dtype)


def gated_middle(rows: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, activation: str = "silu",
                 execution=None) -> torch.Tensor:
    """Middle activation ``act(x W1^T) * (x W3^T)`` of routed rows: one tensor-core product against
    the stacked gate / up matrices and the fused activation kernel (``scoring.gated_middle``)."""

    if execution is not None:
        return execution.decode_middle(rows, w1, w3, activation)
    if activation not in ("silu", "situ"):
        raise ValueError(f"unknown activation {activation!r}")
    from . import scoring

    return scoring.gated_middle(rows, w1, w3, activation)


def quant_args_for(bits: int, device: torch.device, *, seed: int, sv_seed: int, sigma_reg: float = encoder.SIGMA_REG,
                   tailbite_context: int = 128, codebook: str = tables.SQG_XOR_CHEB_T12, **extra) -> dict:
    """The ``quant_args`` dictionary of a uniform-rate encode (qsrt/qsrt_codec_pilot.py:421-452)."""

    args = {
        "K": int(bits),
        "seed": int(seed),
        "sv_seed": int(sv_seed),
        "sigma_reg": float(sigma_reg),
        "devices": [str(device)],
        "device_ratios": None,
        "apply_out_scales": False,
        "ldlq_tf32": False,
        "tailbite_context": int(tailbite_context),
        "sqg_e4m3_lut": tables.sqg_codebook_bytes(bits, codebook),
    }
    args.update(extra)
    return args


def _payload(result, args) -> MatrixPayload:
    proxy, tensors = result
    return MatrixPayload(tensors["trellis"], tensors["suh"], tensors["svh"], int(args["K"]), float(proxy), float(args["g_scale"]))


def decode_matrix(payload: MatrixPayload, lut: torch.Tensor | None = None) -> torch.Tensor:
    """Packed payload -> source-orientation ``[out, in]`` float32 weight."""

    lut = tables.sqg_xor_cheb_t12_bytes(payload.bits) if lut is None else lut
    states = codec.unpack_trellis_states(payload.trellis, payload.bits)
    return codec.decode_exl3_weight(states, payload.suh, payload.svh, lut=lut).T.contiguous()


def verify_payload_roundtrip(payload: MatrixPayload) -> bool:
    """Pack -> decode-to-E4M3 closure: the decoded bytes must equal LUT[states] of a second,
    independent unpack, and the states must close cyclically (bit-exact check on device)."""

    lut = tables.sqg_xor_cheb_t12_bytes(payload.bits).to(payload.trellis.device)
    raw = codec.decode_e4m3(payload.trellis, payload.bits, lut)
    states = codec.unpack_trellis_states(payload.trellis, payload.bits)
    expected = lut[(states.to(torch.int32) & 0xFFFF).long()]
    repacked = codec.pack_trellis_edges(states, payload.bits)
    return bool(torch.equal(raw, expected)) and bool(torch.equal(repacked, payload.trellis))


def encode_expert_batch(experts: list[ExpertSource], *, bits: int, device: torch.device, layer_seed: int = 0,
                        sigma_reg: float = encoder.SIGMA_REG, tailbite_context: int = 128,
                        activation: str = "silu", down_from_reconstruction: bool = False,
                        score: bool = True, h2_max_local_alpha: float = 0.75,
                        coupled_spec=None, shared_scale_scope=None) -> list[ExpertPayload]:
    """Encode a batch of experts at one uniform rate; see the module docstring for the flow.

    With ``coupled_spec`` (a ``coupled.CoupledHadamardSpec``) every expert is first moved into
    the coupled signed block-Hadamard coordinates (``encode_coupled_weights``), its routed rows
    with it (``transform_inputs``), the middle activation is evaluated through
    ``decode_middle`` and the routed error through ``decode_output``
    (``qsrt/pack/qsrt_candidates.py:1157-1180``); the payloads then describe the coupled
    matrices.

    ``shared_scale_scope`` switches on the shared input-scale mode of the production encoder for
    the gate and up matrices (``shared_input_scales_key = (scope, matrix)`` with the global scale
    folded into the output scales, qsrt/pack/qsrt_encoder.py:549-551): every expert encoded under
    the scope stores the input-scale profile of the scope's first tensor, which is expert zero's
    in a canonical layer encode.  A rank whose shard does not start with expert zero
    calls ``prime_shared_scales`` with expert zero's weights first."""

    if not experts:
        return []
    device = torch.device(device)
    if coupled_spec is not None:
        return _encode_coupled_batch(experts, coupled_spec, bits=bits, device=device, layer_seed=layer_seed,
                                     sigma_reg=sigma_reg, tailbite_context=tailbite_context,
                                     activation=activation, down_from_reconstruction=down_from_reconstruction,
                                     score=score, h2_max_local_alpha=h2_max_local_alpha,
                                     shared_scale_scope=shared_scale_scope)

    def shared(matrix: str) -> dict:
        # gate and up only, with the global scale folded into the output scales so that the stored
        # input scales really are one vector per layer and matrix (qsrt/pack/qsrt_encoder.py:549-551)
        if shared_scale_scope is None or matrix not in ("w1", "w3"):
            return {}
        return {"shared_input_scales_key": (shared_scale_scope, matrix), "g_scale_into_sv": True}

    results: list[ExpertPayload] = []
    weights_sq = [ex.gates.float().square() for ex in experts]

    def seed_of(ex, offset):
        return 6 * (layer_seed * 100003 + ex.expert_id) + offset

    # group A: gate and up of every expert; a pair shares its expert's H13
    a_weights, a_h, a_args = [], [], []
    for ex, w in zip(experts, weights_sq):
        h13, _ = hessian.weighted_covariance(ex.rows, w, device=device, return_cpu=False)
        shared_h = encoder.make_shared_h(ex.w1.shape[1], device, h13)
        del h13
        for matrix, offset, name in ((ex.w1, 1, "w1"), (ex.w3, 2, "w3")):
            a_weights.append(matrix.T.float().contiguous())
            a_h.append(shared_h)
            a_args.append(quant_args_for(bits, device, seed=seed_of(ex, 0), sv_seed=seed_of(ex, offset),
                                         sigma_reg=sigma_reg, tailbite_context=tailbite_context, **shared(name)))

    def down_group(middles):
        b_weights, b_h, b_args, infos = [], [], [], []
        for ex, w, middle in zip(experts, weights_sq, middles):
            local_h2, _ = hessian.weighted_covariance(middle, w, device=device, return_cpu=False)
            h2, info = hessian.adaptive_identity_shrinkage(local_h2, w, max_local_alpha=h2_max_local_alpha)
            del local_h2
            b_h.append(encoder.make_shared_h(ex.w2.shape[1], device, h2))
            del h2
            b_args.append(quant_args_for(bits, device, seed=seed_of(ex, 3), sv_seed=seed_of(ex, 4),
                                         sigma_reg=sigma_reg, tailbite_context=tailbite_context, **shared("w2")))
            b_weights.append(ex.w2.T.float().contiguous())
            infos.append(info)
        return (b_weights, b_h, b_args), infos

    if down_from_reconstruction:
        a_out = encoder.quantize_uniform_batch(a_weights, a_h, a_args)
        gate_up = [(_payload(a_out[2 * i], a_args[2 * i]), _payload(a_out[2 * i + 1], a_args[2 * i + 1]))
                   for i in range(len(experts))]
        middles = [gated_middle(ex.rows.float(), decode_matrix(p1), decode_matrix(p3), activation,
                                getattr(ex, "execution", None))
                   for ex, (p1, p3) in zip(experts, gate_up)]
        group_b, evidence = down_group(middles)
        down_args = group_b[2]
        down_out = encoder.quantize_uniform_batch(*group_b)
    else:
        middles = [gated_middle(ex.rows.float(), ex.w1.float(), ex.w3.float(), activation,
                                getattr(ex, "execution", None)) for ex in experts]
        group_b, evidence = down_group(middles)
        down_args = group_b[2]
        # gate/up and down do not depend on each other here: their recursions run concurrently
        a_out, down_out = encoder.quantize_uniform_groups([(a_weights, a_h, a_args), group_b])
        gate_up = [(_payload(a_out[2 * i], a_args[2 * i]), _payload(a_out[2 * i + 1], a_args[2 * i + 1]))
                   for i in range(len(experts))]

    scores = []
    for ex, (p1, p3), res, args, info in zip(experts, gate_up, down_out, down_args, evidence):
        p2 = _payload(res, args)
        payload = ExpertPayload(ex.expert_id, bits, p1, p3, p2, evidence=info)
        payload.payload_bytes = sum(p.trellis.numel() * 2 + p.suh.numel() * 2 + p.svh.numel() * 2 for p in (p1, p3, p2))
        if score:
            scores.append(score_payload(ex, payload, activation))
        results.append(payload)
    # one host synchronisation for the whole batch (the reference defers its row sums the same way,
    # qsrt/pack/qsrt_candidates.py:318-349)
    if scores:
        values = torch.stack([torch.stack(pair) for pair in scores]).cpu()
        for payload, (sse, energy) in zip(results, values.tolist()):
            payload.routed_sse, payload.routed_energy = sse, energy
    return results


def prime_shared_scales(expert_zero: ExpertSource, *, bits: int, device: torch.device, shared_scale_scope,
                        layer_seed: int = 0, sigma_reg: float = encoder.SIGMA_REG, tailbite_context: int = 128) -> None:
    """Seed the shared input-scale profiles of a scope from expert zero's gate and up matrices.

    Under ``shared_scale_scope`` every expert stores the input-scale profile of the scope's first
    tensor - expert zero's in a canonical full-layer encode (qsrt/exl3_encoder_backend.py:2664-2672).
    A rank whose shard does not begin with expert zero calls this once before its first encode,
    as the reference's split workers re-encode expert zero as a primer
    (scripts/pack_qsrt_candidates.py:1282, 1413-1425); only the part of the preparation that the
    profile depends on is run.  ``expert_zero`` needs its weights only (rows may be empty)."""

    device = torch.device(device)
    for matrix, offset, name in ((expert_zero.w1, 1, "w1"), (expert_zero.w3, 2, "w3")):
        args = quant_args_for(bits, device, seed=0,
                              sv_seed=6 * (layer_seed * 100003 + expert_zero.expert_id) + offset, sigma_reg=sigma_reg,
                              tailbite_context=tailbite_context, shared_input_scales_key=(shared_scale_scope, name),
                              g_scale_into_sv=True)
        encoder.prime_shared_input_scales(matrix.to(device).T.float().contiguous(), args)


def score_payload(source: ExpertSource, payload: ExpertPayload, activation: str = "silu"):
    """Routed functional error of a stored expert candidate: its three packed matrices are decoded
    and run against the source expert on the expert's routed rows
    (``sum_rows gate^2 ||student - teacher||^2``; ``functional_sse_by_request`` summed over the
    requests, qsrt/qsrt_candidates.py:621-654).  Returns ``(sse, energy)`` as 0-d float64 device
    tensors; nothing synchronises."""

    from . import scoring

    decoded = (decode_matrix(payload.w1), decode_matrix(payload.w3), decode_matrix(payload.w2))
    return scoring.routed_output_sse(source.rows, source.gates, (source.w1, source.w3, source.w2), decoded, activation)


def _encode_coupled_batch(experts, spec, *, score, activation, **kwargs):
    from . import coupled

    moved, executions, teachers = [], [], []
    for ex in experts:
        execution = coupled.CoupledHadamardExecution(hidden=ex.w1.shape[1], intermediate=ex.w1.shape[0], spec=spec)
        c1, c3, c2 = coupled.encode_coupled_weights((ex.w1, ex.w3, ex.w2), spec)
        rows = execution.transform_inputs(ex.rows)
        moved.append(_CoupledSource(c1, c3, c2, rows, ex.gates, ex.expert_id, execution, activation))
        executions.append(execution)
        if score:
            from . import linalg

            teachers.append(linalg.matmul_nt(gated_middle(ex.rows.float(), ex.w1.float(), ex.w3.float(), activation),
                                             ex.w2.float().contiguous()))
    payloads = encode_expert_batch(moved, score=False, activation=activation, **kwargs)
    if score:
        for payload, src, execution, teacher, ex in zip(payloads, moved, executions, teachers, experts):
            from . import scoring

            decoded = (decode_matrix(payload.w1), decode_matrix(payload.w3), decode_matrix(payload.w2))
            student = execution.execute(ex.rows.float(), decoded, activation)
            w = ex.gates.float().square().double()
            sse, energy = scoring.row_sse(teacher, student, energy=True)
            payload.routed_sse = float((sse * w).sum())
            payload.routed_energy = float((energy * w).sum())
    return payloads


@dataclass
class _CoupledSource(ExpertSource):
    """An expert already moved to coupled coordinates: its middle activation is evaluated by the
    coupled execution (inverse pre-activation transform, activation, post-activation transform)."""

    execution: object = None
    activation: str = "silu"


@dataclass
class LayerSelection:
    """Outcome of the mixed-rate candidate selection of one layer shard."""

    bits: tuple[int, ...]                 # selected rate of every expert of the layer
    table: torch.Tensor                   # [layer_experts, 3, 2] float64 (SSE, bytes), gathered
    selected: dict                        # expert id -> ExpertPayload (local experts only)
    total_sse: float
    baseline_sse: float
    exchanges: int
    trellis_bpw: float


def encode_layer_mixed(experts: list[ExpertSource], *, layer_experts: int, device: torch.device,
                       budget_bpw: float = 3.083333, group=None, experts_per_batch: int = 4,
                       **encode_kwargs) -> LayerSelection:
    """Mixed-rate candidate selection around a K3 baseline.

    Every local expert is encoded completely at K2, K3 and K4; the routed functional error and
    the payload size of each complete-expert candidate are all-gathered
    (``selection.gather_candidate_table``, the path's only collective); every rank then runs the
    same greedy equal-byte K2<->K4 exchange (``selection.equal_byte_exchange``) under the
    trellis budget (3.083333 bpw = all-K3 plus one expert in twelve raised to K4); the selected
    payloads are checked by decoding their packed bitstreams back to E4M3.  ``experts`` is a
    list or any sequence with ``len()`` and slicing that yields ``ExpertSource`` items (they are
    taken ``experts_per_batch`` at a time, so a lazy sequence keeps only one batch resident).
    """

    from . import selection

    rates = (2, 3, 4)
    device = torch.device(device)
    # experts go through the encoder a few at a time (an expert of the full layer shape holds
    # about 1 GB of Hessians and factors while it is being encoded)
    step = max(1, int(experts_per_batch))
    by_rate = {b: [] for b in rates}
    for begin in range(0, len(experts), step):
        for b in rates:
            by_rate[b].extend(encode_expert_batch(experts[begin:begin + step], bits=b, device=device, score=True,
                                                  **encode_kwargs))
    local_ids = [payload.expert_id for payload in by_rate[rates[0]]]
    local = torch.empty((len(experts), 3, 2), dtype=torch.float64, device=device)
    for c, b in enumerate(rates):
        for i, payload in enumerate(by_rate[b]):
            trellis_bytes = sum(m.trellis.numel() * 2 for m in (payload.w1, payload.w3, payload.w2))
            local[i, c, 0] = payload.routed_sse
            local[i, c, 1] = float(trellis_bytes)
    table = selection.gather_candidate_table(local, local_ids, layer_experts, group=group)
    present = torch.isfinite(table[:, 1, 0])
    if not bool(present.all()):
        raise ValueError("the gathered candidate table does not cover every expert of the layer")
    free_upgrades = int(round((budget_bpw - 3.0) * layer_experts + 1e-9))
    allocation = selection.equal_byte_exchange(table, free_upgrades=max(0, free_upgrades))
    chosen = {}
    for i, expert_id in enumerate(local_ids):
        payload = by_rate[allocation.bits[expert_id]][i]
        for matrix in (payload.w1, payload.w3, payload.w2):
            if not verify_payload_roundtrip(matrix):
                raise RuntimeError(f"expert {expert_id}: packed payload failed its decode round trip")
        chosen[expert_id] = payload
    k3_bytes = float(table[:, 1, 1].sum())
    return LayerSelection(allocation.bits, table, chosen, allocation.total_sse, allocation.baseline_sse,
                          allocation.exchanges, 3.0 * allocation.total_bytes / k3_bytes)
