"""Coupled signed block-Hadamard coordinates for gate / up / down (device resident).

Mirrors ``qsrt/qsrt_coupled.py``: ``CoupledHadamardSpec`` (:25-46), ``block_hadamard``
(:49-84), ``rotation_signs`` (:87-107), ``signed_block_hadamard`` (:110-132),
``encode_coupled_weights`` (:145-196) and ``CoupledHadamardExecution`` (:347-543).  Every
butterfly runs in ``qsrtb_signed_block_hadamard`` with the signs fused, in place, in the
reference's operation order, so results match the reference's float32 CPU path bit for bit.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from .pipeline import situ
from .tiles import _stream_ptr

Tensor = torch.Tensor
WeightTriplet = tuple[Tensor, Tensor, Tensor]


@dataclass(frozen=True)
class CoupledHadamardSpec:
    residual_block_size: int = 512
    preactivation_block_size: int = 128
    postactivation_block_size: int = 128
    residual_draw: int = 0
    intermediate_draw: int = 0

    def __post_init__(self) -> None:
        for name, value in (
            ("residual_block_size", self.residual_block_size),
            ("preactivation_block_size", self.preactivation_block_size),
            ("postactivation_block_size", self.postactivation_block_size),
        ):
            if value <= 0 or value & (value - 1):
                raise ValueError(f"{name} must be a positive power of two")
            if value not in (128, 256, 512):
                raise ValueError(f"{name} must be 128, 256 or 512 on the B200 path")
        if self.residual_draw != 0:
            raise ValueError("the coupled profile fixes residual draw zero")
        if not 0 <= self.intermediate_draw < 8:
            raise ValueError("intermediate_draw must lie in 0..7")


def rotation_signs(length: int, *, draw: int, axis: int, device: torch.device) -> Tensor:
    """Deterministic Rademacher vector of the frozen draw family (drawn on the CPU generator,
    as the reference does, then moved)."""

    if length <= 0 or draw < 0:
        raise ValueError("length must be positive and draw nonnegative")
    if draw == 0:
        return torch.ones(length, dtype=torch.float32, device=device)
    generator = torch.Generator(device="cpu")
    generator.manual_seed((0x6A09E667F3BCC909 * draw + 0xBB67AE8584CAA73B * axis) & ((1 << 63) - 1))
    return torch.randint(0, 2, (length,), generator=generator).mul_(2).sub_(1).float().to(device=device)


def _transform_(matrix: Tensor, axis: int, block_size: int, signs: Tensor | None, inverse: bool) -> Tensor:
    """In place on a contiguous CUDA float32 matrix."""

    rows, cols = matrix.shape
    if signs is not None:
        signs = signs.to(device=matrix.device, dtype=torch.float32).contiguous()
    with torch.cuda.device(matrix.device):
        _lib.check(
            _lib.lib().qsrtb_signed_block_hadamard(
                matrix.data_ptr(), rows, cols, cols, axis, block_size,
                signs.data_ptr() if signs is not None else None, int(inverse), _stream_ptr(matrix.device),
            ),
            "qsrtb_signed_block_hadamard",
        )
    return matrix


def _matmul_nt(x: Tensor, w: Tensor) -> Tensor:
    """``x @ w.T`` in float32 accuracy on the tensor cores."""

    from . import linalg

    return linalg.matmul_nt(x.float().contiguous(), w.float().contiguous())


def _as_work_matrix(values: Tensor) -> Tensor:
    if values.ndim != 2 or not torch.is_floating_point(values):
        raise TypeError("block Hadamard input must be a floating point matrix")
    if not values.is_cuda:
        raise ValueError("the B200 coupled transforms require CUDA tensors")
    return values.float().contiguous().clone()


def block_hadamard(values: Tensor, *, block_size: int, dim: int = -1) -> Tensor:
    """Normalised self-inverse block Walsh-Hadamard along ``dim`` of a matrix."""

    if block_size <= 0 or block_size & (block_size - 1):
        raise ValueError("block_size must be a positive power of two")
    axis = dim % 2
    if values.shape[axis] % block_size:
        raise ValueError("Hadamard axis must be divisible by block_size")
    if values.numel() == 0:
        return values.float().contiguous().clone()
    return _transform_(_as_work_matrix(values), axis, block_size, None, False)


def signed_block_hadamard(values: Tensor, *, block_size: int, signs: Tensor, dim: int = -1,
                          inverse: bool = False) -> Tensor:
    """``D H`` on row vectors, or its exact inverse ``H D``."""

    axis = dim % 2
    if signs.ndim != 1 or signs.numel() != values.shape[axis]:
        raise ValueError("rotation signs do not align with the transformed axis")
    if values.shape[axis] % block_size:
        raise ValueError("Hadamard axis must be divisible by block_size")
    if values.numel() == 0:
        return values.float().contiguous().clone()
    return _transform_(_as_work_matrix(values), axis, block_size, signs, inverse)


def _validate_triplet(weights: WeightTriplet) -> tuple[int, int]:
    w1, w3, w2 = weights
    if w1.ndim != 2 or w3.ndim != 2 or w2.ndim != 2 or w1.shape != w3.shape:
        raise ValueError("coupled weights require matching two-dimensional w1/w3")
    intermediate, hidden = w1.shape
    if tuple(w2.shape) != (hidden, intermediate):
        raise ValueError("w2 must have shape [hidden, intermediate]")
    if not all(torch.is_floating_point(value) for value in weights):
        raise TypeError("coupled weights must be floating point")
    if len({value.device for value in weights}) != 1:
        raise ValueError("coupled weights must share one device")
    return intermediate, hidden


def encode_coupled_weights(weights: WeightTriplet, spec: CoupledHadamardSpec) -> WeightTriplet:
    """Reparameterise one full-precision expert into coupled coordinates (:145-196)."""

    w1, w3, w2 = weights
    intermediate, hidden = _validate_triplet(weights)
    if hidden % spec.residual_block_size:
        raise ValueError("hidden size does not close residual Hadamard blocks")
    if 2 * intermediate % spec.preactivation_block_size:
        raise ValueError("interleaved size does not close preactivation blocks")
    if intermediate % spec.postactivation_block_size:
        raise ValueError("intermediate size does not close postactivation blocks")
    device = w1.device
    input_signs = rotation_signs(hidden, draw=spec.residual_draw, axis=0, device=device)
    pre_signs = rotation_signs(2 * intermediate, draw=spec.intermediate_draw, axis=1, device=device)
    post_signs = rotation_signs(intermediate, draw=spec.intermediate_draw, axis=2, device=device)
    output_signs = rotation_signs(hidden, draw=spec.residual_draw, axis=3, device=device)
    upstream = torch.stack((w1.float(), w3.float()), dim=1).reshape(2 * intermediate, hidden).contiguous()
    _transform_(upstream, 1, spec.residual_block_size, input_signs, False)
    _transform_(upstream, 0, spec.preactivation_block_size, pre_signs, False)
    down = w2.float().contiguous().clone()
    _transform_(down, 1, spec.postactivation_block_size, post_signs, False)
    _transform_(down, 0, spec.residual_block_size, output_signs, False)
    return upstream[:intermediate].contiguous(), upstream[intermediate:].contiguous(), down


def encode_coupled_weights_mxfp4(sources, spec: CoupledHadamardSpec, *, round_bf16: bool = True) -> WeightTriplet:
    """``encode_coupled_weights`` for an expert still in its MXFP4 source storage.

    ``sources`` = ``((w1_packed, w1_scale), (w3_packed, w3_scale), (w2_packed, w2_scale))`` with
    packed codes ``[out, in / 2]`` and E8M0 scales ``[out, in / 32]`` (qsrt/io/mxfp4.py:1-63).  The
    dequantiser is fused into the first transform of each matrix (``qsrtb_mxfp4_signed_block_hadamard``):
    the gate and up rows go straight into the interleaved ``[2 I, Hd]`` stack in residual
    coordinates, the down rows into post-activation coordinates; the remaining column-axis
    transforms run in place as in ``encode_coupled_weights``.  With ``round_bf16`` every
    dequantised value is first rounded to bfloat16, the precision in which the source checkpoint
    is held.  Bit-identical to dequantising and calling ``encode_coupled_weights``."""

    (p1, s1), (p3, s3), (p2, s2) = sources
    for packed, scale in sources:
        if packed.dtype != torch.uint8 or scale.dtype != torch.uint8 or packed.ndim != 2 or scale.ndim != 2:
            raise TypeError("MXFP4 sources are uint8 matrices of packed codes and block scales")
        if not packed.is_cuda or scale.device != packed.device:
            raise ValueError("the B200 coupled transforms require CUDA tensors")
        if scale.shape != (packed.shape[0], packed.shape[1] * 2 // 32):
            raise ValueError("scale blocks do not cover the packed codes")
    intermediate, hidden = p1.shape[0], p1.shape[1] * 2
    if p3.shape != p1.shape or tuple(p2.shape) != (hidden, intermediate // 2):
        raise ValueError("coupled weights require matching w1/w3 and w2 [hidden, intermediate]")
    if hidden % spec.residual_block_size:
        raise ValueError("hidden size does not close residual Hadamard blocks")
    if 2 * intermediate % spec.preactivation_block_size:
        raise ValueError("interleaved size does not close preactivation blocks")
    if intermediate % spec.postactivation_block_size:
        raise ValueError("intermediate size does not close postactivation blocks")
    device = p1.device
    input_signs = rotation_signs(hidden, draw=spec.residual_draw, axis=0, device=device)
    pre_signs = rotation_signs(2 * intermediate, draw=spec.intermediate_draw, axis=1, device=device)
    post_signs = rotation_signs(intermediate, draw=spec.intermediate_draw, axis=2, device=device)
    output_signs = rotation_signs(hidden, draw=spec.residual_draw, axis=3, device=device)

    def ingest(packed, scale, out, row_step, row_offset, block, signs):
        packed, scale = packed.contiguous(), scale.contiguous()
        with torch.cuda.device(device):
            _lib.check(
                _lib.lib().qsrtb_mxfp4_signed_block_hadamard(
                    packed.data_ptr(), scale.data_ptr(), packed.shape[0], packed.shape[1] * 2, out.data_ptr(),
                    out.stride(0), row_step, row_offset, block, signs.data_ptr(), int(round_bf16), _stream_ptr(device)),
                "qsrtb_mxfp4_signed_block_hadamard")

    upstream = torch.empty((2 * intermediate, hidden), dtype=torch.float32, device=device)
    ingest(p1, s1, upstream, 2, 0, spec.residual_block_size, input_signs)
    ingest(p3, s3, upstream, 2, 1, spec.residual_block_size, input_signs)
    _transform_(upstream, 0, spec.preactivation_block_size, pre_signs, False)
    down = torch.empty((hidden, intermediate), dtype=torch.float32, device=device)
    ingest(p2, s2, down, 1, 0, spec.postactivation_block_size, post_signs)
    _transform_(down, 0, spec.residual_block_size, output_signs, False)
    return upstream[:intermediate].contiguous(), upstream[intermediate:].contiguous(), down


@dataclass(frozen=True)
class CoupledHadamardExecution:
    """Calibration and scoring operations for one transformed expert basis (:347-543)."""

    hidden: int
    intermediate: int
    spec: CoupledHadamardSpec

    def _signs(self, axis: int, *, device: torch.device) -> Tensor:
        lengths = (self.hidden, 2 * self.intermediate, self.intermediate, self.hidden)
        draw = self.spec.residual_draw if axis in (0, 3) else self.spec.intermediate_draw
        return rotation_signs(lengths[axis], draw=draw, axis=axis, device=device)

    def transform_inputs(self, rows: Tensor) -> Tensor:
        if rows.ndim != 2 or rows.shape[1] != self.hidden:
            raise ValueError("input rows do not match the hidden dimension")
        return signed_block_hadamard(rows, block_size=self.spec.residual_block_size,
                                     signs=self._signs(0, device=rows.device), dim=1)

    def transform_postactivation_rows(self, rows: Tensor) -> Tensor:
        if rows.ndim != 2 or rows.shape[1] != self.intermediate:
            raise ValueError("postactivation rows do not match the intermediate dimension")
        return signed_block_hadamard(rows, block_size=self.spec.postactivation_block_size,
                                     signs=self._signs(2, device=rows.device), dim=1)

    def _congruence(self, hessian: Tensor, axis_id: int, block: int) -> Tensor:
        signs = self._signs(axis_id, device=hessian.device)
        work = _as_work_matrix(hessian)
        _transform_(work, 0, block, signs, False)
        _transform_(work, 1, block, signs, False)
        return work

    def transform_h13(self, hessian: Tensor) -> Tensor:
        if tuple(hessian.shape) != (self.hidden, self.hidden):
            raise ValueError("H13 does not match the hidden dimension")
        return self._congruence(hessian, 0, self.spec.residual_block_size)

    def transform_h2(self, hessian: Tensor) -> Tensor:
        if tuple(hessian.shape) != (self.intermediate, self.intermediate):
            raise ValueError("H2 does not match the intermediate dimension")
        return self._congruence(hessian, 2, self.spec.postactivation_block_size)

    def transform_output_hessian(self, hessian: Tensor) -> Tensor:
        if tuple(hessian.shape) != (self.hidden, self.hidden):
            raise ValueError("output Hessian does not match the hidden dimension")
        return self._congruence(hessian, 3, self.spec.residual_block_size)

    def decode_middle(self, rows: Tensor, w1: Tensor, w3: Tensor, activation: str = "situ") -> Tensor:
        transformed = _matmul_nt(rows, torch.cat((w1, w3), dim=0))
        recovered = _transform_(transformed.float(), 1, self.spec.preactivation_block_size,
                                self._signs(1, device=rows.device), True)
        gate, up = recovered[:, 0::2], recovered[:, 1::2]
        middle = situ(gate, up) if activation == "situ" else torch.nn.functional.silu(gate) * up
        return signed_block_hadamard(middle, block_size=self.spec.postactivation_block_size,
                                     signs=self._signs(2, device=rows.device), dim=1)

    def decode_output(self, transformed: Tensor) -> Tensor:
        if transformed.ndim != 2 or transformed.shape[1] != self.hidden:
            raise ValueError("output rows do not match the hidden dimension")
        return signed_block_hadamard(transformed, block_size=self.spec.residual_block_size,
                                     signs=self._signs(3, device=transformed.device), dim=1, inverse=True)

    def execute(self, rows: Tensor, weights: WeightTriplet, activation: str = "situ") -> Tensor:
        _validate_triplet(weights)
        transformed_rows = self.transform_inputs(rows)
        middle = self.decode_middle(transformed_rows, weights[0], weights[1], activation)
        return self.decode_output(_matmul_nt(middle, weights[2]))
