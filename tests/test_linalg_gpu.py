"""Tensor-core products and the on-device Cholesky against float64 (torch on the same device).

Tolerances: a float32 product summed in a different order than float64 agrees to a few 1e-7
relative Frobenius; the three-product TF32 scheme drops the tail-times-tail term (2^-22 relative
per product), so 3e-6 is asserted for products and 1e-5 (the bound the encoder tests put on the
feedback factor's input) for the factorisation of moderately conditioned matrices.
"""

import numpy as np
import pytest
import torch

from qsrt_b200 import linalg

pytestmark = pytest.mark.gpu


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-300))


def test_split_gives_exact_tf32_head_and_small_tail(cuda_device):
    g = torch.Generator().manual_seed(1)
    x = (torch.randn((70, 100), generator=g) * torch.exp(2.0 * torch.randn((70, 100), generator=g))).to(cuda_device)
    planes = linalg.split_tf32(x)
    assert planes.hi.shape == x.shape
    assert int((planes.hi.view(torch.int32) & 0x1FFF).abs().max()) == 0     # 10 mantissa bits kept
    assert int((planes.lo.view(torch.int32) & 0x1FFF).abs().max()) == 0
    assert float(((planes.hi.double() + planes.lo.double() - x.double()).abs() / x.double().abs()).max()) < 2.0 ** -21
    turned = linalg.split_tf32(x, transpose=True)
    assert torch.equal(turned.hi, planes.hi.T) and torch.equal(turned.lo, planes.lo.T)
    stack = torch.stack([x, 2 * x, -x])
    batched = linalg.split_tf32(stack, transpose=True)
    assert torch.equal(batched.hi[1], (2 * planes.hi).T) and torch.equal(batched.lo[2], (-planes.lo).T)
    # a slice of a wider matrix
    wide = torch.zeros((70, 228), device=cuda_device)
    wide[:, 64:164] = x
    assert torch.equal(linalg.split_tf32(wide[:, 64:164]).hi, planes.hi)


@pytest.mark.parametrize("m,n,k", [(128, 128, 32), (256, 384, 128), (200, 132, 100), (1000, 640, 2048), (64, 16, 96)])
def test_product_matches_float64(cuda_device, m, n, k):
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn((m, k), generator=g).to(cuda_device)
    b = (torch.randn((n, k), generator=g) * torch.exp(torch.randn(k, generator=g))).to(cuda_device)
    want = a.double() @ b.double().T
    pa, pb = linalg.split_tf32(a), linalg.split_tf32(b)
    out = torch.full((m, n), float("nan"), device=cuda_device)
    linalg.gemm_nt(pa, pb, out)
    linalg.check_status(cuda_device)
    assert _rel(out, want) < 3e-6
    # alpha / beta and the transposed store
    base = torch.randn((n, m), generator=g).to(cuda_device)
    out_t = base.clone()
    linalg.gemm_nt(pa, pb, out_t, alpha=-0.5, beta=2.0, transposed_out=True)
    assert _rel(out_t, -0.5 * want.T + 2.0 * base.double()) < 3e-6
    # the plain convenience entry
    assert _rel(linalg.matmul_nt(a, b), want) < 3e-6


def test_product_on_views_batches_and_lower_tiles(cuda_device):
    g = torch.Generator().manual_seed(9)
    big = torch.randn((3, 300, 512), generator=g).to(cuda_device)
    planes = linalg.split_tf32(big)
    # stack of three, operands are column slices (k = 128 of 512) of the planes, output a row slice
    a = linalg.Planes(planes.hi[:, :256, 128:256], planes.lo[:, :256, 128:256])
    b = linalg.Planes(planes.hi[:, 44:300, 256:384], planes.lo[:, 44:300, 256:384])
    out_full = torch.zeros((3, 300, 256), device=cuda_device)
    out = out_full[:, 20:276]
    linalg.gemm_nt(a, b, out)
    want = torch.bmm(big[:, :256, 128:256].double(), big[:, 44:300, 256:384].double().transpose(1, 2))
    assert _rel(out, want) < 3e-6
    assert float(out_full[:, :20].abs().max()) == 0.0 and float(out_full[:, 276:].abs().max()) == 0.0
    # symmetric rank-k update on the lower tiles only: tiles above the diagonal stay untouched
    x = torch.randn((384, 128), generator=g).to(cuda_device)
    px = linalg.split_tf32(x)
    c = torch.ones((384, 384), device=cuda_device)
    linalg.gemm_nt(px, px, c, alpha=-1.0, beta=1.0, lower_only=True)
    want = 1.0 - x.double() @ x.double().T
    for bi in range(3):
        for bj in range(3):
            block = c[bi * 128:(bi + 1) * 128, bj * 128:(bj + 1) * 128]
            if bj <= bi:
                assert _rel(block, want[bi * 128:(bi + 1) * 128, bj * 128:(bj + 1) * 128]) < 3e-6
            else:
                assert float((block - 1.0).abs().max()) == 0.0
    linalg.check_status(cuda_device)


def _spd(n, seed, device):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((n + n // 2, n), generator=g) * torch.exp(0.5 * torch.randn(n, generator=g))
    h = (x.T @ x / x.shape[0]).float()
    h.diagonal().add_(0.025 * h.diagonal().mean())
    return h.to(device)


@pytest.mark.parametrize("n", [16, 128, 144, 384, 528, 2048])
def test_cholesky_matches_float64(cuda_device, n):
    h = _spd(n, 100 + n, cuda_device)
    want = torch.linalg.cholesky(h.double())
    # the strict upper triangle must not be read: poison it
    work = torch.where(torch.tril(torch.ones_like(h)) > 0, h, torch.full_like(h, float("nan")))
    info = linalg.cholesky_(work)
    assert info == 0
    got = torch.tril(work)
    assert not torch.isnan(got).any()
    assert _rel(got, want) < 1e-5
    assert _rel(got.double() @ got.double().T, h) < 2e-6


def test_cholesky_reports_the_failing_column_and_keeps_the_context(cuda_device):
    h = _spd(512, 7, cuda_device)
    bad = h.clone()
    bad[300, 300] = -1.0
    info = linalg.cholesky_(bad)
    assert info == 301
    nan = h.clone()
    nan[5, 5] = float("nan")
    assert linalg.cholesky_(nan) == 6
    # the device is fine afterwards: the same call on the good matrix succeeds
    good = h.clone()
    assert linalg.cholesky_(good) == 0
    assert _rel(torch.tril(good), torch.linalg.cholesky(h.double())) < 1e-5
    assert linalg.cholesky_(torch.zeros((0, 0), device=cuda_device)) == 0
