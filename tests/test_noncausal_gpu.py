"""GPU parity of the non-causal forward/backward and of the bucket-probability producer."""
from __future__ import annotations

import pytest
import torch

from oracle import race_oracle as ro

pytestmark = pytest.mark.gpu


def _rk():
    import race_attention_kernel_b200 as rk
    return rk


SHAPES = [(4, 4096, 4, 16, 64), (3, 1, 4, 16, 64), (2, 33, 4, 16, 64), (2, 1000, 2, 4, 64),
          (2, 300, 1, 32, 64), (2, 200, 2, 8, 32), (2, 300, 4, 16, 128), (2, 300, 8, 64, 128)]


@pytest.mark.parametrize("N,T,L,R,dk", SHAPES)
def test_forward_backward_fp32(N, T, L, R, dk):
    rk = _rk()
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=T + dk)
    dO = torch.randn(N, T, dk, generator=torch.Generator().manual_seed(2))
    ref = ro.noncausal_forward(pQ.double(), pK.double(), V.double())
    g_ref = ro.noncausal_backward_autograd(pQ.double(), pK.double(), V.double(), dO.double())
    q, k, v = (t.cuda().requires_grad_(True) for t in (pQ, pK, V))
    out = rk.race_noncausal(q, k, v)
    assert ro.rel_l2(out, ref) <= 1e-4
    out.backward(dO.cuda())
    # dPK = V.dBs + dA cancels almost completely when a bucket holds very few keys (T = 1: E = V
    # up to eps), so its error is judged against the size of the two terms, not of their difference
    S = L * R
    A = pK.double().reshape(N, T, S).sum(1)
    dBs = pQ.double().reshape(N, T, S).transpose(1, 2).bmm(dO.double()) / (A.unsqueeze(-1) + 1e-6)
    term = V.double().bmm(dBs.transpose(1, 2)).norm().item()
    for got, want, name in zip((q.grad, k.grad, v.grad), g_ref, ("dPQ", "dPK", "dV")):
        if name == "dPK":
            err = (got.double().cpu() - want).norm().item()
            assert err <= 1e-4 * max(term, want.norm().item()), name
        else:
            assert ro.rel_l2(got, want) <= 1e-4, name


@pytest.mark.parametrize("N,T,L,R,dk", [(4, 4096, 4, 16, 64), (2, 300, 8, 64, 128)])
def test_forward_backward_bf16(N, T, L, R, dk):
    rk = _rk()
    pQ, pK, V = (t.bfloat16() for t in ro.synthetic_probs(N, T, L, R, dk, seed=3))
    dO = torch.randn(N, T, dk, generator=torch.Generator().manual_seed(4)).bfloat16()
    ref = ro.noncausal_forward(pQ.double(), pK.double(), V.double())
    g_ref = ro.noncausal_backward_autograd(pQ.double(), pK.double(), V.double(), dO.double())
    q, k, v = (t.cuda().requires_grad_(True) for t in (pQ, pK, V))
    out = rk.race_noncausal(q, k, v)
    assert out.dtype == torch.bfloat16 and ro.rel_l2(out, ref) <= 2e-2
    out.backward(dO.cuda())
    for got, want in zip((q.grad, k.grad, v.grad), g_ref):
        assert ro.rel_l2(got, want) <= 2e-2


def test_expanded_gradient_and_partial_needs():
    rk = _rk()
    pQ, pK, V = (t.cuda() for t in ro.synthetic_probs(2, 100, 4, 16, 64, seed=9))
    v = V.clone().requires_grad_(True)
    rk.race_noncausal(pQ, pK, v).sum().backward()      # stride-0 expanded ones as grad
    _, _, dV = ro.noncausal_backward_autograd(pQ.double().cpu(), pK.double().cpu(), V.double().cpu(),
                                              torch.ones(2, 100, 64, dtype=torch.float64))
    assert ro.rel_l2(v.grad, dV) <= 1e-4


def test_last_causal_token_equals_noncausal():
    rk = _rk()
    pQ, pK, V = (t.cuda() for t in ro.synthetic_probs(3, 500, 4, 16, 64, seed=10))
    a = rk.race_causal_prefix(pQ, pK, V)[:, -1]
    b = rk.race_noncausal(pQ, pK, V)[:, -1]
    assert ro.rel_l2(a, b) <= 1e-5


@pytest.mark.parametrize("dk,K,L,rows", [(64, 4, 4, 1000), (64, 2, 2, 77), (64, 5, 1, 64),
                                         (128, 6, 8, 130), (32, 3, 2, 1), (64, 1, 3, 50), (128, 6, 8, 20007)])
def test_bucket_probs(dk, K, L, rows):
    rk = _rk()
    torch.manual_seed(1234)
    planes_T, protos_T = ro.make_planes(dk, K, L), ro.make_protos(K)
    x = torch.randn(1, rows, dk, generator=torch.Generator().manual_seed(0))
    ref = ro.bucket_probs(x.double(), planes_T.double(), protos_T.double(), L, K)
    got = rk.bucket_probs(x.cuda(), planes_T.T.contiguous().cuda(), L, K)
    assert got.shape == ref.shape
    assert ro.rel_l2(got, ref) <= 1e-5
    assert torch.allclose(got.sum(-1).cpu(), torch.ones(1, rows, L), atol=1e-5)
    got16 = rk.bucket_probs(x.bfloat16().cuda(), planes_T.T.contiguous().cuda(), L, K)
    ref16 = ro.bucket_probs(x.bfloat16().double(), planes_T.double(), protos_T.double(), L, K)
    assert got16.dtype == torch.bfloat16 and ro.rel_l2(got16, ref16) <= 1e-2


def test_bucket_probs_wide_geometry_mixed_dtypes():
    """The tensor-core producer of the d_k = 128, L = 8, K = 6 geometry: fp32 rows to bf16 probabilities and bf16
    rows to fp32 probabilities, a row count that is no multiple of the 16-row blocks, and rows past one grid pass."""
    rk = _rk()
    dk, K, L, rows = 128, 6, 8, 70003
    torch.manual_seed(1234)
    planes_T, protos_T = ro.make_planes(dk, K, L), ro.make_protos(K)
    planes = planes_T.T.contiguous().cuda()
    x = torch.randn(1, rows, dk, generator=torch.Generator().manual_seed(3))
    ref = ro.bucket_probs(x[:, -3000:].double(), planes_T.double(), protos_T.double(), L, K)
    got = rk.bucket_probs(x.cuda(), planes, L, K, out_dtype=torch.bfloat16)
    assert got.dtype == torch.bfloat16 and ro.rel_l2(got[:, -3000:], ref) <= 1e-2
    xb = x.bfloat16()
    refb = ro.bucket_probs(xb[:, -3000:].double(), planes_T.double(), protos_T.double(), L, K)
    gotb = rk.bucket_probs(xb.cuda(), planes, L, K, out_dtype=torch.float32)
    assert gotb.dtype == torch.float32 and ro.rel_l2(gotb[:, -3000:], refb) <= 1e-5
    assert torch.allclose(gotb.sum(-1).cpu(), torch.ones(1, rows, L), atol=1e-5)


@pytest.mark.parametrize("M,B,T,H,dk,K,L", [(1, 1, 300, 8, 64, 4, 4), (2, 2, 37, 3, 32, 3, 2), (1, 2, 130, 2, 128, 6, 8),
                                            (1, 1, 257, 1, 64, 1, 3), (2, 1, 1, 4, 64, 2, 2)])
def test_bucket_probs_streams(M, B, T, H, dk, K, L):
    """The producer reading the operator layout [M,B,T,H,d_k] equals flatten-then-produce
    (src/race_baseline.py:35-44), bit for bit, and matches the oracle."""
    rk = _rk()
    torch.manual_seed(1234)
    planes_T, protos_T = ro.make_planes(dk, K, L), ro.make_protos(K)
    x = torch.randn(M, B, T, H, dk, generator=torch.Generator().manual_seed(5))
    planes = planes_T.T.contiguous().cuda()
    got = rk.bucket_probs_streams(x.cuda(), planes, L, K)
    x2 = ro.to_streams(x)
    flat = rk.bucket_probs(x2.cuda().contiguous(), planes, L, K)
    assert got.shape == (M * B * H, T, L, 1 << K)
    assert torch.equal(got, flat)
    ref = ro.bucket_probs(x2.double(), planes_T.double(), protos_T.double(), L, K)
    assert ro.rel_l2(got, ref) <= 1e-5
