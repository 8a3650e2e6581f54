"""Pin the CPU oracle against outputs of the reference's own implementation (golden .npz
written by tests/golden/make_golden.py from BatchedACE / chunked_forward)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import draw_kvq
from oracle import race_oracle as ro

FULL_CASES = ["small_k4l4", "small_k2l2", "small_k5l1", "small_k6l8_d128", "mb_k3l2_d32"]


def _cfg(golden, name):
    M, B, H, dk, K, L, T, stride = (int(x) for x in golden[f"{name}/cfg"])
    return M, B, H, dk, K, L, T, stride


@pytest.mark.parametrize("name", FULL_CASES)
def test_operator_matches_reference_bitwise(golden, name):
    # Same ATen ops in the same order on the same inputs: the restatement must reproduce the
    # reference's output exactly (chunk >= T degenerates to it, src/test_equivalence.py:50).
    M, B, H, dk, K, L, T, _ = _cfg(golden, name)
    Kh, Vh, Qh = (torch.from_numpy(golden[f"{name}/{k}"]) for k in "KVQ")
    planes_T = torch.from_numpy(golden[f"{name}/planes_T"])
    protos_T = torch.from_numpy(golden[f"{name}/protos_T"])
    assert torch.equal(protos_T, ro.make_protos(K, protos_T.dtype))
    got = ro.batched_ace_forward(planes_T, protos_T, Kh, Vh, Qh, L, K)
    ref = torch.from_numpy(golden[f"{name}/out"])
    assert got.shape == ref.shape
    tol = 0.0 if ref.dtype == torch.float64 else 1e-6
    assert (got - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())


def test_seeded_buffers_match_reference(golden):
    # planes drawn after torch.manual_seed(1234) (src/test_equivalence.py:28)
    M, B, H, dk, K, L, T, _ = _cfg(golden, "small_k4l4")
    torch.manual_seed(1234)
    planes_T = ro.make_planes(dk, K, L)
    assert np.array_equal(planes_T.numpy(), golden["small_k4l4/planes_T"])
    Kh, Vh, Qh = draw_kvq(M, B, T, H, dk, torch.float32)
    assert np.array_equal(Kh.numpy(), golden["small_k4l4/K"])
    assert np.array_equal(Qh.numpy(), golden["small_k4l4/Q"])


def test_config1_matches_reference(golden):
    # the reference benchmark configuration: N=8, T=4096, d_k=64, L=4, K=4, fp32; stored every 64th token.
    M, B, H, dk, K, L, T, stride = _cfg(golden, "c1_t4096")
    Kh, Vh, Qh = draw_kvq(M, B, T, H, dk, torch.float32)
    planes_T = torch.from_numpy(golden["c1_t4096/planes_T"])
    got = ro.batched_ace_forward(planes_T, ro.make_protos(K), Kh, Vh, Qh, L, K, chunk=1024)
    ref = torch.from_numpy(golden["c1_t4096/out"])
    # carried form vs one cumsum: fp32 accumulation-order noise only (tolerance of
    # src/test_equivalence.py:55, 1e-4 max-abs)
    assert (got[:, :, ::stride] - ref).abs().max().item() <= 1e-4


@pytest.mark.parametrize("T,chunk", [(2048, 300), (2048, 512)])
def test_chunked_matches_reference_chunked(golden, T, chunk):
    name = f"chunked_t{T}_c{chunk}"
    M, B, H, dk, K, L, T_, stride = _cfg(golden, name)
    Kh, Vh, Qh = draw_kvq(M, B, T_, H, dk, torch.float32)
    planes_T = torch.from_numpy(golden[f"{name}/planes_T"])
    got = ro.batched_ace_forward(planes_T, ro.make_protos(K), Kh, Vh, Qh, L, K, chunk=chunk)
    ref = torch.from_numpy(golden[f"{name}/out"])
    assert (got[:, :, ::stride] - ref).abs().max().item() <= 1e-6


def test_probs_level_equals_operator():
    # bridge: BatchedACE(K,V,Q) == causal_prefix(probs(Q), probs(K), V) bit for bit
    torch.manual_seed(1234)
    dk, K, L = 64, 4, 4
    planes_T, protos_T = ro.make_planes(dk, K, L), ro.make_protos(K)
    Kh, Vh, Qh = draw_kvq(1, 1, 128, 4, dk, torch.float32)
    full = ro.batched_ace_forward(planes_T, protos_T, Kh, Vh, Qh, L, K)
    pK = ro.bucket_probs(ro.to_streams(Kh), planes_T, protos_T, L, K)
    pQ = ro.bucket_probs(ro.to_streams(Qh), planes_T, protos_T, L, K)
    out = ro.causal_prefix(pQ, pK, ro.to_streams(Vh))
    assert torch.equal(ro.from_streams(out, 1, 1, 4), full)


@pytest.mark.parametrize("T,chunk,tol,dtype", [
    (512, 512, 0.0, torch.float32), (1024, 300, 1e-4, torch.float32),
    (512, 1, 1e-4, torch.float32), (1024, 300, 1e-12, torch.float64),
    (256, 1, 1e-12, torch.float64)])
def test_chunked_equals_unchunked(T, chunk, tol, dtype):
    # the reference's equivalence claims (src/test_equivalence.py:49-63) for the oracle itself
    pQ, pK, V = ro.synthetic_probs(4, T, 4, 16, 64, seed=3, dtype=dtype)
    a = ro.causal_prefix(pQ, pK, V)
    b, A, B = ro.causal_prefix_chunked(pQ, pK, V, chunk=chunk, return_state=True)
    assert (a - b).abs().max().item() <= tol
    At, Bt = ro.tile_totals(pK, V)
    assert torch.allclose(A, At, rtol=1e-5, atol=1e-5)
    assert torch.allclose(B, Bt, rtol=1e-4, atol=1e-4)


def test_known_answers():
    # T = 1: O_0 = v_0 * sum_s pQ*pK/(pK+eps)  (~ L * v_0: no 1/L in this estimator,
    # docs/causal_v2_design.md:86); constant V = c gives ~ L * c at every token.
    pQ, pK, V = ro.synthetic_probs(2, 1, 4, 16, 8, seed=5, dtype=torch.float64)
    out = ro.causal_prefix(pQ, pK, V)
    w = (pQ * pK / (pK + ro.EPS)).sum(dim=(2, 3))
    assert torch.allclose(out, V * w.unsqueeze(-1), atol=1e-14)
    pQ, pK, V = ro.synthetic_probs(2, 64, 4, 16, 8, seed=6, dtype=torch.float64)
    V = torch.full_like(V, 0.75)
    out = ro.causal_prefix(pQ, pK, V)
    assert (out - 4 * 0.75).abs().max().item() < 1e-3


def test_causality():
    # outputs up to t do not change when later keys/values change (method of
    # src/causal_v2/tests/test_reference.py:133-150, restated for this estimator)
    pQ, pK, V = ro.synthetic_probs(2, 96, 2, 8, 16, seed=7, dtype=torch.float64)
    a = ro.causal_prefix(pQ, pK, V)
    pK2, V2 = pK.clone(), V.clone()
    pK2[:, 50:] = torch.softmax(torch.randn(2, 46, 2, 8, dtype=torch.float64), -1)
    V2[:, 50:] = 9.0
    b = ro.causal_prefix(pQ, pK2, V2)
    assert torch.equal(a[:, :50], b[:, :50]) and not torch.equal(a[:, 50:], b[:, 50:])


def test_noncausal_closed_form_matches_autograd():
    pQ, pK, V = ro.synthetic_probs(3, 40, 2, 8, 16, seed=8, dtype=torch.float64)
    dO = torch.randn(3, 40, 16, dtype=torch.float64, generator=torch.Generator().manual_seed(9))
    g1 = ro.noncausal_backward_closed_form(pQ, pK, V, dO)
    g2 = ro.noncausal_backward_autograd(pQ, pK, V, dO)
    for a, b in zip(g1, g2):
        assert (a - b).abs().max().item() < 1e-11
    # last causal token sees every key: equals the non-causal output at that token
    last = ro.causal_prefix(pQ, pK, V)[:, -1]
    assert torch.allclose(last, ro.noncausal_forward(pQ, pK, V)[:, -1], atol=1e-12)


from conftest import GLOBAL_CASES, global_case  # noqa: E402


@pytest.mark.parametrize("name", GLOBAL_CASES)
def test_global_form_matches_reference(golden_global, name):
    # the restatement of src/causal_v2/reference.py:106-127 against that function's own output
    pQ, pK, V, ref = global_case(golden_global, name)
    tol = 1e-12 if ref.dtype == torch.float64 else 1e-5
    for chunk in (256, 33):
        got = ro.causal_prefix_global(pQ, pK, V, chunk=chunk)
        assert ro.rel_l2(got, ref) <= tol
    # carried state: two halves equal one pass
    h = pQ.shape[1] // 2
    o1, A, B = ro.causal_prefix_global(pQ[:, :h], pK[:, :h], V[:, :h], return_state=True)
    o2 = ro.causal_prefix_global(pQ[:, h:], pK[:, h:], V[:, h:], carry=(A, B))
    assert ro.rel_l2(torch.cat([o1, o2], 1), ref) <= tol


@pytest.mark.parametrize("N,T,L,R,dk", [(2, 70, 4, 16, 64), (1, 33, 2, 4, 8), (2, 20, 8, 64, 16)])
def test_causal_closed_form_matches_autograd(N, T, L, R, dk):
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=T, dtype=torch.float64)
    dO = torch.randn(N, T, dk, generator=torch.Generator().manual_seed(T + 1), dtype=torch.float64)
    got = ro.causal_backward_closed_form(pQ, pK, V, dO)
    ref = ro.causal_backward_autograd(pQ, pK, V, dO)
    for g, r in zip(got, ref):
        assert ro.rel_l2(g, r) <= 1e-12


@pytest.mark.parametrize("name", ["grad_k4l4", "grad_k3l2_d32"])
def test_oracle_gradients_match_reference_autograd(name):
    """The restated operator under torch.autograd reproduces the reference module's own gradients
    w.r.t. K, V, Q (fixture written by tests/golden/make_golden_grad.py, fp64)."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "race_grad_golden.npz"))
    M, B, H, dk, K, L, T = (int(x) for x in g[f"{name}/cfg"])
    planes_T = torch.from_numpy(g[f"{name}/planes_T"])
    Kh, Vh, Qh = (torch.from_numpy(g[f"{name}/{k}"]).requires_grad_(True) for k in "KVQ")
    out = ro.batched_ace_forward(planes_T, ro.make_protos(K, torch.float64), Kh, Vh, Qh, L, K)
    assert (out - torch.from_numpy(g[f"{name}/out"])).abs().max().item() <= 1e-12
    out.backward(torch.from_numpy(g[f"{name}/dO"]))
    for t, key in ((Kh, "dK"), (Vh, "dV"), (Qh, "dQ")):
        assert ro.rel_l2(t.grad, torch.from_numpy(g[f"{name}/{key}"])) <= 1e-12, key
