"""GPU parity tests of the causal forward that forms the bucket probabilities inside the prefix kernels
(race_b200_causal_fwd_qkv), through the C-ABI, against the CPU oracle of the whole operator
(src/race_baseline.py:34-52) and against the two-step path (producer kernel, then prefix kernels).

Tolerance: rel-L2 <= 1e-4 against the fp64 oracle (fp32 path)."""
from __future__ import annotations

import pytest
import torch

from oracle import race_oracle as ro

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
L, K, R, DK = 4, 4, 16, 64


def _ops():
    import race_attention_kernel_b200 as rk
    return rk


def _planes(seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(L * K, DK, generator=g)          # [L*K, d_k] = planes_T.T


def _draw(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(shape, generator=g) for _ in range(3)]


def _oracle_streams(Q, Kx, V, planes, carry=None, return_state=False):
    pT, protos = planes.T.double().contiguous(), ro.make_protos(K, torch.float64)
    pQ = ro.bucket_probs(Q.double(), pT, protos, L, K)
    pK = ro.bucket_probs(Kx.double(), pT, protos, L, K)
    return ro.causal_prefix(pQ, pK, V.double(), carry=carry, return_state=return_state)


@pytest.mark.parametrize("N,T", [(2, 1), (3, 63), (2, 64), (3, 65), (2, 1000), (1, 2048), (2, 2049), (8, 4096),
                                 (1, 20000)])
def test_qkv_matches_operator_oracle(N, T):
    rk = _ops()
    planes = _planes(7)
    Q, Kx, V = _draw((N, T, DK), seed=T)
    assert rk.ops.qkv_is_supported(N, T, L, K, DK)
    out, A, B = rk.ops.race_causal_qkv(Q.cuda(), Kx.cuda(), V.cuda(), planes.cuda(), L, K, return_state=True)
    ref, A_ref, B_ref = _oracle_streams(Q, Kx, V, planes, return_state=True)
    assert ro.rel_l2(out, ref) <= FP32_TOL
    assert ro.rel_l2(A, A_ref) <= 1e-5 and ro.rel_l2(B, B_ref) <= FP32_TOL
    # causality: the outputs of a prefix do not depend on what follows it
    if T >= 65:
        cut = T // 2 + 1
        head = rk.ops.race_causal_qkv(Q[:, :cut].contiguous().cuda(), Kx[:, :cut].contiguous().cuda(),
                                      V[:, :cut].contiguous().cuda(), planes.cuda(), L, K)
        assert ro.rel_l2(head, out[:, :cut]) <= 1e-5


@pytest.mark.parametrize("N,T,tile", [(3, 100, 2048), (2, 2048, 2048), (2, 64, 64), (1, 1024, 1024)])
def test_qkv_single_tile_is_bitwise_the_two_step_path(N, T, tile):
    """With one state tile and no carry nothing but the probabilities differs between the two paths, and those are
    formed by the same instructions: the outputs agree bit for bit."""
    rk = _ops()
    planes = _planes(11).cuda()
    Q, Kx, V = (t.cuda() for t in _draw((N, T, DK), seed=N * T))
    pQ, pK = rk.bucket_probs(Q, planes, L, K), rk.bucket_probs(Kx, planes, L, K)
    two_step = rk.race_causal_prefix(pQ, pK, V, variant="tensor", tile_tokens=tile)
    fused = rk.ops.race_causal_qkv(Q, Kx, V, planes, L, K, tile_tokens=tile)
    assert torch.equal(fused, two_step)


def test_qkv_many_tiles_close_to_the_two_step_path():
    # the running A is summed in another order, nothing else differs: far inside the fp32 tolerance
    rk = _ops()
    planes = _planes(3).cuda()
    Q, Kx, V = (t.cuda() for t in _draw((4, 9000, DK), seed=5))
    pQ, pK = rk.bucket_probs(Q, planes, L, K), rk.bucket_probs(Kx, planes, L, K)
    for norm in ("bucket", "global"):
        two_step, A0, B0 = rk.race_causal_prefix(pQ, pK, V, variant="tensor", tile_tokens=512, return_state=True,
                                                 normalization=norm)
        fused, A1, B1 = rk.ops.race_causal_qkv(Q, Kx, V, planes, L, K, tile_tokens=512, return_state=True,
                                               normalization=norm)
        assert ro.rel_l2(fused, two_step) <= 1e-6, norm
        assert torch.equal(B0, B1) and ro.rel_l2(A1, A0) <= 1e-6


@pytest.mark.parametrize("M,B,T,H", [(1, 1, 4096, 8), (2, 2, 333, 3), (1, 2, 2049, 2)])
def test_qkv_operator_layout(M, B, T, H):
    """Q, K, V and out in the operator's layout [M,B,T,H,d_k]: equal to the call on flattened streams, and to the
    oracle of the whole operator."""
    rk = _ops()
    planes = _planes(5)
    Q5, K5, V5 = _draw((M, B, T, H, DK), seed=H)
    got = rk.ops.race_causal_qkv(Q5.cuda(), K5.cuda(), V5.cuda(), planes.cuda(), L, K)
    assert got.shape == (M, B, T, H, DK)
    flat = rk.ops.race_causal_qkv(*(ro.to_streams(t).cuda() for t in (Q5, K5, V5)), planes.cuda(), L, K)
    assert torch.equal(ro.to_streams(got.cpu()), flat.cpu())
    ref = ro.batched_ace_forward(planes.T.double().contiguous(), ro.make_protos(K, torch.float64), K5.double(),
                                 V5.double(), Q5.double(), L, K)
    assert ro.rel_l2(got, ref) <= FP32_TOL


def test_qkv_chunked_carry_equals_one_call():
    # the carried form of src/race_chunked.py:54-63 over ragged cuts
    rk = _ops()
    planes = _planes(9).cuda()
    N, T = 3, 5000
    Q, Kx, V = (t.cuda() for t in _draw((N, T, DK), seed=1))
    whole, A_w, B_w = rk.ops.race_causal_qkv(Q, Kx, V, planes, L, K, return_state=True)
    carry, parts = None, []
    for a, b in ((0, 1), (1, 700), (700, 4097), (4097, T)):
        o, A, Bs = rk.ops.race_causal_qkv(Q[:, a:b].contiguous(), Kx[:, a:b].contiguous(), V[:, a:b].contiguous(),
                                          planes, L, K, carry_in=carry, return_state=True)
        carry = (A, Bs)
        parts.append(o)
    assert ro.rel_l2(torch.cat(parts, 1), whole) <= 1e-5
    assert ro.rel_l2(carry[0], A_w) <= 1e-6 and ro.rel_l2(carry[1], B_w) <= 1e-5


def test_qkv_global_form_matches_oracle():
    rk = _ops()
    planes = _planes(2)
    Q, Kx, V = _draw((2, 3000, DK), seed=4)
    pT, protos = planes.T.double().contiguous(), ro.make_protos(K, torch.float64)
    ref = ro.causal_prefix_global(ro.bucket_probs(Q.double(), pT, protos, L, K),
                                  ro.bucket_probs(Kx.double(), pT, protos, L, K), V.double())
    got = rk.ops.race_causal_qkv(Q.cuda(), Kx.cuda(), V.cuda(), planes.cuda(), L, K, normalization="global")
    assert ro.rel_l2(got, ref) <= FP32_TOL


def test_qkv_operator_uses_it_and_matches_the_two_step_operator():
    rk = _ops()
    torch.manual_seed(21)
    ace = rk.BatchedACE(DK, K, L, 1).cuda()
    K5, V5, Q5 = (t.cuda() for t in _draw((1, 2, 1500, 4, DK), seed=8))
    fused = ace(K5, V5, Q5)
    ace.fuse_producer = False
    two_step = ace(K5, V5, Q5)
    assert ro.rel_l2(fused, two_step) <= 1e-6
    ref = ro.batched_ace_forward(ace.planes_T.cpu().double(), ace.protos_T.cpu().double(), K5.cpu().double(),
                                 V5.cpu().double(), Q5.cpu().double(), L, K)
    assert ro.rel_l2(fused, ref) <= FP32_TOL


def test_qkv_rejections():
    rk = _ops()
    planes = _planes(1).cuda()
    Q, Kx, V = (t.cuda() for t in _draw((2, 128, DK), seed=0))
    assert not rk.ops.qkv_is_supported(2, 128, 2, 4, DK)            # L = 2
    assert not rk.ops.qkv_is_supported(2, 128, 4, 3, DK)            # K = 3
    assert not rk.ops.qkv_is_supported(2, 128, 4, 4, 128)           # d_k = 128
    assert not rk.ops.qkv_is_supported(2, 128, 4, 4, DK, torch.bfloat16)
    with pytest.raises(RuntimeError):
        rk.ops.race_causal_qkv(Q.bfloat16(), Kx.bfloat16(), V.bfloat16(), planes, L, K)
    with pytest.raises(RuntimeError):
        rk.ops.race_causal_qkv(Q, Kx[:, :64].contiguous(), V, planes, L, K)
    with pytest.raises(RuntimeError):
        rk.ops.race_causal_qkv(Q, Kx, V, planes[:8], L, K)
    with pytest.raises(RuntimeError):
        rk.ops.race_causal_qkv(Q, Kx, V, planes, L, K, tile_tokens=100)      # not a multiple of the chunk
    # an empty sequence passes the carry through
    e = torch.empty(2, 0, DK, device="cuda")
    out, A, Bs = rk.ops.race_causal_qkv(e, e, e, planes, L, K, return_state=True)
    assert out.shape == (2, 0, DK) and float(A.abs().sum()) == 0.0 and float(Bs.abs().sum()) == 0.0
