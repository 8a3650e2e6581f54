"""GPU parity tests of the causal prefix path, through the C-ABI, against the CPU oracle.

Tolerances are the ones the task fixes: rel-L2 <= 1e-4 for fp32; <= 2e-2 for bf16 measured
against the fp32/fp64 oracle evaluated on the same bf16-rounded inputs."""
from __future__ import annotations

import itertools

import numpy as np
import pytest
import torch

from conftest import draw_kvq
from oracle import race_oracle as ro

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
BF16_TOL = 2e-2


def _ops():
    import race_attention_kernel_b200 as rk
    return rk


def _variants(N, T, L, R, dk, dtype):
    rk = _ops()
    return [v for v in ("simt", "tensor", "tensor_single_pass") if rk.is_supported(N, max(T, 1), L, R, dk, dtype, v)]


def _oracle(pQ, pK, V, **kw):
    # fp64 oracle on the identical inputs (chunked: O(chunk) memory)
    return ro.causal_prefix_chunked(pQ.double(), pK.double(), V.double(), chunk=512, **kw)


SHAPES = [
    # N, T, L, R, dk
    (8, 4096, 4, 16, 64),       # config 1 at the probabilities boundary
    (2, 1, 4, 16, 64), (2, 31, 4, 16, 64), (2, 32, 4, 16, 64), (2, 33, 4, 16, 64),
    (2, 63, 4, 16, 64), (2, 64, 4, 16, 64), (2, 65, 4, 16, 64), (3, 127, 4, 16, 64),
    (3, 129, 4, 16, 64), (1, 2047, 4, 16, 64), (1, 2049, 4, 16, 64), (2, 4097, 4, 16, 64),
    (1, 20000, 4, 16, 64),
    (2, 300, 2, 4, 64),         # K=2, L=2: S=8
    (2, 300, 1, 32, 64),        # K=5, L=1
    (3, 150, 2, 8, 32),         # K=3, L=2, d_k=32
    (2, 300, 4, 16, 128),       # d_k=128
    (2, 300, 8, 64, 128),       # config 3's bucket geometry (S=512, cluster of 8 groups)
    (1, 100, 2, 64, 64),        # S=128: two groups
]


@pytest.mark.parametrize("N,T,L,R,dk", SHAPES)
def test_fp32_parity(N, T, L, R, dk):
    rk = _ops()
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=N * 1000 + T)
    ref = _oracle(pQ, pK, V)
    for variant in _variants(N, T, L, R, dk, torch.float32):
        out = rk.race_causal_prefix(pQ.cuda(), pK.cuda(), V.cuda(), variant=variant)
        err = ro.rel_l2(out, ref)
        assert err <= FP32_TOL, f"{variant}: rel-L2 {err:.3e}"
        assert torch.isfinite(out).all()


@pytest.mark.parametrize("N,T,L,R,dk", [(8, 4096, 4, 16, 64), (2, 333, 4, 16, 64),
                                        (2, 300, 8, 64, 128), (2, 257, 4, 16, 128),
                                        (2, 300, 1, 32, 64), (2, 1000, 2, 64, 64), (2, 700, 4, 64, 128),
                                        (3, 5000, 8, 64, 128), (1, 65, 8, 64, 128),
                                        (2, 500, 4, 64, 64), (1, 2177, 8, 64, 64)])
def test_bf16_parity(N, T, L, R, dk):
    rk = _ops()
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=7 + T)
    pQ, pK, V = pQ.bfloat16(), pK.bfloat16(), V.bfloat16()
    ref = _oracle(pQ, pK, V)
    for variant in _variants(N, T, L, R, dk, torch.bfloat16):
        out = rk.race_causal_prefix(pQ.cuda(), pK.cuda(), V.cuda(), variant=variant)
        assert out.dtype == torch.bfloat16
        err = ro.rel_l2(out, ref)
        assert err <= BF16_TOL, f"{variant}: rel-L2 {err:.3e}"


def test_bf16_wide_kernel_under_load():
    """Config 3's geometry (S = 512, d_k = 128, bf16) with full 2048-token tiles (256 items per CTA) and several
    waves of CTAs, so that the roles of the wide tensor kernel drift apart the way they do at the bench size:
    against the CUDA-core kernels on the whole output and against the oracle on the head of one stream."""
    rk = _ops()
    N, T, L, R, dk = 40, 8192, 8, 64, 128
    g = torch.Generator(device="cuda").manual_seed(3)
    pQ = torch.softmax(torch.randn(N, T, L, R, device="cuda", generator=g), -1).bfloat16()
    pK = torch.softmax(torch.randn(N, T, L, R, device="cuda", generator=g), -1).bfloat16()
    V = torch.randn(N, T, dk, device="cuda", generator=g).bfloat16()
    for _ in range(3):   # the status word is checked after every call (conftest sets RACE_B200_CHECK_STATUS)
        out = rk.race_causal_prefix(pQ, pK, V, variant="tensor", tile_tokens=2048)
    ref_simt = rk.race_causal_prefix(pQ, pK, V, variant="simt")
    assert ro.rel_l2(out, ref_simt) <= BF16_TOL
    w = 1536
    ref = _oracle(pQ[:1, :w].cpu(), pK[:1, :w].cpu(), V[:1, :w].cpu())
    assert ro.rel_l2(out[:1, :w], ref) <= BF16_TOL


@pytest.mark.parametrize("L,R,dk", [(8, 64, 128), (4, 64, 64), (2, 64, 128)])
def test_bf16_wide_carry_and_short_tiles(L, R, dk):
    """The wide bf16 tensor kernels (2, 4 and 8 bucket groups) with a carried-in state (the chunked form of
    src/race_chunked.py:54-63) and with tiles of two chunks, so that every tile starts from a scanned carry."""
    rk = _ops()
    N, T = 2, 900
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=77)
    pQ, pK, V = pQ.bfloat16(), pK.bfloat16(), V.bfloat16()
    ref, A_ref, B_ref = _oracle(pQ, pK, V, return_state=True)
    q, k, v = pQ.cuda(), pK.cuda(), V.cuda()
    cut = 385
    o1, A1, B1 = rk.race_causal_prefix(q[:, :cut].contiguous(), k[:, :cut].contiguous(), v[:, :cut].contiguous(),
                                       return_state=True, variant="tensor")
    o2, A2, B2 = rk.race_causal_prefix(q[:, cut:].contiguous(), k[:, cut:].contiguous(), v[:, cut:].contiguous(),
                                       carry_in=(A1, B1), return_state=True, variant="tensor")
    assert ro.rel_l2(torch.cat([o1, o2], dim=1), ref) <= BF16_TOL
    assert ro.rel_l2(A2, A_ref) <= 1e-3 and ro.rel_l2(B2, B_ref) <= 1e-3
    short = rk.race_causal_prefix(q, k, v, variant="tensor", tile_tokens=128)
    assert ro.rel_l2(short, ref) <= BF16_TOL


@pytest.mark.parametrize("tile,L,R,dk", [(64, 8, 64, 128), (256, 8, 64, 128), (256, 4, 64, 64), (128, 2, 64, 128),
                                         (128, 4, 16, 64), (128, 4, 16, 128)])
def test_bf16_tensor_kernels_are_bitwise_reproducible(tile, L, R, dk):
    """Run-to-run bitwise equality of the bf16 tensor kernels (one, two, four and eight bucket groups) with short tiles:
    every CTA then starts cold and reads its first tiles the moment they land, which is where a pQ slot handed back to
    the TMA thread without a proxy fence showed in the kernel of four and eight groups."""
    rk = _ops()
    N, T = 4, 4200
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=2 + T)
    q, k, v = pQ.bfloat16().cuda(), pK.bfloat16().cuda(), V.bfloat16().cuda()
    first = None
    for i in range(10):
        junk = torch.full((16 << 20,), float(i), device="cuda")   # the allocations of a run reuse dirtied memory
        del junk
        out = rk.race_causal_prefix(q, k, v, variant="tensor", tile_tokens=tile)
        if first is None:
            first = out.clone()
        else:
            assert torch.equal(out, first), f"run {i} differs in {int((out != first).sum())} values"


def test_fp32_tensor_paths_are_bitwise_reproducible():
    """The same for the fp32 tensor paths: the forward with one-chunk tiles, the forward that forms the probabilities
    itself, the single-pass form and the backward, each run several times on dirtied memory."""
    rk = _ops()
    N, T, L, R, dk = 4, 4200, 4, 16, 64
    pQ, pK, V = (t.cuda() for t in ro.synthetic_probs(N, T, L, R, dk, seed=5))
    g = torch.Generator().manual_seed(9)
    Q, Kx = torch.randn(N, T, dk, generator=g).cuda(), torch.randn(N, T, dk, generator=g).cuda()
    planes, dO = torch.randn(L * 4, dk, generator=g).cuda(), torch.randn(N, T, dk, generator=g).cuda()
    calls = {
        "forward, tile 64": lambda: (rk.race_causal_prefix(pQ, pK, V, variant="tensor", tile_tokens=64),),
        "forward, single pass": lambda: (rk.race_causal_prefix(pQ, pK, V, variant="tensor_single_pass", tile_tokens=128),),
        "forward from Q, K": lambda: (rk.ops.race_causal_qkv(Q, Kx, V, planes, L, 4, tile_tokens=64),),
        "backward": lambda: rk.race_causal_backward(pQ, pK, V, dO),
    }
    for name, fn in calls.items():
        first = None
        for i in range(6):
            junk = torch.full((16 << 20,), float(i), device="cuda")
            del junk
            outs = [o.clone() for o in fn()]
            if first is None:
                first = outs
            else:
                assert all(torch.equal(a, b) for a, b in zip(outs, first)), f"{name}: run {i} differs"


@pytest.mark.parametrize("tile", [32, 64, 128, 512, 4096])
def test_forced_tile_lengths_agree(tile):
    rk = _ops()
    N, T, L, R, dk = 2, 1500, 4, 16, 64
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=11)
    ref = _oracle(pQ, pK, V)
    for variant in _variants(N, T, L, R, dk, torch.float32):
        chunk = 32 if variant == "simt" else 64
        if tile % chunk:
            continue
        out = rk.race_causal_prefix(pQ.cuda(), pK.cuda(), V.cuda(), variant=variant, tile_tokens=tile)
        assert ro.rel_l2(out, ref) <= FP32_TOL


def test_operator_matches_reference_golden(golden):
    # BatchedACE drop-in on the GPU vs outputs of the reference's own BatchedACE
    rk = _ops()
    for name in ["small_k4l4", "small_k2l2", "small_k5l1", "small_k6l8_d128", "mb_k3l2_d32"]:
        M, B, H, dk, K, L, T, _ = (int(x) for x in golden[f"{name}/cfg"])
        ace = rk.BatchedACE(dk, K, L, M)
        ace.planes_T = torch.from_numpy(golden[f"{name}/planes_T"]).float()
        ace = ace.cuda()
        Kh, Vh, Qh = (torch.from_numpy(golden[f"{name}/{k}"]).float().cuda() for k in "KVQ")
        out = ace(Kh, Vh, Qh)
        ref = torch.from_numpy(golden[f"{name}/out"])
        assert out.shape == ref.shape
        assert ro.rel_l2(out, ref) <= FP32_TOL, name


def test_operator_config1_golden(golden):
    rk = _ops()
    M, B, H, dk, K, L, T, stride = (int(x) for x in golden["c1_t4096/cfg"])
    torch.manual_seed(1234)
    ace = rk.BatchedACE(dk, K, L, M)     # seeded construction reproduces the reference planes
    assert np.array_equal(ace.planes_T.numpy(), golden["c1_t4096/planes_T"])
    ace = ace.cuda()
    Kh, Vh, Qh = draw_kvq(M, B, T, H, dk, torch.float32)
    out = ace(Kh.cuda(), Vh.cuda(), Qh.cuda())
    ref = torch.from_numpy(golden["c1_t4096/out"])
    assert ro.rel_l2(out[:, :, ::stride], ref) <= FP32_TOL
    # the reference's own acceptance bound for chunked vs baseline: 1e-4 max-abs
    # (src/test_equivalence.py:55)
    assert (out[:, :, ::stride].cpu() - ref).abs().max().item() <= 1e-3
    # host tensors are accepted and come back on the host
    out_h = ace(Kh, Vh, Qh)
    assert not out_h.is_cuda and torch.equal(out_h, out.cpu())


def test_carry_in_and_state_out():
    rk = _ops()
    N, T, L, R, dk = 3, 700, 4, 16, 64
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=21)
    ref, A_ref, B_ref = _oracle(pQ, pK, V, return_state=True)
    q, k, v = pQ.cuda(), pK.cuda(), V.cuda()
    for variant in _variants(N, T, L, R, dk, torch.float32):
        cut = 257
        o1, A1, B1 = rk.race_causal_prefix(q[:, :cut].contiguous(), k[:, :cut].contiguous(),
                                           v[:, :cut].contiguous(), return_state=True, variant=variant)
        o2, A2, B2 = rk.race_causal_prefix(q[:, cut:].contiguous(), k[:, cut:].contiguous(),
                                           v[:, cut:].contiguous(), carry_in=(A1, B1),
                                           return_state=True, variant=variant)
        out = torch.cat([o1, o2], dim=1)
        assert ro.rel_l2(out, ref) <= FP32_TOL
        assert ro.rel_l2(A2, A_ref) <= 1e-5 and ro.rel_l2(B2, B_ref) <= 1e-5
        A_t, B_t = rk.race_tile_totals(k, v)
        assert ro.rel_l2(A_t, A_ref) <= 1e-5 and ro.rel_l2(B_t, B_ref) <= 1e-5


def test_totals_then_resume_equals_one_call():
    # the two halves the sequence-sharded driver uses: totals pass, then scan + outputs from the
    # per-tile totals left in the workspace; same kernels, same tile -> bitwise equal
    rk = _ops()
    N, T, L, R, dk = 4, 9000, 4, 16, 64
    pQ, pK, V = (t.cuda() for t in ro.synthetic_probs(N, T, L, R, dk, seed=61))
    A0 = torch.rand(N, L, R, device="cuda")
    B0 = torch.randn(N, L, R, dk, device="cuda")
    for variant in _variants(N, T, L, R, dk, torch.float32):
        ref, A_ref, B_ref = rk.race_causal_prefix(pQ, pK, V, carry_in=(A0, B0), return_state=True,
                                                  variant=variant)
        A_t, B_t, ws = rk.race_tile_totals(pK, V, variant=variant, return_workspace=True)
        out, A, B = rk.race_causal_prefix(pQ, pK, V, carry_in=(A0, B0), return_state=True,
                                          variant=variant, totals_workspace=ws)
        assert torch.equal(out, ref) and torch.equal(B, B_ref)
        assert ro.rel_l2(A_t + A0, A_ref) <= 1e-6 and ro.rel_l2(B_t + B0, B_ref) <= 1e-5


def test_known_answers_and_causality():
    rk = _ops()
    N, T, L, R, dk = 2, 200, 4, 16, 64
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=31)
    q, k, v = pQ.cuda(), pK.cuda(), V.cuda()
    for variant in _variants(N, T, L, R, dk, torch.float32):
        out = rk.race_causal_prefix(q, k, v, variant=variant)
        # O_0 = v_0 * sum_s pQ pK/(pK+eps)
        w0 = (pQ[:, 0] * pK[:, 0] / (pK[:, 0] + 1e-6)).sum(dim=(1, 2))
        assert torch.allclose(out[:, 0].cpu(), V[:, 0] * w0[:, None], rtol=1e-4, atol=1e-5)
        # constant V = c comes back as ~ L*c
        outc = rk.race_causal_prefix(q, k, torch.full_like(v, 0.75), variant=variant)
        assert (outc - L * 0.75).abs().max().item() < 2e-3
        # later keys/values cannot change earlier outputs: bitwise
        k2, v2 = k.clone(), v.clone()
        k2[:, 130:] = torch.softmax(torch.randn(N, T - 130, L, R, device="cuda"), -1)
        v2[:, 130:] = 9.0
        out2 = rk.race_causal_prefix(q, k2, v2, variant=variant)
        assert torch.equal(out[:, :130], out2[:, :130])
        assert not torch.equal(out[:, 130:], out2[:, 130:])
        # run-to-run bitwise equality (a race would show up here)
        assert torch.equal(out, rk.race_causal_prefix(q, k, v, variant=variant))


def test_nan_in_one_stream_does_not_leak():
    # a NaN value poisons its own stream from its chunk on, never another stream
    # (the reference pins the cross-stream half, test_forward_cuda.py:238-248)
    rk = _ops()
    N, T, L, R, dk = 4, 300, 4, 16, 64
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=41)
    V[2, 170] = float("nan")
    for variant in _variants(N, T, L, R, dk, torch.float32):
        out = rk.race_causal_prefix(pQ.cuda(), pK.cuda(), V.cuda(), variant=variant)
        assert torch.isfinite(out[[0, 1, 3]]).all()
        # tokens of earlier chunks (chunk lengths are 32 or 64) stay finite
        assert torch.isfinite(out[2, :128]).all() and not torch.isfinite(out[2, 170:]).any()


def test_empty_sequence_and_rejections():
    rk = _ops()
    q = torch.empty(2, 0, 4, 16, device="cuda")
    v = torch.empty(2, 0, 64, device="cuda")
    out, A, B = rk.race_causal_prefix(q, q, v, return_state=True)
    assert out.shape == v.shape and not A.any() and not B.any()
    pQ, pK, V = (t.cuda() for t in ro.synthetic_probs(2, 64, 4, 16, 64, seed=1))
    bad = {
        "fp16": (pQ.half(), pK.half(), V.half()),
        "cpu k": (pQ, pK.cpu(), V),
        "non-contiguous v": (pQ, pK, V.transpose(1, 2).contiguous().transpose(1, 2)),
        "mixed dtype": (pQ.bfloat16(), pK, V),
        "shape mismatch": (pQ, pK[:, :32].contiguous(), V),
        "V wrong T": (pQ, pK, V[:, :32].contiguous()),
        "d_k 96*2": (pQ, pK, torch.randn(2, 64, 192, device="cuda")),
    }
    for label, args in bad.items():
        with pytest.raises(RuntimeError):
            rk.race_causal_prefix(*args)
            pytest.fail(f"accepted {label}")
    with pytest.raises(RuntimeError):
        rk.race_causal_prefix(pQ, pK, V, tile_tokens=48, variant="simt")
    with pytest.raises(RuntimeError):
        rk.race_causal_prefix(pQ, pK, V, tile_tokens=-64, variant="simt")
    # misaligned base pointer
    buf = torch.empty(2 * 64 * 64 + 1, device="cuda")
    with pytest.raises(RuntimeError):
        rk.race_causal_prefix(pQ, pK, buf[1:].view(2, 64, 64))


def test_host_entry_matches_device_entry():
    rk = _ops()
    N, T, L, R, dk = 2, 5000, 4, 16, 64
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=51)
    ref, A_ref, B_ref = _oracle(pQ, pK, V, return_state=True)
    pin = [t.pin_memory() for t in (pQ, pK, V)]
    out, A, B = rk.race_causal_prefix_host(*pin, return_state=True, segment_tokens=2048)
    assert not out.is_cuda
    assert ro.rel_l2(out, ref) <= FP32_TOL
    assert ro.rel_l2(B, B_ref) <= 1e-5
    out1 = rk.race_causal_prefix_host(*pin)       # one segment
    assert ro.rel_l2(out1, ref) <= FP32_TOL


@pytest.mark.parametrize("variant", ["simt", "tensor"])
def test_host_entry_short_last_segment(variant):
    """A last segment much shorter than the others must run with the tile length (and inside the
    workspace) chosen for the full segments: 8 streams, segments of 32 768 tokens, 4 108 tokens left over."""
    rk = _ops()
    N, L, R, dk, seg = 8, 4, 16, 64, 32768
    T = seg + 4108
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=77)
    out, A, B = rk.race_causal_prefix_host(pQ.pin_memory(), pK.pin_memory(), V.pin_memory(), return_state=True,
                                           segment_tokens=seg, variant=variant)
    w = 2048
    A0, B0 = ro.tile_totals(pK[:, : T - w].double(), V[:, : T - w].double())
    ref, A1, B1 = ro.causal_prefix(pQ[-1:, T - w:].double(), pK[-1:, T - w:].double(), V[-1:, T - w:].double(),
                                   carry=(A0[-1:], B0[-1:]), return_state=True)
    assert ro.rel_l2(out[-1:, T - w:], ref) <= FP32_TOL
    assert ro.rel_l2(A[-1:], A1) <= 1e-5 and ro.rel_l2(B[-1:], B1) <= 1e-4
    head = ro.causal_prefix(pQ[:1, :1024].double(), pK[:1, :1024].double(), V[:1, :1024].double())
    assert ro.rel_l2(out[:1, :1024], head) <= FP32_TOL


def test_long_sequence_spot_check():
    # T = 2^18 per stream: the oracle runs on a window of one stream, fed with the true carry
    # (the method of the reference's 2^31-element test, test_forward_cuda.py:306-318)
    rk = _ops()
    N, T, L, R, dk = 8, 1 << 18, 4, 16, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    pQ = torch.softmax(torch.randn(N, T, L, R, device="cuda", generator=g), -1)
    pK = torch.softmax(torch.randn(N, T, L, R, device="cuda", generator=g), -1)
    V = torch.randn(N, T, dk, device="cuda", generator=g)
    out, A, B = rk.race_causal_prefix(pQ, pK, V, return_state=True)
    n, w = N - 1, 2048
    A0 = pK[n, : T - w].double().sum(0).cpu()[None]
    B0 = torch.einsum("tlr,tc->lrc", pK[n, : T - w].double(), V[n, : T - w].double()).cpu()[None]
    ref, A1, B1 = ro.causal_prefix(pQ[n:, T - w:].double().cpu(), pK[n:, T - w:].double().cpu(),
                                   V[n:, T - w:].double().cpu(), carry=(A0, B0), return_state=True)
    assert ro.rel_l2(out[n:, T - w:], ref) <= FP32_TOL
    assert ro.rel_l2(A[n:], A1) <= 1e-5 and ro.rel_l2(B[n:], B1) <= 1e-4


@pytest.mark.parametrize("M,B,T,H", [(1, 1, 4096, 8), (2, 2, 333, 3), (1, 2, 2049, 2), (1, 1, 64, 1)])
def test_heads_layout_equals_flattened_streams(M, B, T, H):
    """V and out in the operator's layout [M,B,T,H,d_k] (stream flattening of
    src/race_baseline.py:35-40 done by the kernels' addressing) give bit-identical results to the
    flattened call, for the whole forward and for the totals / resume pair."""
    rk = _ops()
    L, R, dk = 4, 16, 64
    N = M * B * H
    pQ, pK, V2 = ro.synthetic_probs(N, T, L, R, dk, seed=H + T)
    V5 = V2.view(M, B, H, T, dk).permute(0, 1, 3, 2, 4).contiguous()      # [M,B,T,H,d_k]
    q, k = pQ.cuda(), pK.cuda()
    assert rk.is_supported(N, T, L, R, dk, torch.float32, "auto", heads=H)
    flat, A0, B0 = rk.race_causal_prefix(q, k, V2.cuda(), return_state=True)
    got, A1, B1 = rk.race_causal_prefix(q, k, V5.cuda(), return_state=True)
    assert got.shape == (M, B, T, H, dk)
    assert torch.equal(got.permute(0, 1, 3, 2, 4).reshape(N, T, dk), flat)
    assert torch.equal(A0, A1) and torch.equal(B0, B1)
    At, Bt, ws = rk.race_tile_totals(k, V5.cuda(), return_workspace=True)
    assert torch.equal(At, A0) and torch.equal(Bt, B0)
    again = rk.race_causal_prefix(q, k, V5.cuda(), totals_workspace=ws)
    assert torch.equal(again, got)
    ref = ro.causal_prefix(pQ.double(), pK.double(), V2.double())
    assert ro.rel_l2(flat, ref) <= 1e-4


@pytest.mark.parametrize("M,B,T,H,L,R,dk", [(1, 1, 1000, 4, 8, 64, 128), (2, 1, 257, 3, 4, 64, 64), (1, 2, 4200, 2, 8, 64, 128)])
def test_heads_layout_bf16_wide_equals_flattened_streams(M, B, T, H, L, R, dk):
    """The same for the bf16 tensor kernels of four and eight bucket groups: V and out as [M,B,T,H,d_k]."""
    rk = _ops()
    N = M * B * H
    pQ, pK, V2 = ro.synthetic_probs(N, T, L, R, dk, seed=H + T)
    pQ, pK, V2 = pQ.bfloat16(), pK.bfloat16(), V2.bfloat16()
    V5 = V2.view(M, B, H, T, dk).permute(0, 1, 3, 2, 4).contiguous()      # [M,B,T,H,d_k]
    q, k = pQ.cuda(), pK.cuda()
    assert rk.is_supported(N, T, L, R, dk, torch.bfloat16, "auto", heads=H)
    flat, A0, B0 = rk.race_causal_prefix(q, k, V2.cuda(), return_state=True)
    got, A1, B1 = rk.race_causal_prefix(q, k, V5.cuda(), return_state=True)
    assert got.shape == (M, B, T, H, dk)
    assert torch.equal(got.permute(0, 1, 3, 2, 4).reshape(N, T, dk), flat)
    assert torch.equal(A0, A1) and torch.equal(B0, B1)
    ref = ro.causal_prefix(pQ.double(), pK.double(), V2.double())
    assert ro.rel_l2(flat, ref) <= BF16_TOL


def test_heads_layout_rejected_where_not_built():
    rk = _ops()
    assert not rk.is_supported(8, 256, 4, 16, 64, torch.bfloat16, "auto", heads=4)   # bf16 path, one bucket group
    assert not rk.is_supported(8, 256, 2, 64, 64, torch.bfloat16, "auto", heads=4)   # bf16 path, two bucket groups
    assert not rk.is_supported(8, 256, 4, 16, 64, torch.float32, "simt", heads=4)    # CUDA-core path
    assert not rk.is_supported(8, 256, 8, 64, 128, torch.float32, "auto", heads=4)   # no tensor path: S=512 fp32
    assert not rk.is_supported(8, 256, 4, 16, 64, torch.float32, "auto", heads=3)    # 8 streams / 3 heads


DECODE_SHAPES = [
    # N, prefill, steps (tokens per step), L, R, dk
    (8, 256, (1, 1, 1, 1), 4, 16, 64),      # config 1's geometry, token by token after a prefill
    (3, 0, (1, 2, 5, 64), 4, 16, 64),       # from an empty state, ragged step lengths up to the limit
    (2, 100, (1, 3), 8, 64, 128),           # config 3's bucket geometry (S = 512, d_k = 128)
    (5, 33, (1, 7), 2, 8, 40),              # d_k not a multiple of the 32-column slice
    (200, 16, (1, 1), 4, 16, 64),           # more streams than SMs
    (3001, 0, (1, 1), 4, 16, 64),           # several streams per CTA (pipelined small-state kernel), odd tail
    (2500, 0, (1, 1), 2, 8, 32),            # the same with d_k = 32: four rows of the state per warp access
]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, FP32_TOL), (torch.bfloat16, BF16_TOL)])
@pytest.mark.parametrize("N,prefill,steps,L,R,dk", DECODE_SHAPES)
def test_decode_steps_equal_full_forward(N, prefill, steps, L, R, dk, dtype, tol):
    """Prefill with the full forward, then advance with race_decode_step: every step's outputs and the
    final state equal the oracle's forward over the whole sequence (src/race_chunked.py:54-63)."""
    rk = _ops()
    T = prefill + sum(steps)
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=7 * N + T, dtype=dtype)
    ref, A_ref, B_ref = _oracle(pQ, pK, V, return_state=True)
    q, k, v = pQ.cuda(), pK.cuda(), V.cuda()
    got = torch.empty(N, T, dk, dtype=dtype, device="cuda")
    if prefill:
        o, A, B = rk.race_causal_prefix(q[:, :prefill].contiguous(), k[:, :prefill].contiguous(),
                                        v[:, :prefill].contiguous(), return_state=True)
        got[:, :prefill] = o
        state = rk.pack_state(A, B)
    else:
        state = torch.zeros(N, L * R * (dk + 1), device="cuda")
    t0 = prefill
    for i, n_new in enumerate(steps):
        sl = slice(t0, t0 + n_new)
        args = (q[:, sl].contiguous(), k[:, sl].contiguous(), v[:, sl].contiguous())
        if i % 2 == 0:      # in place
            got[:, sl] = rk.race_decode_step(*args, state)
        else:               # into a second buffer, the source left untouched
            before = state.clone()
            nxt = torch.empty_like(state)
            got[:, sl] = rk.race_decode_step(*args, state, state_out=nxt)
            assert torch.equal(state, before)
            state = nxt
        t0 += n_new
    err = ro.rel_l2(got, ref)
    assert err <= tol, f"outputs rel-L2 {err:.3e}"
    A, B = rk.unpack_state(state, L, R, dk)
    assert ro.rel_l2(A, A_ref) <= tol and ro.rel_l2(B, B_ref) <= tol


def test_decode_step_rejections():
    rk = _ops()
    pQ, pK, V = ro.synthetic_probs(2, 65, 4, 16, 64, seed=1)
    state = torch.zeros(2, 64 * 65, device="cuda")
    with pytest.raises(RuntimeError):       # more new tokens than one step takes
        rk.race_decode_step(pQ.cuda(), pK.cuda(), V.cuda(), state)
    with pytest.raises(RuntimeError):       # state of the wrong size
        rk.race_decode_step(pQ[:, :1].contiguous().cuda(), pK[:, :1].contiguous().cuda(),
                            V[:, :1].contiguous().cuda(), state[:, :-1].contiguous())
    out = rk.race_decode_step(pQ[:, :0].contiguous().cuda(), pK[:, :0].contiguous().cuda(),
                              V[:, :0].contiguous().cuda(), state)
    assert out.shape == (2, 0, 64) and not state.any()


from conftest import GLOBAL_CASES, global_case  # noqa: E402


@pytest.mark.parametrize("name", GLOBAL_CASES)
def test_global_form_matches_reference_vectors(golden_global, name):
    """normalization="global" against the outputs of the reference's race_causal_reference
    (src/causal_v2/reference.py:106-127) on the features that function computed."""
    rk = _ops()
    pQ, pK, V, ref = global_case(golden_global, name)
    N, T, L, R = pK.shape
    variants = _variants(N, T, L, R, V.shape[-1], torch.float32)
    if name == "g_k4l4":
        assert "tensor" in variants      # the reference kernels' own geometry runs on the tcgen05 kernels too
    for variant in variants:
        out = rk.race_causal_prefix(pQ.float().cuda(), pK.float().cuda(), V.float().cuda(), normalization="global",
                                    variant=variant)
        assert ro.rel_l2(out, ref) <= FP32_TOL, variant
        assert torch.isfinite(out).all()


@pytest.mark.parametrize("N,T,L,R,dk,dtype,tol", [
    (8, 4096, 4, 16, 64, torch.float32, FP32_TOL),      # config 1's geometry, several tiles
    (2, 4097, 4, 16, 64, torch.float32, FP32_TOL),
    (2, 300, 8, 64, 128, torch.float32, FP32_TOL),      # S = 512: eight bucket groups share the denominator
    (1, 100, 2, 64, 64, torch.float32, FP32_TOL),
    (3, 150, 2, 8, 32, torch.float32, FP32_TOL),
    (2, 1000, 4, 16, 64, torch.bfloat16, BF16_TOL),
    (2, 700, 4, 16, 128, torch.bfloat16, BF16_TOL),
    (2, 300, 8, 64, 128, torch.bfloat16, BF16_TOL),
])
def test_global_form_parity_and_carry(N, T, L, R, dk, dtype, tol):
    rk = _ops()
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=11 * N + T, dtype=dtype)
    ref, A_ref, B_ref = ro.causal_prefix_global(pQ.double(), pK.double(), V.double(), return_state=True)
    q, k, v = pQ.cuda(), pK.cuda(), V.cuda()
    variants = ["simt"] + (["tensor", "tensor_single_pass"]
                           if dtype == torch.float32 and "tensor" in _variants(N, T, L, R, dk, dtype) else [])
    if dtype == torch.bfloat16 and L * R == 64:
        variants.append("tensor")        # the one-group bf16 tensor kernel has this form too
    for variant in variants:
        out, A, B = rk.race_causal_prefix(q, k, v, normalization="global", return_state=True, variant=variant)
        assert ro.rel_l2(out, ref) <= tol, variant
        assert ro.rel_l2(A, A_ref) <= tol and ro.rel_l2(B, B_ref) <= tol
        # two calls with the carried state equal one call; small tiles exercise the scan
        h = T // 3
        t1, t2 = (32, 64) if variant == "simt" else (64, 128)
        o1, A1, B1 = rk.race_causal_prefix(q[:, :h].contiguous(), k[:, :h].contiguous(), v[:, :h].contiguous(),
                                           normalization="global", return_state=True, tile_tokens=t1, variant=variant)
        o2 = rk.race_causal_prefix(q[:, h:].contiguous(), k[:, h:].contiguous(), v[:, h:].contiguous(),
                                   normalization="global", carry_in=(A1, B1), tile_tokens=t2, variant=variant)
        assert ro.rel_l2(torch.cat([o1, o2], 1), ref) <= tol, variant


def test_global_form_zero_denominator_and_rejections():
    rk = _ops()
    pQ, pK, V = ro.synthetic_probs(2, 64, 4, 16, 64, seed=3)
    pK[0, :10] = 0          # stream 0 has no key mass for its first ten tokens: those rows are 0
    ref = ro.causal_prefix_global(pQ.double(), pK.double(), V.double())
    for variant in ("simt", "tensor", "tensor_single_pass", "auto"):
        out = rk.race_causal_prefix(pQ.cuda(), pK.cuda(), V.cuda(), normalization="global", variant=variant)
        assert not out[0, :10].any() and torch.isfinite(out).all(), variant
        assert ro.rel_l2(out, ref) <= FP32_TOL, variant
    pQw, pKw, Vw = (t.bfloat16().cuda() for t in ro.synthetic_probs(2, 64, 8, 64, 128, seed=4))
    with pytest.raises(RuntimeError):     # the wide bf16 tensor kernel does not have this form
        rk.race_causal_prefix(pQw, pKw, Vw, normalization="global", variant="tensor")
    with pytest.raises(RuntimeError):
        rk.race_causal_prefix(pQ.cuda(), pK.cuda(), V.cuda(), normalization="paper")


BWD_SHAPES = [
    # N, T, L, R, dk
    (2, 70, 4, 16, 64), (2, 2100, 4, 16, 64),   # config 1's geometry; the second spans many state tiles
    (1, 32, 4, 16, 64), (1, 33, 1, 32, 64),
    (3, 150, 2, 8, 32), (2, 300, 4, 16, 128), (5, 97, 2, 4, 40),
    (2, 300, 8, 64, 128),       # config 3's bucket geometry: S = 512, a cluster of eight bucket groups
    (1, 100, 2, 64, 64),        # S = 128: two groups
]


def _grad_out(N, T, dk, dtype, seed):
    return torch.randn(N, T, dk, generator=torch.Generator().manual_seed(seed)).to(dtype)


@pytest.mark.parametrize("N,T,L,R,dk", BWD_SHAPES)
def test_causal_backward_fp32(N, T, L, R, dk):
    """The backward kernels against the hand-derived gradients evaluated in fp64 (which the CPU suite
    checks against torch.autograd through the restated reference forward, src/race_baseline.py:45-51)."""
    rk = _ops()
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=5 * N + T)
    dO = _grad_out(N, T, dk, torch.float32, T)
    ref = ro.causal_backward_closed_form(pQ.double(), pK.double(), V.double(), dO.double())
    got = rk.race_causal_backward(pQ.cuda(), pK.cuda(), V.cuda(), dO.cuda())
    for name, g, r in zip(("dPQ", "dPK", "dV"), got, ref):
        err = ro.rel_l2(g, r)
        assert err <= FP32_TOL, f"{name}: rel-L2 {err:.3e}"
        assert torch.isfinite(g).all()


def test_causal_backward_single_token():
    """T = 1: dPK is the difference of two terms that cancel to O(eps) (analytically
    pQ (v.dO) eps / (pK+eps)^2), so it is held to an absolute bound on the scale of those terms;
    dPQ and dV keep the relative bound."""
    rk = _ops()
    pQ, pK, V = ro.synthetic_probs(3, 1, 4, 16, 64, seed=6)
    dO = _grad_out(3, 1, 64, torch.float32, 1)
    ref = ro.causal_backward_closed_form(pQ.double(), pK.double(), V.double(), dO.double())
    got = rk.race_causal_backward(pQ.cuda(), pK.cuda(), V.cuda(), dO.cuda())
    assert ro.rel_l2(got[0], ref[0]) <= FP32_TOL and ro.rel_l2(got[2], ref[2]) <= FP32_TOL
    scale = ((pQ / (pK + 1e-6)).abs().amax() * (V * dO).sum(-1).abs().amax()).item()
    assert (got[1].cpu().double() - ref[1]).abs().max().item() <= 1e-5 * scale


def test_causal_backward_bf16_and_autograd():
    rk = _ops()
    N, T, L, R, dk = 2, 500, 4, 16, 64
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=9, dtype=torch.bfloat16)
    dO = _grad_out(N, T, dk, torch.bfloat16, 10)
    ref = ro.causal_backward_closed_form(pQ.double(), pK.double(), V.double(), dO.double())
    got = rk.race_causal_backward(pQ.cuda(), pK.cuda(), V.cuda(), dO.cuda())
    for name, g, r in zip(("dPQ", "dPK", "dV"), got, ref):
        assert ro.rel_l2(g, r) <= BF16_TOL, name
    # through autograd, fp32, against torch.autograd of the oracle forward
    pQ, pK, V = ro.synthetic_probs(N, 200, L, R, dk, seed=4)
    dO = _grad_out(N, 200, dk, torch.float32, 5)
    ref = ro.causal_backward_autograd(pQ.double(), pK.double(), V.double(), dO.double())
    q, k, v = (t.cuda().requires_grad_(True) for t in (pQ, pK, V))
    out = rk.race_causal(q, k, v)
    assert ro.rel_l2(out, ro.causal_prefix(pQ.double(), pK.double(), V.double())) <= FP32_TOL
    out.backward(dO.cuda())
    for g, r in zip((q.grad, k.grad, v.grad), ref):
        assert ro.rel_l2(g, r) <= FP32_TOL


def test_causal_backward_rejections():
    rk = _ops()
    pQ, pK, V = ro.synthetic_probs(1, 40, 3, 32, 64, seed=2)      # S = 96: outside the backward's range
    with pytest.raises(RuntimeError):
        rk.race_causal_backward(pQ.cuda(), pK.cuda(), V.cuda(), torch.zeros_like(V).cuda())
    pQ, pK, V = ro.synthetic_probs(1, 40, 4, 16, 64, seed=2)
    with pytest.raises(RuntimeError):
        rk.race_causal_backward(pQ.cuda(), pK.cuda(), V.cuda(), torch.zeros(1, 39, 64).cuda())


def test_operator_step_continues_the_reference_output(golden):
    """Prefill with BatchedACE.forward(return_state=True), then BatchedACE.step token groups: the pieces equal
    the reference's own BatchedACE output over the whole sequence (golden vectors)."""
    rk = _ops()
    for name, prefill in (("small_k4l4", 64), ("mb_k3l2_d32", 0), ("small_k6l8_d128", 17)):
        M, B, H, dk, K, L, T, _ = (int(x) for x in golden[f"{name}/cfg"])
        ace = rk.BatchedACE(dk, K, L, M)
        ace.planes_T = torch.from_numpy(golden[f"{name}/planes_T"]).float()
        ace = ace.cuda()
        Kh, Vh, Qh = (torch.from_numpy(golden[f"{name}/{k}"]).float().cuda() for k in "KVQ")
        ref = torch.from_numpy(golden[f"{name}/out"])
        got = torch.empty(M, B, T, H, dk, device="cuda")
        if prefill:
            o, A, Bs = ace(Kh[:, :, :prefill], Vh[:, :, :prefill], Qh[:, :, :prefill], return_state=True)
            got[:, :, :prefill] = o
            state = rk.pack_state(A, Bs)
        else:
            state = torch.zeros(M * B * H, L * (1 << K) * (dk + 1), device="cuda")
        t0 = prefill
        for n_new in itertools.cycle((1, 3, 1, 8)):
            if t0 >= T:
                break
            t1 = min(T, t0 + n_new)
            got[:, :, t0:t1] = ace.step(Kh[:, :, t0:t1], Vh[:, :, t0:t1], Qh[:, :, t0:t1], state)
            t0 = t1
        assert ro.rel_l2(got, ref) <= FP32_TOL, name


@pytest.mark.parametrize("N,T,L,R,dk,cuts", [(2, 300, 4, 16, 64, (0, 100, 164, 300)), (2, 90, 2, 64, 32, (0, 1, 50, 90))])
def test_causal_backward_through_chunks(N, T, L, R, dk, cuts):
    """Chunks chained through the carried state (src/race_chunked.py:45-63) back-propagate to the same
    gradients as the whole sequence at once."""
    rk = _ops()
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=21)
    dO = _grad_out(N, T, dk, torch.float32, 22)
    ref = ro.causal_backward_autograd(pQ.double(), pK.double(), V.double(), dO.double())
    q, k, v = (t.cuda().requires_grad_(True) for t in (pQ, pK, V))
    state = torch.zeros(N, L * R * (dk + 1), device="cuda")
    outs = []
    for a, b in zip(cuts[:-1], cuts[1:]):
        o, state = rk.race_causal_chunk(q[:, a:b].contiguous(), k[:, a:b].contiguous(), v[:, a:b].contiguous(), state)
        outs.append(o)
    out = torch.cat(outs, 1)
    assert ro.rel_l2(out, ro.causal_prefix(pQ.double(), pK.double(), V.double())) <= FP32_TOL
    out.backward(dO.cuda())
    for name, g, r in zip(("dPQ", "dPK", "dV"), (q.grad, k.grad, v.grad), ref):
        assert ro.rel_l2(g, r) <= FP32_TOL, name


def test_causal_backward_long_sequence():
    """20 000 tokens (ten state tiles of 2048, suffix sums over 625 chunks): accumulated rounding stays inside
    the fp32 bound."""
    rk = _ops()
    N, T, L, R, dk = 1, 20000, 4, 16, 64
    pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=77)
    dO = _grad_out(N, T, dk, torch.float32, 78)
    ref = ro.causal_backward_closed_form(pQ.double(), pK.double(), V.double(), dO.double())
    got = rk.race_causal_backward(pQ.cuda(), pK.cuda(), V.cuda(), dO.cuda())
    for name, g, r in zip(("dPQ", "dPK", "dV"), got, ref):
        assert ro.rel_l2(g, r) <= FP32_TOL, name


def test_bounded_wait_runs_out_and_device_stays_usable():
    """A wait that nothing satisfies must end by its limit: the producer of the first CTA withholds one
    chunk's load, every wait is limited to about a millisecond, and the kernel has to return with the
    status word set -- after which an ordinary forward on the same device is bit-identical to one run
    before.  No memory fault and no unbounded spin is involved."""
    rk = _ops()
    N, T, L, R, dk = 2, 32768, 4, 16, 64
    pQ, pK, V = (t.cuda() for t in ro.synthetic_probs(N, T, L, R, dk, seed=99))
    for variant in ("tensor", "tensor_single_pass"):
        _bounded_wait_case(rk, pQ, pK, V, variant)


def _bounded_wait_case(rk, pQ, pK, V, variant):
    N, T, L, R = pK.shape
    dk = V.shape[-1]
    assert rk.select_tile_tokens(N, T, L, R, dk, variant=variant) >= 6 * 64      # chunks 0, 1 and 5 exist in a tile
    before = rk.race_causal_prefix(pQ, pK, V, variant=variant)
    assert rk.ops.device_status() == 0
    for chunk in (0, 1, 5):
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        out, code = rk.ops.selftest_bounded_wait(pQ, pK, V, wait_cycles=2_000_000, withhold_chunk=chunk,
                                                 variant=variant)
        t1.record()
        torch.cuda.synchronize()
        assert code != 0, "the withheld load went unnoticed"
        assert 100 <= code < 600, code                    # one of the kernels' wait codes
        assert t0.elapsed_time(t1) < 1000.0               # ended by the limit (~1 ms), not by the default (~1 s)
        # tiles of the other stream never depended on the withheld chunk
        assert torch.equal(out[1], before[1])
        assert rk.ops.device_status() == 0                # the self-test used its own status word
        again = rk.race_causal_prefix(pQ, pK, V, variant=variant)
        assert torch.equal(again, before)
    # a chunk index beyond the tile: nothing is withheld, nothing runs out
    out, code = rk.ops.selftest_bounded_wait(pQ, pK, V, wait_cycles=2_000_000, withhold_chunk=10_000, variant=variant)
    assert code == 0 and torch.equal(out, before)


def test_operator_gradients_match_reference():
    """BatchedACE under autograd: gradients w.r.t. K, V, Q against the reference module's own autograd
    gradients (tests/golden/make_golden_grad.py, fp64), through the forward and backward kernels."""
    import os

    import numpy as np
    rk = _ops()
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "race_grad_golden.npz"))
    for name in ("grad_k4l4", "grad_k3l2_d32"):
        M, B, H, dk, K, L, T = (int(x) for x in g[f"{name}/cfg"])
        ace = rk.BatchedACE(dk, K, L, M)
        ace.planes_T = torch.from_numpy(g[f"{name}/planes_T"]).float()
        ace = ace.cuda()
        Kh, Vh, Qh = (torch.from_numpy(g[f"{name}/{k}"]).float().cuda().requires_grad_(True) for k in "KVQ")
        out = ace(Kh, Vh, Qh)
        assert out.requires_grad
        assert ro.rel_l2(out, torch.from_numpy(g[f"{name}/out"])) <= FP32_TOL
        out.backward(torch.from_numpy(g[f"{name}/dO"]).float().cuda())
        for t, key in ((Kh, "dK"), (Vh, "dV"), (Qh, "dQ")):
            assert ro.rel_l2(t.grad, torch.from_numpy(g[f"{name}/{key}"])) <= 5e-4, (name, key)
        # without gradients the same call takes the pure kernel path and agrees
        with torch.no_grad():
            plain = ace(Kh, Vh, Qh)
        assert not plain.requires_grad and ro.rel_l2(plain, out) <= 1e-5


def test_decode_stepper_matches_general_wrapper():
    rk = _ops()
    N, L, R, dk = 8, 4, 16, 64
    pQ, pK, V = (t.cuda() for t in ro.synthetic_probs(N, 40, L, R, dk, seed=21))
    step = rk.DecodeStepper(N, L, R, dk, torch.float32, torch.device("cuda", torch.cuda.current_device()))
    s1 = torch.zeros(N, L * R * (dk + 1), device="cuda")
    s2 = torch.zeros_like(s1)
    for t in range(40):
        q, k, v = (x[:, t:t + 1].contiguous() for x in (pQ, pK, V))
        a = step(q, k, v, s1).clone()
        b = rk.race_decode_step(q, k, v, s2)
        assert torch.equal(a, b)
    assert torch.equal(s1, s2)
    with pytest.raises(RuntimeError):
        step(pQ[:, :2].contiguous(), pK[:, :2].contiguous(), V[:, :2].contiguous(), s1)


@pytest.mark.parametrize("N,T", [(8, 20000), (3, 4097), (2, 1 << 16), (1, 100)])
def test_single_pass_equals_three_launches_bitwise(N, T):
    """The persistent single-pass kernel (tile tickets, decoupled look-back in tile order, tile re-read from L2)
    and the three launches (totals, scan, outputs) run the same arithmetic in the same order: for equal tile
    lengths outputs and final states are bit-identical, with and without a carried state; and the single-pass
    form meets the oracle at its own automatic tile length."""
    rk = _ops()
    L, R, dk = 4, 16, 64
    pQ, pK, V = (t.cuda() for t in ro.synthetic_probs(N, T, L, R, dk, seed=T))
    carry = rk.pack_state(torch.rand(N, L, R, device="cuda") * 5, torch.randn(N, L, R, dk, device="cuda"))
    for tile in (64, 512, 1024, 2048):
        for cin in (None, carry):
            a, Aa, Ba = rk.race_causal_prefix(pQ, pK, V, carry_in=cin, return_state=True, variant="tensor",
                                              tile_tokens=tile)
            b, Ab, Bb = rk.race_causal_prefix(pQ, pK, V, carry_in=cin, return_state=True,
                                              variant="tensor_single_pass", tile_tokens=tile)
            assert torch.equal(a, b), (tile, cin is None)
            assert torch.equal(Aa, Ab) and torch.equal(Ba, Bb)
    out = rk.race_causal_prefix(pQ, pK, V, variant="tensor_single_pass")
    ref = _oracle(pQ.cpu(), pK.cpu(), V.cpu())
    assert ro.rel_l2(out, ref) <= FP32_TOL
    # run to run: the look-back may stop at different tiles, the sum is the same
    again = rk.race_causal_prefix(pQ, pK, V, variant="tensor_single_pass")
    assert torch.equal(out, again)
