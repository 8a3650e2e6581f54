"""The allocation-free entry point (race_b200_causal_fwd_static).

Who needs it: callers that may not allocate device memory at the moment they run the forward --
code inside an open stream capture, allocator hooks, memory-planned serving loops.  The entry
point therefore takes its workspace from an array compiled into the library.  The checks: called
through the C ABI it gives the same output as the ordinary entry point (bitwise: same kernels,
same tile length), on two calls in a row that share the built-in array, with the second call
using a different shape so that stale contents of the array would show; and shapes beyond the
array are refused with a clear error.  This file sorts last on purpose, so that a failure here
stops a fail-fast run only after every other test has run."""
from __future__ import annotations

import ctypes

import pytest
import torch

from oracle import race_oracle as ro
from race_attention_kernel_b200 import _lib


def test_scratch_limit_is_refused_without_launch():
    L = _lib.lib()
    limit = L.race_b200_static_scratch_bytes()
    assert limit == 16 << 20
    # 8 streams x 2^20 tokens needs 68 MB of tile states: refused before any pointer is looked at
    big = _lib.RaceShape(8, 1 << 20, 4, 16, 64, 0, 1e-6, 0)
    assert L.race_b200_causal_workspace_bytes(ctypes.byref(big), 0, 1) > limit
    rc = L.race_b200_causal_fwd_static(None, None, None, None, None, None, ctypes.byref(big), 0, 1,
                                       None, None)
    assert rc == -8
    assert b"scratch" in L.race_b200_error_string(rc)


@pytest.mark.gpu
def test_static_scratch_matches_ordinary_entry_twice():
    import race_attention_kernel_b200 as rk

    torch.cuda.set_device(0)
    # second call: other sizes, fewer tiles, a carry-in and the final state
    cases = [(8, 20000, 4, 16, 64, False), (3, 4097, 4, 16, 64, True)]
    for variant in ("simt", "tensor", "tensor_single_pass"):
        for N, T, L, R, dk, with_state in cases:
            if not rk.is_supported(N, T, L, R, dk, torch.float32, variant):
                continue
            pQ, pK, V = (t.cuda() for t in ro.synthetic_probs(N, T, L, R, dk, seed=T))
            carry = None
            if with_state:
                A0 = torch.rand(N, L, R, device="cuda") * 3
                B0 = torch.randn(N, L, R, dk, device="cuda")
                carry = rk.pack_state(A0, B0)
            res = rk.race_causal_prefix(pQ, pK, V, carry_in=carry, return_state=with_state,
                                        variant=variant)
            ref = res[0] if with_state else res
            # everything the call touches exists before the call
            out = torch.full_like(V, float("nan"))
            state = torch.empty(N, L * R * (dk + 1), device="cuda") if with_state else None
            before = torch.cuda.memory_allocated()
            rk.race_causal_prefix_static(pQ, pK, V, out, carry_in=carry, state_out=state,
                                         variant=variant)
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated() == before     # torch's allocator was not used
            assert torch.equal(out, ref), (variant, N, T)
            if with_state:
                A, B = rk.unpack_state(state, L, R, dk)
                assert torch.equal(A, res[1]) and torch.equal(B, res[2])
            # and against the oracle, with the tolerance of the other fp32 tests
            want = ro.causal_prefix_chunked(
                pQ.double().cpu(), pK.double().cpu(), V.double().cpu(), chunk=512,
                carry=None if carry is None else (A0.double().cpu(), B0.double().cpu()))
            assert ro.rel_l2(out, want) <= 1e-4
    assert rk.ops.device_status() == 0


@pytest.mark.gpu
def test_static_wrapper_allocates_nothing_as_first_call():
    """The Python wrapper must not create the per-device status word on the fly: with the word absent
    (a process whose first operator call is the allocation-free one) the call still allocates nothing."""
    import race_attention_kernel_b200 as rk
    from race_attention_kernel_b200 import ops

    torch.cuda.set_device(0)
    N, T, L, R, dk = 2, 1000, 4, 16, 64
    pQ, pK, V = (t.cuda() for t in ro.synthetic_probs(N, T, L, R, dk, seed=5))
    ref = rk.race_causal_prefix(pQ, pK, V)
    out = torch.full_like(V, float("nan"))
    saved = dict(ops._STATUS)
    ops._STATUS.clear()
    try:
        before = torch.cuda.memory_allocated()
        rk.race_causal_prefix_static(pQ, pK, V, out)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert not ops._STATUS                      # still absent: nothing was created behind the caller's back
    finally:
        ops._STATUS.update(saved)
    assert torch.equal(out, ref)
    # bad carry / state arguments are refused before they reach the device
    with pytest.raises(RuntimeError):
        rk.race_causal_prefix_static(pQ, pK, V, out, carry_in=torch.zeros(N, L * R * (dk + 1)))          # host tensor
    with pytest.raises(RuntimeError):
        rk.race_causal_prefix_static(pQ, pK, V, out, state_out=torch.zeros(N, 8, device="cuda"))           # too short
    with pytest.raises(RuntimeError):
        rk.race_causal_prefix_static(pQ, pK, V, out, carry_in=torch.zeros(N, L * R * (dk + 1), device="cuda",
                                                                          dtype=torch.float64))
