"""CPU checks of the C-ABI boundary: the library loads, exports every symbol the public header
declares, and rejects bad arguments with its documented codes (no kernel is launched)."""
from __future__ import annotations

import ctypes
import os
import re

import pytest

from conftest import ROOT
from race_attention_kernel_b200 import _lib


def _declared():
    text = open(os.path.join(ROOT, "include", "race_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(race_b200_\w+)\s*\(", text)))


def test_header_symbols_exported():
    names = _declared()
    assert len(names) >= 13
    L = _lib.lib()
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/race_b200.h but not exported"
    assert sorted(_lib.EXPORTS) == names


def test_version_and_error_strings():
    L = _lib.lib()
    assert L.race_b200_version() >= 1000
    assert L.race_b200_error_string(0) == b"ok"
    for code in range(-8, 0):
        assert L.race_b200_error_string(code) not in (b"", b"unknown error")


def _shape(N=8, T=4096, L=4, R=16, dk=64, dtype=0, eps=1e-6, heads=0):
    return _lib.RaceShape(N, T, L, R, dk, dtype, eps, heads)


def test_state_floats_and_support():
    L = _lib.lib()
    sh = _shape()
    assert L.race_b200_state_floats(ctypes.byref(sh)) == 8 * 64 * 65
    assert L.race_b200_is_supported(ctypes.byref(sh), 1) == 1
    assert L.race_b200_is_supported(ctypes.byref(_shape(dk=96 * 4)), 1) == 0     # d_k > 128
    assert L.race_b200_is_supported(ctypes.byref(_shape(L=3, R=32)), 1) == 0      # S=96: not /64
    assert L.race_b200_is_supported(ctypes.byref(_shape(L=8, R=64, dk=128, dtype=1)), 1) == 1
    assert L.race_b200_is_supported(ctypes.byref(_shape(L=8, R=64, dk=128, dtype=1)), 2) == 1   # tensor, cluster of 8
    assert L.race_b200_is_supported(ctypes.byref(_shape(L=3, R=64, dk=128, dtype=1)), 2) == 0   # 3 groups
    assert L.race_b200_is_supported(ctypes.byref(_shape(dk=128)), 2) == 0                       # fp32 d_k=128
    assert L.race_b200_is_supported(ctypes.byref(_shape(dtype=7)), 0) == 0
    assert L.race_b200_is_supported(ctypes.byref(_shape(heads=3)), 0) == 0
    # the heads layout of V / out: fp32 tensor kernels, bf16 tensor kernels with four or eight bucket groups
    assert L.race_b200_is_supported(ctypes.byref(_shape(heads=4)), 0) == 1
    assert L.race_b200_is_supported(ctypes.byref(_shape(heads=4)), 1) == 0                                   # CUDA-core path
    assert L.race_b200_is_supported(ctypes.byref(_shape(L=8, R=64, dk=128, dtype=1, heads=4)), 0) == 1
    assert L.race_b200_is_supported(ctypes.byref(_shape(L=4, R=64, dk=64, dtype=1, heads=2)), 2) == 1
    assert L.race_b200_is_supported(ctypes.byref(_shape(L=2, R=64, dk=64, dtype=1, heads=2)), 0) == 0        # two groups
    assert L.race_b200_is_supported(ctypes.byref(_shape(dtype=1, heads=2)), 0) == 0                          # one group
    assert L.race_b200_is_supported(ctypes.byref(_shape(N=9, L=8, R=64, dk=128, dtype=1, heads=4)), 0) == 0  # 9 streams / 4


@pytest.mark.parametrize("kw,code", [
    (dict(dtype=5), -2), (dict(N=-1), -2), (dict(L=0), -2), (dict(eps=-1.0), -2),
    (dict(heads=3), -2), (dict(), -1),      # a valid shape then fails on the NULL pointers
])
def test_argument_errors_without_launch(kw, code):
    L = _lib.lib()
    sh = _shape(**kw)
    rc = L.race_b200_causal_fwd(None, None, None, None, None, None, None, 0, ctypes.byref(sh), 0, 1,
                                None, None)
    assert rc == code


def test_misaligned_rows_and_tiles():
    L = _lib.lib()
    # S = 6 fp32 = 24-byte rows: not a multiple of 16
    rc = L.race_b200_causal_fwd(None, None, None, None, None, None, None, 0,
                                ctypes.byref(_shape(L=1, R=6)), 0, 1, None, None)
    assert rc == -3
    # tile that is not a multiple of the 32-token chunk, negative tile
    for tile in (48, -64):
        rc = L.race_b200_causal_fwd(None, None, None, None, None, None, None, 0,
                                    ctypes.byref(_shape()), tile, 1, None, None)
        assert rc == -5
    # unknown variant
    rc = L.race_b200_causal_fwd(None, None, None, None, None, None, None, 0,
                                ctypes.byref(_shape()), 0, 9, None, None)
    assert rc == -6
    # NULL shape
    assert L.race_b200_causal_fwd(None, None, None, None, None, None, None, 0, None, 0, 1, None, None) == -1


def test_workspace_and_tile_selection():
    L = _lib.lib()
    sh = _shape(T=1 << 20)
    tile = ctypes.c_int(0)
    assert L.race_b200_select_tile_tokens(ctypes.byref(sh), 1, ctypes.byref(tile)) == 0
    assert tile.value % 32 == 0 and 32 <= tile.value <= 4096
    ws = L.race_b200_causal_workspace_bytes(ctypes.byref(sh), tile.value, 1)
    tiles = ((1 << 20) + tile.value - 1) // tile.value
    assert ws == 8 * tiles * 64 * 65 * 4
    short = ctypes.c_int(0)
    L.race_b200_select_tile_tokens(ctypes.byref(_shape(N=1, T=100)), 1, ctypes.byref(short))
    assert short.value == 32   # a short sequence gets the smallest tile


def test_python_binding_rejects_cpu_tensors():
    import torch

    from race_attention_kernel_b200 import race_causal_prefix
    pq = torch.rand(1, 8, 2, 4)
    with pytest.raises(RuntimeError):
        race_causal_prefix(pq, pq, torch.rand(1, 8, 4))


def test_decode_step_argument_errors_without_launch():
    L = _lib.lib()
    call = lambda sh, state=None: L.race_b200_decode_step(None, None, None, None, None, state, ctypes.byref(sh), None)
    assert call(_shape(T=1)) == -1                       # state_out is required
    assert call(_shape(T=65), 256) == -2                 # more new tokens than one step takes
    assert call(_shape(T=1, heads=8), 256) == -2         # the heads layout is not read by this entry point
    assert call(_shape(T=1, L=64, R=64), 256) == -2      # S > 2048
    assert call(_shape(T=1), 256) == -1                  # valid shape, NULL token pointers
    assert call(_shape(N=0, T=1), 256) == 0              # nothing to do


def test_global_form_argument_errors_without_launch():
    L = _lib.lib()
    call = lambda sh, variant=0: L.race_b200_causal_fwd_global(None, None, None, None, None, None, None, 0,
                                                               ctypes.byref(sh), 0, variant, None, None)
    assert call(_shape(heads=8), 1) == -6               # the heads layout is read by the fp32 tensor kernels only
    assert call(_shape(heads=8)) == -1                  # ... which AUTO picks: valid shape, NULL pointers
    assert call(_shape(dk=96 * 4), 1) == -6             # outside the CUDA-core kernels' range
    assert call(_shape(dk=96 * 4)) == -2                # no kernel family takes it
    assert call(_shape(dtype=1, L=8, R=64, dk=128), 2) == -6   # the wide bf16 tensor kernel does not have this form
    assert call(_shape(dtype=1), 2) == -1               # bf16, S = 64: valid, NULL pointers
    assert call(_shape()) == -1                         # valid shape, NULL pointers
    assert call(_shape(T=0)) == 0                       # nothing to launch


def test_causal_backward_argument_errors_without_launch():
    L = _lib.lib()
    call = lambda sh: L.race_b200_causal_bwd(None, None, None, None, None, None, None, None, 0, ctypes.byref(sh), None,
                                             None)
    assert call(_shape(L=3, R=32)) == -2                 # S = 96: neither <= 64 nor a multiple of 64
    assert call(_shape(dk=96 * 4)) == -2
    assert call(_shape(heads=8)) == -2
    assert call(_shape()) == -1                          # valid shape, NULL pointers
    assert call(_shape(T=0)) == 0
    assert L.race_b200_causal_bwd_workspace_bytes(ctypes.byref(_shape(L=3, R=32))) == 0
    assert L.race_b200_causal_bwd_workspace_bytes(ctypes.byref(_shape())) >= 2 * 8 * 4096 * 64 * 4


def test_causal_backward_carry_argument_errors_without_launch():
    L = _lib.lib()
    call = lambda sh: L.race_b200_causal_bwd_carry(None, None, None, None, None, None, None, None, None, None, None, 0,
                                                   ctypes.byref(sh), None, None)
    assert call(_shape(L=3, R=32)) == -2
    assert call(_shape()) == -1
    assert call(_shape(T=0)) == 0        # no tokens and no d_carry_in requested: nothing to do


def test_bounded_wait_selftest_argument_errors_without_launch():
    L = _lib.lib()
    call = lambda sh, cycles=2_000_000, chunk=1, status=256, variant=2: L.race_b200_selftest_bounded_wait(
        None, None, None, None, None, 0, ctypes.byref(sh), variant, cycles, chunk, None, status)
    assert call(_shape(), status=None) == -1             # the status word is required
    assert call(_shape(), cycles=10) == -2               # limit below the accepted range
    assert call(_shape(), chunk=-1) == -2
    assert call(_shape(dtype=1)) == -6                   # fp32 tensor kernels only
    assert call(_shape(L=3, R=32)) == -6                 # S = 96: not a tensor-kernel shape
    assert call(_shape()) == -1                          # valid arguments, NULL tensors
    assert call(_shape(), variant=3) == -1               # the single-pass form too
    assert call(_shape(), variant=1) == -6               # not a tensor-kernel family


def test_single_pass_variant_sizes():
    L = _lib.lib()
    sh = _shape(T=1 << 20)
    three = L.race_b200_causal_workspace_bytes(ctypes.byref(sh), 1024, 2)
    single = L.race_b200_causal_workspace_bytes(ctypes.byref(sh), 1024, 3)
    tiles = 8 * 1024
    assert three == tiles * 64 * 65 * 4
    assert single >= 2 * three + tiles * 4 + 8           # totals + inclusive prefixes + flags + ticket
    assert L.race_b200_is_supported(ctypes.byref(sh), 3) == 1
    assert L.race_b200_is_supported(ctypes.byref(_shape(dtype=1)), 3) == 0      # fp32 only
    assert L.race_b200_is_supported(ctypes.byref(_shape(L=8, R=64, dk=128)), 3) == 0
    tile = ctypes.c_int(0)
    assert L.race_b200_select_tile_tokens(ctypes.byref(sh), 3, ctypes.byref(tile)) == 0
    assert tile.value == 1024                            # tiles in flight on all SMs stay inside the L2
    # too small a workspace for the single-pass form is refused, not silently switched
    rc = L.race_b200_causal_fwd(256, 256, 256, 256, None, None, 256, three, ctypes.byref(sh), 1024, 3, None, None)
    assert rc == -4


def test_qkv_entry_argument_errors_without_launch():
    """race_b200_causal_fwd_qkv: supported geometry and the argument errors that come before any launch."""
    L = _lib.lib()
    ok = _shape()
    assert L.race_b200_qkv_is_supported(ctypes.byref(ok), 4) == 1
    assert L.race_b200_qkv_is_supported(ctypes.byref(_shape(heads=4)), 4) == 1          # the operator's layout
    assert L.race_b200_qkv_is_supported(ctypes.byref(_shape(L=2)), 4) == 0              # two tables
    assert L.race_b200_qkv_is_supported(ctypes.byref(_shape(R=8)), 3) == 0              # three planes per table
    assert L.race_b200_qkv_is_supported(ctypes.byref(_shape(dk=128)), 4) == 0
    assert L.race_b200_qkv_is_supported(ctypes.byref(_shape(dtype=1)), 4) == 0          # bf16
    assert L.race_b200_qkv_is_supported(ctypes.byref(ok), 3) == 0                       # R != 2^K
    buf = ctypes.create_string_buffer(4096 + 16)
    p = (ctypes.addressof(buf) + 15) & ~15

    def call(shape, q=p, k=p, v=p, planes=p, out=p, ws=p, ws_bytes=1 << 40, n_planes=4, tile=0):
        return L.race_b200_causal_fwd_qkv(q, k, v, planes, out, None, None, ws, ws_bytes, ctypes.byref(shape),
                                          n_planes, tile, 0, None, None)
    assert call(ok, n_planes=3) == -2                    # RACE_ERR_SHAPE: n_buckets != 2^K
    assert call(_shape(dtype=1)) == -6                   # RACE_ERR_VARIANT: bf16 has no such kernel
    assert call(_shape(L=2)) == -6
    assert call(ok, tile=100) == -5                      # RACE_ERR_TILE
    assert call(ok, q=None) == -1                        # RACE_ERR_NULL
    assert call(ok, planes=None) == -1
    assert call(ok, k=p + 4) == -3                       # RACE_ERR_ALIGN
    assert call(ok, ws_bytes=16) == -4                   # RACE_ERR_WORKSPACE
    assert call(_shape(N=0)) == 0                        # nothing to do
