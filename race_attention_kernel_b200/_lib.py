"""ctypes binding of the C-ABI library (``include/race_b200.h``).

The library is the product: there is no Python or CPU fallback.  ``lib()`` raises if the
shared object is missing or cannot be loaded, and every wrapper raises ``RuntimeError`` on a
non-zero return code, mirroring the reference binding's TORCH_CHECK / C10_CUDA_CHECK behaviour
(src/causal_v2/kernels/torch_binding.cpp:74-90, 139-168).
"""
from __future__ import annotations

import ctypes
import functools
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "librace_b200.so")

DTYPE_F32, DTYPE_BF16 = 0, 1
VARIANTS = {"auto": 0, "simt": 1, "tensor": 2, "tensor_single_pass": 3}

EXPORTS = [
    "race_b200_version", "race_b200_error_string", "race_b200_is_supported",
    "race_b200_state_floats", "race_b200_select_tile_tokens", "race_b200_causal_workspace_bytes",
    "race_b200_causal_fwd", "race_b200_tile_totals", "race_b200_causal_fwd_resume",
    "race_b200_noncausal_fwd",
    "race_b200_noncausal_bwd_workspace_bytes", "race_b200_noncausal_bwd",
    "race_b200_bucket_probs", "race_b200_bucket_probs_streams", "race_b200_causal_fwd_host",
    "race_b200_static_scratch_bytes", "race_b200_causal_fwd_static", "race_b200_decode_step",
    "race_b200_causal_fwd_global", "race_b200_causal_bwd_workspace_bytes", "race_b200_causal_bwd",
    "race_b200_causal_bwd_carry", "race_b200_selftest_bounded_wait", "race_b200_host_release",
    "race_b200_qkv_is_supported", "race_b200_causal_fwd_qkv",
]


class RaceShape(ctypes.Structure):
    _fields_ = [
        ("n_streams", ctypes.c_int64), ("seq_len", ctypes.c_int64),
        ("n_tables", ctypes.c_int32), ("n_buckets", ctypes.c_int32),
        ("head_dim", ctypes.c_int32), ("dtype", ctypes.c_int32),
        ("eps", ctypes.c_float), ("heads", ctypes.c_int32),
    ]


@functools.cache
def lib() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m race_attention_kernel_b200.build` "
            "(there is no CPU or PyTorch fallback for the kernels)")
    L = ctypes.CDLL(LIB_PATH)
    vp, sz, i32, i64 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int64
    shp = ctypes.POINTER(RaceShape)
    L.race_b200_version.restype = i32
    L.race_b200_error_string.restype = ctypes.c_char_p
    L.race_b200_error_string.argtypes = [i32]
    L.race_b200_is_supported.restype = i32
    L.race_b200_is_supported.argtypes = [shp, i32]
    L.race_b200_state_floats.restype = sz
    L.race_b200_state_floats.argtypes = [shp]
    L.race_b200_select_tile_tokens.restype = i32
    L.race_b200_select_tile_tokens.argtypes = [shp, i32, ctypes.POINTER(i32)]
    L.race_b200_causal_workspace_bytes.restype = sz
    L.race_b200_causal_workspace_bytes.argtypes = [shp, i32, i32]
    L.race_b200_causal_fwd.restype = i32
    L.race_b200_causal_fwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, sz, shp, i32, i32, vp, vp]
    L.race_b200_tile_totals.restype = i32
    L.race_b200_tile_totals.argtypes = [vp, vp, vp, vp, sz, shp, i32, i32, vp, vp]
    L.race_b200_causal_fwd_resume.restype = i32
    L.race_b200_causal_fwd_resume.argtypes = [vp, vp, vp, vp, vp, vp, vp, sz, shp, i32, i32, vp, vp]
    L.race_b200_noncausal_fwd.restype = i32
    L.race_b200_noncausal_fwd.argtypes = [vp, vp, vp, vp, vp, vp, sz, shp, vp]
    L.race_b200_noncausal_bwd_workspace_bytes.restype = sz
    L.race_b200_noncausal_bwd_workspace_bytes.argtypes = [shp]
    L.race_b200_noncausal_bwd.restype = i32
    L.race_b200_noncausal_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, shp, vp]
    L.race_b200_bucket_probs.restype = i32
    L.race_b200_bucket_probs.argtypes = [vp, vp, vp, i64, i32, i32, i32, i32, i32, vp]
    L.race_b200_bucket_probs_streams.restype = i32
    L.race_b200_bucket_probs_streams.argtypes = [vp, vp, vp, i64, i64, i32, i32, i32, i32, i32, i32, vp]
    L.race_b200_causal_fwd_host.restype = i32
    L.race_b200_causal_fwd_host.argtypes = [vp, vp, vp, vp, vp, vp, shp, i64, i32, i32]
    L.race_b200_host_release.restype = i32
    L.race_b200_host_release.argtypes = [i32]
    L.race_b200_static_scratch_bytes.restype = sz
    L.race_b200_static_scratch_bytes.argtypes = []
    L.race_b200_causal_fwd_static.restype = i32
    L.race_b200_causal_fwd_static.argtypes = [vp, vp, vp, vp, vp, vp, shp, i32, i32, vp, vp]
    L.race_b200_causal_fwd_global.restype = i32
    L.race_b200_causal_fwd_global.argtypes = [vp, vp, vp, vp, vp, vp, vp, sz, shp, i32, i32, vp, vp]
    L.race_b200_qkv_is_supported.restype = i32
    L.race_b200_qkv_is_supported.argtypes = [shp, i32]
    L.race_b200_causal_fwd_qkv.restype = i32
    L.race_b200_causal_fwd_qkv.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, sz, shp, i32, i32, i32, vp, vp]
    L.race_b200_selftest_bounded_wait.restype = i32
    L.race_b200_selftest_bounded_wait.argtypes = [vp, vp, vp, vp, vp, sz, shp, i32, i64, i32, vp, vp]
    L.race_b200_causal_bwd_workspace_bytes.restype = sz
    L.race_b200_causal_bwd_workspace_bytes.argtypes = [shp]
    L.race_b200_causal_bwd.restype = i32
    L.race_b200_causal_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, sz, shp, vp, vp]
    L.race_b200_causal_bwd_carry.restype = i32
    L.race_b200_causal_bwd_carry.argtypes = [vp] * 10 + [vp, sz, shp, vp, vp]
    L.race_b200_decode_step.restype = i32
    L.race_b200_decode_step.argtypes = [vp, vp, vp, vp, vp, vp, shp, vp]
    return L


def check(code: int, what: str) -> None:
    if code != 0:
        msg = lib().race_b200_error_string(code).decode()
        raise RuntimeError(f"{what}: {msg} (code {code})")
