"""Probabilities-level operators on the C-ABI library.

``race_causal_prefix`` is the hot path: what ``BatchedACE.forward`` does after it has the
bucket probabilities (src/race_baseline.py:45-51), with an optional carried state
(src/race_chunked.py:54-63).  ``race_noncausal`` is the full-sequence form with gradients.
Tensors must be CUDA, contiguous, fp32 or bf16; violations raise ``RuntimeError`` the way the
reference's binding does (src/causal_v2/kernels/torch_binding.cpp:74-90).
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib

_DTYPES = {torch.float32: _lib.DTYPE_F32, torch.bfloat16: _lib.DTYPE_BF16}


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_STATUS: dict[int, torch.Tensor] = {}


def _status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 status word the kernels raise when a bounded device-side wait runs out."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _STATUS:
        _STATUS[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _STATUS[idx]


def prepare(device=None) -> None:
    """Create the per-device status word now.  Callers that must not allocate later (stream capture,
    ``race_causal_prefix_static``) call this once per device at start-up; without it the static wrapper
    runs without a status word rather than allocating one."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    _status_word(dev)


def _existing_status(device: torch.device):
    idx = device.index if device.index is not None else torch.cuda.current_device()
    return _STATUS.get(idx)


def _check_state(name, st, V, n_floats):
    if st is None:
        return
    if (not isinstance(st, torch.Tensor) or not st.is_cuda or st.device != V.device or st.dtype != torch.float32
            or not st.is_contiguous() or st.numel() != n_floats):
        raise RuntimeError(f"{name} must be a contiguous fp32 CUDA state of N*S*(d_k+1) floats on V's device")


def device_status(device=None, reset: bool = True) -> int:
    """Synchronise and return the status word of `device` (0 = every kernel ran to completion;
    non-zero = code of the first wait that gave up).  Reading it costs a device sync, so the
    operators never do it themselves unless RACE_B200_CHECK_STATUS=1 is set."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = _status_word(dev)
    val = int(word.item())
    if reset and val:
        word.zero_()
    return val


def _raise_on_wait(device, what: str) -> None:
    """With RACE_B200_CHECK_STATUS=1 (the test-suite sets it): synchronise and raise if a kernel gave up a wait."""
    if os.environ.get("RACE_B200_CHECK_STATUS") == "1":
        code = device_status(device)
        if code:
            raise RuntimeError(f"{what}: a bounded device-side wait ran out (code {code})")


def _check_inputs(probsQ, probsK, V, need_q=True):
    tensors = [("probsK", probsK), ("V", V)] + ([("probsQ", probsQ)] if need_q else [])
    for name, t in tensors:
        if not isinstance(t, torch.Tensor):
            raise RuntimeError(f"{name} must be a tensor")
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor (there is no CPU path)")
        if t.dtype not in _DTYPES:
            raise RuntimeError(f"{name}: dtype {t.dtype} not supported (float32 or bfloat16)")
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
        if t.device != V.device or t.dtype != V.dtype:
            raise RuntimeError(f"{name}: device/dtype differ from V")
    if probsK.dim() != 4 or V.dim() not in (3, 5):
        raise RuntimeError("expected probs [N,T,L,R] and V [N,T,d_k] (or [M,B,T,H,d_k])")
    if need_q and probsQ.shape != probsK.shape:
        raise RuntimeError("probsQ and probsK shapes differ")
    N, T, L, R = probsK.shape
    if V.dim() == 5:   # the operator's layout: stream n = (m*B + b)*H + h
        if V.shape[0] * V.shape[1] * V.shape[3] != N or V.shape[2] != T:
            raise RuntimeError("V [M,B,T,H,d_k] does not match probs in M*B*H or T")
    elif V.shape[0] != N or V.shape[1] != T:
        raise RuntimeError("V does not match probs in N or T")
    return N, T, L, R, V.shape[-1]


def _heads(V) -> int:
    return int(V.shape[3]) if V.dim() == 5 else 0


def make_shape(N, T, L, R, dk, dtype, eps, heads: int = 0) -> _lib.RaceShape:
    return _lib.RaceShape(N, T, L, R, dk, _DTYPES[dtype], float(eps), heads)


def pack_state(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """(A [N,L,R], B [N,L,R,d_k]) -> packed fp32 state [N, S*d_k + S] (B first, then A)."""
    N = A.shape[0]
    dt = torch.float64 if B.dtype == torch.float64 else torch.float32   # fp64 only in CPU tests
    return torch.cat([B.reshape(N, -1).to(dt), A.reshape(N, -1).to(dt)], dim=1).contiguous()


def unpack_state(state: torch.Tensor, L: int, R: int, dk: int):
    N = state.shape[0]
    S = L * R
    return state[:, S * dk:].reshape(N, L, R), state[:, : S * dk].reshape(N, L, R, dk)


def select_tile_tokens(N, T, L, R, dk, dtype=torch.float32, variant="auto") -> int:
    sh = make_shape(N, T, L, R, dk, dtype, 1e-6)
    out = ctypes.c_int(0)
    _lib.check(_lib.lib().race_b200_select_tile_tokens(ctypes.byref(sh), _lib.VARIANTS[variant],
                                                       ctypes.byref(out)), "select_tile_tokens")
    return out.value


def is_supported(N, T, L, R, dk, dtype=torch.float32, variant="auto", heads: int = 0) -> bool:
    """heads = H > 1 asks for V / out in the operator's layout [N/H, T, H, d_k]."""
    sh = make_shape(N, T, L, R, dk, dtype, 1e-6, heads)
    return bool(_lib.lib().race_b200_is_supported(ctypes.byref(sh), _lib.VARIANTS[variant]))


def race_causal_prefix(probsQ, probsK, V, eps: float = 1e-6, *, carry_in=None,
                       return_state: bool = False, tile_tokens: int = 0, variant: str = "auto",
                       out: torch.Tensor | None = None, totals_workspace: torch.Tensor | None = None,
                       normalization: str = "bucket"):
    """out[n,t,:] = sum_s pQ[n,t,s] * B_t[n,s,:] / (A_t[n,s] + eps) with inclusive prefixes
    A_t, B_t (src/race_baseline.py:45-51).

    V may also be given in the operator's layout [M,B,T,H,d_k] (stream n = (m*B+b)*H + h, the order of
    src/race_baseline.py:35-40); the output then has that layout too and no flattened copy is made
    (fp32 with S = 64, d_k = 64, and bf16 with 256 or 512 buckets: see ``is_supported(..., heads=H)``).

    carry_in: None, a packed state [N, S*d_k+S] or a tuple (A [N,L,R], B [N,L,R,d_k]) holding the
    sums over tokens before this call's first token.  return_state=True also returns (A, B)
    after the last token.  tile_tokens / variant are test hooks (0 / "auto" = automatic);
    variant="tensor_single_pass" runs the fp32 tensor forward as one persistent kernel (tile tickets, decoupled
    look-back, second read of a tile from L2: 1.05x instead of 1.5x the algorithmic DRAM traffic), bit-identical
    to "tensor" for equal tile_tokens.

    normalization="global" computes the global-normalisation estimator instead (one denominator per
    token, no eps: out_t = (pQ_t . B_t) / (pQ_t . A_t), src/causal_v2/reference.py:106-127): on the
    tcgen05 kernels for fp32 S = 64, d_k = 64 and for bf16 S = 64, else on the CUDA-core kernels; states and
    carries are the same quantities in both forms.
    """
    N, T, L, R, dk = _check_inputs(probsQ, probsK, V)
    if variant not in _lib.VARIANTS:
        raise RuntimeError(f"unknown variant {variant!r}")
    L_ = _lib.lib()
    sh = make_shape(N, T, L, R, dk, V.dtype, eps, _heads(V))
    var = _lib.VARIANTS[variant]
    if normalization not in ("bucket", "global"):
        raise RuntimeError(f"unknown normalization {normalization!r}")
    glob = normalization == "global"
    if glob:
        if totals_workspace is not None or V.dim() != 3:
            raise RuntimeError("normalization='global' takes V [N,T,d_k] and no totals_workspace")
        if V.dtype != torch.float32 and variant == "auto" and L * R != 64:
            var = _lib.VARIANTS["simt"]     # the wide bf16 tensor kernel does not have this form
    carry = None
    if carry_in is not None:
        carry = pack_state(*carry_in) if isinstance(carry_in, (tuple, list)) else carry_in
        _check_state("carry_in", carry, V, N * L * R * (dk + 1))
    with torch.cuda.device(V.device):
        if out is None:
            out = torch.empty_like(V)
        state = torch.empty(N, L * R * (dk + 1), dtype=torch.float32, device=V.device) \
            if return_state else None
        ws_bytes = L_.race_b200_causal_workspace_bytes(ctypes.byref(sh), tile_tokens, var)
        if totals_workspace is not None:
            # second half after race_tile_totals(..., return_workspace=True) with the same
            # tile_tokens / variant: the per-tile totals are already in the workspace
            if totals_workspace.numel() < ws_bytes or totals_workspace.device != V.device:
                raise RuntimeError("totals_workspace does not belong to this shape")
            entry, ws = L_.race_b200_causal_fwd_resume, totals_workspace
        else:
            entry, ws = L_.race_b200_causal_fwd, torch.empty(max(ws_bytes, 16), dtype=torch.uint8,
                                                             device=V.device)
        if glob:
            rc = L_.race_b200_causal_fwd_global(_ptr(probsQ), _ptr(probsK), _ptr(V), _ptr(out), _ptr(carry),
                                                _ptr(state), _ptr(ws), ws_bytes, ctypes.byref(sh), tile_tokens,
                                                var, _stream(), _ptr(_status_word(V.device)))
        else:
            rc = entry(_ptr(probsQ), _ptr(probsK), _ptr(V), _ptr(out), _ptr(carry),
                       _ptr(state), _ptr(ws), ws_bytes, ctypes.byref(sh),
                       tile_tokens, var, _stream(), _ptr(_status_word(V.device)))
    _lib.check(rc, "race_b200_causal_fwd")
    _raise_on_wait(V.device, "race_b200_causal_fwd")
    if return_state:
        A, B = unpack_state(state, L, R, dk)
        return out, A, B
    return out


def qkv_is_supported(N, T, L, K, dk, dtype=torch.float32, heads: int = 0) -> bool:
    """Whether ``race_causal_qkv`` takes this geometry (fp32, d_k = 64, L = 4, K = 4)."""
    sh = make_shape(N, T, L, 1 << K, dk, dtype, 1e-6, heads)
    return bool(_lib.lib().race_b200_qkv_is_supported(ctypes.byref(sh), K))


def race_causal_qkv(Q, K, V, planes, L: int, n_planes: int, eps: float = 1e-6, *, carry_in=None,
                    return_state: bool = False, tile_tokens: int = 0, out: torch.Tensor | None = None,
                    normalization: str = "bucket"):
    """The causal forward of ``BatchedACE`` from Q, K, V and the hyperplanes (src/race_baseline.py:41-51) with the
    bucket probabilities formed inside the prefix kernels: they never exist in device memory.

    Q, K, V: fp32 CUDA tensors of one shape, [N,T,d_k] or the operator's layout [M,B,T,H,d_k] (stream
    n = (m*B+b)*H + h); planes: fp32 [L*n_planes, d_k] (``planes_T.T``).  Geometry: ``qkv_is_supported``.
    carry_in / return_state / normalization as in ``race_causal_prefix``; the output has the layout of V."""
    if not (Q.shape == K.shape == V.shape) or V.dim() not in (3, 5):
        raise RuntimeError("Q, K, V must have one shape, [N,T,d_k] or [M,B,T,H,d_k]")
    for name, t in (("Q", Q), ("K", K), ("V", V)):
        if not t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous() or t.device != V.device:
            raise RuntimeError(f"{name} must be a contiguous fp32 CUDA tensor on V's device")
    if normalization not in ("bucket", "global"):
        raise RuntimeError(f"unknown normalization {normalization!r}")
    dk, R = V.shape[-1], 1 << n_planes
    if V.dim() == 5:
        M, B, T, H, _ = V.shape
        N = M * B * H
    else:
        (N, T, _), H = V.shape, 0
    planes = planes.to(device=V.device, dtype=torch.float32).contiguous()
    if planes.shape != (L * n_planes, dk):
        raise RuntimeError(f"planes must be [L*K, d_k] = [{L * n_planes}, {dk}]")
    L_ = _lib.lib()
    sh = make_shape(N, T, L, R, dk, V.dtype, eps, H)
    if not L_.race_b200_qkv_is_supported(ctypes.byref(sh), n_planes):
        raise RuntimeError("race_causal_qkv: geometry not supported (fp32, d_k = 64, L = 4, K = 4); use "
                           "bucket_probs_streams + race_causal_prefix")
    carry = None
    if carry_in is not None:
        carry = pack_state(*carry_in) if isinstance(carry_in, (tuple, list)) else carry_in
        _check_state("carry_in", carry, V, N * L * R * (dk + 1))
    with torch.cuda.device(V.device):
        if out is None:
            out = torch.empty_like(V)
        state = torch.empty(N, L * R * (dk + 1), dtype=torch.float32, device=V.device) if return_state else None
        ws_bytes = L_.race_b200_causal_workspace_bytes(ctypes.byref(sh), tile_tokens, _lib.VARIANTS["tensor"])
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=V.device)
        rc = L_.race_b200_causal_fwd_qkv(_ptr(Q), _ptr(K), _ptr(V), _ptr(planes), _ptr(out), _ptr(carry),
                                         _ptr(state), _ptr(ws), ws_bytes, ctypes.byref(sh), n_planes, tile_tokens,
                                         1 if normalization == "global" else 0, _stream(),
                                         _ptr(_status_word(V.device)))
    _lib.check(rc, "race_b200_causal_fwd_qkv")
    _raise_on_wait(V.device, "race_b200_causal_fwd_qkv")
    if return_state:
        A, B = unpack_state(state, L, R, dk)
        return out, A, B
    return out


def race_decode_step(probsQ, probsK, V, state: torch.Tensor, eps: float = 1e-6, *,
                     state_out: torch.Tensor | None = None) -> torch.Tensor:
    """Incremental step: outputs of T <= 64 new tokens per stream (typically one) given the packed
    running state [N, S*d_k+S] of everything before them, which is advanced IN PLACE (or written to
    ``state_out``, leaving ``state`` untouched).  One chunk step of src/race_chunked.py:54-63; start
    from ``torch.zeros`` or from the state a ``race_causal_prefix(..., return_state=True)`` prefill
    returned (``pack_state(A, B)``)."""
    N, T, L, R, dk = _check_inputs(probsQ, probsK, V)
    if V.dim() != 3:
        raise RuntimeError("race_decode_step takes V as [N,T,d_k]")
    dst = state if state_out is None else state_out
    for st in (state, dst):
        if (not st.is_cuda or st.device != V.device or st.dtype != torch.float32 or not st.is_contiguous()
                or st.numel() != N * L * R * (dk + 1)):
            raise RuntimeError("state must be a contiguous fp32 CUDA state of N*S*(d_k+1) floats")
    sh = make_shape(N, T, L, R, dk, V.dtype, eps)
    with torch.cuda.device(V.device):
        out = torch.empty_like(V)
        rc = _lib.lib().race_b200_decode_step(_ptr(probsQ), _ptr(probsK), _ptr(V), _ptr(out), _ptr(state),
                                              _ptr(dst), ctypes.byref(sh), _stream())
    _lib.check(rc, "race_b200_decode_step")
    return out


class DecodeStepper:
    """``race_decode_step`` for a serving loop: shape, dtype and device are fixed and checked once, the
    output buffer is allocated once, and a call is little more than the C-ABI call itself (the general
    wrapper spends most of a one-token step on Python-side validation).

        step = DecodeStepper(N, L, R, d_k, torch.float32, device)
        out = step(pQ_t, pK_t, V_t, state)      # [N, tokens, d_k]; `state` advanced in place

    The returned tensor is the stepper's own buffer: it is overwritten by the next call."""

    def __init__(self, N: int, L: int, R: int, dk: int, dtype=torch.float32, device=None, tokens: int = 1,
                 eps: float = 1e-6):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.shape = make_shape(N, tokens, L, R, dk, dtype, eps)
        self._shape_ref = ctypes.byref(self.shape)
        self._fn = _lib.lib().race_b200_decode_step
        self._probs = (N, tokens, L, R)
        self._v = (N, tokens, dk)
        self._state_floats = N * L * R * (dk + 1)
        self._dtype = dtype
        self.out = torch.empty(N, tokens, dk, dtype=dtype, device=self.device)
        # one validated call-through of the general wrapper's checks, on zeros
        z = torch.zeros(N, tokens, L, R, dtype=dtype, device=self.device)
        race_decode_step(z, z, torch.zeros(N, tokens, dk, dtype=dtype, device=self.device),
                         torch.zeros(N, L * R * (dk + 1), device=self.device))

    def __call__(self, probsQ, probsK, V, state):
        if (probsQ.shape != self._probs or probsK.shape != self._probs or V.shape != self._v
                or state.numel() != self._state_floats or state.dtype != torch.float32
                or probsQ.dtype != self._dtype or probsK.dtype != self._dtype or V.dtype != self._dtype
                or probsQ.device != self.device or probsK.device != self.device or V.device != self.device
                or state.device != self.device
                or not (probsQ.is_contiguous() and probsK.is_contiguous() and V.is_contiguous()
                        and state.is_contiguous())):
            raise RuntimeError("DecodeStepper: tensors do not match the shape/dtype/device it was built for")
        sp = state.data_ptr()
        rc = self._fn(probsQ.data_ptr(), probsK.data_ptr(), V.data_ptr(), self.out.data_ptr(), sp, sp,
                      self._shape_ref, torch.cuda.current_stream(self.device).cuda_stream)
        if rc:
            _lib.check(rc, "race_b200_decode_step")
        return self.out


def race_tile_totals(probsK, V, *, tile_tokens: int = 0, variant: str = "auto",
                     return_workspace: bool = False):
    """(A [N,L,R], B [N,L,R,d_k]) summed over all T tokens (pass 1 of the sequence-sharded
    driver; the final carry of src/race_chunked.py:62-63).  With return_workspace=True the
    workspace holding the per-tile totals is returned as a third value; pass it to
    ``race_causal_prefix(..., totals_workspace=...)`` to finish the forward without reducing
    pK and V again."""
    N, T, L, R, dk = _check_inputs(None, probsK, V, need_q=False)
    L_ = _lib.lib()
    sh = make_shape(N, T, L, R, dk, V.dtype, 1e-6, _heads(V))
    var = _lib.VARIANTS[variant]
    with torch.cuda.device(V.device):
        state = torch.empty(N, L * R * (dk + 1), dtype=torch.float32, device=V.device)
        ws_bytes = L_.race_b200_causal_workspace_bytes(ctypes.byref(sh), tile_tokens, var)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=V.device)
        rc = L_.race_b200_tile_totals(_ptr(probsK), _ptr(V), _ptr(state), _ptr(ws), ws_bytes,
                                      ctypes.byref(sh), tile_tokens, var, _stream(),
                                      _ptr(_status_word(V.device)))
    _lib.check(rc, "race_b200_tile_totals")
    A, B = unpack_state(state, L, R, dk)
    return (A, B, ws) if return_workspace else (A, B)


def bucket_probs(x: torch.Tensor, planes: torch.Tensor, L: int, K: int,
                 out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """x [..., d_k] -> probs [..., L, 2**K]  (src/race_baseline.py:41-44).

    planes: fp32 [L*K, d_k] row-major (``planes_T.T``)."""
    if not x.is_cuda or x.dtype not in _DTYPES or not x.is_contiguous():
        raise RuntimeError("x must be a contiguous fp32/bf16 CUDA tensor")
    dk = x.shape[-1]
    planes = planes.to(device=x.device, dtype=torch.float32).contiguous()
    if planes.shape != (L * K, dk):
        raise RuntimeError(f"planes must be [L*K, d_k] = [{L * K}, {dk}]")
    out_dtype = out_dtype or x.dtype
    rows = x.numel() // dk
    with torch.cuda.device(x.device):
        probs = torch.empty(*x.shape[:-1], L, 1 << K, dtype=out_dtype, device=x.device)
        rc = _lib.lib().race_b200_bucket_probs(_ptr(x), _ptr(planes), _ptr(probs), rows, dk, L, K,
                                               _DTYPES[x.dtype], _DTYPES[out_dtype], _stream())
    _lib.check(rc, "race_b200_bucket_probs")
    return probs


def bucket_probs_streams(x: torch.Tensor, planes: torch.Tensor, L: int, K: int,
                         out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """x [M, B, T, H, d_k] (the operator's layout) -> probs [M*B*H, T, L, 2**K]: the stream flattening
    of src/race_baseline.py:35-40 fused into the producer of :41-44; no flattened copy of x is made.

    planes: fp32 [L*K, d_k] row-major (``planes_T.T``)."""
    if not x.is_cuda or x.dtype not in _DTYPES or not x.is_contiguous() or x.dim() != 5:
        raise RuntimeError("x must be a contiguous fp32/bf16 CUDA tensor [M,B,T,H,d_k]")
    M, B, T, H, dk = x.shape
    planes = planes.to(device=x.device, dtype=torch.float32).contiguous()
    if planes.shape != (L * K, dk):
        raise RuntimeError(f"planes must be [L*K, d_k] = [{L * K}, {dk}]")
    out_dtype = out_dtype or x.dtype
    with torch.cuda.device(x.device):
        probs = torch.empty(M * B * H, T, L, 1 << K, dtype=out_dtype, device=x.device)
        rc = _lib.lib().race_b200_bucket_probs_streams(_ptr(x), _ptr(planes), _ptr(probs), M * B, T, H, dk,
                                                       L, K, _DTYPES[x.dtype], _DTYPES[out_dtype], _stream())
    _lib.check(rc, "race_b200_bucket_probs_streams")
    return probs


class _RaceCausal(torch.autograd.Function):
    """The causal forward (``race_causal_prefix``) with the hand-written backward kernels.  Only the
    three inputs are saved: the backward recomputes the prefix states tile by tile."""

    @staticmethod
    def forward(ctx, probsQ, probsK, V, eps):
        out = race_causal_prefix(probsQ, probsK, V, eps)
        ctx.save_for_backward(probsQ, probsK, V)
        ctx.eps = eps
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_out):
        probsQ, probsK, V = ctx.saved_tensors
        if not any(ctx.needs_input_grad[:3]):
            return None, None, None, None
        dpq, dpk, dv = race_causal_backward(probsQ, probsK, V, grad_out, ctx.eps)
        g = ctx.needs_input_grad
        return (dpq if g[0] else None, dpk if g[1] else None, dv if g[2] else None, None)


def race_causal_backward(probsQ, probsK, V, grad_out, eps: float = 1e-6, *, carry_in=None, grad_state=None,
                         return_grad_carry: bool = False):
    """(d probsQ, d probsK, d V) of ``race_causal_prefix(probsQ, probsK, V, eps)`` for the output
    gradient ``grad_out`` [N,T,d_k] (derivative of src/race_baseline.py:45-51; L*R <= 64 or a multiple of 64
    up to 512, d_k <= 128).

    For one chunk of a longer sequence: ``carry_in`` is the packed state the forward was given,
    ``grad_state`` the gradient reaching the packed state it returned, and ``return_grad_carry=True``
    appends the gradient of ``carry_in`` to the result."""
    N, T, L, R, dk = _check_inputs(probsQ, probsK, V)
    if V.dim() != 3:
        raise RuntimeError("race_causal_backward takes V as [N,T,d_k]")
    if grad_out.shape != V.shape or not grad_out.is_cuda:
        raise RuntimeError("grad_out must be a CUDA tensor shaped like V")
    # autograd may hand over an expanded (stride-0) gradient: the kernels need dense rows
    grad_out = grad_out.to(V.dtype).contiguous()
    L_ = _lib.lib()
    sh = make_shape(N, T, L, R, dk, V.dtype, eps)
    with torch.cuda.device(V.device):
        dpq, dpk, dv = torch.empty_like(probsQ), torch.empty_like(probsK), torch.empty_like(V)
        ws_bytes = L_.race_b200_causal_bwd_workspace_bytes(ctypes.byref(sh))
        ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=V.device)
        for st in (carry_in, grad_state):
            if st is not None and (not st.is_cuda or st.dtype != torch.float32 or not st.is_contiguous()
                                   or st.numel() != N * L * R * (dk + 1)):
                raise RuntimeError("carry_in / grad_state must be contiguous fp32 CUDA states of N*S*(d_k+1) floats")
        dcarry = torch.empty(N, L * R * (dk + 1), dtype=torch.float32, device=V.device) if return_grad_carry else None
        rc = L_.race_b200_causal_bwd_carry(_ptr(probsQ), _ptr(probsK), _ptr(V), _ptr(grad_out), _ptr(carry_in),
                                           _ptr(grad_state), _ptr(dpq), _ptr(dpk), _ptr(dv), _ptr(dcarry), _ptr(ws),
                                           ws_bytes, ctypes.byref(sh), _stream(), _ptr(_status_word(V.device)))
    _lib.check(rc, "race_b200_causal_bwd_carry")
    _raise_on_wait(V.device, "race_b200_causal_bwd_carry")
    return (dpq, dpk, dv, dcarry) if return_grad_carry else (dpq, dpk, dv)


class _RaceCausalChunk(torch.autograd.Function):
    """One chunk of a longer sequence: (out, state_out) = forward(pQ, pK, V, state_in), differentiable in all
    four, so that chained chunks back-propagate through the carried state."""

    @staticmethod
    def forward(ctx, probsQ, probsK, V, state, eps):
        N, T, L, R = probsK.shape
        out, A, B = race_causal_prefix(probsQ, probsK, V, eps, carry_in=state, return_state=True)
        ctx.save_for_backward(probsQ, probsK, V, state)
        ctx.eps = eps
        return out, pack_state(A, B)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_out, grad_state):
        probsQ, probsK, V, state = ctx.saved_tensors
        gs = None if grad_state is None else grad_state.float().contiguous()
        dpq, dpk, dv, dcarry = race_causal_backward(probsQ, probsK, V, grad_out, ctx.eps, carry_in=state,
                                                    grad_state=gs, return_grad_carry=True)
        g = ctx.needs_input_grad
        return (dpq if g[0] else None, dpk if g[1] else None, dv if g[2] else None, dcarry if g[3] else None, None)


def race_causal_chunk(probsQ, probsK, V, state, eps: float = 1e-6):
    """Differentiable chunk step for sequences processed in pieces (the loop of src/race_chunked.py:45-63 with
    gradients): returns (out, new_state); ``state`` is the packed [N, S*(d_k+1)] running state (zeros before
    the first chunk).  Chain the calls and call ``backward`` once: autograd walks the chunks in reverse."""
    return _RaceCausalChunk.apply(probsQ, probsK, V, state, eps)


def race_causal(probsQ, probsK, V, eps: float = 1e-6) -> torch.Tensor:
    """Differentiable causal per-bucket forward: ``race_causal_prefix`` with gradients for all three
    inputs (the training-time form; the reference has none)."""
    return _RaceCausal.apply(probsQ, probsK, V, eps)


class _RaceNonCausal(torch.autograd.Function):
    """out = pQ . (pK^T V / (sum_t pK + eps)) with the hand-written backward kernels.

    Saved for backward: the three inputs and the reduced sums (Bs, A) -- the same choice the
    reference's autograd wrapper makes (src/noncausal/ops.py:29-33)."""

    @staticmethod
    def forward(ctx, probsQ, probsK, V, eps):
        N, T, L, R, dk = _check_inputs(probsQ, probsK, V)
        if V.dim() != 3:
            raise RuntimeError("race_noncausal takes V as [N,T,d_k]")
        L_ = _lib.lib()
        sh = make_shape(N, T, L, R, dk, V.dtype, eps)
        with torch.cuda.device(V.device):
            out = torch.empty_like(V)
            totals = torch.empty(N, L * R * (dk + 1), dtype=torch.float32, device=V.device)
            ws_bytes = L_.race_b200_causal_workspace_bytes(ctypes.byref(sh), 0, _lib.VARIANTS["auto"])
            ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=V.device)
            rc = L_.race_b200_noncausal_fwd(_ptr(probsQ), _ptr(probsK), _ptr(V), _ptr(out),
                                            _ptr(totals), _ptr(ws), ws_bytes, ctypes.byref(sh),
                                            _stream())
        _lib.check(rc, "race_b200_noncausal_fwd")
        ctx.save_for_backward(probsQ, probsK, V, totals)
        ctx.eps = eps
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_out):
        probsQ, probsK, V, totals = ctx.saved_tensors
        if not any(ctx.needs_input_grad[:3]):
            return None, None, None, None
        N, T, L, R = probsK.shape
        dk = V.shape[-1]
        # autograd may hand over an expanded (stride-0) gradient: the kernels need dense rows
        grad_out = grad_out.to(V.dtype).contiguous()
        L_ = _lib.lib()
        sh = make_shape(N, T, L, R, dk, V.dtype, ctx.eps)
        with torch.cuda.device(V.device):
            dpq, dpk, dv = torch.empty_like(probsQ), torch.empty_like(probsK), torch.empty_like(V)
            ws_bytes = L_.race_b200_noncausal_bwd_workspace_bytes(ctypes.byref(sh))
            ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=V.device)
            rc = L_.race_b200_noncausal_bwd(_ptr(probsQ), _ptr(probsK), _ptr(V), _ptr(totals),
                                            _ptr(grad_out), _ptr(dpq), _ptr(dpk), _ptr(dv), _ptr(ws),
                                            ws_bytes, ctypes.byref(sh), _stream())
        _lib.check(rc, "race_b200_noncausal_bwd")
        g = ctx.needs_input_grad
        return (dpq if g[0] else None, dpk if g[1] else None, dv if g[2] else None, None)


def race_noncausal(probsQ, probsK, V, eps: float = 1e-6) -> torch.Tensor:
    """Non-causal per-bucket RACE attention, differentiable in probsQ, probsK and V
    (upstream scaling/benchmark_time.py:155-162 as quoted at analysis/hot-path.md:157-162)."""
    return _RaceNonCausal.apply(probsQ, probsK, V, float(eps))


def race_causal_prefix_host(probsQ, probsK, V, eps: float = 1e-6, *, carry_in=None,
                            return_state: bool = False, segment_tokens: int = 0,
                            variant: str = "auto", device: int | None = None,
                            out: torch.Tensor | None = None):
    """Same result as ``race_causal_prefix`` for tensors in HOST memory (pin them for full copy
    bandwidth): the library stages the sequence through the device in segments and returns
    after the last copy back has finished."""
    for name, t in (("probsQ", probsQ), ("probsK", probsK), ("V", V)):
        if t.is_cuda or not t.is_contiguous() or t.dtype not in _DTYPES or t.dtype != V.dtype:
            raise RuntimeError(f"{name} must be a contiguous fp32/bf16 host tensor")
    N, T, L, R = probsK.shape
    dk = V.shape[-1]
    if probsQ.shape != probsK.shape or V.shape[:2] != (N, T):
        raise RuntimeError("shape mismatch")
    sh = make_shape(N, T, L, R, dk, V.dtype, eps)
    carry = None
    if carry_in is not None:
        carry = (pack_state(*carry_in) if isinstance(carry_in, (tuple, list)) else carry_in)
        carry = carry.float().contiguous().cpu()
    if out is None:
        out = torch.empty_like(V)
    state = torch.empty(N, L * R * (dk + 1), dtype=torch.float32) if return_state else None
    dev = torch.cuda.current_device() if device is None else device
    rc = _lib.lib().race_b200_causal_fwd_host(_ptr(probsQ), _ptr(probsK), _ptr(V), _ptr(out),
                                              _ptr(carry), _ptr(state), ctypes.byref(sh),
                                              segment_tokens, _lib.VARIANTS[variant], dev)
    _lib.check(rc, "race_b200_causal_fwd_host")
    if return_state:
        A, B = unpack_state(state, L, R, dk)
        return out, A, B
    return out


def race_causal_prefix_static(probsQ, probsK, V, out, eps: float = 1e-6, *, carry_in=None,
                              state_out: torch.Tensor | None = None, tile_tokens: int = 0,
                              variant: str = "auto") -> torch.Tensor:
    """``race_causal_prefix`` for callers that cannot allocate device memory when they call.

    Examples of such callers: code that runs while a CUDA stream capture is open, hooks that the
    caching allocator itself invokes, serving loops that pre-plan all device memory.  This
    wrapper allocates nothing either: `out` (and `state_out`, a packed fp32 state
    [N, S*(d_k+1)], if the final state is wanted) must be passed in, `carry_in` must already be a
    packed state, and the kernels' workspace is the 16 MiB array built into the library.
    Shapes that need more raise ``RuntimeError`` (RACE_ERR_SCRATCH).  All calls share that array:
    issue them on one stream or order them with events.  Make the first call on each device
    outside of stream capture (it looks up the array's device address).  The kernels report a
    wait that ran out through the per-device status word only if that word already exists
    (``prepare(device)`` at start-up, or any other operator of this module called before): this
    wrapper does not create it."""
    N, T, L, R, dk = _check_inputs(probsQ, probsK, V)
    if (not isinstance(out, torch.Tensor) or out.shape != V.shape or out.dtype != V.dtype
            or not out.is_contiguous() or out.device != V.device):
        raise RuntimeError("out must be a contiguous tensor like V")
    if variant not in _lib.VARIANTS:
        raise RuntimeError(f"unknown variant {variant!r}")
    _check_state("carry_in", carry_in, V, N * L * R * (dk + 1))
    _check_state("state_out", state_out, V, N * L * R * (dk + 1))
    sh = make_shape(N, T, L, R, dk, V.dtype, eps, _heads(V))
    with torch.cuda.device(V.device):
        rc = _lib.lib().race_b200_causal_fwd_static(
            _ptr(probsQ), _ptr(probsK), _ptr(V), _ptr(out), _ptr(carry_in), _ptr(state_out),
            ctypes.byref(sh), tile_tokens, _lib.VARIANTS[variant], _stream(),
            _ptr(_existing_status(V.device)))
    _lib.check(rc, "race_b200_causal_fwd_static")
    return out


def selftest_bounded_wait(probsQ, probsK, V, wait_cycles: int = 2_000_000, withhold_chunk: int = 1,
                          variant: str = "tensor"):
    """Diagnostics: run the fp32 tensor forward with every device-side wait limited to ``wait_cycles``
    SM cycles while the first CTA's load of one chunk is withheld (``race_b200_selftest_bounded_wait``).
    Returns ``(out, code)``: ``code`` is the status the kernels raised (non-zero when the wait ran out as
    designed); the rows of ``out`` that belong to the first tile of stream 0 are unspecified."""
    N, T, L, R, dk = _check_inputs(probsQ, probsK, V)
    if V.dim() != 3:
        raise RuntimeError("selftest_bounded_wait takes V as [N,T,d_k]")
    L_ = _lib.lib()
    sh = make_shape(N, T, L, R, dk, V.dtype, 1e-6)
    var = _lib.VARIANTS[variant]
    with torch.cuda.device(V.device):
        out = torch.empty_like(V)
        word = torch.zeros(1, dtype=torch.int32, device=V.device)
        ws_bytes = L_.race_b200_causal_workspace_bytes(ctypes.byref(sh), 0, var)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=V.device)
        rc = L_.race_b200_selftest_bounded_wait(_ptr(probsQ), _ptr(probsK), _ptr(V), _ptr(out), _ptr(ws), ws_bytes,
                                                ctypes.byref(sh), var, int(wait_cycles), int(withhold_chunk), _stream(),
                                                _ptr(word))
        _lib.check(rc, "race_b200_selftest_bounded_wait")
        code = int(word.item())
    return out, code
