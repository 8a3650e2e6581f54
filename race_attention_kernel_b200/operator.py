"""Drop-in operator: ``BatchedACE`` with the reference's constructor and call signature.

    ace = BatchedACE(d_k, K, L, M)            # buffers drawn like the reference (CPU RNG)
    ace = ace.cuda()
    out = ace(Khf, Vhf, Qhf)                  # argument order K, V, Q; each [M,B,T,H,d_k]

(src/race_baseline.py:21-52).  Buffers keep the reference's names and shapes (``planes_T``
[d_k, L*K], ``protos_T`` [K, R]) so code that overwrites ``ace.planes_T`` keeps working.
The forward runs on the GPU only: bucket probabilities come from the producer kernel and the
cumsum/divide/bmm of the reference is replaced by the prefix kernel.  Host tensors are
accepted and streamed through the device; there is no CPU compute path.

Gradients: the reference module is differentiable through K, V and Q (plain autograd over
src/race_baseline.py:41-51).  Here, when autograd is recording and an input requires a gradient,
``forward`` forms the bucket probabilities with differentiable torch ops on the GPU (the producer
kernel has no backward) and runs the prefix path through ``ops.race_causal`` -- the same forward
kernels with the hand-written backward kernels.  Without gradients it is the pure kernel path.
"""
from __future__ import annotations

import itertools

import torch
from torch import nn

from . import ops


class BatchedACE(nn.Module):
    def __init__(self, d_k, K, L, M, device="cpu", share_planes=True):
        super().__init__()
        assert share_planes, "reference config uses shared planes"
        self.d_k, self.K, self.L, self.M = d_k, K, L, M
        self.R = 1 << K
        # drawn exactly like the reference (src/race_baseline.py:27-32) so that a seeded
        # construction gives the same planes
        planes = torch.randn(L, K, d_k, device=device)
        self.register_buffer("planes_T", planes.view(L * K, d_k).T)
        corners = torch.tensor(list(itertools.product([-1.0, 1.0], repeat=K)), device=device)
        self.register_buffer("protos_T", corners.T)
        self.eps = 1e-6
        self.variant = "auto"
        # form the bucket probabilities inside the prefix kernels where that path exists (fp32, d_k = 64, L = 4,
        # K = 4); False keeps the producer kernel and the probabilities in device memory
        self.fuse_producer = True

    def _streams(self, x: torch.Tensor) -> torch.Tensor:
        M, B, T, H, dk = x.shape
        return x.permute(0, 1, 3, 2, 4).contiguous().view(M * B * H, T, dk)

    def bucket_probs(self, x2: torch.Tensor) -> torch.Tensor:
        """[N,T,d_k] -> [N,T,L,R] with this module's planes."""
        planes = self.planes_T.T.contiguous().float()
        return ops.bucket_probs(x2, planes, self.L, self.K)

    def _probs_autograd(self, x2: torch.Tensor) -> torch.Tensor:
        """src/race_baseline.py:41-44 with torch ops (differentiable); x2 [N,T,d_k] on the GPU."""
        N, T, dk = x2.shape
        planes_T = self.planes_T.to(device=x2.device, dtype=torch.float32)
        protos_T = self.protos_T.to(device=x2.device, dtype=torch.float32)
        proj = (x2.float() @ planes_T).view(N, T, self.L, self.K)
        logits = proj.tanh().div(dk ** 0.5) @ protos_T
        return torch.softmax(logits, dim=-1).to(x2.dtype)

    def _forward_autograd(self, Khf, Vhf, Qhf):
        M, B, T, H, dk = Khf.shape
        dev = self.planes_T.device if self.planes_T.is_cuda else torch.device("cuda", torch.cuda.current_device())
        K2, V2, Q2 = (self._streams(t.to(dev)) for t in (Khf, Vhf, Qhf))
        out2 = ops.race_causal(self._probs_autograd(Q2), self._probs_autograd(K2), V2, self.eps)
        out = out2.view(M, B, H, T, dk).permute(0, 1, 3, 2, 4)
        return out if Khf.is_cuda else out.cpu()

    def forward(self, Khf, Vhf, Qhf, *, carry_in=None, return_state=False):
        if not (Khf.shape == Vhf.shape == Qhf.shape) or Khf.dim() != 5:
            raise RuntimeError("expected K, V, Q of identical shape [M,B,T,H,d_k]")
        M, B, T, H, dk = Khf.shape
        if dk != self.d_k:
            raise RuntimeError(f"d_k mismatch: module {self.d_k}, input {dk}")
        if torch.is_grad_enabled() and (Khf.requires_grad or Vhf.requires_grad or Qhf.requires_grad):
            if carry_in is not None or return_state:
                raise RuntimeError("carry_in / return_state are inference-only; chain ops.race_causal_chunk "
                                   "for differentiable chunked sequences")
            if Khf.dtype not in (torch.float32, torch.bfloat16):
                raise RuntimeError("fp32 or bf16 inputs only")
            return self._forward_autograd(Khf, Vhf, Qhf)
        with torch.no_grad():
            return self._forward_kernels(Khf, Vhf, Qhf, carry_in, return_state)

    def _forward_kernels(self, Khf, Vhf, Qhf, carry_in, return_state):
        M, B, T, H, dk = Khf.shape
        host = not Khf.is_cuda
        dev = self.planes_T.device if self.planes_T.is_cuda else torch.device("cuda", torch.cuda.current_device())
        if host:
            Khf, Vhf, Qhf = (t.to(dev, non_blocking=True) for t in (Khf, Vhf, Qhf))
        if Khf.dtype not in (torch.float32, torch.bfloat16):
            raise RuntimeError("fp32 or bf16 inputs only")
        planes = self.planes_T.T.contiguous().float()
        if self.fuse_producer and self.variant == "auto" and ops.qkv_is_supported(M * B * H, T, self.L, self.K, dk, Khf.dtype, heads=H):
            # the prefix kernels form the bucket probabilities themselves: Q, K, V in, out back, nothing else
            res = ops.race_causal_qkv(Qhf.contiguous(), Khf.contiguous(), Vhf.contiguous(), planes, self.L, self.K,
                                      self.eps, carry_in=carry_in, return_state=return_state)
            out = res[0] if return_state else res
            if host:
                out = out.cpu()
            return (out, res[1], res[2]) if return_state else out
        # K and Q are only read by the producer, which flattens [M,B,T,H,d_k] -> streams on the fly;
        # V is consumed by the prefix kernels as [N,T,d_k] and is copied once
        pK = ops.bucket_probs_streams(Khf.contiguous(), planes, self.L, self.K)
        pQ = ops.bucket_probs_streams(Qhf.contiguous(), planes, self.L, self.K)
        N, S_l, S_r = M * B * H, self.L, 1 << self.K
        if self.variant == "auto" and ops.is_supported(N, T, S_l, S_r, dk, Vhf.dtype, "auto", heads=H):
            # the prefix kernels read V and write the output in [M,B,T,H,d_k] directly
            res = ops.race_causal_prefix(pQ, pK, Vhf.contiguous(), self.eps, carry_in=carry_in,
                                         return_state=return_state, variant=self.variant)
            out = res[0] if return_state else res
        else:
            V2 = self._streams(Vhf)
            res = ops.race_causal_prefix(pQ, pK, V2, self.eps, carry_in=carry_in,
                                         return_state=return_state, variant=self.variant)
            out2 = res[0] if return_state else res
            out = out2.view(M, B, H, T, dk).permute(0, 1, 3, 2, 4)
        if host:
            out = out.cpu()
        return (out, res[1], res[2]) if return_state else out

    @torch.no_grad()
    def step(self, Khf, Vhf, Qhf, state: torch.Tensor):
        """Token-by-token generation: outputs for the ``t`` <= 64 NEW tokens ``[M,B,t,H,d_k]`` given the
        packed running state ``[M*B*H, S*(d_k+1)]`` of everything before them (``torch.zeros`` or
        ``ops.pack_state(A, B)`` of a ``forward(..., return_state=True)`` prefill); ``state`` is advanced
        in place.  Equals continuing the reference's chunked evaluation (src/race_chunked.py:54-63) by a
        chunk of ``t`` tokens."""
        if not (Khf.shape == Vhf.shape == Qhf.shape) or Khf.dim() != 5:
            raise RuntimeError("expected K, V, Q of identical shape [M,B,t,H,d_k]")
        M, B, T, H, dk = Khf.shape
        if dk != self.d_k:
            raise RuntimeError(f"d_k mismatch: module {self.d_k}, input {dk}")
        if not (Khf.is_cuda and state.is_cuda):
            raise RuntimeError("step() takes CUDA tensors (there is no CPU path)")
        planes = self.planes_T.T.contiguous().float()
        pK = ops.bucket_probs_streams(Khf.contiguous(), planes, self.L, self.K)
        pQ = ops.bucket_probs_streams(Qhf.contiguous(), planes, self.L, self.K)
        out2 = ops.race_decode_step(pQ, pK, self._streams(Vhf), state, self.eps)
        return out2.view(M, B, H, T, dk).permute(0, 1, 3, 2, 4)
