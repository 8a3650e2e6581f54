"""CPU oracle for RACE attention's per-bucket prefix-sum path.  TEST INFRASTRUCTURE ONLY.

This module restates, with plain torch ops on the CPU, what the reference computes for the
path this library accelerates.  It is the checker the tests, the smoke test and the
benchmark's CPU-baseline leg compare against; nothing the library ships may import it.

Pinning status: PINNED.  ``tests/golden/make_golden.py`` imports the reference's own
``BatchedACE`` / ``chunked_forward`` and stores their outputs as fixtures; the CPU test-suite
checks every function here against those fixtures (``tests/test_oracle_golden.py``).  The
non-causal *per-bucket* form has no test in the reference (its kernels implement another
estimator); for that one the oracle is the restatement of the four lines the reference
quotes from upstream plus torch.autograd, and its parity is "unpinned" in that sense.

Conventions (the reference's, docs/causal_v2_design.md:37-48):
  N = M*B*H independent streams, T tokens, d_k head dim, K hash bits, R = 2**K buckets,
  L tables, S = L*R bucket features per token.  State of a stream = (A [L,R], B [L,R,d_k]).
"""
from __future__ import annotations

import itertools
import math

import torch
import torch.nn.functional as F

EPS = 1e-6  # src/race_baseline.py:47 adds 1e-6 to A before the divide


# --------------------------------------------------------------------------------------
# operator buffers and the stream view          (src/race_baseline.py:22-40)
# --------------------------------------------------------------------------------------
def make_planes(d_k: int, K: int, L: int, dtype=torch.float32) -> torch.Tensor:
    """planes_T [d_k, L*K]: a randn [L,K,d_k] draw viewed [L*K,d_k] and transposed
    (src/race_baseline.py:27-28).  Consumes the global torch RNG exactly like the reference."""
    planes = torch.randn(L, K, d_k)
    return planes.view(L * K, d_k).T.to(dtype)


def make_protos(K: int, dtype=torch.float32) -> torch.Tensor:
    """protos_T [K, R]: the 2**K sign corners, corner r has +1 on plane t iff bit (K-1-t)
    of r is set (src/race_baseline.py:29-32)."""
    corners = torch.tensor(list(itertools.product([-1.0, 1.0], repeat=K)), dtype=dtype)
    return corners.T.contiguous()


def to_streams(x: torch.Tensor) -> torch.Tensor:
    """[M,B,T,H,d_k] -> [N,T,d_k] contiguous, N = M*B*H (src/race_baseline.py:35-40)."""
    M, B, T, H, dk = x.shape
    return x.permute(0, 1, 3, 2, 4).contiguous().view(M * B * H, T, dk)


def from_streams(y: torch.Tensor, M: int, B: int, H: int) -> torch.Tensor:
    """[N,T,d_k] -> [M,B,T,H,d_k] (a permuted view, src/race_baseline.py:52)."""
    N, T, dk = y.shape
    return y.view(M, B, H, T, dk).permute(0, 1, 3, 2, 4)


# --------------------------------------------------------------------------------------
# bucket-probability producer                   (src/race_baseline.py:41-44)
# --------------------------------------------------------------------------------------
def bucket_probs(x: torch.Tensor, planes_T: torch.Tensor, protos_T: torch.Tensor,
                 L: int, K: int) -> torch.Tensor:
    """x [N,T,d_k] -> probs [N,T,L,R] = softmax(tanh(x @ planes_T)/sqrt(d_k) @ protos_T)."""
    N, T, dk = x.shape
    proj = (x @ planes_T).view(N, T, L, K)
    return F.softmax(proj.tanh().div(math.sqrt(dk)) @ protos_T, dim=-1)


# --------------------------------------------------------------------------------------
# THE hot path: cumsum prefixes, per-bucket divide, bmm     (src/race_baseline.py:45-51)
# --------------------------------------------------------------------------------------
def causal_prefix(probsQ: torch.Tensor, probsK: torch.Tensor, V: torch.Tensor,
                  eps: float = EPS, carry=None, return_state: bool = False):
    """out[n,t,:] = sum_s pQ[n,t,s] * B_t[n,s,:] / (A_t[n,s] + eps).

    A_t, B_t are inclusive prefixes over tokens <= t of pK and pK (x) v
    (src/race_baseline.py:45-47); the contraction with pQ is the M=1 bmm of :49-51.
    ``carry = (A0 [N,L,R], B0 [N,L,R,d_k])`` is added before the divide exactly as
    src/race_chunked.py:54-56 does for a chunk that follows earlier tokens.
    Materialises the 5-D tensor: use for T where N*T*S*d_k*elt*3 bytes fit in RAM.
    """
    N, T, L, R = probsK.shape
    dk = V.shape[-1]
    S = L * R
    A_pref = probsK.cumsum(dim=1)
    B_pref = (probsK.unsqueeze(-1) * V.unsqueeze(2).unsqueeze(3)).cumsum(dim=1)
    if carry is not None:
        A_pref = carry[0].unsqueeze(1) + A_pref
        B_pref = carry[1].unsqueeze(1) + B_pref
    E_pref = B_pref.div(A_pref.unsqueeze(-1).add(eps))
    out = torch.bmm(probsQ.reshape(N * T, 1, S), E_pref.reshape(N * T, S, dk)).view(N, T, dk)
    if return_state:
        if T == 0:
            z = carry if carry is not None else (
                torch.zeros(N, L, R, dtype=V.dtype), torch.zeros(N, L, R, dk, dtype=V.dtype))
            return out, z[0].clone(), z[1].clone()
        return out, A_pref[:, -1].clone(), B_pref[:, -1].clone()
    return out


def causal_prefix_chunked(probsQ, probsK, V, chunk: int = 4096, eps: float = EPS,
                          carry=None, return_state: bool = False):
    """Long-T form: the same arithmetic one chunk at a time with the running (A,B) carried
    between chunks (src/race_chunked.py:41-63).  Peak memory O(N*chunk*S*d_k)."""
    N, T, L, R = probsK.shape
    dk = V.shape[-1]
    if carry is None:
        A = torch.zeros(N, L, R, dtype=V.dtype)
        B = torch.zeros(N, L, R, dk, dtype=V.dtype)
    else:
        A, B = carry[0].clone(), carry[1].clone()
    out = torch.empty(N, T, dk, dtype=V.dtype)
    for t0 in range(0, T, chunk):
        t1 = min(t0 + chunk, T)
        o, A, B = causal_prefix(probsQ[:, t0:t1], probsK[:, t0:t1], V[:, t0:t1], eps,
                                carry=(A, B), return_state=True)
        out[:, t0:t1] = o
    if return_state:
        return out, A, B
    return out


def causal_prefix_global(probsQ: torch.Tensor, probsK: torch.Tensor, V: torch.Tensor, carry=None,
                         return_state: bool = False, chunk: int = 256):
    """Global-normalisation causal form (paper Algorithm 1 made causal; the estimator of the
    reference's own CUDA kernels): out[n,t,:] = (pQ_t . B_t) / (pQ_t . A_t) with the same inclusive
    prefixes A_t, B_t as ``causal_prefix``, one denominator per token, no eps, and an output row of 0
    where the denominator is exactly 0 (src/causal_v2/reference.py:77-81,106-127), evaluated a block of
    tokens at a time with the running (A, B) carried (:84-103)."""
    N, T, L, R = probsK.shape
    dk = V.shape[-1]
    S = L * R
    if carry is None:
        A = torch.zeros(N, L, R, dtype=V.dtype)
        B = torch.zeros(N, L, R, dk, dtype=V.dtype)
    else:
        A, B = carry[0].clone(), carry[1].clone()
    out = torch.empty(N, T, dk, dtype=V.dtype)
    for t0 in range(0, T, chunk):
        t1 = min(t0 + chunk, T)
        pk, q, v = probsK[:, t0:t1], probsQ[:, t0:t1].reshape(N, t1 - t0, S), V[:, t0:t1]
        mass = A.unsqueeze(1) + pk.cumsum(dim=1)
        values = B.unsqueeze(1) + (pk.unsqueeze(-1) * v.unsqueeze(2).unsqueeze(3)).cumsum(dim=1)
        num = torch.einsum("nts,ntsd->ntd", q, values.reshape(N, t1 - t0, S, dk))
        den = torch.einsum("nts,nts->nt", q, mass.reshape(N, t1 - t0, S)).unsqueeze(-1)
        empty = den == 0
        out[:, t0:t1] = torch.where(empty, torch.zeros_like(num), num / torch.where(empty, torch.ones_like(den), den))
        A, B = mass[:, -1].clone(), values[:, -1].clone()
    if return_state:
        return out, A, B
    return out


def tile_totals(probsK: torch.Tensor, V: torch.Tensor):
    """(A_tot [N,L,R], B_tot [N,L,R,d_k]) over all T tokens: the ``pref[:, -1:]`` carry of
    src/race_chunked.py:62-63 without forming the prefixes."""
    N, T, L, R = probsK.shape
    A = probsK.sum(dim=1)
    B = torch.einsum("ntlr,ntc->nlrc", probsK, V)
    return A, B


def batched_ace_forward(planes_T, protos_T, Khf, Vhf, Qhf, L: int, K: int, eps: float = EPS,
                        chunk: int | None = None):
    """The full operator (src/race_baseline.py:34-52): argument order K, V, Q, each
    [M,B,T,H,d_k]; returns [M,B,T,H,d_k].  ``chunk`` switches to the carried form
    (src/race_chunked.py:24-65) for long T."""
    M, B, T, H, dk = Khf.shape
    K2, Q2, V2 = to_streams(Khf), to_streams(Qhf), to_streams(Vhf)
    if chunk is None:
        pK = bucket_probs(K2, planes_T, protos_T, L, K)
        pQ = bucket_probs(Q2, planes_T, protos_T, L, K)
        out = causal_prefix(pQ, pK, V2, eps)
    else:
        N = M * B * H
        R = 1 << K
        A = torch.zeros(N, L, R, dtype=Khf.dtype)
        Bs = torch.zeros(N, L, R, dk, dtype=Khf.dtype)
        out = torch.empty(N, T, dk, dtype=Khf.dtype)
        for t0 in range(0, T, chunk):
            t1 = min(t0 + chunk, T)
            pK = bucket_probs(K2[:, t0:t1], planes_T, protos_T, L, K)
            pQ = bucket_probs(Q2[:, t0:t1], planes_T, protos_T, L, K)
            out[:, t0:t1], A, Bs = causal_prefix(pQ, pK, V2[:, t0:t1], eps, carry=(A, Bs),
                                                 return_state=True)
    return from_streams(out, M, B, H)


# --------------------------------------------------------------------------------------
# non-causal per-bucket form   (upstream scaling/benchmark_time.py:155-162 as quoted at
#                               analysis/hot-path.md:157-162)
# --------------------------------------------------------------------------------------
def noncausal_forward(probsQ, probsK, V, eps: float = EPS):
    """Bs = pK^T V [N,S,d_k]; A = sum_t pK [N,S]; E = Bs/(A+eps); out = pQ E [N,T,d_k]."""
    N, T, L, R = probsK.shape
    S = L * R
    pK = probsK.reshape(N, T, S)
    pQ = probsQ.reshape(N, T, S)
    b_sum = pK.transpose(1, 2).bmm(V)
    A = pK.sum(dim=1)
    E = b_sum / (A.unsqueeze(-1) + eps)
    return pQ.bmm(E)


def noncausal_backward_closed_form(probsQ, probsK, V, dO, eps: float = EPS):
    """Gradients of ``noncausal_forward`` w.r.t. (probsQ, probsK, V), written out by hand:
    dPQ = dO E^T; dE = PQ^T dO; dBs = dE/(A+eps); dA[s] = -sum_c dE[s,c] E[s,c]/(A[s]+eps);
    dV = PK dBs; dPK[t,s] = V[t].dBs[s] + dA[s].  Checked against torch.autograd in the tests."""
    N, T, L, R = probsK.shape
    S = L * R
    pK = probsK.reshape(N, T, S)
    pQ = probsQ.reshape(N, T, S)
    Bs = pK.transpose(1, 2).bmm(V)
    A = pK.sum(dim=1)
    inv = 1.0 / (A + eps)
    E = Bs * inv.unsqueeze(-1)
    dPQ = dO.bmm(E.transpose(1, 2))
    dE = pQ.transpose(1, 2).bmm(dO)
    dBs = dE * inv.unsqueeze(-1)
    dA = -(dE * E).sum(-1) * inv
    dV = pK.bmm(dBs)
    dPK = V.bmm(dBs.transpose(1, 2)) + dA.unsqueeze(1)
    return dPQ.view_as(probsQ), dPK.view_as(probsK), dV


def noncausal_backward_autograd(probsQ, probsK, V, dO, eps: float = EPS):
    pq = probsQ.detach().clone().requires_grad_(True)
    pk = probsK.detach().clone().requires_grad_(True)
    v = V.detach().clone().requires_grad_(True)
    out = noncausal_forward(pq, pk, v, eps)
    out.backward(dO)
    return pq.grad, pk.grad, v.grad


def causal_backward_autograd(probsQ, probsK, V, dO, eps: float = EPS):
    """Gradients of ``causal_prefix`` (src/race_baseline.py:45-51) w.r.t. (probsQ, probsK, V) by
    torch.autograd through the restated cumsum / divide / bmm.  The reference has no causal backward
    (its design note only outlines one for the global form), so this is the checker."""
    pq = probsQ.detach().clone().requires_grad_(True)
    pk = probsK.detach().clone().requires_grad_(True)
    v = V.detach().clone().requires_grad_(True)
    out = causal_prefix(pq, pk, v, eps)
    out.backward(dO)
    return pq.grad, pk.grad, v.grad


def causal_backward_closed_form(probsQ, probsK, V, dO, eps: float = EPS):
    """The same gradients written out by hand, the arithmetic the kernels follow.  With
    inv_t = 1/(A_t+eps), W_t = pQ_t*inv_t (prefixes A_t, B_t as in ``causal_prefix``):
      X_t[s] = B_t[s,:].dO_t ;  dPQ_t = X_t*inv_t ;  g_t = -X_t*W_t*inv_t   (gradient reaching A_t)
      SA_j = sum_{t>=j} g_t ;  SB_j = sum_{t>=j} W_t (x) dO_t                (suffix sums)
      dPK_j[s] = SA_j[s] + SB_j[s,:].V_j ;  dV_j = sum_s pK_j[s] SB_j[s,:].
    Checked against ``causal_backward_autograd`` in the tests."""
    N, T, L, R = probsK.shape
    S = L * R
    pK, pQ = probsK.reshape(N, T, S), probsQ.reshape(N, T, S)
    A = pK.cumsum(dim=1)
    B = (pK.unsqueeze(-1) * V.unsqueeze(2)).cumsum(dim=1)            # [N,T,S,d]
    inv = 1.0 / (A + eps)
    W = pQ * inv
    X = torch.einsum("ntsd,ntd->nts", B, dO)
    dPQ = X * inv
    g = -X * W * inv
    SA = g.flip(1).cumsum(dim=1).flip(1)
    SB = (W.unsqueeze(-1) * dO.unsqueeze(2)).flip(1).cumsum(dim=1).flip(1)
    dPK = SA + torch.einsum("ntsd,ntd->nts", SB, V)
    dV = torch.einsum("nts,ntsd->ntd", pK, SB)
    return dPQ.view_as(probsQ), dPK.view_as(probsK), dV


# --------------------------------------------------------------------------------------
# helpers shared by the tests
# --------------------------------------------------------------------------------------
def rel_l2(got: torch.Tensor, ref: torch.Tensor) -> float:
    """||got-ref||_2 / ||ref||_2 in fp64 over all elements."""
    g = got.detach().double().cpu()
    r = ref.detach().double().cpu()
    den = r.norm().item()
    return (g - r).norm().item() / (den if den > 0 else 1.0)


def synthetic_probs(N: int, T: int, L: int, R: int, dk: int, seed: int = 0, dtype=torch.float32):
    """Seeded stand-in inputs: probsQ/probsK rows are a softmax over R of N(0,1) logits,
    V ~ N(0,1).  Generation order pQ, pK, V from one torch.Generator."""
    g = torch.Generator().manual_seed(seed)
    pQ = torch.softmax(torch.randn(N, T, L, R, generator=g), dim=-1).to(dtype)
    pK = torch.softmax(torch.randn(N, T, L, R, generator=g), dim=-1).to(dtype)
    V = torch.randn(N, T, dk, generator=g).to(dtype)
    return pQ, pK, V
