"""Multi-GPU driver: one process per GPU, ``torch.distributed`` for the plumbing.

Two ways the path shards (streams never interact; tokens interact only through the running
state (A, B)):

* **streams** -- ``shard_streams``: each rank takes a contiguous block of the N = M*B*H streams
  and runs the single-GPU kernel on it.  No communication on the data path.

* **sequence** -- ``sequence_sharded_prefix``: each rank holds a contiguous range of tokens of
  every stream.  Pass 1 reduces the local range to its totals (A_tot, B_tot); the ranks then
  pass the running state down the chain (rank r receives the state before its first token from
  rank r-1, adds its own totals and sends the sum to rank r+1: N*L*R*(d_k+1) floats per hop,
  NCCL send/recv over NVLink); pass 2 is the ordinary causal kernel with that state as
  ``carry_in``.  The per-bucket divide makes outputs non-linear in the carry, so the carry has
  to be known before outputs are formed: there is no cheaper "fix-up" of finished outputs.
  The reference has no multi-GPU path; the carried form it does have is the serial chunk loop
  of src/race_chunked.py:41-63, which this distributes.

The compute callables are parameters so that the exchange logic can be exercised by CPU ranks
(gloo) in the tests; the defaults are the CUDA operators.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

from . import ops


def shard_streams(n_streams: int, world: int, rank: int) -> slice:
    """Contiguous block of streams owned by `rank` (blocks differ by at most one stream)."""
    base, extra = divmod(n_streams, world)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


def shard_tokens(n_tokens: int, world: int, rank: int) -> slice:
    """Contiguous token range of `rank` for the sequence-sharded mode."""
    return shard_streams(n_tokens, world, rank)


def _pack(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    return ops.pack_state(A, B)


def exchange_carry(totals: torch.Tensor, group=None, mode: str = "chain") -> torch.Tensor:
    """Exclusive prefix over ranks of the packed per-rank totals [N, S*(d_k+1)].

    mode "chain":     send/recv down the rank order; rank r gets sum_{r' < r} totals[r'] with the
                      additions done in rank order (deterministic).
    mode "allgather": one all_gather, every rank adds the lower ranks' totals in rank order.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if world == 1:
        return torch.zeros_like(totals)
    if mode == "allgather":
        parts = [torch.empty_like(totals) for _ in range(world)]
        dist.all_gather(parts, totals.contiguous(), group=group)
        carry = torch.zeros_like(totals)
        for r in range(rank):
            carry += parts[r]
        return carry
    if mode != "chain":
        raise ValueError(f"unknown exchange mode {mode!r}")
    carry = torch.zeros_like(totals)
    ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
    if rank > 0:
        dist.recv(carry, src=ranks[rank - 1], group=group)
    if rank < world - 1:
        dist.send((carry + totals).contiguous(), dst=ranks[rank + 1], group=group)
    return carry


def sequence_sharded_prefix(probsQ: torch.Tensor, probsK: torch.Tensor, V: torch.Tensor,
                            eps: float = 1e-6, *, group=None, mode: str = "chain",
                            return_state: bool = False,
                            totals_fn: Callable | None = None, prefix_fn: Callable | None = None):
    """Causal prefix forward of a sequence whose tokens are sharded contiguously over the ranks
    of `group` (this rank passes its local [N, T_local, ...] tensors).  Returns the local outputs
    (and, with return_state, the state after this rank's last token)."""
    totals_fn = totals_fn or ops.race_tile_totals
    prefix_fn = prefix_fn or ops.race_causal_prefix
    N, T, L, R = probsK.shape
    dk = V.shape[-1]
    kw = {}
    if totals_fn is ops.race_tile_totals and prefix_fn is ops.race_causal_prefix:
        # pass 1 leaves its per-tile totals in the workspace; pass 2 scans them instead of
        # reducing pK and V again
        A_tot, B_tot, ws = totals_fn(probsK, V, return_workspace=True)
        kw["totals_workspace"] = ws
    else:
        A_tot, B_tot = totals_fn(probsK, V)                    # pass 1: local totals
    carry = exchange_carry(_pack(A_tot, B_tot), group, mode)   # one small message per hop
    A0, B0 = ops.unpack_state(carry, L, R, dk)
    return prefix_fn(probsQ, probsK, V, eps, carry_in=(A0.contiguous(), B0.contiguous()),
                     return_state=return_state, **kw)          # pass 2: outputs with the carry


def emulate_sequence_shards(probsQ, probsK, V, shards: int, eps: float = 1e-6,
                            totals_fn: Callable | None = None, prefix_fn: Callable | None = None):
    """The same two passes with the ranks played one after the other on one device (no process
    group): used to check the two-pass arithmetic where fewer GPUs than ranks are available."""
    totals_fn = totals_fn or ops.race_tile_totals
    prefix_fn = prefix_fn or ops.race_causal_prefix
    N, T, L, R = probsK.shape
    dk = V.shape[-1]
    outs, carry = [], None
    for r in range(shards):
        sl = shard_tokens(T, shards, r)
        q, k, v = (t[:, sl].contiguous() for t in (probsQ, probsK, V))
        kw = {}
        if totals_fn is ops.race_tile_totals and prefix_fn is ops.race_causal_prefix:
            A_tot, B_tot, ws = totals_fn(k, v, return_workspace=True)
            kw["totals_workspace"] = ws
        else:
            A_tot, B_tot = totals_fn(k, v)
        totals = _pack(A_tot, B_tot)
        if carry is None:
            carry = torch.zeros_like(totals)
        A0, B0 = ops.unpack_state(carry, L, R, dk)
        outs.append(prefix_fn(q, k, v, eps, carry_in=(A0.contiguous(), B0.contiguous()), **kw))
        carry = carry + totals
    return torch.cat(outs, dim=1)
