"""Host logic of the multi-GPU driver, run by CPU ranks over gloo (world size 2 and 3) with the
oracle standing in for the kernels, and on one GPU with the ranks played in sequence."""
from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import race_oracle as ro


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cpu_totals(pK, V):
    return ro.tile_totals(pK, V)


def _cpu_prefix(pQ, pK, V, eps, carry_in=None, return_state=False):
    return ro.causal_prefix(pQ, pK, V, eps, carry=carry_in, return_state=return_state)


def _worker(rank, world, port, mode, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from race_attention_kernel_b200 import multigpu as mg
        N, T, L, R, dk = 3, 101, 2, 8, 16
        pQ, pK, V = ro.synthetic_probs(N, T, L, R, dk, seed=5, dtype=torch.float64)
        sl = mg.shard_tokens(T, world, rank)
        out, A, B = mg.sequence_sharded_prefix(
            pQ[:, sl].contiguous(), pK[:, sl].contiguous(), V[:, sl].contiguous(), mode=mode,
            return_state=True, totals_fn=_cpu_totals, prefix_fn=_cpu_prefix)
        ref, A_ref, B_ref = ro.causal_prefix(pQ, pK, V, return_state=True)
        err = (out - ref[:, sl]).abs().max().item()
        state_err = 0.0
        if rank == world - 1:
            state_err = max((A - A_ref).abs().max().item(), (B - B_ref).abs().max().item())
        # stream sharding: blocks tile the streams exactly
        blocks = [mg.shard_streams(7, world, r) for r in range(world)]
        cover = sorted(i for b in blocks for i in range(b.start, b.stop))
        q.put((rank, err, state_err, cover == list(range(7))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,mode", [(2, "chain"), (3, "chain"), (2, "allgather")])
def test_sequence_sharding_over_gloo(world, mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, state_err, tiled in results:
        assert err < 1e-12 and state_err < 1e-11 and tiled, (rank, err, state_err)


def test_emulated_shards_cpu():
    from race_attention_kernel_b200 import multigpu as mg
    pQ, pK, V = ro.synthetic_probs(2, 77, 2, 8, 16, seed=6, dtype=torch.float64)
    out = mg.emulate_sequence_shards(pQ, pK, V, 4, totals_fn=_cpu_totals, prefix_fn=_cpu_prefix)
    assert (out - ro.causal_prefix(pQ, pK, V)).abs().max().item() < 1e-12


@pytest.mark.gpu
@pytest.mark.parametrize("shards", [2, 4, 8])
def test_emulated_shards_gpu(shards):
    # the two-pass arithmetic of the sequence-sharded mode on the real kernels, ranks in sequence
    from race_attention_kernel_b200 import multigpu as mg
    pQ, pK, V = ro.synthetic_probs(8, 5000, 4, 16, 64, seed=7)
    out = mg.emulate_sequence_shards(pQ.cuda(), pK.cuda(), V.cuda(), shards)
    ref = ro.causal_prefix_chunked(pQ.double(), pK.double(), V.double(), chunk=512)
    assert ro.rel_l2(out, ref) <= 1e-4
