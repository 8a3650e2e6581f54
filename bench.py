"""Benchmark of the causal per-bucket prefix forward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--seq-len T]

Workload (the causal fp32 sweep configuration at its headline length): N=8 streams per GPU, T=1,048,576 tokens,
d_k=64, L=4 tables, R=16 buckets, fp32; probsQ/probsK rows are a softmax of N(0,1) logits and
V ~ N(0,1) (seeded synthetic data -- the reference measures on synthetic randn data too).
One step = one forward over all streams.  Metric: M tokens/s = streams*T / seconds / 1e6.

  value     inputs resident in HBM, CUDA-event timed, max over ranks
  e2e       the same forward through the host-buffer C-ABI entry point: pinned host tensors in,
            host tensor out, every copy inside the timed region
  roofline  algorithmic bytes elt*(2S+2d_k) per token-stream / measured forward time, against the
            measured HBM copy peak (MEASURED_PEAKS.json) or the stated fallback
  cpu_baseline   the CPU oracle (port of the reference's path) on this box's host cores
  c4, c3    sub-records of the same line: the sequence-sharded configuration (N=8, T=4,194,304 fp32 cut
            over the ranks, carry chain over NCCL send/recv) and the bf16 configuration (256 streams,
            T=262,144, S=512, d_k=128, split over the ranks, walked in batches of 32 streams)

  operator, causal_bwd   sub-records: BatchedACE.forward at T=2^20 (probabilities formed in-kernel, the two-step
            time beside it) and the causal backward at N=8, T=2^20
Other workloads (--workload): sweep (lengths up to what fits, each with its parity figure), c3, c4, c5, bwd, next
(incremental step, global form, backward) and operator (--dtype bf16: the operator at the bf16 multi-head geometry,
H=32, d_k=128, K=6, L=8, T=65,536).

With N > 1 (torchrun) every rank runs its own N=8 streams: streams are independent, so ranks
share nothing on the data path ("weak" scaling); only timing uses a collective.

Parity gates (a kernel that fails one is not timed): the first 1024 tokens of stream 0, the LAST 2048
tokens of the last stream against the oracle fed the true fp64 carry of everything before them, and the
returned final state of every stream against fp64 totals -- at the full headline length.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

CFG = dict(N=8, L=4, R=16, dk=64)
FALLBACK_HBM_GBS = 6650.0


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seq-len", type=int, default=1 << 20)
    ap.add_argument("--variant", default="auto")
    ap.add_argument("--dtype", default="f32", choices=["f32", "bf16"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-sub", action="store_true", help="skip the c4 / c3 sub-records")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--workload", default="c2", choices=["c2", "sweep", "c3", "c4", "c5", "operator", "next", "bwd"],
                    help="c2 (default): the contract line; the others print extra measurement lines")
    return ap.parse_args()


# ----------------------------------------------------------------------------------------------
# clocks during the timed region
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def mark(self):
        """Host time stamp to bracket the timed region with (summary(t0, t1) keeps the samples in between)."""
        return time.time()

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def _window(self, t0, t1):
        # a sample describes the period before it arrives, so the window is widened by one period and a bit
        return [r for ts, r in self.rows if t0 is None or t0 <= ts <= t1 + 0.03]

    def count(self, t0, t1):
        return len(self._window(t0, t1))

    def summary(self, t0=None, t1=None):
        """Median SM clock and the throttle reasons seen in the samples that arrived during [t0, t1]."""
        rows = self._window(t0, t1)
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------------------
# CPU arm: the oracle port on host cores
# ----------------------------------------------------------------------------------------------
def cpu_run(T_sample: int, steps: int, warmup: int, dtype=torch.float32):
    from oracle import race_oracle as ro

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    N, L, R, dk = CFG["N"], CFG["L"], CFG["R"], CFG["dk"]
    pQ, pK, V = ro.synthetic_probs(N, T_sample, L, R, dk, seed=0, dtype=dtype)
    times = []
    with torch.no_grad():
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            ro.causal_prefix_chunked(pQ, pK, V, chunk=4096)
            dt = time.perf_counter() - t0
            if i >= warmup:
                times.append(dt)
    times.sort()
    med = times[len(times) // 2]
    return {"value": N * T_sample / med / 1e6, "unit": "Mtok/s", "cores": torch.get_num_threads(),
            "kind": "port",
            "sample": f"N={N} T={T_sample} chunked(4096) fp32 oracle, median of {steps} after {warmup} warm-up",
            "seconds_per_step": med}


def _time_ms(fn, warmup, steps):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    # a bounded device-side wait that ran out makes the kernels return early: such a time is not a measurement
    import race_attention_kernel_b200 as rk
    code = rk.ops.device_status(torch.device("cuda", torch.cuda.current_device()))
    if code:
        raise SystemExit(f"a bounded device-side wait ran out while timing (code {code})")
    return e0.elapsed_time(e1) / steps


def fp64_state(pK_n, V_n, upto: int, block: int = 1 << 19):
    """fp64 (A [L,R], B [L,R,d_k]) over tokens [0, upto) of ONE stream (pK_n [T,L,R], V_n [T,d_k] on the
    device), accumulated block by block so that the fp64 temporaries stay small."""
    Tn, L, R = pK_n.shape
    dk = V_n.shape[-1]
    A = torch.zeros(L * R, dtype=torch.float64, device=pK_n.device)
    B = torch.zeros(L * R, dk, dtype=torch.float64, device=pK_n.device)
    for t0 in range(0, upto, block):
        t1 = min(upto, t0 + block)
        k = pK_n[t0:t1].reshape(t1 - t0, L * R).double()
        A += k.sum(0)
        B += k.T @ V_n[t0:t1].double()
    return A.view(L, R), B.view(L, R, dk)


def window_parity(ro, pQ, pK, V, out, A=None, B=None, window: int = 2048, carry=None):
    """rel-L2 of the last `window` tokens of the last stream against the oracle fed the fp64 state of all
    tokens before them (+ `carry`, the fp64 state before this tensor's first token), and, when the final
    state (A, B) is given, its worst rel-L2 over the streams against fp64 totals.  The method of the
    reference's large-tensor test (src/causal_v2/tests/test_forward_cuda.py:306-318)."""
    N, T = pK.shape[0], pK.shape[1]
    n, w = N - 1, min(window, T)
    A0, B0 = fp64_state(pK[n], V[n], T - w)
    if carry is not None:
        A0, B0 = A0 + carry[0], B0 + carry[1]
    ref, A1, B1 = ro.causal_prefix(pQ[n:, T - w:].double().cpu(), pK[n:, T - w:].double().cpu(),
                                   V[n:, T - w:].double().cpu(), carry=(A0.cpu()[None], B0.cpu()[None]),
                                   return_state=True)
    tail = ro.rel_l2(out[n:, T - w:], ref)
    state = None
    if A is not None:
        state = max(ro.rel_l2(A[n:], A1), ro.rel_l2(B[n:], B1))
        for m in range(N - 1):
            Am, Bm = fp64_state(pK[m], V[m], T)
            state = max(state, ro.rel_l2(A[m], Am), ro.rel_l2(B[m], Bm))
    return tail, state


def _probs_on_device(N, T, L, R, dtype, g, dev):
    # generated stream by stream to bound the fp32 temporaries
    out = torch.empty(N, T, L, R, dtype=dtype, device=dev)
    for n in range(N):
        out[n] = torch.softmax(torch.randn(T, L, R, device=dev, generator=g), -1).to(dtype)
    return out


def sub_c4(rk, ro, dev, rank, world, steps=5, warmup=2):
    """Sequence-sharded configuration on the ranks of this run: N=8, T=4,194,304 fp32, contiguous T/world tokens
    per rank; local totals, carry chain (NCCL send/recv of N*S*(d_k+1) floats per hop), output pass with
    the received carry.  Strong scaling: the total work is fixed."""
    import torch.distributed as dist

    from race_attention_kernel_b200 import multigpu as mg
    N, L, R, dk, T = 8, 4, 16, 64, 4194304

    def reduce_max(x):
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def run(q, k, v):
        if world > 1:
            return mg.sequence_sharded_prefix(q, k, v, mode="chain")
        return rk.race_causal_prefix(q, k, v)

    # gate 1: a short sequence, the same inputs on every rank, each rank's slice against the oracle
    Ts = 20000
    pQ, pK, V = ro.synthetic_probs(N, Ts, L, R, dk, seed=3)
    sl = mg.shard_tokens(Ts, world, rank)
    ref = ro.causal_prefix_chunked(pQ.double(), pK.double(), V.double(), chunk=512)[:, sl]
    err_short = reduce_max(ro.rel_l2(run(pQ[:, sl].contiguous().to(dev), pK[:, sl].contiguous().to(dev),
                                         V[:, sl].contiguous().to(dev)), ref))
    if not err_short <= 1e-4:
        raise SystemExit(f"c4 parity gate failed: rel-L2 {err_short:.3e}")
    Tl = T // world
    g = torch.Generator(device=dev).manual_seed(4000 + rank)
    q = _probs_on_device(N, Tl, L, R, torch.float32, g, dev)
    k = _probs_on_device(N, Tl, L, R, torch.float32, g, dev)
    v = torch.randn(N, Tl, dk, device=dev, generator=g)
    # gate 2, at full size: the last 2048 tokens of the last stream on the LAST rank, against the oracle fed
    # the fp64 state of all tokens before them on every rank
    out = run(q, k, v)
    A_own, B_own = fp64_state(k[N - 1], v[N - 1], Tl)
    packed = torch.cat([A_own.reshape(-1), B_own.reshape(-1)])
    parts = [torch.empty_like(packed) for _ in range(world)]
    if world > 1:
        dist.all_gather(parts, packed)
    err_tail = 0.0
    if rank == world - 1:
        carry = torch.zeros_like(packed)
        for r in range(world - 1):
            carry += parts[r]
        cA, cB = carry[: L * R].view(L, R), carry[L * R:].view(L, R, dk)
        err_tail, _ = window_parity(ro, q, k, v, out, carry=(cA, cB))
    err_tail = reduce_max(err_tail)
    if not err_tail <= 1e-4:
        raise SystemExit(f"c4 tail parity gate failed: rel-L2 {err_tail:.3e}")
    del out
    if world > 1:
        dist.barrier()
    ms = reduce_max(_time_ms(lambda: run(q, k, v), warmup, steps))
    return {"workload": f"C4 causal fwd f32 N={N} T={T} sharded over {world} rank(s), carry chain send/recv",
            "ranks": world, "tokens_per_rank": Tl, "ms_per_step": ms, "value": N * T / ms / 1e3, "unit": "Mtok/s",
            "scaling": "strong", "steps": steps, "warmup": warmup, "carry_bytes_per_hop": N * L * R * (dk + 1) * 4,
            "parity_rel_l2": max(err_short, err_tail), "parity_short_rel_l2": err_short,
            "parity_tail_rel_l2": err_tail}


def sub_c3(rk, ro, dev, rank, world, peak, steps=2, warmup=1):
    """bf16 configuration: 256 streams of T=262,144 tokens, S=512 (L=8, R=64), d_k=128, split over the ranks with
    no communication; a rank walks its streams in batches of 32 through one set of device buffers (all
    256 streams are 172 GB of probabilities and do not fit one GPU)."""
    import torch.distributed as dist

    from race_attention_kernel_b200 import multigpu as mg
    L, R, dk, T, N_total, batch = 8, 64, 128, 262144, 256, 32
    mine = mg.shard_streams(N_total, world, rank)
    n_mine = mine.stop - mine.start
    # gate: a small case of the same geometry through the same kernels against the fp64 oracle
    pQ, pK, V = (t.bfloat16() for t in ro.synthetic_probs(2, 300, L, R, dk, seed=33))
    ref = ro.causal_prefix_chunked(pQ.double(), pK.double(), V.double(), chunk=128)
    err = ro.rel_l2(rk.race_causal_prefix(pQ.to(dev), pK.to(dev), V.to(dev)), ref)
    if not err <= 2e-2:
        raise SystemExit(f"c3 parity gate failed: rel-L2 {err:.3e}")
    g = torch.Generator(device=dev).manual_seed(3000 + rank)
    nb = min(batch, n_mine)
    q = _probs_on_device(nb, T, L, R, torch.bfloat16, g, dev)
    k = _probs_on_device(nb, T, L, R, torch.bfloat16, g, dev)
    v = torch.randn(nb, T, dk, device=dev, generator=g).bfloat16()
    out = torch.empty_like(v)
    batches = (n_mine + nb - 1) // nb

    def step():
        for _ in range(batches):
            rk.race_causal_prefix(q, k, v, out=out)

    if world > 1:
        dist.barrier()
    ms = _time_ms(step, warmup, steps)
    t = torch.tensor([ms, err], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, err = t[0].item(), t[1].item()
    gbs = n_mine * T * 2 * (2 * L * R + 2 * dk) / (ms * 1e-3) / 1e9     # this rank's algorithmic bytes
    return {"workload": f"C3 causal fwd bf16 {N_total} streams T={T} d_k={dk} L={L} R={R}, streams split over "
                        f"{world} rank(s), batches of {nb}",
            "ranks": world, "streams_per_rank": n_mine, "batches_per_step": batches, "ms_per_step": ms,
            "value": N_total * T / ms / 1e3, "unit": "Mtok/s", "scaling": "strong", "steps": steps, "warmup": warmup,
            "GB_s_per_gpu": gbs, "frac": gbs / peak, "parity_rel_l2": err}


def sub_operator(rk, ro, dev, rank, world, peak, steps=5, warmup=2):
    """The drop-in operator BatchedACE.forward(K, V, Q) on the device (M=B=1, H=8, d_k=64, K=4, L=4, fp32, T=2^20;
    one replica per rank): with the bucket probabilities formed inside the prefix kernels (the default) and with the
    producer kernel writing them to device memory first.  Gate: the first 512 tokens of head 0 against the oracle of
    the whole operator."""
    import torch.distributed as dist
    M, B, H, dk, K, L, T = 1, 1, 8, 64, 4, 4, 1 << 20
    torch.manual_seed(1234)
    ace = rk.BatchedACE(dk, K, L, M, device=dev)
    g = torch.Generator(device=dev).manual_seed(4000 + rank)
    Kh, Vh, Qh = (torch.randn(M, B, T, H, dk, device=dev, generator=g) for _ in range(3))
    w = 512
    ref = ro.batched_ace_forward(ace.planes_T.cpu().double(), ace.protos_T.cpu().double(),
                                 *(t[:, :, :w, :1].cpu().double() for t in (Kh, Vh, Qh)), L, K)
    res = {}
    for mode in ("fused", "two_step"):
        ace.fuse_producer = mode == "fused"
        with torch.no_grad():
            err = ro.rel_l2(ace(Kh, Vh, Qh)[:, :, :w, :1], ref)
            if not err <= 1e-4:
                raise SystemExit(f"operator parity gate failed ({mode}): rel-L2 {err:.3e}")
            if world > 1:
                dist.barrier()
            ms = _time_ms(lambda: ace(Kh, Vh, Qh), warmup, steps)
        t = torch.tensor([ms, err], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res[mode] = (t[0].item(), t[1].item())
    n_tok = M * B * H * T
    ms_f, ms_t = res["fused"][0], res["two_step"][0]
    return {"workload": f"BatchedACE.forward f32 M=B=1 H={H} T={T} d_k={dk} K={K} L={L}, one replica per rank",
            "ranks": world, "ms_per_step": ms_f, "value": world * n_tok / ms_f / 1e3, "unit": "Mtok/s",
            "frac": n_tok * 4 * dk * 4 / (ms_f * 1e-3) / 1e9 / peak,
            "algorithmic_bytes_per_token_stream": 4 * dk * 4,
            "two_step_ms_per_step": ms_t, "steps": steps, "warmup": warmup,
            "parity_rel_l2": max(res["fused"][1], res["two_step"][1]),
            "path": "race_b200_causal_fwd_qkv (probabilities formed in-kernel); two_step = "
                    "race_b200_bucket_probs_streams x2 + race_b200_causal_fwd"}


def sub_bwd(rk, ro, dev, rank, world, peak, steps=3, warmup=1):
    """The causal backward (fp32, N=8 streams per rank, T=2^20, d_k=64, L=4, R=16): dPQ, dPK, dV from pQ, pK, V, dO.
    Gate: a small case through the same kernels against the oracle's closed form in fp64."""
    import torch.distributed as dist
    N, T, L, R, dk = 8, 1 << 20, 4, 16, 64
    pQ, pK, V = ro.synthetic_probs(2, 4500, L, R, dk, seed=41)
    dO = torch.randn(2, 4500, dk, generator=torch.Generator().manual_seed(42))
    ref = ro.causal_backward_closed_form(pQ.double(), pK.double(), V.double(), dO.double())
    got = rk.race_causal_backward(pQ.to(dev), pK.to(dev), V.to(dev), dO.to(dev))
    err = max(ro.rel_l2(a, b) for a, b in zip(got[:3], ref[:3]))
    if not err <= 1e-4:
        raise SystemExit(f"backward parity gate failed: rel-L2 {err:.3e}")
    g = torch.Generator(device=dev).manual_seed(5000 + rank)
    q = _probs_on_device(N, T, L, R, torch.float32, g, dev)
    k = _probs_on_device(N, T, L, R, torch.float32, g, dev)
    v = torch.randn(N, T, dk, device=dev, generator=g)
    do = torch.randn(N, T, dk, device=dev, generator=g)
    if world > 1:
        dist.barrier()
    ms = _time_ms(lambda: rk.race_causal_backward(q, k, v, do), warmup, steps)
    t = torch.tensor([ms, err], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, err = t[0].item(), t[1].item()
    bb = N * T * 4 * (4 * L * R + 3 * dk)
    return {"workload": f"causal backward f32 N={N}/GPU T={T} d_k={dk} L={L} R={R}", "ranks": world,
            "ms_per_step": ms, "value": world * N * T / ms / 1e3, "unit": "Mtok/s",
            "GB_s_per_gpu": bb / (ms * 1e-3) / 1e9, "frac": bb / (ms * 1e-3) / 1e9 / peak,
            "algorithmic_bytes_per_token_stream": 4 * (4 * L * R + 3 * dk), "steps": steps, "warmup": warmup,
            "parity_rel_l2": err}


def workload_c4(args):
    """The sequence-sharded configuration alone (run under torchrun for more than one rank)."""
    import torch.distributed as dist

    import race_attention_kernel_b200 as rk
    from oracle import race_oracle as ro
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rec = sub_c4(rk, ro, dev, rank, world, steps=args.steps, warmup=args.warmup)
    if rank == 0:
        print(json.dumps(rec), flush=True)
    if world > 1:
        dist.destroy_process_group()


def extra_workloads(args):
    """Measurement lines for the other benchmark configurations on one GPU (not the contract line)."""
    if args.workload == "c4":
        return workload_c4(args)
    import race_attention_kernel_b200 as rk
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peak = FALLBACK_HBM_GBS
    try:
        peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        pass

    def probs(N, T, L, R, dtype, g):
        # generated stream by stream to bound the fp32 temporaries
        out = torch.empty(N, T, L, R, dtype=dtype, device=dev)
        for n in range(N):
            out[n] = torch.softmax(torch.randn(T, L, R, device=dev, generator=g), -1).to(dtype)
        return out

    g = torch.Generator(device=dev).manual_seed(0)
    if args.workload == "sweep":
        N, L, R, dk = 8, 4, 16, 64
        T = 4096
        while True:
            try:
                pQ, pK = probs(N, T, L, R, torch.float32, g), probs(N, T, L, R, torch.float32, g)
                V = torch.randn(N, T, dk, device=dev, generator=g)
                out = torch.empty_like(V)
                ms = _time_ms(lambda: rk.race_causal_prefix(pQ, pK, V, out=out), 3, 10 if T <= (1 << 21) else 3)
                # parity spot check at this length: last window of the last stream with the fp64 carry
                from oracle import race_oracle as ro
                tail, _ = window_parity(ro, pQ, pK, V, out)
            except (torch.OutOfMemoryError, RuntimeError) as e:
                print(json.dumps({"workload": "sweep", "T": T, "failed": str(e)[:80]}), flush=True)
                break
            gbs = N * T * 1024 / (ms * 1e-3) / 1e9
            print(json.dumps({"workload": "sweep", "N": N, "T": T, "ms": round(ms, 4),
                              "Mtok_s": round(N * T / ms / 1e3, 1), "GB_s": round(gbs, 1),
                              "frac_measured_peak": round(gbs / peak, 4),
                              "peak_GiB": round(torch.cuda.max_memory_allocated() / 2**30, 2),
                              "parity_tail_rel_l2": tail, "parity_ok": bool(tail <= 1e-4),
                              "status": rk.ops.device_status(dev)}), flush=True)
            if not tail <= 1e-4:
                break
            del pQ, pK, V, out
            torch.cuda.empty_cache()
            torch.cuda.reset_peak_memory_stats()
            T = T * 2 if T < (1 << 24) else T + (1 << 22)
            if T > (3 << 23):
                break
    elif args.workload == "c3":
        # multi-head batched bf16 configuration: bf16, d_k=128, L=8, R=64 (S=512); per-GPU share of the 256 streams
        L, R, dk = 8, 64, 128
        # --seq-len other than the default picks that one length (small captures under a profiler)
        for N, T in (((32, 65536), (32, 262144)) if args.seq_len == 1 << 20 else ((32, args.seq_len),)):
            pQ, pK = probs(N, T, L, R, torch.bfloat16, g), probs(N, T, L, R, torch.bfloat16, g)
            V = torch.randn(N, T, dk, device=dev, generator=g).bfloat16()
            out = torch.empty_like(V)
            ms = _time_ms(lambda: rk.race_causal_prefix(pQ, pK, V, out=out), 2, 3)
            gbs = N * T * 2560 / (ms * 1e-3) / 1e9
            print(json.dumps({"workload": "c3", "dtype": "bf16", "N": N, "T": T, "ms": round(ms, 3),
                              "Mtok_s": round(N * T / ms / 1e3, 1), "GB_s": round(gbs, 1),
                              "frac_measured_peak": round(gbs / peak, 4), "variant": "auto"}),
                  flush=True)
            del pQ, pK, V, out
            torch.cuda.empty_cache()
    elif args.workload == "c5":
        # non-causal configuration: forward + backward, B=64, H=12 (N=768), T=4096, S=64, d_k=64
        N, T, L, R, dk = 768, 4096, 4, 16, 64
        for dtype, elt in ((torch.float32, 4), (torch.bfloat16, 2)):
            pQ = probs(N, T, L, R, dtype, g).requires_grad_(True)
            pK = probs(N, T, L, R, dtype, g).requires_grad_(True)
            V = torch.randn(N, T, dk, device=dev, generator=g).to(dtype).requires_grad_(True)
            dO = torch.randn(N, T, dk, device=dev, generator=g).to(dtype)
            with torch.no_grad():
                ms_f = _time_ms(lambda: rk.race_noncausal(pQ, pK, V), 3, 10)

            def fb():
                pQ.grad = pK.grad = V.grad = None
                rk.race_noncausal(pQ, pK, V).backward(dO)
            ms_fb = _time_ms(fb, 3, 10)
            bf, bb = N * T * elt * (2 * 64 + 2 * 64), N * T * elt * (4 * 64 + 3 * 64)
            print(json.dumps({"workload": "c5", "dtype": str(dtype), "N": N, "T": T,
                              "fwd_ms": round(ms_f, 3), "fwd_bwd_ms": round(ms_fb, 3),
                              "fwd_GB_s": round(bf / ms_f / 1e6, 1),
                              "fwd_bwd_GB_s": round((bf + bb) / ms_fb / 1e6, 1),
                              "fwd_frac": round(bf / ms_f / 1e6 / peak, 4),
                              "fwd_bwd_frac": round((bf + bb) / ms_fb / 1e6 / peak, 4),
                              "Mtok_s_fwd_bwd": round(N * T / ms_fb / 1e3, 1)}), flush=True)
            del pQ, pK, V, dO
    elif args.workload == "next":
        # the widened rows: incremental step, causal backward, global-normalisation forward (CUDA cores)
        for N, L, R, dk, dtype in ((8192, 4, 16, 64, torch.float32), (1024, 8, 64, 128, torch.bfloat16)):
            pQ, pK = probs(N, 1, L, R, dtype, g), probs(N, 1, L, R, dtype, g)
            V = torch.randn(N, 1, dk, device=dev, generator=g).to(dtype)
            state = torch.rand(N, L * R * (dk + 1), device=dev)
            ms = _time_ms(lambda: rk.race_decode_step(pQ, pK, V, state), 5, 50)
            byts = 2 * state.numel() * 4
            print(json.dumps({"workload": "decode_step", "dtype": str(dtype), "N": N, "S": L * R, "d_k": dk,
                              "us_per_step": round(ms * 1e3, 1), "state_GB_s": round(byts / ms / 1e6, 1),
                              "frac_measured_peak": round(byts / ms / 1e6 / peak, 4),
                              "Mtok_s": round(N / ms / 1e3, 2)}), flush=True)
            del pQ, pK, V, state
        # launch path of a one-token step at N=8 streams: general wrapper vs the pre-validated stepper
        N, L, R, dk = 8, 4, 16, 64
        pQ, pK = probs(N, 1, L, R, torch.float32, g), probs(N, 1, L, R, torch.float32, g)
        V = torch.randn(N, 1, dk, device=dev, generator=g)
        state = torch.rand(N, L * R * (dk + 1), device=dev)
        stepper = rk.DecodeStepper(N, L, R, dk, torch.float32, dev)
        for name, fn in (("race_decode_step", lambda: rk.race_decode_step(pQ, pK, V, state)),
                         ("DecodeStepper", lambda: stepper(pQ, pK, V, state))):
            for _ in range(20):
                fn()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(2000):
                fn()
            torch.cuda.synchronize()
            print(json.dumps({"workload": "decode_step_launch_path", "api": name, "N": N,
                              "us_per_call": round((time.perf_counter() - t0) / 2000 * 1e6, 2)}), flush=True)
        del pQ, pK, V, state
        N, T, L, R, dk = 8, 131072, 4, 16, 64
        pQ, pK = probs(N, T, L, R, torch.float32, g), probs(N, T, L, R, torch.float32, g)
        V = torch.randn(N, T, dk, device=dev, generator=g)
        dO = torch.randn(N, T, dk, device=dev, generator=g)
        ms = _time_ms(lambda: rk.race_causal_backward(pQ, pK, V, dO), 3, 10)
        bb = N * T * 4 * (4 * 64 + 3 * 64)
        print(json.dumps({"workload": "causal_bwd", "dtype": "f32", "N": N, "T": T, "ms": round(ms, 3),
                          "Mtok_s": round(N * T / ms / 1e3, 1), "GB_s": round(bb / ms / 1e6, 1),
                          "frac_measured_peak": round(bb / ms / 1e6 / peak, 4)}), flush=True)
        # the same at the headline length
        Tb = 1 << 20
        qb, kb = probs(N, Tb, L, R, torch.float32, g), probs(N, Tb, L, R, torch.float32, g)
        vb = torch.randn(N, Tb, dk, device=dev, generator=g)
        dob = torch.randn(N, Tb, dk, device=dev, generator=g)
        ms = _time_ms(lambda: rk.race_causal_backward(qb, kb, vb, dob), 2, 5)
        bb2 = N * Tb * 4 * (4 * 64 + 3 * 64)
        print(json.dumps({"workload": "causal_bwd", "dtype": "f32", "N": N, "T": Tb, "ms": round(ms, 3),
                          "Mtok_s": round(N * Tb / ms / 1e3, 1), "GB_s": round(bb2 / ms / 1e6, 1),
                          "frac_measured_peak": round(bb2 / ms / 1e6 / peak, 4)}), flush=True)
        del qb, kb, vb, dob
        torch.cuda.empty_cache()
        # the global-normalisation form on the tcgen05 kernels at the size the reference quotes its own tensor-core
        # kernel on (bf16, d=64, N*T = 16.8 M token-streams: 14.7 ms on H100, benchmarks/h100_run.md:47)
        for dt in (torch.float32, torch.bfloat16):
            N2, T2 = 8, 1 << 21
            q2, k2 = probs(N2, T2, L, R, dt, g), probs(N2, T2, L, R, dt, g)
            v2 = torch.randn(N2, T2, dk, device=dev, generator=g).to(dt)
            o2 = torch.empty_like(v2)
            for norm in ("bucket", "global"):
                ms2 = _time_ms(lambda: rk.race_causal_prefix(q2, k2, v2, variant="tensor", normalization=norm, out=o2), 3, 10)
                print(json.dumps({"workload": "causal_fwd_tcgen05", "normalization": norm, "dtype": str(dt), "N": N2,
                                  "T": T2, "ms": round(ms2, 3), "Mtok_s": round(N2 * T2 / ms2 / 1e3, 1)}), flush=True)
            del q2, k2, v2, o2
        for norm in ("bucket", "global"):
            ms = _time_ms(lambda: rk.race_causal_prefix(pQ, pK, V, variant="simt", normalization=norm), 3, 10)
            print(json.dumps({"workload": "causal_fwd_cuda_cores", "normalization": norm, "N": N, "T": T,
                              "ms": round(ms, 3), "Mtok_s": round(N * T / ms / 1e3, 1),
                              "frac_measured_peak": round(N * T * 1024 / ms / 1e6 / peak, 4)}), flush=True)
    elif args.workload == "bwd":
        # the causal backward alone (fp32, N=8, d_k=64, L=4, R=16) at --seq-len: the line of the "next" workload,
        # as a command of its own for launch lists
        N, T, L, R, dk = 8, args.seq_len, 4, 16, 64
        pQ, pK = probs(N, T, L, R, torch.float32, g), probs(N, T, L, R, torch.float32, g)
        V = torch.randn(N, T, dk, device=dev, generator=g)
        dO = torch.randn(N, T, dk, device=dev, generator=g)
        ms = _time_ms(lambda: rk.race_causal_backward(pQ, pK, V, dO), 2, 5)
        bb = N * T * 4 * (4 * 64 + 3 * 64)
        print(json.dumps({"workload": "causal_bwd", "dtype": "f32", "N": N, "T": T, "ms": round(ms, 3),
                          "Mtok_s": round(N * T / ms / 1e3, 1), "GB_s": round(bb / ms / 1e6, 1),
                          "frac_measured_peak": round(bb / ms / 1e6 / peak, 4)}), flush=True)
    elif args.workload == "operator":
        # the drop-in operator end to end on the device: BatchedACE.forward(K, V, Q); fp32, M=1, B=1, H=8, d_k=64,
        # K=4, L=4 (the reference CPU configuration at longer T).  "fused": the prefix kernels form the bucket
        # probabilities themselves (Q, K, V in, out back: 4 d_k elt = 1024 B per token-stream, the same
        # algorithmic bytes as the probabilities-level path); "two_step": producer kernel writes the
        # probabilities to HBM, the prefix kernels read them back.  A parity gate against the oracle of the
        # whole operator (first 512 tokens of stream 0) runs before the timing.
        # --dtype bf16: the operator at the geometry of the bf16 multi-head configuration (H=32 streams, d_k=128, K=6,
        # L=8, T=65536 unless --seq-len says otherwise): producer kernel, then the wide bf16 prefix kernels.
        from oracle import race_oracle as ro
        wide = args.dtype == "bf16"
        M, B, H, dk, K, L = (1, 1, 32, 128, 6, 8) if wide else (1, 1, 8, 64, 4, 4)
        dt, elt, tol = (torch.bfloat16, 2, 2e-2) if wide else (torch.float32, 4, 1e-4)
        default_T = (65536,) if wide else (4096, 131072, 1048576)
        # --seq-len other than the default picks that one length (small captures under a profiler)
        for T in (default_T if args.seq_len == 1 << 20 else (args.seq_len,)):
            torch.manual_seed(1234)
            ace = rk.BatchedACE(dk, K, L, M, device=dev)
            Kh, Vh, Qh = (torch.randn(M, B, T, H, dk, device=dev, generator=g).to(dt) for _ in range(3))
            n_tok = M * B * H * T
            w = min(T, 256 if wide else 512)
            ref = ro.batched_ace_forward(ace.planes_T.cpu().double(), ace.protos_T.cpu().double(),
                                         *(t[:, :, :w, :1].cpu().double() for t in (Kh, Vh, Qh)), L, K)
            for mode in (("two_step",) if wide else ("fused", "two_step")):
                ace.fuse_producer = mode == "fused"
                with torch.no_grad():
                    err = ro.rel_l2(ace(Kh, Vh, Qh)[:, :, :w, :1], ref)
                    if not err <= tol:
                        raise SystemExit(f"operator parity gate failed ({mode}): rel-L2 {err:.3e}")
                    ms = _time_ms(lambda: ace(Kh, Vh, Qh), 3, 10)
                    ms_prod = _time_ms(lambda: ace.bucket_probs(Kh.view(M * B * T, H, dk)), 3, 10) if wide else None
                rec = {"workload": "operator", "mode": mode, "dtype": args.dtype, "M,B,H": [M, B, H], "T": T,
                       "d_k,K,L": [dk, K, L], "ms": round(ms, 4), "Mtok_s": round(n_tok / ms / 1e3, 1),
                       "qkvo_GB_s": round(n_tok * 4 * dk * elt / ms / 1e6, 1),
                       "frac_measured_peak": round(n_tok * 4 * dk * elt / ms / 1e6 / peak, 4),
                       "parity_rel_l2": err, "peak_GiB": round(torch.cuda.max_memory_allocated() / 2**30, 2)}
                if ms_prod is not None:
                    rec["producer_ms_per_tensor"] = round(ms_prod, 4)
                print(json.dumps(rec), flush=True)
            del Kh, Vh, Qh
            torch.cuda.empty_cache()


# DRAM traffic of one forward per algorithmic byte, by kernel, from the ncu capture summarised under
# profiles/ (causal_out_tc_N8_T131072_ncu_full.md: T=131072, 1073.7 MB of algorithmic bytes per launch set;
# traffic grows in proportion to the tokens processed).  Update together with that file.
TRAFFIC_MB_PER_1073_7 = {"causal_out_tc": 1053.7, "tile_totals_tc": 547.9, "tile_scan": 17.0}
# the single-pass kernel in the same units (profiles/causal_fused_tc_N8_T131072_ncu.md): 851.7 MB read + 272.9 MB
# written per 1073.7 MB
TRAFFIC_SINGLE_PASS_PER_ALG = (851.7 + 272.9) / 1073.7


def reference_arm(args, workload):
    """The reference's own CPU path for this workload -- its memory-light chunked restatement
    (src/race_chunked.py), which it uses as the timing baseline for long T -- as restated by the oracle, on
    the box's host cores with all threads, at the FULL sequence length of the workload.  A full-size step
    takes about a minute, so the step counts actually run (and printed) are small: 1 warm-up + 2 timed."""
    T = args.seq_len
    steps, warmup = min(args.steps, 2), min(args.warmup, 1)
    res = cpu_run(T, steps, warmup)
    return {"impl": "reference", "metric": "causal_fwd_tokens_per_s", "value": res["value"],
            "unit": "Mtok/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
            "steps_requested": args.steps, "warmup_requested": args.warmup,
            "ms_per_step": res["seconds_per_step"] * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload},
            "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": res["value"], "unit": "Mtok/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}


def main():
    args = parse()
    if args.workload != "c2":
        return extra_workloads(args)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    N, L, R, dk = CFG["N"], CFG["L"], CFG["R"], CFG["dk"]
    T = args.seq_len
    S = L * R
    workload = f"C2 causal fwd {args.dtype} N={N}/GPU T={T} d_k={dk} L={L} R={R} (probs-in)"

    if args.impl == "reference":
        if rank == 0:      # rank 0 alone runs the CPU arm; the other ranks have nothing to do
            print(json.dumps(reference_arm(args, workload)), flush=True)
        return

    import torch.distributed as dist

    import race_attention_kernel_b200 as rk
    from oracle import race_oracle as ro

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    tdtype = torch.float32 if args.dtype == "f32" else torch.bfloat16
    elt = 4 if args.dtype == "f32" else 2
    tol = 1e-4 if args.dtype == "f32" else 2e-2
    peak, peak_src = FALLBACK_HBM_GBS, "fallback"
    try:
        peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
        peak_src = "measured"
    except Exception:
        pass

    # synthetic inputs generated on the device for the resident-input leg (8.6 GB at T=2^20)
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    pQ = torch.softmax(torch.randn(N, T, L, R, device=dev, generator=g), -1).to(tdtype)
    pK = torch.softmax(torch.randn(N, T, L, R, device=dev, generator=g), -1).to(tdtype)
    V = torch.randn(N, T, dk, device=dev, generator=g).to(tdtype)
    out = torch.empty_like(V)

    variant = args.variant
    if variant == "auto":
        variant = "tensor" if rk.is_supported(N, T, L, R, dk, tdtype, "tensor") else "simt"
    launches_per_step = 3   # tile totals, scan over tiles, output pass

    def step():
        rk.race_causal_prefix(pQ, pK, V, variant=variant, out=out)

    # parity gates before timing, at the full length: a wrong kernel is not timed
    _, A_fin, B_fin = rk.race_causal_prefix(pQ, pK, V, variant=variant, out=out, return_state=True)
    torch.cuda.synchronize()
    w = min(T, 1024)
    ref = ro.causal_prefix(pQ[:1, :w].double().cpu(), pK[:1, :w].double().cpu(), V[:1, :w].double().cpu())
    err_head = ro.rel_l2(out[:1, :w], ref)
    err_tail, err_state = window_parity(ro, pQ, pK, V, out, A_fin, B_fin)
    del A_fin, B_fin
    if not (err_head <= tol and err_tail <= tol and err_state <= tol):
        raise SystemExit(f"parity gate failed: rel-L2 head {err_head:.3e} tail {err_tail:.3e} "
                         f"state {err_state:.3e} > {tol}")

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:      # sampling starts before the warm-up: nvidia-smi needs a moment to come up
        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t_wall0 = clk.mark()
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        t_wall1 = clk.mark()
        # the timed region lasts tens of milliseconds, a few sampling periods: only where no sample at all fell
        # inside it do the same steps go on (untimed) for a quarter of a second, and those samples are reported
        # (a longer run of back-to-back steps draws more power and may show lower clocks than the timed region saw)
        t_wall2 = t_wall1
        if clk.count(t_wall0, t_wall1) < 1:
            while time.time() - t_wall1 < 0.25:
                step()
            torch.cuda.synchronize()
            t_wall2 = clk.mark()
    clocks = clk.summary(t_wall0, t_wall2)
    clocks["window"] = ("timed region" if t_wall2 == t_wall1
                        else "timed region and the same steps repeated for 0.25 s after it")
    ms = e0.elapsed_time(e1)
    code = rk.ops.device_status(dev)
    if code:
        raise SystemExit(f"a bounded device-side wait ran out during the timed region (code {code})")
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    ms_step = ms / args.steps
    tokens_total = N * T * world
    value = tokens_total / (ms_step * 1e-3) / 1e6

    # roofline of the forward: algorithmic bytes / measured time of one forward on this rank
    alg_bytes = N * T * elt * (2 * S + 2 * dk)
    achieved = alg_bytes / (ms_step * 1e-3) / 1e9
    traffic = (alg_bytes * sum(TRAFFIC_MB_PER_1073_7.values()) / 1073.7
               if (variant == "tensor" and args.dtype == "f32") else None)
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
                "kernel": "causal forward (tile_totals_tc + tile_scan + causal_out_tc of one step)",
                "algorithmic_bytes_per_launch": alg_bytes}
    # the same workload through the single-pass form of the forward (one persistent kernel, decoupled look-back,
    # second read of a tile from L2), gated bitwise against the form timed above
    single = None
    if variant == "tensor" and args.dtype == "f32" and not args.no_sub:
        tile_sp = rk.select_tile_tokens(N, T, L, R, dk, tdtype, "tensor_single_pass")
        same = torch.equal(rk.race_causal_prefix(pQ, pK, V, variant="tensor_single_pass", tile_tokens=tile_sp),
                           rk.race_causal_prefix(pQ, pK, V, variant="tensor", tile_tokens=tile_sp, out=out))
        if not same:
            raise SystemExit("single-pass form differs from the three launches at the same tile length")
        out_sp = torch.empty_like(V)
        ms_sp = _time_ms(lambda: rk.race_causal_prefix(pQ, pK, V, variant="tensor_single_pass", out=out_sp),
                         args.warmup, args.steps)
        if world > 1:
            t = torch.tensor([ms_sp], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_sp = t.item()
        single = {"variant": "tensor_single_pass", "tile_tokens": tile_sp, "ms_per_step": ms_sp,
                  "value": tokens_total / ms_sp / 1e3, "unit": "Mtok/s", "bitwise_equal_to_three_launches": True,
                  "frac": alg_bytes / (ms_sp * 1e-3) / 1e9 / peak,
                  "traffic": alg_bytes * TRAFFIC_SINGLE_PASS_PER_ALG, "gpu_launches": args.steps}
        del out_sp
    del pQ, pK, V, out
    torch.cuda.empty_cache()

    # sub-records: the sequence-sharded and the bf16 configuration on the same ranks
    c4 = c3 = operator = bwd = None
    if not args.no_sub and args.dtype == "f32" and T == (1 << 20):
        c4 = sub_c4(rk, ro, dev, rank, world)
        torch.cuda.empty_cache()
        c3 = sub_c3(rk, ro, dev, rank, world, peak)
        torch.cuda.empty_cache()
        operator = sub_operator(rk, ro, dev, rank, world, peak)
        torch.cuda.empty_cache()
        bwd = sub_bwd(rk, ro, dev, rank, world, peak)
        torch.cuda.empty_cache()
        code = rk.ops.device_status(dev)
        if code:
            raise SystemExit(f"a bounded device-side wait ran out in a sub-record (code {code})")

    # e2e: host buffers through the C-ABI host entry point
    e2e = None
    if not args.no_e2e:
        gh = torch.Generator().manual_seed(rank)
        hq = torch.softmax(torch.randn(N, T, L, R, generator=gh), -1).to(tdtype).pin_memory()
        hk = torch.softmax(torch.randn(N, T, L, R, generator=gh), -1).to(tdtype).pin_memory()
        hv = torch.randn(N, T, dk, generator=gh).to(tdtype).pin_memory()
        ho = torch.empty_like(hv).pin_memory()
        rk.race_causal_prefix_host(hq, hk, hv, out=ho, variant=variant, device=local)  # warm-up
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            rk.race_causal_prefix_host(hq, hk, hv, out=ho, variant=variant, device=local)
        dt = (time.perf_counter() - t0) / args.e2e_steps
        # the floor of that step: the same bytes moved by plain pinned copies, both directions at once
        dq, dk_, dv = (torch.empty_like(t, device=dev) for t in (hq, hk, hv))
        do = torch.empty_like(hv, device=dev)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

        def copies():
            with torch.cuda.stream(s_in):
                dq.copy_(hq, non_blocking=True)
                dk_.copy_(hk, non_blocking=True)
                dv.copy_(hv, non_blocking=True)
            with torch.cuda.stream(s_out):
                ho.copy_(do, non_blocking=True)
            s_in.synchronize()
            s_out.synchronize()
        copies()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            copies()
        dt_copy = (time.perf_counter() - t0) / args.e2e_steps
        if world > 1:
            t = torch.tensor([dt, dt_copy], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt, dt_copy = t[0].item(), t[1].item()
        h2d, d2h = N * T * elt * (2 * S + dk), N * T * elt * dk
        e2e = {"value": tokens_total / dt / 1e6, "unit": "Mtok/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": dt * 1e3, "steps": args.e2e_steps,
               "copy_only_ms_per_step": dt_copy * 1e3,
               "copy_only_GB_s_per_rank": (h2d + d2h) / dt_copy / 1e9,
               "frac_of_copy_only": dt_copy / dt,
               "api": "race_b200_causal_fwd_host (pinned host tensors, segmented copy/compute pipeline); "
                      "copy_only = the same bytes as plain pinned cudaMemcpyAsync, both directions at once"}
        del dq, dk_, dv, do, hq, hk, hv, ho

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        res = cpu_run(min(T, 65536), 3, 1)
        cpu = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}

    if rank == 0:
        line = {"metric": "causal_fwd_tokens_per_s", "value": value, "unit": "Mtok/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": args.dtype, "data": "synthetic",
                "config": {"workload": workload, "variant": variant, "l2": "inputs larger than L2",
                           "parity_gate_rel_l2": max(err_head, err_tail),
                           "parity_head_rel_l2": err_head, "parity_tail_rel_l2": err_tail,
                           "parity_state_rel_l2": err_state,
                           "parity_gate": "first 1024 tokens of stream 0; last 2048 tokens of the last stream vs the "
                                          "oracle with the fp64 carry; final state of every stream vs fp64 totals"},
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "c4": c4, "c3": c3, "single_pass": single,
                "operator": operator, "causal_bwd": bwd,
                "gpu_launches": launches_per_step * args.steps, "clocks": clocks}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
