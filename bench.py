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

With N > 1 (torchrun) every rank runs its own N=8 streams: streams are independent, so ranks
share nothing on the data path ("weak" scaling); only timing uses a collective.
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
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--workload", default="c2", choices=["c2", "sweep", "c3", "c4", "c5", "operator", "next"],
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
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
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
    return e0.elapsed_time(e1) / steps


def workload_c4(args):
    """Single ultra-long sequence configuration: one long sequence per stream (N=8, T=4,194,304, fp32) sharded contiguously
    over the ranks (run under torchrun); carry chain over NCCL send/recv."""
    import torch.distributed as dist

    import race_attention_kernel_b200 as rk
    from oracle import race_oracle as ro
    from race_attention_kernel_b200 import multigpu as mg
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    N, L, R, dk, T = 8, 4, 16, 64, 4194304

    def reduce_max(x):
        t = torch.tensor([x], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    # parity on a short sequence first: every rank builds the same inputs and takes its slice
    Ts = 20000
    pQ, pK, V = ro.synthetic_probs(N, Ts, L, R, dk, seed=3)
    sl = mg.shard_tokens(Ts, world, rank)
    ref = ro.causal_prefix_chunked(pQ.double(), pK.double(), V.double(), chunk=512)[:, sl]
    run = (lambda q, k, v, mode: mg.sequence_sharded_prefix(q, k, v, mode=mode)) if world > 1 else \
          (lambda q, k, v, mode: rk.race_causal_prefix(q, k, v))
    err = reduce_max(ro.rel_l2(run(pQ[:, sl].contiguous().cuda(), pK[:, sl].contiguous().cuda(),
                                   V[:, sl].contiguous().cuda(), "chain"), ref))
    if not err <= 1e-4:
        raise SystemExit(f"parity gate failed: rel-L2 {err:.3e}")
    Tl = T // world
    g = torch.Generator(device=dev).manual_seed(rank)
    q = torch.softmax(torch.randn(N, Tl, L, R, device=dev, generator=g), -1)
    k = torch.softmax(torch.randn(N, Tl, L, R, device=dev, generator=g), -1)
    v = torch.randn(N, Tl, dk, device=dev, generator=g)
    for mode in (("chain", "allgather") if world > 1 else ("single",)):
        ms = reduce_max(_time_ms(lambda: run(q, k, v, mode), args.warmup, args.steps))
        if rank == 0:
            print(json.dumps({"workload": "c4", "mode": mode, "n_gpus": world, "N": N, "T": T,
                              "ms_per_step": round(ms, 3), "Mtok_s": round(N * T / ms / 1e3, 1),
                              "scaling": "strong", "parity_rel_l2": err}), flush=True)
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
            except (torch.OutOfMemoryError, RuntimeError) as e:
                print(json.dumps({"workload": "sweep", "T": T, "failed": str(e)[:80]}), flush=True)
                break
            gbs = N * T * 1024 / (ms * 1e-3) / 1e9
            print(json.dumps({"workload": "sweep", "N": N, "T": T, "ms": round(ms, 4),
                              "Mtok_s": round(N * T / ms / 1e3, 1), "GB_s": round(gbs, 1),
                              "frac_measured_peak": round(gbs / peak, 4),
                              "peak_GiB": round(torch.cuda.max_memory_allocated() / 2**30, 2),
                              "status": rk.ops.device_status(dev)}), flush=True)
            del pQ, pK, V, out
            torch.cuda.empty_cache()
            torch.cuda.reset_peak_memory_stats()
            T = T * 2 if T < (1 << 24) else T + (1 << 22)
            if T > (3 << 23):
                break
    elif args.workload == "c3":
        # multi-head batched bf16 configuration: bf16, d_k=128, L=8, R=64 (S=512); per-GPU share of the 256 streams
        L, R, dk = 8, 64, 128
        for N, T in ((32, 65536), (32, 262144)):
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
        N, T, L, R, dk = 8, 131072, 4, 16, 64
        pQ, pK = probs(N, T, L, R, torch.float32, g), probs(N, T, L, R, torch.float32, g)
        V = torch.randn(N, T, dk, device=dev, generator=g)
        dO = torch.randn(N, T, dk, device=dev, generator=g)
        ms = _time_ms(lambda: rk.race_causal_backward(pQ, pK, V, dO), 3, 10)
        bb = N * T * 4 * (4 * 64 + 3 * 64)
        print(json.dumps({"workload": "causal_bwd", "dtype": "f32", "N": N, "T": T, "ms": round(ms, 3),
                          "Mtok_s": round(N * T / ms / 1e3, 1), "GB_s": round(bb / ms / 1e6, 1),
                          "frac_measured_peak": round(bb / ms / 1e6 / peak, 4)}), flush=True)
        for norm in ("bucket", "global"):
            ms = _time_ms(lambda: rk.race_causal_prefix(pQ, pK, V, variant="simt", normalization=norm), 3, 10)
            print(json.dumps({"workload": "causal_fwd_cuda_cores", "normalization": norm, "N": N, "T": T,
                              "ms": round(ms, 3), "Mtok_s": round(N * T / ms / 1e3, 1),
                              "frac_measured_peak": round(N * T * 1024 / ms / 1e6 / peak, 4)}), flush=True)
    elif args.workload == "operator":
        # the drop-in operator end to end on the device: BatchedACE.forward(K, V, Q) = stream flattening +
        # bucket-probability producer (probabilities written to HBM) + causal prefix kernels; fp32,
        # M=1, B=1, H=8, d_k=64, K=4, L=4 (the reference CPU configuration at longer T)
        M, B, H, dk, K, L = 1, 1, 8, 64, 4, 4
        for T in (4096, 131072, 1048576):
            torch.manual_seed(1234)
            ace = rk.BatchedACE(dk, K, L, M, device=dev)
            Kh, Vh, Qh = (torch.randn(M, B, T, H, dk, device=dev, generator=g) for _ in range(3))
            with torch.no_grad():
                ms = _time_ms(lambda: ace(Kh, Vh, Qh), 3, 10)
            n_tok = M * B * H * T
            print(json.dumps({"workload": "operator", "M,B,H": [M, B, H], "T": T, "ms": round(ms, 4),
                              "Mtok_s": round(n_tok / ms / 1e3, 1),
                              "qkvo_GB_s": round(n_tok * 4 * dk * 4 / ms / 1e6, 1),
                              "peak_GiB": round(torch.cuda.max_memory_allocated() / 2**30, 2)}), flush=True)
            del Kh, Vh, Qh
            torch.cuda.empty_cache()


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
        # the reference's own CPU path (its memory-light chunked restatement, which it uses as the
        # timing baseline for long T) on a bounded sample of the same workload; rank 0 only
        if rank != 0:
            return
        T_s = min(T, 32768)
        res = cpu_run(T_s, max(1, min(args.steps, 3)), max(1, min(args.warmup, 1)))
        line = {"impl": "reference", "metric": "causal_fwd_tokens_per_s", "value": res["value"],
                "unit": "Mtok/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": res["seconds_per_step"] * 1e3, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": workload, "sample_T": T_s},
                "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": res["value"], "unit": "Mtok/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return

    import torch.distributed as dist

    import race_attention_kernel_b200 as rk

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    tdtype = torch.float32 if args.dtype == "f32" else torch.bfloat16
    elt = 4 if args.dtype == "f32" else 2

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

    # parity gate on a window before timing: a wrong kernel is not timed
    from oracle import race_oracle as ro
    step()
    torch.cuda.synchronize()
    w = min(T, 1024)
    ref = ro.causal_prefix(pQ[:1, :w].double().cpu(), pK[:1, :w].double().cpu(), V[:1, :w].double().cpu())
    err = ro.rel_l2(out[:1, :w], ref)
    tol = 1e-4 if args.dtype == "f32" else 2e-2
    if not err <= tol:
        raise SystemExit(f"parity gate failed: rel-L2 {err:.3e} > {tol}")

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
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
    peak, peak_src = FALLBACK_HBM_GBS, "fallback"
    try:
        peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
        peak_src = "measured"
    except Exception:
        pass
    achieved = alg_bytes / (ms_step * 1e-3) / 1e9
    # DRAM traffic of one forward from the ncu capture in profiles/ (T=131072: output pass 1053.7 MB,
    # totals pass 547.9 MB, scan 17 MB per 1073.7 MB of algorithmic bytes), scaled by tokens
    traffic = alg_bytes * (1053.7 + 547.9 + 17.0) / 1073.7 if (variant == "tensor" and args.dtype == "f32") else None
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
                "kernel": "causal forward (tile_totals_tc + tile_scan + causal_out_tc of one step)",
                "algorithmic_bytes_per_launch": alg_bytes}

    # e2e: host buffers through the C-ABI host entry point
    e2e = None
    if not args.no_e2e:
        del pQ, pK, V, out
        torch.cuda.empty_cache()
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
        if world > 1:
            t = torch.tensor([dt], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = t.item()
        e2e = {"value": tokens_total / dt / 1e6, "unit": "Mtok/s",
               "h2d_bytes_per_step": N * T * elt * (2 * S + dk), "d2h_bytes_per_step": N * T * elt * dk,
               "ms_per_step": dt * 1e3, "steps": args.e2e_steps,
               "api": "race_b200_causal_fwd_host (pinned host tensors, segmented copy/compute pipeline)"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        res = cpu_run(min(T, 32768), 3, 1)
        cpu = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}

    if rank == 0:
        line = {"metric": "causal_fwd_tokens_per_s", "value": value, "unit": "Mtok/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": args.dtype, "data": "synthetic",
                "config": {"workload": workload, "variant": variant, "l2": "inputs larger than L2",
                           "parity_gate_rel_l2": err},
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
                "gpu_launches": launches_per_step * args.steps, "clocks": clk.summary()}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
