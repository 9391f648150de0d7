"""Headline benchmark: causal-adjusted attention TFLOPS of one public fwd+bwd call (quantisation included) on the
reference's headline cell b4 s4096 h16 d128 causal, MXFP8 route (flash_attn_fp8 defaults), synthetic seeded inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--route fp8|fp4] [--dense]

One process per GPU (torchrun for N > 1). The path has no collective: every rank runs its own slice of a global batch of
4 N rows (weak scaling by (batch, head)); only the timing is reduced (max over ranks). Prints ONE JSON line on rank 0.
FLOP rule (the reference benchmark's): fwd = 4 b h d pairs, pairs = s (s + 1) / 2 causal | s^2 dense; step = 3.5 x fwd.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

B, S, H, HKV, D = 4, 4096, 16, 16, 128


def shard_groups(n_groups: int, rank: int, world: int):
    """Contiguous slice [lo, hi) of the n_groups independent (batch, kv-head) groups owned by `rank`."""
    base, rem = divmod(n_groups, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def flops_fwd(b, s, h, d, causal):
    pairs = s * (s + 1) / 2 if causal else s * s
    return 4.0 * b * h * d * pairs


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        m = json.load(open(p))
        return m.get("bf16_tflops_sustained", 1399.2), m.get("bf16_tflops", 1647.9), m.get("hbm_gbs", 6542.7), "measured"
    return 1400.0, 1590.0, 6650.0, "fallback"


class ClockSampler:
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms",
                                          "20", "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                                         text=True)
        except OSError:
            pass

    def stop(self, window=None):
        """window = (t0, t1) wall-clock seconds of the timed region: samples inside it are preferred."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        import datetime
        rows, mx = [], None
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(f[1]), [n for n, val in zip(
                    ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9])
                    if val.lower().startswith("active")]))
                mx = float(f[2])
            except ValueError:
                continue
        inside = [r for r in rows if window and window[0] <= r[0] <= window[1]]
        scope = "timed region"
        if not inside:      # a region shorter than the sampling period: the samples under load around it
            inside = [r for r in rows if mx and r[1] > 0.5 * mx] or rows
            scope = "whole run under load"
        sm = [r[1] for r in inside]
        reasons = sorted({n for r in inside for n in r[2]})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": reasons,
                "samples": len(sm), "scope": scope}


def cpu_reference_slice(causal, threads=None, n_slices=8):
    """n_slices (batch, head) slices of the workload through the CPU oracle (quantise-dequantise emulation + fp32
    attention forward and backward): the reference's own CPU statement of the path. Returns (seconds, flops)."""
    import torch
    from oracle import attention_oracle as A
    from tests.inputs import attention_inputs
    if threads:
        torch.set_num_threads(threads)
    q, k, v, g = attention_inputs(1, S, n_slices, n_slices, D, seed=0)
    t0 = time.perf_counter()
    A.qdq_attention(q, k, v, g, causal=causal, rotate_qk=True)
    dt = time.perf_counter() - t0
    return dt, 3.5 * flops_fwd(1, S, n_slices, D, causal)


def run_reference(args, rank, world):
    """--impl reference: the CPU port of the reference's emulation on the host cores; rank 0 only."""
    if rank != 0:
        return
    import torch
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    causal = not args.dense
    # one step = a bounded sample of the cell; fewer slices per step when many steps are asked for, so that the whole run
    # stays within a few minutes (about 0.2 s per slice on 16 cores)
    n_sl = 8 if args.steps <= 30 else (4 if args.steps <= 100 else 2)
    for _ in range(min(args.warmup, 1)):
        cpu_reference_slice(causal, n_slices=n_sl)
    times, fl = [], 0.0
    for _ in range(args.steps):
        dt, fl = cpu_reference_slice(causal, n_slices=n_sl)
        times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    val = fl / (ms * 1e-3) / 1e12
    sample = f"{n_sl} (batch, head) slices of b{B} s{S} h{H} d{D} per step: oracle quantise + fp32 fwd+bwd"
    print(json.dumps({
        "impl": "reference", "metric": "attention fwd+bwd step TFLOPS (causal-adjusted), MXFP8", "value": val,
        "unit": "TFLOPS", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"b{B} s{S} h{H} d{D} {'causal' if causal else 'dense'} fwd+bwd, MXFP8 QDQ emulation on CPU",
                   "sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOPS", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--route", default="fp8", choices=["fp8", "fp4"])
    ap.add_argument("--dense", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of replaying one captured step")
    ap.add_argument("--profile-case", action="store_true",
                    help="run `--steps` plain steps of a reduced cell (b2, same s/h/d) and exit: the command profilers wrap; "
                         "prints no bench value")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from flamia_blackwell_attention_b200 import flash_attn_fp4, flash_attn_fp8, kernels as K
    from tests.inputs import attention_inputs
    fn = flash_attn_fp8 if args.route == "fp8" else flash_attn_fp4
    causal = not args.dense
    if args.profile_case:
        pq, pk, pv, pg = (t.to(dev) for t in attention_inputs(2, S, H, HKV, D, seed=0))
        pq.requires_grad_(True); pk.requires_grad_(True); pv.requires_grad_(True)
        for _ in range(args.warmup + args.steps):
            pq.grad = pk.grad = pv.grad = None
            fn(pq, pk, pv, causal=causal).backward(pg)
        torch.cuda.synchronize()
        print(json.dumps({"profile_case": f"b2 s{S} h{H} d{D}", "steps": args.warmup + args.steps, "launches_per_step": 8}))
        return
    W = max(args.warmup, 3)

    # this rank's slice of the global batch of 4 * world rows: rows [lo, hi) of the (batch, head) groups
    lo, hi = shard_groups(B * world * HKV, rank, world)
    assert (hi - lo) == B * HKV
    qh, kh, vh, gh = (t.pin_memory() for t in attention_inputs(B, S, H, HKV, D, seed=rank))
    q, k, v, g = (t.to(dev, non_blocking=True) for t in (qh, kh, vh, gh))
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    torch.cuda.synchronize()

    # per-kernel event pairs around the two tensor-core kernels (same stream as the launches)
    ev = {"fwd": [], "bwd": []}
    timing = {"on": False}
    _fwd, _bwd = K.attn_fwd, K.attn_bwd

    def timed(name, f):
        def w(*a, **kw):
            if not timing["on"]:
                return f(*a, **kw)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = f(*a, **kw)
            e1.record()
            ev[name].append((e0, e1))
            return r
        return w
    K.attn_fwd, K.attn_bwd = timed("fwd", _fwd), timed("bwd", _bwd)
    import flamia_blackwell_attention_b200._routes as R
    R.K = K

    def step():
        q.grad = k.grad = v.grad = None
        out = fn(q, k, v, causal=causal)
        out.backward(g)
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    for _ in range(W):
        step()
    barrier()
    # per-kernel event pairs: a short eager pass (event records cannot be timed inside a captured graph)
    timing["on"] = True
    for _ in range(min(args.steps, 20)):
        step()
    torch.cuda.synchronize()
    timing["on"] = False
    k_fwd = sum(a.elapsed_time(b) for a, b in ev["fwd"]) / max(len(ev["fwd"]), 1)
    k_bwd = sum(a.elapsed_time(b) for a, b in ev["bwd"]) / max(len(ev["bwd"]), 1)
    # the timed steps replay one captured step (8 launches + the status-word fill): no host launch gaps between kernels
    run_step, mode = step, "eager"
    if not args.no_graph:
        try:
            q.grad = k.grad = v.grad = None
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                fn(q, k, v, causal=causal).backward(g)
            run_step, mode = graph.replay, "cuda graph replay"
            for _ in range(3):
                run_step()
        except Exception as exc:      # capture is an optimisation of the launch path only
            print(f"bench: graph capture failed ({exc!r}); timing eager launches", file=sys.stderr)
            torch.cuda.synchronize()
            run_step, mode = step, "eager"
    barrier()
    wall0 = time.time()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        run_step()
    t1.record()
    barrier()
    wall1 = time.time()
    ms = t0.elapsed_time(t1) / args.steps
    clocks = sampler.stop((wall0, wall1)) if sampler else None

    # ---- end to end through the public call with HOST buffers: every step copies q, k, v, dO in from pinned host memory
    # and O, dQ, dK, dV back out. Three streams (copy in, compute, copy out) and two device input sets: the copy-in of
    # step i + 1 and the copy-out of step i - 1 run beside the kernels of step i, so the steady state is bound by the slower
    # PCIe direction rather than by their sum.
    oh, dqh, dkh, dvh = (torch.empty_like(t).pin_memory() for t in (qh, qh, kh, vh))
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    dev_in = [[torch.empty_like(t, device=dev) for t in (qh, kh, vh, gh)] for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_used = [torch.cuda.Event() for _ in range(2)]
    ev_out = torch.cuda.Event()

    def e2e_run(n):
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        for i in range(n + 1):
            if i < n:
                with torch.cuda.stream(s_in):
                    if i >= 2:
                        s_in.wait_event(ev_used[i % 2])          # the kernels of step i - 2 are done with this set
                    for d_t, h_t in zip(dev_in[i % 2], (qh, kh, vh, gh)):
                        d_t.copy_(h_t, non_blocking=True)
                    ev_in[i % 2].record(s_in)
            if i >= 1:
                j = i - 1
                main.wait_event(ev_in[j % 2])
                qd, kd, vd, gd = dev_in[j % 2]
                qd = qd.detach().requires_grad_(True); kd = kd.detach().requires_grad_(True); vd = vd.detach().requires_grad_(True)
                out = fn(qd, kd, vd, causal=causal)
                out.backward(gd)
                ev_used[j % 2].record(main)
                res = (out.detach(), qd.grad, kd.grad, vd.grad)
                s_out.wait_event(ev_used[j % 2])
                with torch.cuda.stream(s_out):
                    for h_t, d_t in zip((oh, dqh, dkh, dvh), res):
                        d_t.record_stream(s_out)
                        h_t.copy_(d_t, non_blocking=True)
                    ev_out.record(s_out)
        main.wait_event(ev_out)

    e2e_run(3)
    barrier()
    n_e2e = max(4, min(args.steps, 20))
    t0.record()
    e2e_run(n_e2e)
    t1.record()
    barrier()
    ms_e2e = t0.elapsed_time(t1) / n_e2e
    status_ok = True

    tt = torch.tensor([ms, ms_e2e, k_fwd, k_bwd], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms, ms_e2e, k_fwd, k_bwd = tt.tolist()
    if rank == 0:
        f_fwd = flops_fwd(B, S, H, D, causal)
        f_step = 3.5 * f_fwd * world
        value = f_step / (ms * 1e-3) / 1e12
        e2e_val = f_step / (ms_e2e * 1e-3) / 1e12
        sust, burst, hbm, how = _peaks()
        peak = 2.0 * sust      # E4M3 tensor rate = 2 x the dense bf16 rate; the kernel is timed inside a long step
        f_bwd = 2.5 * f_fwd
        # mixed route: the S recompute (1 of 5 backward GEMMs) runs at the E2M1 rate (2 x E4M3)
        t_min = (f_bwd / (peak * 1e12)) if args.route == "fp8" else (0.2 * f_bwd / (2 * peak * 1e12) + 0.8 * f_bwd / (peak * 1e12))
        achieved = f_bwd / (k_bwd * 1e-3) / 1e12
        line = {
            "metric": "attention fwd+bwd step TFLOPS (causal-adjusted), " + ("MXFP8" if args.route == "fp8" else "NVFP4/FP8"),
            "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps, "warmup": W, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "e4m3" if args.route == "fp8" else "e2m1+e4m3",
            "data": "synthetic",
            "config": {"workload": f"b{B} s{S} h{H} d{D} {'causal' if causal else 'dense'} fwd+bwd per GPU, flash_attn_{args.route} "
                                   "defaults (token-block scales, Hadamard on), quantisation included",
                       "global_batch": B * world, "seq_len": S, "parallelism": f"batch-sharded x{world}, no collective",
                       "l2": "inputs 268 MB per step > 126 MB L2, no flush needed", "launch": mode,
                       "published_reference_ms": 0.865 if causal else 1.416},
            "ms_fwd_kernel": k_fwd, "ms_bwd_kernel": k_bwd,
            "tflops_fwd_kernel": f_fwd / (k_fwd * 1e-3) / 1e12, "tflops_bwd_kernel": achieved,
            "roofline": {"bound": "tensor", "kernel": "bwd_kernel_pipelined", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": (t_min / (k_bwd * 1e-3)),
                         # dram read + write bytes of one launch: 151.4 MB captured by ncu on the b2 cell of
                         # --profile-case, scaled by the batch (traffic is proportional to b); fp8 route, causal
                         "traffic": 151.4e6 * B / 2 if (args.route == "fp8" and causal) else None,
                         "note": f"peak = 2 x {sust} TF/s dense bf16 sustained ({how}); of {how}"},
            "e2e": {"value": e2e_val, "unit": "TFLOPS", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in (qh, kh, vh, gh)),
                    "d2h_bytes_per_step": sum(t.numel() * t.element_size() for t in (oh, dqh, dkh, dvh))},
            "gpu_launches": 8 * args.steps,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            dt, fl = cpu_reference_slice(causal, cores, n_slices=16)
            line["cpu_baseline"] = {"value": fl / dt / 1e12, "unit": "TFLOPS", "cores": cores, "kind": "port",
                                    "sample": f"16 (batch, head) slices of the workload (s{S} d{D}): oracle quantise + fp32 "
                                              f"fwd+bwd, {dt:.1f} s"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
