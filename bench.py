#!/usr/bin/env python
"""Benchmark of the operator hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload ("step"): FlashAttention forward + backward, bf16, q/k/v
[4, 4096, 16, 128], no bias, non-causal — the third benchmark configuration,
the one the TFLOPS metric is quoted on.  The norm / RoPE half of the metric
(HBM GB/s) is measured in the same run on the second configuration
(FusedLNRoPE forward + backward, q/k [8, 4096, 16, 128] bf16) and reported
under ``norm_rope``.  With N > 1 (launched by torchrun, one rank per GPU)
every rank runs the full workload on its own GPU (weak scaling, no collective
on the data path); time is the max over ranks.

One JSON line is printed by rank 0.  ``--impl reference`` times the equivalent
torch-eager path on the host CPU cores instead (the reference has no CPU
implementation of its own; its kernels are GPU-only Triton).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CFG3 = dict(B=4, T=4096, H=16, D=128)          # attention
CFG2 = dict(B=8, T=4096, H=16, D=128, R=64)    # FusedLNRoPE
METRIC = "attn fwd+bwd TFLOPS (bf16,T=4096,d=128) + norm/RoPE HBM GB/s at 1/2/4/8 B200"


def attn_flops(B, T, H, D):
    fwd = 4.0 * B * H * T * T * D
    return fwd, 2.5 * fwd


def lnrope_bytes(B, T, H, D):
    per = B * T * H * D * 2            # one bf16 tensor
    return 4 * per, 6 * per            # fwd: q,k in + out; bwd: q,k,dqo,dko in + dq,dk out


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"], d["bf16_tflops"], d.get("bf16_tflops_sustained", d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "20"], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.05)
            self.proc.terminate()
            self.proc.wait(timeout=5)
            self.t.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        busy = [s for s in sm if s > 0.5 * max(sm)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def synth_attn(cfg, device, seed=0):
    """Seeded N(0,1) bf16 inputs generated on the CPU in fp32, then cast."""
    g = torch.Generator().manual_seed(seed)
    shape = (cfg["B"], cfg["T"], cfg["H"], cfg["D"])
    host = [torch.randn(*shape, generator=g).to(torch.bfloat16).pin_memory() if device != "cpu"
            else torch.randn(*shape, generator=g).to(torch.bfloat16) for _ in range(4)]
    return host   # q, k, v, do


def rotary_table(P, R, dtype):
    inv = 1.0 / (10000.0 ** (torch.arange(0, R, 2, dtype=torch.float32) / R))
    ang = (torch.arange(P, dtype=torch.float32)[:, None] * inv[None, :]).repeat_interleave(2, dim=-1)
    return torch.stack([ang.sin(), ang.cos()]).to(dtype)


# ---------------------------------------------------------------------------
# CPU side: torch-eager equivalents (baseline / reference arm)
# ---------------------------------------------------------------------------
def cpu_attn_step(q, k, v, do):
    """fwd+bwd of eager attention on the CPU, chunked per batch element."""
    scale = 1.0 / math.sqrt(q.shape[-1])
    for b in range(q.shape[0]):
        qb, kb, vb = (t[b:b + 1].detach().requires_grad_(True) for t in (q, k, v))
        s = torch.einsum("bthd,bshd->bhts", qb * scale, kb)
        o = torch.einsum("bhts,bshd->bthd", torch.softmax(s, dim=-1), vb)
        torch.autograd.grad(o, (qb, kb, vb), do[b:b + 1])


def cpu_baseline(cfg, seconds_budget=25.0):
    """Eager attention fwd+bwd on the host cores for a bounded sample (whole
    batch elements of the headline workload), reported in the metric's unit."""
    q, k, v, do = synth_attn(dict(cfg, B=1), "cpu")
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    cpu_attn_step(q, k, v, do)                     # untimed
    t0 = time.perf_counter()
    reps = 0
    while True:
        cpu_attn_step(q, k, v, do)
        reps += 1
        if time.perf_counter() - t0 > seconds_budget / 2 or reps >= 3:
            break
    dt = (time.perf_counter() - t0) / reps
    f, b = attn_flops(1, cfg["T"], cfg["H"], cfg["D"])
    return {"value": (f + b) / dt / 1e12, "unit": "TFLOPS", "cores": cores, "kind": "port",
            "sample": f"1 of {cfg['B']} batch elements (q/k/v [1,{cfg['T']},{cfg['H']},{cfg['D']}] bf16), "
                      f"torch eager fwd+bwd, {reps} timed repetition(s), {dt:.2f} s each"}


def run_reference(args):
    """Reference arm: the torch-eager path on the host CPU, same workload/metric."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    cfg = CFG3
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    q, k, v, do = synth_attn(dict(cfg, B=1), "cpu")
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_attn_step(q, k, v, do)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_attn_step(q, k, v, do)
    dt = (time.perf_counter() - t0) / args.steps
    f, b = attn_flops(1, cfg["T"], cfg["H"], cfg["D"])
    val = (f + b) / dt / 1e12
    sample = (f"each step = 1 of {cfg['B']} batch elements of the workload (bounded sample), torch eager fwd+bwd "
              f"on {cores} host threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "config3 FlashAttention fwd+bwd bf16 q/k/v [4,4096,16,128] no bias non-causal",
                   "sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOPS", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ---------------------------------------------------------------------------
# GPU side
# ---------------------------------------------------------------------------
def op_table(dev, steps, hbm_peak):
    """HBM GB/s of every norm / RoPE operator, forward and backward timed
    separately with CUDA events, at the benchmark configurations' shapes.
    L2 is flushed before every timed launch: a 512 MiB fill evicts the
    operator's tensors, then a 256 MiB read-only pass pushes the fill's dirty
    lines out so their write-back does not compete with the timed kernel.  The
    flush also keeps the GPU busy while the host enqueues the operator, so the
    events bracket kernel time and not launch latency."""
    from rgd_triton_b200 import ops
    bf = torch.bfloat16
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    clean = torch.zeros(64 << 20, dtype=torch.float32, device=dev)     # 256 MiB, only ever read
    g = torch.Generator().manual_seed(2)

    def rn(*shape, dtype=bf):
        return torch.randn(*shape, generator=g).to(dtype).to(dev)

    def nbytes(*ts):
        return sum(t.numel() * t.element_size() for t in ts)

    def timed(run):
        ts = []
        for _ in range(steps + 2):
            flush.fill_(1)          # evicts the operator's tensors from L2 ...
            clean.sum()             # ... and a read pass drains the fill's dirty lines before the timed launch
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            run()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts[2:])

    def case(name, fwd, inputs, grads_of, upstream, extra_bwd_bytes=0):
        ins = [t.requires_grad_(True) for t in inputs]
        outs = fwd(*ins)
        outs = outs if isinstance(outs, tuple) else (outs,)
        fwd_b = nbytes(*inputs) + nbytes(*outs)
        bwd_b = nbytes(*inputs) + nbytes(*upstream) + nbytes(*inputs) + extra_bwd_bytes
        with torch.no_grad():
            t_f = timed(lambda: fwd(*ins))
        wrt = ins + grads_of
        t_b = timed(lambda: torch.autograd.grad(outs, wrt, upstream, retain_graph=True))
        # Yardstick: a plain device copy moving the same number of bytes as the forward (half
        # read, half written), timed the same way.  The measured peak comes from a 2 GiB copy;
        # at these sizes (tens of microseconds) ramp-up and tail cost even a copy a good part of it.
        src = torch.empty(fwd_b // 2, dtype=torch.uint8, device=dev)
        dst = torch.empty_like(src)
        t_c = timed(lambda: dst.copy_(src))
        del src, dst
        return {"op": name, "fwd_bytes": fwd_b, "bwd_bytes": bwd_b, "fwd_ms": t_f, "bwd_ms": t_b,
                "fwd_gbs": fwd_b / t_f / 1e6, "bwd_gbs": bwd_b / t_b / 1e6,
                "fwd_frac": fwd_b / t_f / 1e6 / hbm_peak, "bwd_frac": bwd_b / t_b / 1e6 / hbm_peak,
                "copy_same_bytes_gbs": fwd_b / t_c / 1e6, "copy_same_bytes_frac": fwd_b / t_c / 1e6 / hbm_peak}

    rows = []
    # config 1: FusedRMSNorm fp32 [4,256,1024]
    m = ops.FusedRMSNorm(1024).to(dev)
    rows.append(case("FusedRMSNorm f32 [4,256,1024] (config1)", m, [rn(4, 256, 1024, dtype=torch.float32)],
                     [m.weight], [rn(4, 256, 1024, dtype=torch.float32)]))
    # config 2: FusedLNRoPE bf16 [8,4096,16,128]
    pos = rotary_table(4097, 64, bf).to(dev)
    f = ops.FusedLNRoPE()
    rows.append(case("FusedLNRoPE bf16 q,k [8,4096,16,128] (config2)",
                     lambda a, b: f(a, b, pos, (4096, 4096), False, 1e-5),
                     [rn(8, 4096, 16, 128), rn(8, 4096, 16, 128)], [], [rn(8, 4096, 16, 128), rn(8, 4096, 16, 128)]))
    # config 5, per GPU (batch 2)
    m2 = ops.FusedRMSNorm2((3072, 3072), dtype=bf).to(dev)
    rows.append(case("FusedRMSNorm2 bf16 [2,512,3072]+[2,4096,3072] (config5)", m2,
                     [rn(2, 512, 3072), rn(2, 4096, 3072)], [m2.weight1, m2.weight2],
                     [rn(2, 512, 3072), rn(2, 4096, 3072)]))
    pos5 = rotary_table(4609, 64, bf).to(dev)
    hl, rp, l2, l22 = ops.FusedHeadLayerNorm(), ops.RoPE(), ops.L2Normalize(), ops.FusedL2Normalize2()
    qk = lambda: [rn(2, 4608, 24, 128), rn(2, 4608, 24, 128)]
    rows.append(case("FusedHeadLayerNorm bf16 q,k [2,4608,24,128] (config5)",
                     lambda a, b: hl(a, b, False, 1e-6), qk(), [], qk()))
    r = case("RoPE bf16 q,k [2,4608,24,128] R=64 cutoff 4096 (config5)",
             lambda a, b: rp(a, b, pos5, 4096, False), qk(), [], qk())
    r["bwd_bytes"] = r["fwd_bytes"]          # the backward reads only the upstream gradients
    r["bwd_gbs"] = r["bwd_bytes"] / r["bwd_ms"] / 1e6
    r["bwd_frac"] = r["bwd_gbs"] / hbm_peak
    rows.append(r)
    rows.append(case("L2Normalize bf16 [2,4096,3072]", lambda a: l2(a), [rn(2, 4096, 3072)], [],
                     [rn(2, 4096, 3072)]))
    rows.append(case("FusedL2Normalize2 bf16 [2,512,3072]+[2,4096,3072]", lambda a, b: l22(a, b),
                     [rn(2, 512, 3072), rn(2, 4096, 3072)], [], [rn(2, 512, 3072), rn(2, 4096, 3072)]))
    del flush, clean
    return rows


def profile_case(name, dev):
    """A small case of one operator for profiler captures: inputs larger than
    the 126 MB L2 in total but well under 1 GB, three forward+backward passes."""
    from rgd_triton_b200 import ops
    g = torch.Generator().manual_seed(3)
    bf = torch.bfloat16

    def rn(*shape, dtype=bf):
        return torch.randn(*shape, generator=g).to(dtype).to(dev).requires_grad_(True)

    if name in ("attn", "attn64"):
        d = 128 if name == "attn" else 64
        H = 16 if name == "attn" else 24
        dt = bf if name == "attn" else torch.float16
        q, k, v = rn(1, 4096, H, d, dtype=dt), rn(1, 4096, H, d, dtype=dt), rn(1, 4096, H, d, dtype=dt)
        do = torch.randn(1, 4096, H, d, generator=g).to(dt).to(dev)
        bias = None
        if name == "attn64":
            bias = torch.randn(1, H, 4096, 4096, generator=g).to(dt).to(dev)
        m = ops.FlashAttention()
        for _ in range(3):
            o = m(q, k, v, bias)
            torch.autograd.grad(o, (q, k, v), do)
    elif name == "lnrope":
        q, k = rn(2, 4096, 16, 128), rn(2, 4096, 16, 128)
        gq, gk = torch.randn_like(q), torch.randn_like(k)
        pos = rotary_table(4097, 64, bf).to(dev)
        m = ops.FusedLNRoPE()
        for _ in range(3):
            qo, ko = m(q, k, pos, (4096, 4096), False, 1e-5)
            torch.autograd.grad((qo, ko), (q, k), (gq, gk))
    else:
        m = ops.FusedRMSNorm2((3072, 3072), dtype=bf).to(dev)
        a, b = rn(2, 512, 3072), rn(2, 4096, 3072)
        ga, gb = torch.randn_like(a), torch.randn_like(b)
        for _ in range(3):
            ya, yb = m(a, b)
            torch.autograd.grad((ya, yb), (a, b, m.weight1, m.weight2), (ga, gb))
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": name, "ok": True}), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ops-only", action="store_true", help="only the per-operator norm / RoPE table")
    ap.add_argument("--no-config4", action="store_true", help="skip the dense-bias attention measurement")
    ap.add_argument("--profile", default=None, choices=["attn", "attn64", "lnrope", "rms2"],
                    help="run a small fixed case of one operator (1 warm-up + 2 fwd+bwd passes) for ncu captures")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    args.warmup = max(args.warmup, 3)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    import torch.distributed as dist
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local)

    from rgd_triton_b200 import _lib, ops
    lib = _lib.load()
    if lib.rgd_device_supported(local) != 1:
        raise RuntimeError("bench.py needs a compute-capability-10 GPU (B200)")

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    hbm_peak, tf_burst, tf_sust, peak_src = peaks()
    if args.profile:
        return profile_case(args.profile, dev)
    if args.ops_only:
        rows = op_table(dev, args.steps, hbm_peak)
        if rank == 0:
            print(json.dumps({"ops": rows, "hbm_peak_gbs": hbm_peak, "peak_source": peak_src}), flush=True)
        return 0

    # ---------------- attention, config 3 ----------------
    cfg = CFG3
    hq, hk, hv, hdo = synth_attn(cfg, "cuda")
    q, k, v, do = (t.to(dev, non_blocking=True) for t in (hq, hk, hv, hdo))
    attn = ops.FlashAttention()

    def attn_step(q, k, v, do, ev=None):
        qi, ki, vi = q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
        if ev:
            ev[0].record()
        o = attn(qi, ki, vi)
        if ev:
            ev[1].record()
        grads = torch.autograd.grad(o, (qi, ki, vi), do)
        if ev:
            ev[2].record()
        return o, grads

    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    # the sampler starts before the warm-up (same load as the timed steps), so that short
    # timed regions still get clock samples under load
    with ClockSampler(local) as clk:
        for _ in range(args.warmup):
            attn_step(q, k, v, do)
        barrier()
        launches0 = lib.rgd_launch_count()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for i in range(args.steps):
            attn_step(q, k, v, do, evs[i])
        end.record()
        barrier()
    launches = lib.rgd_launch_count() - launches0
    ms_total = max_over_ranks(start.elapsed_time(end))
    ms_step = ms_total / args.steps
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in evs)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in evs)
    f_fwd, f_bwd = attn_flops(**cfg)
    tflops = world * (f_fwd + f_bwd) / (ms_step * 1e-3) / 1e12
    clocks = clk.summary()
    dom = ("attention backward (delta + dK/dV + dQ kernels)", f_bwd, bwd_ms) if bwd_ms >= fwd_ms else \
          ("attention forward kernel", f_fwd, fwd_ms)
    achieved = dom[1] / (dom[2] * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": dom[0], "achieved": achieved, "peak": tf_burst, "unit": "TFLOP/s",
                "frac": achieved / tf_burst, "peak_source": peak_src,
                # DRAM bytes (read + write) of the prep, dK/dV and dQ launches: ncu capture of the quarter-size
                # case (16 of the 64 (batch, head) pairs, profiles/attention_tmem_kernels_small_case.md) scaled x4
                "traffic": 4 * (33.82e6 + 67.85e6 + 8.40e6 + 67.70e6 + 4.39e6),
                "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
                "fwd_tflops": f_fwd / (fwd_ms * 1e-3) / 1e12, "bwd_tflops": f_bwd / (bwd_ms * 1e-3) / 1e12}

    # ---------------- end to end: host buffers through the module API ----------------
    # Every step copies its inputs from pinned host memory, runs forward + backward through
    # ops.FlashAttention and copies all four results back.  Steps rotate over three CUDA
    # streams, each with its own pinned result buffers, so one step's device-to-host copies
    # overlap the next step's host-to-device copies and kernels (PCIe is full duplex and the
    # copy engines are separate); within a stream everything stays in order.
    n_slots = 3        # measured on B200: 1 stream 12.0 ms per step, 2 streams 6.9, 3 streams 6.3, 4 streams 6.3
    slots = []
    for _ in range(n_slots):
        slots.append({"stream": torch.cuda.Stream(device=dev),
                      "ho": torch.empty_like(hq).pin_memory(),
                      "hgrads": [torch.empty_like(hq).pin_memory() for _ in range(3)]})

    def e2e_step(i):
        sl = slots[i % n_slots]
        with torch.cuda.stream(sl["stream"]):
            dq_, dk_, dv_, ddo = (t.to(dev, non_blocking=True) for t in (hq, hk, hv, hdo))
            o, grads = attn_step(dq_, dk_, dv_, ddo)
            sl["ho"].copy_(o.detach(), non_blocking=True)
            for h, g_ in zip(sl["hgrads"], grads):
                h.copy_(g_, non_blocking=True)

    def e2e_run(n):
        main = torch.cuda.current_stream()
        for sl in slots:
            sl["stream"].wait_stream(main)
        for i in range(n):
            e2e_step(i)
        for sl in slots:
            main.wait_stream(sl["stream"])

    e2e_steps = max(4, min(args.steps, 10))
    e2e_run(2)
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    e2e_run(e2e_steps)
    e2.record()
    barrier()
    e2e_ms = max_over_ranks(s2.elapsed_time(e2)) / e2e_steps
    nbytes = hq.numel() * hq.element_size()
    e2e = {"value": world * (f_fwd + f_bwd) / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": 4 * nbytes, "d2h_bytes_per_step": 4 * nbytes, "steps": e2e_steps,
           "overlap": "steps rotate over 3 CUDA streams: D2H of step i overlaps H2D + kernels of the next steps"}
    del slots
    del q, k, v, do
    torch.cuda.empty_cache()

    # ---------------- FusedLNRoPE, config 2 (HBM-bound half of the metric) ----------------
    c2 = CFG2
    g = torch.Generator().manual_seed(1)
    shp = (c2["B"], c2["T"], c2["H"], c2["D"])
    q2, k2, gq2, gk2 = (torch.randn(*shp, generator=g).to(torch.bfloat16).to(dev) for _ in range(4))
    pos = rotary_table(c2["T"] + 1, c2["R"], torch.bfloat16).to(dev)
    lnrope = ops.FusedLNRoPE()

    def lnrope_step(ev=None):
        qi, ki = q2.requires_grad_(True), k2.requires_grad_(True)
        if ev:
            ev[0].record()
        qo, ko = lnrope(qi, ki, pos, seq_cutoff=(c2["T"], c2["T"]), heads_second=False, eps=1e-5)
        if ev:
            ev[1].record()
        torch.autograd.grad((qo, ko), (qi, ki), (gq2, gk2))
        if ev:
            ev[2].record()

    for _ in range(args.warmup):
        lnrope_step()
    barrier()
    evs2 = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    s3, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s3.record()
    for i in range(args.steps):
        lnrope_step(evs2[i])
    e3.record()
    barrier()
    ln_ms = max_over_ranks(s3.elapsed_time(e3)) / args.steps
    b_fwd, b_bwd = lnrope_bytes(c2["B"], c2["T"], c2["H"], c2["D"])
    ln_fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in evs2)
    ln_bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in evs2)
    norm_rope = {
        "workload": "config2 FusedLNRoPE fwd+bwd bf16 q/k [8,4096,16,128] heads_second=False R=64",
        "value": world * (b_fwd + b_bwd) / (ln_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ln_ms,
        "roofline": {"bound": "hbm", "peak": hbm_peak, "unit": "GB/s", "peak_source": peak_src,
                     "fwd_gbs": b_fwd / (ln_fwd_ms * 1e-3) / 1e9, "bwd_gbs": b_bwd / (ln_bwd_ms * 1e-3) / 1e9,
                     "fwd_frac": b_fwd / (ln_fwd_ms * 1e-3) / 1e9 / hbm_peak,
                     "bwd_frac": b_bwd / (ln_bwd_ms * 1e-3) / 1e9 / hbm_peak,
                     "fwd_ms": ln_fwd_ms, "bwd_ms": ln_bwd_ms, "traffic": None},
        "l2": "working set 1.3 GB per step, larger than the 126 MB L2",
    }
    del q2, k2, gq2, gk2
    norm_rope["ops"] = op_table(dev, min(args.steps, 10), hbm_peak)

    # ---------------- attention with a dense additive bias, config 4 ----------------
    def config4(broadcast):
        g4 = torch.Generator().manual_seed(4)
        B4, T4, H4, D4 = 2, 4096, 24, 64
        q4, k4, v4, do4 = (torch.randn(B4, T4, H4, D4, generator=g4).to(torch.float16).to(dev) for _ in range(4))
        bb = 1 if broadcast else B4
        bias = torch.randn(bb, H4, T4, T4, generator=g4, dtype=torch.float16)
        blk = (torch.rand(bb, H4, T4 // 64, T4 // 64, generator=g4) < 0.1) & ~torch.eye(T4 // 64, dtype=torch.bool)
        bias = (bias.float() - 1e4 * blk.repeat_interleave(64, 2).repeat_interleave(64, 3)).to(torch.float16).to(dev)
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(max(3, min(args.steps, 10)))]
        for i in range(-2, len(ev)):
            qi, ki, vi = q4.requires_grad_(True), k4.requires_grad_(True), v4.requires_grad_(True)
            if i >= 0:
                ev[i][0].record()
            o = attn(qi, ki, vi, bias)
            if i >= 0:
                ev[i][1].record()
            torch.autograd.grad(o, (qi, ki, vi), do4)
            if i >= 0:
                ev[i][2].record()
        torch.cuda.synchronize()
        fwd = statistics.median(e[0].elapsed_time(e[1]) for e in ev)
        bwd = statistics.median(e[1].elapsed_time(e[2]) for e in ev)
        ff, fb = attn_flops(B4, T4, H4, D4)
        nbias = bias.numel() * 2
        return {"workload": f"config4 FlashAttention fwd+bwd fp16 q/k/v [2,4096,24,64] bias [{bb},24,4096,4096]",
                "fwd_ms": fwd, "bwd_ms": bwd, "tflops": (ff + fb) / ((fwd + bwd) * 1e-3) / 1e12,
                "fwd_bias_gbs": nbias / (fwd * 1e-3) / 1e9, "bias_bytes_per_pass": nbias,
                "roofline_ms": sum(max(f / (tf_burst * 1e12), nbias / (hbm_peak * 1e9)) for f in (ff, fb)) * 1e3}

    cfg4 = [config4(False), config4(True)] if not args.no_config4 else None
    torch.cuda.empty_cache()

    base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        base = cpu_baseline(cfg)

    if rank == 0:
        line = {
            "metric": METRIC, "value": tflops, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "config3 FlashAttention fwd+bwd bf16 q/k/v [4,4096,16,128] no bias non-causal, "
                                   "per GPU", "l2": "inputs+outputs 256 MiB per step, larger than the 126 MB L2",
                       "parallelism": f"replicas x{world} (batch x heads shard, no collective)"},
            "roofline": roofline, "norm_rope": norm_rope, "e2e": e2e, "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if cfg4 is not None:
            line["config4"] = cfg4
        if base is not None:
            line["cpu_baseline"] = base
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
