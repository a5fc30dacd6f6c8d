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
on the data path); time is the max over ranks, and every rank's own time and
clocks are listed under ``per_rank``.

One JSON line is printed by rank 0.  Besides the headline it carries:
``roofline`` (dominant phase against the measured tensor peak), ``sustained``
(the same step looped for seconds, against the sustained peak), ``e2e`` (host
buffers through the module API), ``norm_rope`` (configuration 2 and a table of
every norm / RoPE operator), ``config4`` (dense-bias attention), ``config5``
(the MMDiT joint-attention block per GPU), ``host_us_per_call`` (host time of a
call through the module API), ``reference_triton`` (the reference's own Triton
kernels on the same GPU, when that project is installed under baseline/_ref),
``verify`` (a batch x heads shard of the workload per rank, gathered and
compared bit for bit with the unsharded result) and ``cpu_baseline``.

``--impl reference`` times the equivalent torch-eager path on the host CPU
cores instead (the reference has no CPU implementation of its own; its kernels
are GPU-only Triton).
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


def dram_traffic_table():
    """DRAM bytes per launch from profiler captures of small cases, kept as a tracked table
    (kernel -> bytes per (batch, head) pair of that case); None when the table is absent."""
    p = ROOT / "profiles" / "dram_traffic_per_unit.json"
    try:
        return json.loads(p.read_text())
    except (OSError, ValueError):
        return None


class ClockSampler:
    """Samples SM clocks and throttle reasons of the node's GPUs with ONE nvidia-smi
    process while a region runs (only the rank that owns it starts one)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, enabled: bool = True, period_ms: int = 20):
        self.enabled, self.period_ms, self.proc, self.lines = enabled, period_ms, None, []

    def __enter__(self):
        if not self.enabled:
            return self
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", str(self.period_ms)], stdout=subprocess.PIPE, text=True)
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

    def summary(self, index: int):
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                if int(f[0]) != index:
                    continue
                s_, m_ = float(f[1]), float(f[2])
            except ValueError:
                continue
            sm.append(s_)
            mx.append(m_)
            try:
                pw.append(float(f[3]))
            except ValueError:
                pass
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        busy = [s for s in sm if s > 0.5 * max(sm)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_mhz_min": min(busy), "sm_max_mhz": max(mx),
                "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons), "samples": len(sm)}


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


def shard_units(n_units: int, world: int, rank: int) -> range:
    """Contiguous, balanced split of independent (batch, head) units over ranks."""
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


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
    """Reference arm: the torch-eager path on the host CPU, same workload/metric.
    Under torchrun rank 0 alone runs; the other ranks exit without work."""
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
              f"on {cores} host threads; one CPU process whatever --gpus says")
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
# GPU side: timing helpers
# ---------------------------------------------------------------------------
class L2Flush:
    """Evicts an operator's tensors from L2 before a timed launch: a 512 MiB fill, then a
    256 MiB read-only pass that pushes the fill's dirty lines out so their write-back does
    not compete with the timed kernel.  The flush also keeps the GPU busy while the host
    enqueues the operator, so the events bracket kernel time and not launch latency."""

    def __init__(self, dev):
        self.flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
        self.clean = torch.zeros(64 << 20, dtype=torch.float32, device=dev)

    def __call__(self):
        self.flush.fill_(1)
        self.clean.sum()


def timed_median(run, steps, flush=None, warm=2):
    ts = []
    for _ in range(steps + warm):
        if flush is not None:
            flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        run()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts[warm:])


def graph_time_ms(step, replays=5):
    """GPU time of one call of `step` with no host launch time in it: the call is captured
    into a CUDA graph after warm-up and the replays are timed with events.  Returns
    (ms, "graph") or, when the call cannot be captured, the event time of back-to-back eager
    calls and "eager" (host launch gaps included)."""
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    try:
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            step()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        with torch.cuda.graph(g):
            step()
        g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(replays):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        del g
        return statistics.median(ts), "graph"
    except Exception:
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(replays):
            step()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / replays, "eager"


def op_cases(dev, bf=torch.bfloat16):
    """The norm / RoPE operators at the benchmark configurations' shapes:
    (name, module-call, inputs, extra tensors to differentiate, upstream gradients)."""
    from rgd_triton_b200 import ops
    g = torch.Generator().manual_seed(2)

    def rn(*shape, dtype=bf):
        return torch.randn(*shape, generator=g).to(dtype).to(dev)

    cases = []
    m = ops.FusedRMSNorm(1024).to(dev)
    cases.append(("FusedRMSNorm f32 [4,256,1024] (config1)", m, [rn(4, 256, 1024, dtype=torch.float32)],
                  [m.weight], [rn(4, 256, 1024, dtype=torch.float32)], None))
    pos = rotary_table(4097, 64, bf).to(dev)
    f = ops.FusedLNRoPE()
    cases.append(("FusedLNRoPE bf16 q,k [8,4096,16,128] (config2)",
                  lambda a, b: f(a, b, pos, (4096, 4096), False, 1e-5),
                  [rn(8, 4096, 16, 128), rn(8, 4096, 16, 128)], [], [rn(8, 4096, 16, 128), rn(8, 4096, 16, 128)], None))
    m2 = ops.FusedRMSNorm2((3072, 3072), dtype=bf).to(dev)
    cases.append(("FusedRMSNorm2 bf16 [2,512,3072]+[2,4096,3072] (config5)", m2,
                  [rn(2, 512, 3072), rn(2, 4096, 3072)], [m2.weight1, m2.weight2],
                  [rn(2, 512, 3072), rn(2, 4096, 3072)], None))
    pos5 = rotary_table(4609, 64, bf).to(dev)
    hl, rp, l2, l22 = ops.FusedHeadLayerNorm(), ops.RoPE(), ops.L2Normalize(), ops.FusedL2Normalize2()
    qk = lambda: [rn(2, 4608, 24, 128), rn(2, 4608, 24, 128)]
    cases.append(("FusedHeadLayerNorm bf16 q,k [2,4608,24,128] (config5)",
                  lambda a, b: hl(a, b, False, 1e-6), qk(), [], qk(), None))
    # the RoPE backward reads only the upstream gradients
    cases.append(("RoPE bf16 q,k [2,4608,24,128] R=64 cutoff 4096 (config5)",
                  lambda a, b: rp(a, b, pos5, 4096, False), qk(), [], qk(), "bwd_bytes=fwd_bytes"))
    cases.append(("L2Normalize bf16 [2,4096,3072]", lambda a: l2(a), [rn(2, 4096, 3072)], [],
                  [rn(2, 4096, 3072)], None))
    cases.append(("FusedL2Normalize2 bf16 [2,512,3072]+[2,4096,3072]", lambda a, b: l22(a, b),
                  [rn(2, 512, 3072), rn(2, 4096, 3072)], [], [rn(2, 512, 3072), rn(2, 4096, 3072)], None))
    return cases


def op_table(dev, steps, hbm_peak):
    """HBM GB/s of every norm / RoPE operator, forward and backward timed
    separately with CUDA events, L2 flushed before every timed launch."""
    flush = L2Flush(dev)

    def nbytes(*ts):
        return sum(t.numel() * t.element_size() for t in ts)

    rows = []
    for name, fwd, inputs, grads_of, upstream, note in op_cases(dev):
        ins = [t.requires_grad_(True) for t in inputs]
        outs = fwd(*ins)
        outs = outs if isinstance(outs, tuple) else (outs,)
        fwd_b = nbytes(*inputs) + nbytes(*outs)
        bwd_b = fwd_b if note else nbytes(*inputs) + nbytes(*upstream) + nbytes(*inputs)
        with torch.no_grad():
            t_f = timed_median(lambda: fwd(*ins), steps, flush)
        wrt = ins + grads_of
        t_b = timed_median(lambda: torch.autograd.grad(outs, wrt, upstream, retain_graph=True), steps, flush)
        # Yardstick: a plain device copy moving the same number of bytes as the forward (half
        # read, half written), timed the same way.  The measured peak comes from a 2 GiB copy;
        # at these sizes (tens of microseconds) ramp-up and tail cost even a copy a good part of it.
        src = torch.empty(fwd_b // 2, dtype=torch.uint8, device=dev)
        dst = torch.empty_like(src)
        t_c = timed_median(lambda: dst.copy_(src), steps, flush)
        del src, dst
        rows.append({"op": name, "fwd_bytes": fwd_b, "bwd_bytes": bwd_b, "fwd_ms": t_f, "bwd_ms": t_b,
                     "fwd_gbs": fwd_b / t_f / 1e6, "bwd_gbs": bwd_b / t_b / 1e6,
                     "fwd_frac": fwd_b / t_f / 1e6 / hbm_peak, "bwd_frac": bwd_b / t_b / 1e6 / hbm_peak,
                     "copy_same_bytes_gbs": fwd_b / t_c / 1e6, "copy_same_bytes_frac": fwd_b / t_c / 1e6 / hbm_peak})
    return rows


def host_us_per_call(dev, reps=40):
    """Host wall time of one call through the module API with the GPU idle (synchronised
    before every call, clock stopped when the call returns, i.e. when its launches are
    enqueued): what the Python layer, ctypes and the C entry point cost per call.  Small
    tensors, so that nothing but the host path is measured; second and later calls, so the
    module cache is warm."""
    from rgd_triton_b200 import ops
    bf = torch.bfloat16
    g = torch.Generator().manual_seed(5)
    rn = lambda *s, dtype=bf: torch.randn(*s, generator=g).to(dtype).to(dev)

    def wall(fn):
        ts = []
        for _ in range(reps + 5):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            fn()
            ts.append((time.perf_counter() - t0) * 1e6)
        return statistics.median(ts[5:])

    out = {}

    def add(name, fwd, inputs, extra=()):
        with torch.no_grad():
            out[name + " fwd"] = wall(lambda: fwd(*inputs))
        ins = [t.clone().requires_grad_(True) for t in inputs]

        def both():
            o = fwd(*ins)
            o = o if isinstance(o, tuple) else (o,)
            torch.autograd.grad(o, ins + list(extra), [torch.ones_like(t) for t in o])
        out[name + " fwd+bwd (autograd)"] = wall(both)

    pos = rotary_table(300, 64, bf).to(dev)
    m1 = ops.FusedRMSNorm(1024).to(dev)
    add("FusedRMSNorm", m1, [rn(4, 256, 1024, dtype=torch.float32)], [m1.weight])
    m2 = ops.FusedRMSNorm2((512, 512), dtype=bf).to(dev)
    add("FusedRMSNorm2", m2, [rn(2, 64, 512), rn(2, 128, 512)], [m2.weight1, m2.weight2])
    l2, l22, hl, rp, lr = (ops.L2Normalize(), ops.FusedL2Normalize2(), ops.FusedHeadLayerNorm(), ops.RoPE(),
                           ops.FusedLNRoPE())
    add("L2Normalize", lambda a: l2(a), [rn(2, 128, 512)])
    add("FusedL2Normalize2", lambda a, b: l22(a, b), [rn(2, 64, 512), rn(2, 128, 512)])
    add("FusedHeadLayerNorm", lambda a, b: hl(a, b, False, 1e-6), [rn(2, 256, 4, 128), rn(2, 256, 4, 128)])
    add("RoPE", lambda a, b: rp(a, b, pos, 256, False), [rn(2, 256, 4, 128), rn(2, 256, 4, 128)])
    add("FusedLNRoPE", lambda a, b: lr(a, b, pos, 256, False, 1e-5), [rn(2, 256, 4, 128), rn(2, 256, 4, 128)])
    fa = ops.FlashAttention()
    add("FlashAttention", lambda a, b, c: fa(a, b, c), [rn(1, 256, 2, 128) for _ in range(3)])
    return {k: round(v, 1) for k, v in out.items()}


def config5_block(dev, steps, hbm_peak, tf_burst):
    """One GPU's share (batch 2) of the MMDiT joint-attention block, forward + backward:
    FusedRMSNorm2 on the text and image streams -> QKV Linear (cuBLAS, outside the operator
    set) on the image-then-text sequence -> FusedHeadLayerNorm on q, k -> RoPE on the image
    tokens -> FlashAttention with a dense bias masking padded text keys."""
    from rgd_triton_b200 import ops
    bf = torch.bfloat16
    g = torch.Generator().manual_seed(5)
    B, Tt, Ti, Cm, H, D = 2, 512, 4096, 3072, 24, 128
    Tn = Ti + Tt
    text = torch.randn(B, Tt, Cm, generator=g).to(bf).to(dev).requires_grad_(True)
    image = torch.randn(B, Ti, Cm, generator=g).to(bf).to(dev).requires_grad_(True)
    rms = ops.FusedRMSNorm2((Cm, Cm), dtype=bf).to(dev)
    with torch.no_grad():
        rms.weight1.copy_((1 + 0.02 * torch.randn(Cm, generator=g)).to(bf))
        rms.weight2.copy_((1 + 0.02 * torch.randn(Cm, generator=g)).to(bf))
    w_qkv = (torch.randn(3 * H * D, Cm, generator=g) / math.sqrt(Cm)).to(bf).to(dev).requires_grad_(True)
    text_len = torch.randint(64, 513, (B,), generator=g).tolist()
    bias = torch.zeros(B, H, Tn, Tn, device=dev, dtype=bf)
    for b, L in enumerate(text_len):
        bias[b, :, :, Ti + L:] = -1e4
    pos = rotary_table(Tn + 1, 64, bf).to(dev)
    do = torch.randn(B, Tn, H, D, generator=g).to(bf).to(dev)
    hl, rp, fa = ops.FusedHeadLayerNorm(), ops.RoPE(), ops.FlashAttention()

    def forward(ev=None):
        mark = (lambda i: ev[i].record()) if ev else (lambda i: None)
        mark(0)
        tn, im = rms(text, image)
        mark(1)
        x = torch.cat([im, tn], dim=1)                               # image tokens first
        qkv = torch.nn.functional.linear(x, w_qkv).view(B, Tn, 3, H, D)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]           # strided views, channel stride 1
        mark(2)
        q, k = hl(q, k, False, 1e-6)
        mark(3)
        q, k = rp(q, k, pos, Ti, False)
        mark(4)
        o = fa(q, k, v, bias)
        mark(5)
        return o

    params = [text, image, rms.weight1, rms.weight2, w_qkv]
    for _ in range(2):
        torch.autograd.grad(forward(), params, do)
    n = max(3, min(steps, 5))
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(7)] for _ in range(n)]
    for i in range(n):
        o = forward(ev[i])
        torch.autograd.grad(o, params, do)
        ev[i][6].record()
    torch.cuda.synchronize()
    med = lambda a, b: statistics.median(e[a].elapsed_time(e[b]) for e in ev)
    # attention alone, forward and backward, on the block's own q, k, v
    with torch.no_grad():
        tn, im = rms(text, image)
        qkv = torch.nn.functional.linear(torch.cat([im, tn], dim=1), w_qkv).view(B, Tn, 3, H, D)
        q, k = rp(*hl(qkv[:, :, 0], qkv[:, :, 1], False, 1e-6), pos, Ti, False)
        v = qkv[:, :, 2]
    qa, ka, va = (t.detach().requires_grad_(True) for t in (q, k, v))
    o = fa(qa, ka, va, bias)
    a_fwd = timed_median(lambda: fa(qa, ka, va, bias), n)
    a_bwd = timed_median(lambda: torch.autograd.grad(o, (qa, ka, va), do, retain_graph=True), n)
    # the same without the block-sparse skip: the bias has been through `fa`'s cache more than once
    # by now, so the calls above visit only key blocks that hold an unmasked key
    from rgd_triton_b200 import functional as F_
    prev = F_.set_skip_masked_tiles(False)
    try:
        fd = ops.FlashAttention()
        od = fd(qa, ka, va, bias)
        d_fwd = timed_median(lambda: fd(qa, ka, va, bias), n)
        d_bwd = timed_median(lambda: torch.autograd.grad(od, (qa, ka, va), do, retain_graph=True), n)
    finally:
        F_.set_skip_masked_tiles(prev)
    nkb = (Tn + 127) // 128
    skipped = sum(nkb - (Ti + L + 127) // 128 for L in text_len) / (B * nkb)
    ff, fb = attn_flops(B, Tn, H, D)
    nbias = bias.numel() * 2
    masked = sum(Tt - L for L in text_len) / (B * Tn)
    # The same block with what the operator set already offers beyond the literal
    # configuration: FusedLNRoPE (LayerNorm and rotary of the image tokens in one pass, the
    # cutoff covering the image-first part of the sequence) instead of FusedHeadLayerNorm + RoPE,
    # and the padded-key mask as a (B, 1, 1, T) vector bias (one value per key, 18 KB) instead of
    # the dense (B, h, T, T) tensor (2 GB): every row of the dense bias holds exactly these values.
    # (The fused LayerNorm + rotary rounds once where the two separate operators round twice, so
    # the block's output differs from the literal form in the last bits.)
    lr = ops.FusedLNRoPE()
    vbias = bias[:, :1, :1, :].contiguous()

    def forward_fused():
        tn, im = rms(text, image)
        qkv = torch.nn.functional.linear(torch.cat([im, tn], dim=1), w_qkv).view(B, Tn, 3, H, D)
        q, k = lr(qkv[:, :, 0], qkv[:, :, 1], pos, Ti, False, 1e-6)
        return fa(q, k, qkv[:, :, 2], vbias)

    with torch.no_grad():
        diff = (forward().float() - forward_fused().float()).abs().max().item()
    fused_ms = timed_median(lambda: torch.autograd.grad(forward_fused(), params, do), n)
    ov = fa(qa, ka, va, vbias)
    v_fwd = timed_median(lambda: fa(qa, ka, va, vbias), n)
    v_bwd = timed_median(lambda: torch.autograd.grad(ov, (qa, ka, va), do, retain_graph=True), n)
    fused = {"what": "FusedLNRoPE (cutoff = image tokens) replaces FusedHeadLayerNorm + RoPE; the padded-key mask "
                     "is passed as a (B,1,1,T) vector bias instead of the dense (B,h,T,T) tensor",
             "block_fwd_bwd_ms": fused_ms, "output_max_abs_diff_vs_literal_form": diff,
             "attention": {"fwd_ms": v_fwd, "bwd_ms": v_bwd, "tflops": (ff + fb) / ((v_fwd + v_bwd) * 1e-3) / 1e12,
                           "bias_bytes_per_pass": vbias.numel() * 2}}
    return {
        "workload": f"config5 MMDiT block per GPU: text [2,512,3072] + image [2,4096,3072] bf16, 24 heads x 128, "
                    f"bias [2,24,{Tn},{Tn}] masking padded text keys (text lengths {text_len})",
        "block_fwd_bwd_ms": med(0, 6), "block_fwd_ms": med(0, 5), "block_bwd_ms": med(5, 6),
        "fwd_ms": {"FusedRMSNorm2": med(0, 1), "cat + QKV Linear (cuBLAS)": med(1, 2), "FusedHeadLayerNorm": med(2, 3),
                   "RoPE": med(3, 4), "FlashAttention": med(4, 5)},
        "attention": {"fwd_ms": a_fwd, "bwd_ms": a_bwd, "tflops": (ff + fb) / ((a_fwd + a_bwd) * 1e-3) / 1e12,
                      "fwd_tflops": ff / (a_fwd * 1e-3) / 1e12, "bwd_tflops": fb / (a_bwd * 1e-3) / 1e12,
                      "fwd_bias_gbs": nbias / (a_fwd * 1e-3) / 1e9, "bias_bytes_per_pass": nbias,
                      "flop_fwd_bwd": ff + fb, "masked_key_fraction": masked,
                      "key_blocks_skipped_fraction": skipped,
                      "tile_lists_used": bool(torch.is_tensor(getattr(fa.cache, "_tiles", [None, None, None])[2])),
                      "without_skip_fwd_ms": d_fwd, "without_skip_bwd_ms": d_bwd,
                      "roofline_ms": sum(max(f / (tf_burst * 1e12), nbias / (hbm_peak * 1e9)) for f in (ff, fb)) * 1e3},
        "fused_form": fused,
    }


def config4(dev, attn, steps, broadcast, hbm_peak, tf_burst):
    """Attention with a dense additive bias: fp16, q/k/v [2,4096,24,64], bias N(0,1) with
    -1e4 on 64x64 blocks chosen Bernoulli(0.1), diagonal blocks kept."""
    g4 = torch.Generator().manual_seed(4)
    B4, T4, H4, D4 = 2, 4096, 24, 64
    q4, k4, v4, do4 = (torch.randn(B4, T4, H4, D4, generator=g4).to(torch.float16).to(dev) for _ in range(4))
    bb = 1 if broadcast else B4
    gd = torch.Generator(device=dev).manual_seed(4)
    bias = torch.randn(bb, H4, T4, T4, generator=gd, device=dev, dtype=torch.float32).to(torch.float16)
    nb = T4 // 64
    blk = (torch.rand(bb, H4, nb, nb, generator=gd, device=dev) < 0.1) & ~torch.eye(nb, dtype=torch.bool, device=dev)
    bias.view(bb, H4, nb, 64, nb, 64).masked_fill_(blk[:, :, :, None, :, None], -1e4)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(max(3, min(steps, 10)))]
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
            "fwd_bias_gbs": nbias / (fwd * 1e-3) / 1e9, "bwd_bias_gbs": nbias / (bwd * 1e-3) / 1e9,
            "bias_bytes_per_pass": nbias, "masked_block_fraction": float(blk.float().mean()),
            "roofline_ms": sum(max(f / (tf_burst * 1e12), nbias / (hbm_peak * 1e9)) for f in (ff, fb)) * 1e3}


def block_sparse_case(dev, steps):
    """The block-sparse skip where it applies: configuration 4's shapes (fp16, [2,4096,24,64]) with a
    bias whose 128 x 128 tiles are masked (-1e4) with probability 0.5, diagonal tiles kept.  The
    module scans the bias on its second use and then visits only unmasked tiles; timed against the
    same module with the skip turned off."""
    from rgd_triton_b200 import functional as F_, ops
    g = torch.Generator().manual_seed(44)
    B, T_, H, D = 2, 4096, 24, 64
    q, k, v, do = (torch.randn(B, T_, H, D, generator=g).to(torch.float16).to(dev) for _ in range(4))
    gd = torch.Generator(device=dev).manual_seed(44)
    bias = torch.randn(B, H, T_, T_, generator=gd, device=dev, dtype=torch.float32).to(torch.float16)
    nb = T_ // 128
    blk = (torch.rand(B, H, nb, nb, generator=gd, device=dev) < 0.5) & ~torch.eye(nb, dtype=torch.bool, device=dev)
    bias.view(B, H, nb, 128, nb, 128).masked_fill_(blk[:, :, :, None, :, None], -1e4)
    out = {"workload": "fp16 q/k/v [2,4096,24,64], bias [2,24,4096,4096] with 128x128 tiles masked Bernoulli(0.5)",
           "masked_tile_fraction": float(blk.float().mean())}
    n = max(3, min(steps, 10))
    for name, enable in (("dense", False), ("skip", True)):
        prev = F_.set_skip_masked_tiles(enable)
        try:
            fa = ops.FlashAttention()
            qi, ki, vi = (t.detach().requires_grad_(True) for t in (q, k, v))
            for _ in range(3):
                o = fa(qi, ki, vi, bias)
                torch.autograd.grad(o, (qi, ki, vi), do)
            o = fa(qi, ki, vi, bias)
            out[name + "_fwd_ms"] = timed_median(lambda: fa(qi, ki, vi, bias), n)
            out[name + "_bwd_ms"] = timed_median(lambda: torch.autograd.grad(o, (qi, ki, vi), do, retain_graph=True), n)
            if enable:
                out["tile_lists_used"] = bool(torch.is_tensor(getattr(fa.cache, "_tiles", [None, None, None])[2]))
        finally:
            F_.set_skip_masked_tiles(prev)
    out["speedup_fwd_bwd"] = (out["dense_fwd_ms"] + out["dense_bwd_ms"]) / (out["skip_fwd_ms"] + out["skip_bwd_ms"])
    return out


def reference_triton(dev):
    """The reference project's own Triton kernels on this GPU next to this library, at
    benchmark configurations 1-4 (forward + backward).  Runs only when the unmodified
    reference is importable from baseline/_ref; its entries are called with
    kernel_cache=None.  Times are GPU time of one forward + backward (CUDA-graph replays, so
    neither side's host launch path is in them); "eager" marks a side that could not be
    captured and was timed as back-to-back eager calls instead."""
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "rgd_triton").is_dir():
        return {"unavailable": "reference project is not installed under baseline/_ref"}
    sys.path.insert(0, str(ref_root))
    try:
        from rgd_triton.triton.flash_attn.flash_attn_triton_cached import flash_attn_func as r_attn
        from rgd_triton.triton.normalization.rmsnorm_cached import triton_rms_func_fn as r_rms
        from rgd_triton.triton.rope.fused_ln_rope_cached import triton_fused_ln_rope_fn as r_lnrope
    except Exception as e:
        return {"unavailable": f"reference kernels cannot be imported: {e!r}"[:200]}
    finally:
        sys.path.remove(str(ref_root))
    from rgd_triton_b200 import functional as F_
    g = torch.Generator().manual_seed(6)
    rn = lambda *s, dtype=torch.bfloat16: torch.randn(*s, generator=g).to(dtype).to(dev)
    rows = []

    def both(name, ref_step, our_step):
        row = {"config": name}
        for key, step in (("reference", ref_step), ("here", our_step)):
            try:
                ms, how = graph_time_ms(step)
                row[key + "_ms"], row[key + "_timing"] = ms, how
            except Exception as e:
                row[key + "_error"] = repr(e)[:160]
            torch.cuda.synchronize()
        if "reference_ms" in row and "here_ms" in row:
            row["speedup"] = row["reference_ms"] / row["here_ms"]
        rows.append(row)

    # config 1
    x, dy = rn(4, 256, 1024, dtype=torch.float32).requires_grad_(True), rn(4, 256, 1024, dtype=torch.float32)
    w = (1 + 0.02 * torch.randn(1024, generator=g)).to(dev).requires_grad_(True)
    both("config1 FusedRMSNorm f32 [4,256,1024]",
         lambda: torch.autograd.grad(r_rms(x, w, 1e-6), (x, w), dy),
         lambda: torch.autograd.grad(F_.triton_rms_func_fn(x, w, 1e-6), (x, w), dy))
    del x, dy, w
    # config 2
    q, k = rn(8, 4096, 16, 128).requires_grad_(True), rn(8, 4096, 16, 128).requires_grad_(True)
    gq, gk = rn(8, 4096, 16, 128), rn(8, 4096, 16, 128)
    pos = rotary_table(4097, 64, torch.bfloat16).to(dev)
    both("config2 FusedLNRoPE bf16 q,k [8,4096,16,128]",
         lambda: torch.autograd.grad(r_lnrope(q, k, pos, (4096, 4096), False, 1e-5), (q, k), (gq, gk)),
         lambda: torch.autograd.grad(F_.triton_fused_ln_rope_fn(q, k, pos, (4096, 4096), False, 1e-5), (q, k), (gq, gk)))
    del q, k, gq, gk
    # config 3
    q, k, v = (rn(4, 4096, 16, 128).requires_grad_(True) for _ in range(3))
    do = rn(4, 4096, 16, 128)
    both("config3 FlashAttention bf16 [4,4096,16,128]",
         lambda: torch.autograd.grad(r_attn(q, k, v), (q, k, v), do),
         lambda: torch.autograd.grad(F_.flash_attn_func(q, k, v), (q, k, v), do))
    del q, k, v, do
    # config 4 (full bias)
    q, k, v = (rn(2, 4096, 24, 64, dtype=torch.float16).requires_grad_(True) for _ in range(3))
    do = rn(2, 4096, 24, 64, dtype=torch.float16)
    gd = torch.Generator(device=dev).manual_seed(4)
    bias = torch.randn(2, 24, 4096, 4096, generator=gd, device=dev, dtype=torch.float32).to(torch.float16)
    both("config4 FlashAttention fp16 [2,4096,24,64] + bias [2,24,4096,4096]",
         lambda: torch.autograd.grad(r_attn(q, k, v, bias), (q, k, v), do),
         lambda: torch.autograd.grad(F_.flash_attn_func(q, k, v, bias), (q, k, v), do))
    del q, k, v, do, bias
    torch.cuda.empty_cache()
    for name in [n for n in sys.modules if n == "rgd_triton" or n.startswith("rgd_triton.")]:
        del sys.modules[name]
    return {"rows": rows, "note": "forward + backward GPU time per call; reference = rgd_triton *_fn(kernel_cache=None)"}


def reference_triton_isolated():
    """reference_triton() in a process of its own, so that nothing the reference's kernels or
    their compiler do (a failed graph capture, a compile error) can take the benchmark down."""
    if not (ROOT / "baseline" / "_ref" / "rgd_triton").is_dir():
        return {"unavailable": "reference project is not installed under baseline/_ref"}
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_PORT")}
    try:
        res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--reference-triton-only"], env=env,
                             capture_output=True, text=True, timeout=900)
    except subprocess.TimeoutExpired:
        return {"unavailable": "the comparison run did not finish within 900 s"}
    for ln in reversed(res.stdout.splitlines()):
        if ln.startswith("{"):
            try:
                return json.loads(ln)
            except ValueError:
                break
    return {"unavailable": f"the comparison run exited with code {res.returncode}: {res.stderr[-300:]}"}


def run_shard(dev, attn, q, k, v, do, world, rank):
    """Forward + backward of the attention workload on this rank's share of its batch x heads
    units (a contiguous range of b * H + h; heads as strided views with the channel dimension
    contiguous).  Returns o, dq, dk, dv of the share, unit-major [units, T, D], padded to the
    largest share so that every rank contributes equally sized buffers to the gather."""
    B, T, H, D = q.shape
    units = shard_units(B * H, world, rank)
    n_max = max(len(shard_units(B * H, world, r)) for r in range(world))
    outs = [torch.zeros(n_max, T, D, dtype=q.dtype, device=dev) for _ in range(4)]
    u = units.start
    while u < units.stop:                      # one call per batch element this range touches
        b, h0 = divmod(u, H)
        h1 = min(H, h0 + (units.stop - u))
        qs, ks, vs = (t[b:b + 1, :, h0:h1].detach().requires_grad_(True) for t in (q, k, v))
        o = attn(qs, ks, vs)
        grads = torch.autograd.grad(o, (qs, ks, vs), do[b:b + 1, :, h0:h1])
        for dst, src in zip(outs, (o.detach(), *grads)):
            dst[u - units.start:u - units.start + (h1 - h0)] = src[0].permute(1, 0, 2)
        u += h1 - h0
    return outs


def compare_gathered(buckets, full, world):
    """buckets[t][r]: tensor t (o, dq, dk, dv) of rank r as run_shard returned it; full: the same
    four tensors of the unsharded run, [B, T, H, D].  Bit-equality is the rule."""
    B, T, H, D = full[0].shape
    ok, worst = True, 0.0
    for per_rank, ref_t in zip(buckets, full):
        got = torch.cat([bk[:len(shard_units(B * H, world, r))] for r, bk in enumerate(per_rank)])
        want = ref_t.detach().permute(0, 2, 1, 3).reshape(B * H, T, D)
        if not torch.equal(got, want):
            ok = False
            worst = max(worst, (got.float() - want.float()).abs().max().item())
    return {"ok": ok, "units": B * H, "ranks": world, "compared": ["o", "dq", "dk", "dv"],
            "rule": "bit-equal to the unsharded result", "max_abs_diff": worst}


def verify_sharded(dev, attn, q, k, v, do, full, world, rank, dist):
    """Shard the workload over ranks, gather every rank's results (the only collective) and
    compare them with the unsharded result computed on this rank's own GPU."""
    mine = run_shard(dev, attn, q, k, v, do, world, rank)
    buckets = []
    for t in mine:
        if world > 1:
            bucket = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(bucket, t)
        else:
            bucket = [t]
        buckets.append(bucket)
    res = compare_gathered(buckets, full, world)
    res["units_this_rank"] = len(shard_units(q.shape[0] * q.shape[2], world, rank))
    return res


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
        # FusedRMSNorm2 at the fifth configuration's shapes x4 in batch (226 MB of inputs)
        m = ops.FusedRMSNorm2((3072, 3072), dtype=bf).to(dev)
        a, b = rn(8, 512, 3072), rn(8, 4096, 3072)
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
    ap.add_argument("--attn-only", action="store_true", help="only the headline attention step (quick A/B runs)")
    ap.add_argument("--no-config4", action="store_true", help="skip the dense-bias attention measurement")
    ap.add_argument("--no-config5", action="store_true", help="skip the MMDiT block measurement")
    ap.add_argument("--no-reference-triton", action="store_true",
                    help="skip the reference's Triton kernels even when baseline/_ref is present")
    ap.add_argument("--reference-triton-only", action="store_true",
                    help="only the comparison with the reference's Triton kernels (one JSON line)")
    ap.add_argument("--sustained-seconds", type=float, default=2.0,
                    help="length of the sustained-clock loop of the headline step (0 = skip)")
    ap.add_argument("--profile", default=None, choices=["attn", "attn64", "lnrope", "rms2"],
                    help="run a small fixed case of one operator (three fwd+bwd passes) for ncu captures")
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

    def gather_objects(obj):
        if world == 1:
            return [obj]
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    def waits_ok(what):
        """The bounded device-side waits of the tensor-memory kernels must all have completed:
        a wait that gave up would have left wrong results and a meaningless time."""
        code = lib.rgd_device_status()
        if code != 0:
            raise RuntimeError(f"{what}: {_lib.status_string(code)} (status {code})")

    hbm_peak, tf_burst, tf_sust, peak_src = peaks()
    if args.profile:
        return profile_case(args.profile, dev)
    if args.reference_triton_only:
        print(json.dumps(reference_triton(dev)), flush=True)
        return 0
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
    # One sampler for the whole node, owned by local rank 0 (a poller per rank costs host time
    # on every rank).  It starts before the warm-up (same load as the timed steps), so that
    # short timed regions still get samples under load.
    with ClockSampler(enabled=(local == 0), period_ms=20 if world == 1 else 50) as clk:
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
    waits_ok("attention, configuration 3")
    my_ms = start.elapsed_time(end) / args.steps
    ms_step = max_over_ranks(my_ms * args.steps) / args.steps
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in evs)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in evs)
    f_fwd, f_bwd = attn_flops(**cfg)
    tflops = world * (f_fwd + f_bwd) / (ms_step * 1e-3) / 1e12
    node_clocks = [clk.summary(i) for i in range(world)] if local == 0 else None
    dom = ("attention backward (delta + dK/dV + dQ kernels)", f_bwd, bwd_ms) if bwd_ms >= fwd_ms else \
          ("attention forward kernel", f_fwd, fwd_ms)
    achieved = dom[1] / (dom[2] * 1e-3) / 1e12
    traffic = None
    tt = dram_traffic_table()
    if tt is not None:
        try:
            per_unit = sum(tt["attention_backward_config3"]["bytes_per_batch_head"].values())
            traffic = per_unit * cfg["B"] * cfg["H"]
        except (KeyError, TypeError):
            traffic = None
    roofline = {"bound": "tensor", "kernel": dom[0], "achieved": achieved, "peak": tf_burst, "unit": "TFLOP/s",
                "frac": achieved / tf_burst, "peak_source": peak_src, "traffic": traffic,
                "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
                "fwd_tflops": f_fwd / (fwd_ms * 1e-3) / 1e12, "bwd_tflops": f_bwd / (bwd_ms * 1e-3) / 1e12,
                "step_frac_of_burst_peak": (f_fwd + f_bwd) / (my_ms * 1e-3) / 1e12 / tf_burst}
    per_rank = gather_objects({"rank": rank, "gpu": local, "ms_per_step": my_ms, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms})

    # ---------------- the same step, sustained ----------------
    sustained = None
    if args.sustained_seconds > 0 and not args.attn_only:
        n_sus = max(50, int(args.sustained_seconds * 1e3 / max(my_ms, 0.1)))
        with ClockSampler(enabled=(local == 0), period_ms=50) as clk2:
            barrier()
            s1, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s1.record()
            for _ in range(n_sus):
                attn_step(q, k, v, do)
            e1.record()
            barrier()
        waits_ok("attention, sustained loop")
        sus_my = s1.elapsed_time(e1) / n_sus
        sus_ms = max_over_ranks(sus_my * n_sus) / n_sus
        sus_clocks = [clk2.summary(i) for i in range(world)] if local == 0 else None
        sus_tf = (f_fwd + f_bwd) / (sus_ms * 1e-3) / 1e12
        sustained = {"steps": n_sus, "seconds": sus_ms * n_sus * 1e-3, "ms_per_step": sus_ms,
                     "tflops_per_gpu": sus_tf, "peak": tf_sust, "frac_of_sustained_peak": sus_tf / tf_sust,
                     "frac_of_burst_peak": sus_tf / tf_burst, "clocks": sus_clocks[0] if sus_clocks else None}
        if sus_clocks and sus_clocks[0].get("sm_mhz"):
            sustained["ms_x_median_mhz"] = sus_ms * sus_clocks[0]["sm_mhz"]
        sus_per_rank = gather_objects({"rank": rank, "ms_per_step": sus_my})
        sustained["per_rank_ms"] = [r["ms_per_step"] for r in sus_per_rank]
        if sus_clocks:
            sustained["per_gpu_clocks"] = sus_clocks

    # ---------------- sharded run, gathered and compared with the unsharded result ----------------
    o_full, g_full = attn_step(q, k, v, do)
    verify = verify_sharded(dev, attn, q.detach(), k.detach(), v.detach(), do, (o_full, *g_full), world, rank, dist)
    verify_all = gather_objects(verify["ok"])
    verify["ok"] = bool(all(verify_all))
    del o_full, g_full
    waits_ok("sharded verification run")

    if args.attn_only:
        if rank == 0:
            print(json.dumps({"value": tflops, "ms_per_step": ms_step, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
                              "verify": verify, "clocks": node_clocks[0] if node_clocks else None}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return 0

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
        main_s = torch.cuda.current_stream()
        for sl in slots:
            sl["stream"].wait_stream(main_s)
        for i in range(n):
            e2e_step(i)
        for sl in slots:
            main_s.wait_stream(sl["stream"])

    e2e_steps = max(4, min(args.steps, 10))
    e2e_run(2)
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    e2e_run(e2e_steps)
    e2.record()
    barrier()
    e2e_my = s2.elapsed_time(e2) / e2e_steps
    e2e_ms = max_over_ranks(e2e_my * e2e_steps) / e2e_steps
    nbytes = hq.numel() * hq.element_size()
    e2e_ranks = gather_objects({"rank": rank, "ms_per_step": e2e_my,
                                "h2d_gbs": 4 * nbytes / (e2e_my * 1e-3) / 1e9,
                                "d2h_gbs": 4 * nbytes / (e2e_my * 1e-3) / 1e9})
    e2e = {"value": world * (f_fwd + f_bwd) / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": 4 * nbytes, "d2h_bytes_per_step": 4 * nbytes, "steps": e2e_steps,
           "overlap": "steps rotate over 3 CUDA streams: D2H of step i overlaps H2D + kernels of the next steps",
           "per_rank": e2e_ranks,
           "node_h2d_gbs": sum(r["h2d_gbs"] for r in e2e_ranks), "node_d2h_gbs": sum(r["d2h_gbs"] for r in e2e_ranks),
           "bound": "pinned-host copies over PCIe: kernels take ms_per_step of the device-timed value, the rest "
                    "of the step is H2D + D2H (all ranks share the host's PCIe / memory path)"}
    waits_ok("end-to-end loop")
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

    # ---------------- dense-bias attention (config 4), the MMDiT block (config 5) ----------------
    cfg4 = None
    if not args.no_config4:
        cfg4 = [config4(dev, attn, args.steps, False, hbm_peak, tf_burst),
                config4(dev, attn, args.steps, True, hbm_peak, tf_burst)]
        torch.cuda.empty_cache()
        waits_ok("attention, configuration 4")
        if rank == 0:
            cfg4.append(block_sparse_case(dev, args.steps))
            torch.cuda.empty_cache()
            waits_ok("attention, block-sparse bias")
    cfg5 = None
    if not args.no_config5:
        cfg5 = config5_block(dev, args.steps, hbm_peak, tf_burst)
        torch.cuda.empty_cache()
        waits_ok("MMDiT block, configuration 5")

    host_us = host_us_per_call(dev) if rank == 0 else None
    ref_tri = None
    if rank == 0 and world == 1 and not args.no_reference_triton:
        torch.cuda.empty_cache()
        ref_tri = reference_triton_isolated()
    base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        base = cpu_baseline(cfg)

    if rank == 0:
        for r, c in zip(per_rank, node_clocks or []):
            r["clocks"] = c
        slowest = max(per_rank, key=lambda r: r["ms_per_step"])
        line = {
            "metric": METRIC, "value": tflops, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "config3 FlashAttention fwd+bwd bf16 q/k/v [4,4096,16,128] no bias non-causal, "
                                   "per GPU", "l2": "inputs+outputs 256 MiB per step, larger than the 126 MB L2",
                       "parallelism": f"replicas x{world} (batch x heads shard, no collective)"},
            "roofline": roofline, "sustained": sustained, "norm_rope": norm_rope, "e2e": e2e,
            "gpu_launches": int(launches), "clocks": (node_clocks or [None])[0],
            "per_rank": per_rank, "slowest_rank": {"rank": slowest["rank"], "ms_per_step": slowest["ms_per_step"],
                                                   "clocks": slowest.get("clocks")},
            "verify": verify, "host_us_per_call": host_us,
        }
        if cfg4 is not None:
            line["config4"] = cfg4
        if cfg5 is not None:
            line["config5"] = cfg5
        if ref_tri is not None:
            line["reference_triton"] = ref_tri
        if base is not None:
            line["cpu_baseline"] = base
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
