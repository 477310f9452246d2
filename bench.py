#!/usr/bin/env python
"""Benchmark of the batched complex training step (forward + Wirtinger backward + SGD update).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload "mixer_dp4096": the token-mixing stack (8 x [FourierTrans(1024) -> Hadamard ->
CGelu -> Linear(1024->1024) -> Residual] -> Linear(1024->10) -> CrossEntropy) at GLOBAL batch 4096,
split evenly over the N ranks (strong scaling), weight gradients all-reduced over NCCL before the
update.  One step = one pass over one synthetic batch.  Prints ONE JSON line on rank 0.

`value`  : samples/s with the batch already resident in HBM.
`e2e`    : samples/s through the public API with pinned HOST buffers: H2D of the batch and D2H of
           the per-sample losses inside the timed region.
`--impl reference`: the reference's own CPU implementation (oracle/_ref, built from the reference
           sources) on the host cores, on a bounded sample of the same workload.

Timing: `--steps K` steps between a barrier + synchronize on both sides, CUDA events on the stream the
step is launched on, max over ranks; that K-step measurement is repeated `--repeats` times (a fixed
count, so that every N runs the same number of updates) and the MEDIAN is reported, with nvidia-smi
clocks sampled over the whole timed region.  `e2e` is host wall-clock time around the same number of
pipelined steps including the final wait for the losses.  `loss_global` is the mean loss of the WHOLE
batch (summed over the ranks) after the last timed resident step: the same number at every N up to
fp32 reassociation.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from cnet_b200 import configs  # noqa: E402

WORKLOADS = {
    # name: (builder, kwargs, global batch, input kind)
    "mixer_dp4096": (configs.build_mixer, dict(n=1024, blocks=8, m=10), 4096, "normal"),
    # config 2: standalone complex Linear 4096 -> 4096 at batch 4096: forward + dX* + dW* (no net around it)
    "linear_4096": (None, dict(n_in=4096, n_out=4096), 4096, "fanin"),
    "mixer_b512": (configs.build_mixer, dict(n=1024, blocks=8, m=10), 512, "normal"),
    "classifier_b64": (configs.build_classifier, dict(n=784, m=10), 64, "image"),
    "embed_lm_b1024": (configs.build_embed_lm, dict(tokens=64, vocab=8192, dim=256, hidden=2048), 1024, None),
}
LR = 0.01


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


def _gemm_flops(spec_kw, batch, name):
    """Algorithmic real flops of the complex GEMMs of one step: 8*M*N*K each."""
    if name.startswith("mixer"):
        n, blocks, m = spec_kw["n"], spec_kw["blocks"], spec_kw["m"]
        return blocks * 3 * 8 * batch * n * n + 3 * 8 * batch * n * m
    if name.startswith("classifier"):
        return 3 * 8 * batch * spec_kw["n"] * spec_kw["m"]
    d = spec_kw["tokens"] * spec_kw["dim"]
    return 3 * 8 * batch * (d * spec_kw["hidden"] + spec_kw["hidden"] * spec_kw["vocab"])


class _Clocks:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index, interval_ms=100):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.Q,
                                       "--format=csv,noheader,nounits", "-lms", str(interval_ms)],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.p is None:
            return out
        time.sleep(0.15)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        rows = [r.split(", ") for r in open(self.f.name).read().strip().splitlines() if r.count(",") >= 8]
        os.unlink(self.f.name)
        if not rows:
            return out
        sm = sorted(float(r[1]) for r in rows)
        out["sm_mhz"] = sm[len(sm) // 2]
        out["sm_max_mhz"] = float(rows[0][2])
        out["samples"] = len(rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for k, nme in enumerate(names):
            if any(r[5 + k].strip() == "Active" for r in rows):
                out["reasons"].append(nme)
        return out


def run_reference(args):
    """The reference's own CPU path on the host cores, on a bounded sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ref
    builder, kw, gbatch, kind = WORKLOADS[args.workload]
    if builder is None:
        builder = configs.build_linear
    if not ref.available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libcnet_ref.so is not built"}))
        return
    # torchrun exports OMP_NUM_THREADS=1 to its ranks: use every host core, as at N = 1
    ref.set_threads(os.cpu_count() or 1)
    net = ref.RefNet()
    spec = builder(net, **kw)
    for uid, (re, im) in configs.init_weights(spec, 0).items():
        net.set_values(uid, re, im)
    cores = ref.max_threads()
    # size the per-step sample so K+W steps end within a few minutes
    data, labels = configs.make_batch(spec, 2, 0, 0, kind)
    t0 = time.perf_counter()
    _run_ref(net, spec, data, labels)
    per_sample = (time.perf_counter() - t0) / 2
    budget = 120.0 / max(1, args.steps + args.warmup)
    sample = int(max(1, min(gbatch, budget / max(per_sample, 1e-6))))
    times = []
    for s in range(args.warmup + args.steps):
        data, labels = configs.make_batch(spec, sample, 0, s, kind)
        t0 = time.perf_counter()
        _run_ref(net, spec, data, labels)
        net.update(LR, sample)
        if s >= args.warmup:
            times.append(time.perf_counter() - t0)
    total = sum(times)
    value = sample * len(times) / total
    line = {
        "impl": "reference", "metric": "train samples/sec (fwd+bwd+update)", "value": value, "unit": "samples/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / len(times) * (gbatch / sample), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "global_batch": gbatch, **kw},
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": cores, "kind": "reference",
                         "sample": "%d of %d samples per step, per-sample loop of the reference trainer "
                                   "(setInput, forward, loss, backward(label)) + update; ms_per_step scaled to the full batch"
                                   % (sample, gbatch)},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def _run_ref(net, spec, data, labels):
    if spec.tokens:
        net.run_batch(spec.main, tokens=data, labels=labels, record=False)
    else:
        net.run_batch(spec.main, x=data, labels=labels, record=False)


def cpu_baseline(workload, seconds=15.0):
    from oracle import ref
    if not ref.available():
        return None
    builder, kw, gbatch, kind = WORKLOADS[workload]
    if builder is None:
        builder = configs.build_linear      # config 2 as a net: the three products + a loss on top
    ref.set_threads(os.cpu_count() or 1)
    net = ref.RefNet()
    spec = builder(net, **kw)
    for uid, (re, im) in configs.init_weights(spec, 0).items():
        net.set_values(uid, re, im)
    data, labels = configs.make_batch(spec, 2, 0, 0, kind)
    t0 = time.perf_counter()
    _run_ref(net, spec, data, labels)
    per = (time.perf_counter() - t0) / 2
    k = int(max(2, min(gbatch, seconds / max(per, 1e-6))))
    data, labels = configs.make_batch(spec, k, 0, 1, kind)
    t0 = time.perf_counter()
    _run_ref(net, spec, data, labels)
    net.update(LR, k)
    dt = time.perf_counter() - t0
    return {"value": k / dt, "unit": "samples/s", "cores": ref.max_threads(), "kind": "reference",
            "sample": "%d of %d samples of the workload through the unmodified reference CPU path "
                      "(oracle/_ref), %.1f s" % (k, gbatch, dt)}


# DRAM traffic of one launch of the dominant kernel from the ncu capture summarised under profiles/
# (dram__bytes_read.sum + dram__bytes_write.sum), keyed by (M, N, K); None where not captured.
NCU_TRAFFIC_BYTES = {(4096, 1024, 1024): 126.3e6}

_TF32 = {}


def _tf32_peak(torch, gpu_index):
    """Dense TF32 throughput of this GPU, measured the way MEASURED_PEAKS.json's bf16 figure was: torch.matmul
    (cuBLAS, fp32 operands with TF32 allowed) at 8192^3, best of 10 launches (burst) and back to back for ~2 s
    (sustained), clocks sampled during the sustained loop.  A measuring stick only: no kernel of the path uses it."""
    if _TF32:
        return _TF32
    n = 8192
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn(n, n, device="cuda")
        b = torch.randn(n, n, device="cuda")
        c = torch.empty(n, n, device="cuda")
        for _ in range(3):
            torch.matmul(a, b, out=c)
        best = 1e30
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b, out=c)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        clocks = _Clocks(gpu_index, interval_ms=50)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        count = 0
        t0 = time.perf_counter()
        e0.record()
        while time.perf_counter() - t0 < 2.0:
            for _ in range(25):
                torch.matmul(a, b, out=c)
            count += 25
            torch.cuda.synchronize()
        e1.record()
        torch.cuda.synchronize()
        clk = clocks.stop()
        flops = 2.0 * n ** 3
        _TF32.update({"tf32_tflops": flops / (best * 1e-3) / 1e12,
                      "tf32_tflops_sustained": flops * count / (e0.elapsed_time(e1) * 1e-3) / 1e12,
                      "sm_mhz_sustained": clk.get("sm_mhz"), "reasons_sustained": clk.get("reasons"),
                      "how": "torch.matmul fp32 with TF32 allowed, 8192^3: best of 10 (burst), back to back for 2 s (sustained)"})
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    del a, b, c
    return _TF32


def _time_launches(torch, fn, reps=20, clocks_for=None):
    """Average device time of fn() in ms: CUDA events on the launching stream, L2 flushed in between.
    clocks_for = GPU index: also the median SM clock sampled while the loop runs."""
    flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda")
    clean = torch.zeros(40 << 20, dtype=torch.float32, device="cuda")
    for _ in range(3):
        fn()
    sampler = _Clocks(clocks_for, interval_ms=20) if clocks_for is not None else None
    tot = 0.0
    for _ in range(reps):
        flush.zero_()          # evict the working set ...
        clean.sum()            # ... then leave L2 full of clean lines, so no write-back lands in the timed launch
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        tot += e0.elapsed_time(e1)
    if sampler is not None:
        return tot / reps, sampler.stop().get("sm_mhz")
    return tot / reps


L2_BYTES = 126 << 20


def _nsets(nbytes, lo=3, hi=48):
    """How many disjoint operand sets a kernel that touches nbytes per launch must rotate over so that a set
    has left L2 (3 x L2 of other traffic) before it is used again."""
    return int(min(hi, max(lo, -(-3 * L2_BYTES // max(1, int(nbytes))))))


def _time_stream(torch, fns, launches=60, clocks_for=None):
    """Average device time per launch, in ms, of the launches fns[0], fns[1], ... issued back to back on the
    stream, round robin, between two CUDA events: each fns[k] works on operands of its own (together larger
    than L2, so nothing is served from cache), as consecutive kernels of a step do.  A spin kernel queued first
    keeps the GPU busy until the host has enqueued all of it, so host launch time is not in the figure."""
    for _ in range(max(1, -(-3 // len(fns)))):
        for f in fns:
            f()
    rounds = max(1, launches // len(fns))
    torch.cuda.synchronize()
    sampler = _Clocks(clocks_for, interval_ms=20) if clocks_for is not None else None
    if hasattr(torch.cuda, "_sleep"):
        torch.cuda._sleep(int(4e4 * rounds * len(fns)))       # ~20 us of head start per launch to come
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(rounds):
        for f in fns:
            f()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / (rounds * len(fns))
    if sampler is not None:
        return ms, sampler.stop().get("sm_mhz")
    return ms


def _hbm_entry(torch, peaks, name, fns, nbytes):
    """One HBM-bound kernel: in-stream average over rotating operand sets (the figure the fraction uses) and a
    single launch between two events after an L2 flush (which adds the launch ramp and the events' own cost:
    a kernel that does nothing measures ~5-8 us that way)."""
    d = _time_stream(torch, fns)
    single = _time_launches(torch, fns[0], reps=10)
    gbs = nbytes / (d * 1e-3) / 1e9
    return {"kernel": name, "GB/s": round(gbs, 1), "frac": round(gbs / peaks["hbm"], 3), "ms": round(d, 4),
            "ms_single": round(single, 4), "frac_single": round(nbytes / (single * 1e-3) / 1e9 / peaks["hbm"], 3),
            "operand_sets": len(fns)}


def _tensor_roof(torch, peaks, dur, mhz, B, n_out, n_in, gpu_index):
    """Roofline of the split complex GEMM.  Every real product of the 8*M*N*K algorithmic flops passes the tensor
    cores three times: hi.hi on the TF32 pipe and the two cross terms on the BF16 pipe, so the time per
    algorithmic flop at peak is 1/TF32 + 2/BF16 (TF32 measured in this run, BF16 from the peaks file).
    frac_3xtf32 = the same launch against the all-TF32 form's roofline (TF32 / 3), for comparison."""
    flops = 8.0 * B * n_in * n_out
    achieved = flops / (dur * 1e-3) / 1e12
    tf = _tf32_peak(torch, gpu_index)
    peak = 1.0 / (1.0 / tf["tf32_tflops"] + 2.0 / peaks["bf16"])
    sustained = 1.0 / (1.0 / tf["tf32_tflops_sustained"] + 2.0 / (peaks["bf16_sustained"] or peaks["bf16"]))
    derived = 1.0 / (2.0 / peaks["bf16"] + 2.0 / peaks["bf16"])      # what the peaks file alone gives: TF32 = bf16 / 2
    return {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
            "frac_derived": achieved / derived, "peak_derived": derived,
            "frac_sustained": achieved / sustained,
            "frac_3xtf32": achieved / (tf["tf32_tflops"] / 3.0), "peak_3xtf32": tf["tf32_tflops"] / 3.0,
            "traffic": NCU_TRAFFIC_BYTES.get((B, n_out, n_in)),
            "kernel": "cgemm_tc_k (tcgen05: TF32 hi.hi + BF16 cross terms)",
            "shape": [B, n_out, n_in], "ms_per_launch": dur, "sm_mhz_during": mhz,
            "ms_x_mhz": (dur * mhz) if mhz else None, "tf32_peak": tf,
            "peak_note": "1 / (1/TF32 + 2/BF16): dense TF32 measured in this run (cuBLAS 8192^3 burst %.1f TFLOP/s, sustained "
                         "%.1f at %s MHz), BF16 burst %.1f of %s; frac_derived = with TF32 taken as BF16 / 2; "
                         "frac_3xtf32 = against TF32 / 3"
                         % (tf["tf32_tflops"], tf["tf32_tflops_sustained"], tf["sm_mhz_sustained"], peaks["bf16"],
                            peaks["source"])}


def _roofline(workload, kw, B, gbatch, step_ms, device, hbm_kernels=True):
    """The dominant kernel of the step (the complex GEMM of the Linear layers, or the skinny head kernel
    when the net has no square Linear) at this rank's shape, plus the HBM-bound kernels of one block."""
    import torch
    from cnet_b200.ops import Context
    peaks = _peaks()
    ctx = Context(device=device, arena_bytes=2 << 30)
    n = kw.get("n", 1024)
    if workload.startswith("embed"):
        n_in, n_out = kw["tokens"] * kw["dim"], kw["hidden"]
    elif workload.startswith("classifier"):
        n_in, n_out = kw["n"], kw["m"]
    else:
        n_in, n_out = n, n
    x = tuple(torch.randn(B, n_in, device="cuda") for _ in range(2))
    w = tuple(torch.randn(n_out, n_in, device="cuda") * n_in ** -0.5 for _ in range(2))
    hbm = []
    if ctx.lib.cnb_linear_split_ok(B, n_in, n_out):
        # operands pre-split; every launch of the timed run has activations and output of its own (the weights
        # are shared, as a layer's are), so no launch finds its operands in L2
        SG = _nsets(24.0 * B * n_in + 8.0 * B * n_out, hi=12)
        ws = ctx.split(w)
        xs = [ctx.split(tuple(torch.randn(B, n_in, device="cuda") for _ in range(2))) for _ in range(SG)]
        ys = [ctx._new(B, n_out) for _ in range(SG)]
        fns = [lambda k=k: ctx.linear_fwd_split(xs[k], ws, B, n_in, n_out, out=ys[k]) for k in range(SG)]
        dur, mhz = _time_stream(torch, fns, launches=200, clocks_for=device)
        roof = _tensor_roof(torch, peaks, dur, mhz, B, n_out, n_in, device)
        roof["ms_single"] = _time_launches(torch, fns[0], reps=20)
        roof["timing"] = ("ms_per_launch: average of 200 launches back to back on the stream over %d operand sets (larger than L2 "
                          "together); ms_single: one launch between two events after an L2 flush" % SG)
        del xs, ys
    else:
        dur = _time_launches(torch, lambda: ctx.linear_fwd(x, w))
        nbytes = 8.0 * B * n_in + 8.0 * n_in * n_out + 8.0 * B * n_out
        achieved = nbytes / (dur * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                "frac": achieved / peaks["hbm"], "traffic": None, "kernel": "skinny_fwd_k (fp32)",
                "shape": [B, n_out, n_in], "ms_per_launch": dur, "peak_note": "copy bandwidth, of " + peaks["source"]}
    roof["step_gemm_tflops"] = _gemm_flops(kw, gbatch, workload) / (step_ms * 1e-3) / 1e12
    # HBM-bound kernels at the same activation shape: algorithmic bytes / time, against the measured copy bandwidth
    import ctypes as C
    L, H_, st = ctx.lib, ctx.h, ctx._stream()

    def P(t):
        return C.c_void_p(t.data_ptr())

    def pair(*shape, fill=None):
        t = ctx._new(*shape)
        if fill == "randn":
            for q in t:
                q.normal_()
        elif fill == "zero":
            for q in t:
                q.zero_()
        return t

    if hbm_kernels and workload.startswith("embed"):
        T, D, V, H = kw["tokens"], kw["dim"], kw["vocab"], kw["hidden"]
        table = tuple(torch.randn(V, D, device="cuda") * 0.02 for _ in range(2))
        dtable = pair(V, D, fill="zero")
        S = _nsets(16.0 * B * V)
        tok = [torch.randint(0, V, (B, T), device="cuda", dtype=torch.int32) for _ in range(S)]
        labels = torch.randint(0, V, (B,), device="cuda", dtype=torch.int32)
        ge = [pair(B, T * D, fill="randn") for _ in range(S)]          # embedding rows / their gradients
        z = [pair(B, V, fill="randn") for _ in range(S)]
        yv = [pair(B, V, fill="randn") for _ in range(S)]
        inv = torch.ones(B, device="cuda")
        loss = torch.empty(B, device="cuda")
        SA = _nsets(16.0 * B * H)
        a = [pair(B, H, fill="randn") for _ in range(SA)]
        ya = [pair(B, H, fill="randn") for _ in range(SA)]
        da = [pair(B, H) for _ in range(SA)]
        gz = [pair(B, V, fill="randn") for _ in range(S)]
        cases = [("embed_fwd_k (gather)",
                  [lambda k=k: L.cnb_embed_fwd(H_, P(table[0]), P(table[1]), P(tok[k]), P(ge[k][0]), P(ge[k][1]), B, T, D, V, st) for k in range(S)],
                  16.0 * B * T * D),
                 ("embed_bwd (scatter-add of dz* rows into the table)",
                  [lambda k=k: L.cnb_embed_bwd(H_, P(ge[k][0]), P(ge[k][1]), P(tok[k]), P(dtable[0]), P(dtable[1]), B, T, D, V, st) for k in range(S)],
                  16.0 * B * T * D),
                 ("softmax_fwd_k (L2 normalise)",
                  [lambda k=k: L.cnb_softmax_fwd(H_, P(z[k][0]), P(z[k][1]), P(yv[k][0]), P(yv[k][1]), P(inv), B, V, st) for k in range(S)],
                  16.0 * B * V),
                 ("softmax_bwd_k",
                  [lambda k=k: L.cnb_softmax_bwd(H_, P(gz[k][0]), P(gz[k][1]), P(z[k][0]), P(z[k][1]), P(inv), P(yv[k][0]), P(yv[k][1]), B, V, 0, st) for k in range(S)],
                  24.0 * B * V),
                 ("crossent_k (loss + dz* seed)",
                  [lambda k=k: L.cnb_crossent_fwd_bwd(H_, P(z[k][0]), P(z[k][1]), P(labels), P(loss), P(yv[k][0]), P(yv[k][1]), B, V, st) for k in range(S)],
                  16.0 * B * V),
                 ("gelu_fwd_k",
                  [lambda k=k: L.cnb_gelu_fwd(H_, P(a[k][0]), P(a[k][1]), P(ya[k][0]), P(ya[k][1]), C.c_size_t(B * H), st) for k in range(SA)],
                  16.0 * B * H),
                 ("gelu_bwd_k",
                  [lambda k=k: L.cnb_gelu_bwd(H_, P(ya[k][0]), P(ya[k][1]), P(a[k][0]), P(a[k][1]), P(da[k][0]), P(da[k][1]), C.c_size_t(B * H), 0, st) for k in range(SA)],
                  24.0 * B * H)]
        for name, fns, nbytes in cases:
            hbm.append(_hbm_entry(torch, peaks, name, fns, nbytes))
        # the second product of the net at its shape (K = hidden)
        x2 = tuple(torch.randn(B, H, device="cuda") for _ in range(2))
        w2 = tuple(torch.randn(V, H, device="cuda") * H ** -0.5 for _ in range(2))
        xs2, ws2 = ctx.split(x2), ctx.split(w2)
        d2 = _time_stream(torch, [lambda k=k: ctx.linear_fwd_split(xs2, ws2, B, H, V, out=yv[k]) for k in range(S)], launches=20)
        roof["second_gemm"] = {"shape": [B, V, H], "ms_per_launch": d2,
                               "frac": 8.0 * B * H * V / (d2 * 1e-3) / 1e12 / roof["peak"],
                               "frac_3xtf32": 8.0 * B * H * V / (d2 * 1e-3) / 1e12 / roof["peak_3xtf32"]}
    elif hbm_kernels:
        N = n_in
        S = _nsets(16.0 * B * N)
        u = [pair(B, N, fill="randn") for _ in range(S)]
        g = [pair(B, N, fill="randn") for _ in range(S)]
        a = [pair(B, N, fill="randn") for _ in range(S)]
        o = [pair(B, N, fill="zero") for _ in range(S)]
        h = tuple(torch.randn(N, device="cuda") for _ in range(2))
        dh = pair(N)
        fft_name = "fft1024_pipe_k<-1> (FourierTrans forward)" if N == 1024 else "FourierTrans forward (N = %d)" % N
        cases = [("hadamard_gelu_fwd_k",
                  [lambda k=k: L.cnb_hadamard_gelu_fwd(H_, P(u[k][0]), P(u[k][1]), P(h[0]), P(h[1]), P(a[k][0]), P(a[k][1]), P(o[k][0]), P(o[k][1]), B, N, st) for k in range(S)],
                  24.0 * B * N),
                 ("colreduce_stage1_k<1> (gelu'+hadamard bwd + dh* partials)",
                  [lambda k=k: L.cnb_hadamard_gelu_bwd(H_, P(g[k][0]), P(g[k][1]), P(a[k][0]), P(a[k][1]), P(u[k][0]), P(u[k][1]), P(h[0]), P(h[1]), P(o[k][0]), P(o[k][1]), 0, P(dh[0]), P(dh[1]), 0, B, N, st) for k in range(S)],
                  32.0 * B * N),
                 ("colreduce_stage1_k<1>, a = u o h recomputed (as in the step)",
                  [lambda k=k: L.cnb_hadamard_gelu_bwd(H_, P(g[k][0]), P(g[k][1]), None, None, P(u[k][0]), P(u[k][1]), P(h[0]), P(h[1]), P(o[k][0]), P(o[k][1]), 0, P(dh[0]), P(dh[1]), 0, B, N, st) for k in range(S)],
                  24.0 * B * N),
                 (fft_name,
                  [lambda k=k: L.cnb_dft_fwd(H_, P(u[k][0]), P(u[k][1]), P(o[k][0]), P(o[k][1]), B, N, st) for k in range(S)],
                  16.0 * B * N)]
        if L.cnb_dft_fused_ok(N):
            # the forms that run inside the step: forward with the Hadamard + CGelu + operand split tail (reads x; writes
            # u and four split planes), backward accumulating into the gradient (reads g, read-modify-writes dx)
            sp = [torch.empty(L.cnb_split_floats(B * N), dtype=torch.float32, device="cuda") for _ in range(S)]
            cases.append(("fft1024_pipe_k<-1> + Hadamard + CGelu + split tail (as in the step)" if N == 1024 else "FourierTrans forward + tail",
                          [lambda k=k: L.cnb_dft_hadamard_gelu_fwd(H_, P(u[k][0]), P(u[k][1]), P(h[0]), P(h[1]), P(o[k][0]), P(o[k][1]), None, None, P(sp[k]), B, N, st) for k in range(S)],
                          32.0 * B * N))
            cases.append(("fft1024_pipe_k<+1> backward, reduce-add into the gradient (as in the step)" if N == 1024 else "FourierTrans backward + accumulate",
                          [lambda k=k: L.cnb_dft_bwd(H_, P(g[k][0]), P(g[k][1]), P(o[k][0]), P(o[k][1]), B, N, 1, st) for k in range(S)],
                          24.0 * B * N))
        n_w = 2 * n_in * n_out * max(1, kw.get("blocks", 1))       # the whole weight arena of the net
        SW = _nsets(16.0 * n_w, lo=2)
        wflat = [torch.randn(n_w, device="cuda") for _ in range(SW)]
        gflat = [torch.randn(n_w, device="cuda") for _ in range(SW)]
        cases.append(("sgd_k",
                      [lambda k=k: L.cnb_sgd_update(H_, P(wflat[k]), P(gflat[k]), C.c_size_t(n_w), C.c_float(1e-3), 1, st) for k in range(SW)],
                      16.0 * n_w))
        for name, fns, nbytes in cases:
            hbm.append(_hbm_entry(torch, peaks, name, fns, nbytes))
    roof["hbm_kernels"] = hbm
    roof["hbm_timing"] = ("ms / frac: average of 60 launches back to back on the stream, each on operands of its own (operand_sets "
                          "of them, together > 3 x L2); ms_single / frac_single: one launch between two events after an L2 flush")
    ctx.close()
    return roof


def _median(v):
    v = sorted(v)
    return v[len(v) // 2]


def run_linear(args, steps=None, repeats=None, quiet=False):
    """Config 2: one complex Linear layer, forward plus both backward products, through the C-ABI
    operators (operands split once per step, three tensor-core GEMMs).  Single GPU."""
    import torch
    from cnet_b200 import lib as cl
    from cnet_b200.ops import Context
    _, kw, B, _ = WORKLOADS["linear_4096"]
    steps = steps or args.steps
    repeats = repeats or args.repeats
    n_in, n_out = kw["n_in"], kw["n_out"]
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        raise SystemExit("linear_4096 is a single-GPU workload")
    torch.cuda.set_device(0)
    lib = cl.load()
    ctx = Context(device=0, arena_bytes=1 << 30)
    r = np.random.Generator(np.random.Philox(key=[0, 77]))
    s = n_in ** -0.5
    host = [torch.from_numpy((r.standard_normal((B, n_in)) * s).astype(np.float32)).pin_memory() for _ in range(2)]
    host += [torch.from_numpy(r.standard_normal((B, n_out)).astype(np.float32)).pin_memory() for _ in range(2)]
    w = tuple(torch.from_numpy((r.standard_normal((n_out, n_in)) * s).astype(np.float32)).cuda() for _ in range(2))
    x = tuple(torch.empty(B, n_in, device="cuda") for _ in range(2))
    g = tuple(torch.empty(B, n_out, device="cuda") for _ in range(2))
    y, dx, dw = ctx._new(B, n_out), ctx._new(B, n_in), ctx._new(n_out, n_in)
    host_y = torch.empty(B, dtype=torch.float32).pin_memory()

    def upload():
        for d, h in zip(x + g, host):
            d.copy_(h, non_blocking=True)

    def step():
        xs, ws, gs = ctx.split(x), ctx.split(w), ctx.split(g)
        ctx.linear_fwd_split(xs, ws, B, n_in, n_out, out=y)
        ctx.linear_bwd_x_split(gs, ws, B, n_in, n_out, out=dx)
        ctx.linear_bwd_w_split(gs, xs, B, n_in, n_out, out=dw)

    def e2e_step():
        upload()
        step()
        host_y.copy_(y[0][:, 0], non_blocking=False)

    def timed(fn, n):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    def walled(fn, n):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        torch.cuda.synchronize()
        return 1e3 * (time.perf_counter() - t0)

    upload()
    for _ in range(max(3, args.warmup)):
        step()
    clocks = _Clocks(0)
    l0 = lib.cnb_launch_count()
    ms = _median([timed(step, steps) for _ in range(repeats)])
    launches = (lib.cnb_launch_count() - l0) // repeats
    e2e_step()
    ms_e2e = _median([walled(e2e_step, steps) for _ in range(max(1, repeats // 3))])
    clk = clocks.stop()
    # parity spot check against float64 on a sample of outputs
    xs = (x[0][:8].double() + 1j * x[1][:8].double())
    want = xs @ (w[0].double() + 1j * w[1].double()).T
    err = float(((y[0][:8].double() + 1j * y[1][:8].double()) - want).norm() / want.norm())
    peaks = _peaks()
    per_step = ms / steps
    tflops = 3 * 8.0 * B * n_in * n_out / (per_step * 1e-3) / 1e12
    xs_, ws_ = ctx.split(x), ctx.split(w)
    dur, mhz = _time_launches(torch, lambda: ctx.linear_fwd_split(xs_, ws_, B, n_in, n_out, out=y), reps=40, clocks_for=0)
    roof = _tensor_roof(torch, peaks, dur, mhz, B, n_out, n_in, 0)
    roof["step_gemm_tflops"] = tflops
    line = {
        "metric": "train samples/sec (fwd+bwd+update)", "value": B / (per_step * 1e-3), "unit": "samples/s",
        "n_gpus": 1, "steps": steps, "warmup": max(3, args.warmup), "repeats": repeats, "ms_per_step": per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "linear_4096", "global_batch": B, **kw, "parallelism": "dp1",
                   "note": "forward + dX* + dW* of one layer, no update (config 2 measures the three products)",
                   "l2": "operands and outputs (> 1 GB per step) exceed the 126 MB L2"},
        "e2e": {"value": B / (ms_e2e / steps * 1e-3), "unit": "samples/s",
                "h2d_bytes_per_step": sum(h.numel() * 4 for h in host), "d2h_bytes_per_step": B * 4,
                "timed": "host wall clock, copies not pipelined"},
        "gpu_launches": int(launches), "clocks": clk, "roofline": roof,
        "forward_relerr_vs_f64": err,
    }
    ctx.close()
    del x, g, w, y, dx, dw
    torch.cuda.empty_cache()
    if not quiet:
        line["cpu_baseline"] = None if args.no_cpu_baseline else cpu_baseline("linear_4096")
        print(json.dumps(line))
    return line


def _measure(args, workload, steps, repeats, hbm_kernels=True):
    """Times one workload on this rank's GPU (all ranks call it together) and returns the JSON line's fields."""
    import gc
    import torch
    import torch.distributed as dist
    from cnet_b200 import lib as cl
    from cnet_b200.dp import DataParallelTrainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    builder, kw, gbatch, kind = WORKLOADS[workload]
    assert gbatch % world == 0
    B = gbatch // world
    lib = cl.load()

    trainer = DataParallelTrainer(builder, kw, global_batch=gbatch, lr=LR, device=local, seed=0)
    spec = trainer.spec
    # pinned host staging of this rank's shard (the e2e leg copies from here every step)
    data, labels = configs.make_batch(spec, gbatch, 0, 0, kind)
    lo, hi = rank * B, (rank + 1) * B
    if spec.tokens:
        host_in = (torch.from_numpy(data[lo:hi].copy()).pin_memory(),)
        h2d = host_in[0].numel() * 4
    else:
        host_in = (torch.from_numpy(data[0][lo:hi].copy()).pin_memory(),
                   torch.from_numpy(data[1][lo:hi].copy()).pin_memory())
        h2d = 2 * host_in[0].numel() * 4
    host_labels = torch.from_numpy(labels[lo:hi].copy()).pin_memory()
    h2d += host_labels.numel() * 4
    host_loss = torch.empty(B, dtype=torch.float32).pin_memory()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def timed(fn, n):
        """Exactly n steps between barrier + synchronize on both sides: CUDA events on the launching stream."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(trainer.stream)          # the stream every kernel of the step is launched on
        for _ in range(n):
            fn()
        e1.record(trainer.stream)
        barrier()
        return over_ranks(e0.elapsed_time(e1))

    def walled(fn, n, finish):
        """The same n steps by the host's clock, up to the arrival of the last step's losses."""
        barrier()
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        finish()
        torch.cuda.synchronize()
        ms = 1e3 * (time.perf_counter() - t0)
        barrier()
        return over_ranks(ms)

    trainer.upload(host_in, host_labels)
    trainer.step_resident()
    if not args.no_graph:
        trainer.capture()
    for _ in range(max(3, args.warmup)):
        trainer.step_resident()
    clocks = _Clocks(local) if rank == 0 else None
    l0 = lib.cnb_launch_count()
    all_ms = [timed(trainer.step_resident, steps) for _ in range(repeats)]
    ms = _median(all_ms)
    launches = (lib.cnb_launch_count() - l0) // repeats
    if trainer.kernels_per_step():
        launches = trainer.kernels_per_step() * steps      # replayed from the captured graph
    trainer.net.sync()
    # mean loss of the WHOLE batch under the weights all those updates produced (forward only)
    with torch.cuda.stream(trainer.stream):
        trainer.net.infer()
    trainer.net.sync()
    tot = torch.tensor([float(trainer.net.losses(B).astype(np.float64).sum())], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tot)
    loss_global = float(tot.item()) / gbatch
    updates = 1 + max(3, args.warmup) + repeats * steps

    # end to end: every step copies its batch from pinned host memory (on the copy stream, overlapping the
    # previous step) and brings its per-sample losses back to the host
    host_loss2 = torch.empty(B, dtype=torch.float32).pin_memory()
    bufs = [host_loss, host_loss2]
    it = [0]

    def e2e_step():
        trainer.step_pipelined(host_in, host_labels, bufs[it[0] & 1])
        it[0] += 1
    trainer.prefetch(host_in, host_labels)
    for _ in range(2):
        e2e_step()
    e2e_ms = _median([walled(e2e_step, steps, trainer.net.wait_losses) for _ in range(max(1, repeats // 3))])
    clk = clocks.stop() if clocks else None
    loss_mean = float(bufs[(it[0] - 1) & 1].mean())
    per_step = ms / steps
    out = {"value": gbatch / (per_step * 1e-3), "ms_per_step": per_step, "world": world, "B": B, "h2d": h2d,
           "e2e_value": gbatch / (e2e_ms / steps * 1e-3), "launches": int(launches), "clocks": clk,
           "loss_rank0": loss_mean, "loss_global": loss_global, "updates_before_loss_global": updates,
           "ms_all": [round(m / steps, 5) for m in all_ms], "kw": kw, "gbatch": gbatch}
    del trainer
    gc.collect()
    torch.cuda.empty_cache()
    out["roofline"] = _roofline(workload, kw, B, gbatch, per_step, local, hbm_kernels) if rank == 0 else None
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    m = _measure(args, args.workload, args.steps, args.repeats)
    others = {}
    if world == 1 and args.workload == "mixer_dp4096" and not args.no_workloads:
        # the other benchmark configurations, briefly (5 steps x 3), so that each has a witnessed number
        for name in ("classifier_b64", "linear_4096", "mixer_b512", "embed_lm_b1024"):
            try:
                if WORKLOADS[name][0] is None:
                    ln = run_linear(args, steps=5, repeats=3, quiet=True)
                    others[name] = {"value": ln["value"], "ms_per_step": ln["ms_per_step"], "e2e": ln["e2e"]["value"],
                                    "kernel": ln["roofline"]["kernel"], "roofline_frac": ln["roofline"]["frac"],
                                    "roofline_bound": "tensor", "gpu_launches_per_step": ln["gpu_launches"] // 5}
                    continue
                o = _measure(args, name, 5, 3, hbm_kernels=name.startswith("embed"))
                r = o["roofline"]
                others[name] = {"value": o["value"], "ms_per_step": o["ms_per_step"], "e2e": o["e2e_value"],
                                "kernel": r["kernel"], "roofline_frac": r["frac"], "roofline_bound": r["bound"],
                                "gpu_launches_per_step": o["launches"] // 5, "loss_global": o["loss_global"]}
                if r.get("hbm_kernels"):
                    others[name]["hbm_kernels"] = r["hbm_kernels"]
                if r.get("second_gemm"):
                    others[name]["second_gemm"] = r["second_gemm"]
            except Exception as e:           # a side workload must not take the headline line with it
                others[name] = {"error": "%s: %s" % (type(e).__name__, e)}
    if rank == 0:
        line = {
            "metric": "train samples/sec (fwd+bwd+update)", "value": m["value"], "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "repeats": args.repeats,
            "ms_per_step": m["ms_per_step"], "ms_per_step_all": m["ms_all"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": args.workload, "global_batch": m["gbatch"], "per_gpu_batch": m["B"], **m["kw"],
                       "parallelism": "dp%d" % world, "lr": LR, "cuda_graph": not args.no_graph,
                       "l2": "per-step working set (activations + gradients, > 1 GB) exceeds the 126 MB L2"},
            "e2e": {"value": m["e2e_value"], "unit": "samples/s",
                    "h2d_bytes_per_step": m["h2d"], "d2h_bytes_per_step": m["B"] * 4,
                    "timed": "host wall clock around the pipelined steps and the wait for the last losses"},
            "gpu_launches": m["launches"], "clocks": m["clocks"], "roofline": m["roofline"],
            "loss": m["loss_rank0"], "loss_global": m["loss_global"],
            "updates_before_loss_global": m["updates_before_loss_global"],
            "cpu_baseline": cpu_baseline(args.workload) if world == 1 and not args.no_cpu_baseline else None,
        }
        if others:
            line["workloads"] = others
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mixer_dp4096", choices=sorted(WORKLOADS))
    ap.add_argument("--repeats", type=int, default=15,
                    help="the K-step measurement is repeated this many times and the median reported")
    ap.add_argument("--global-batch", type=int, default=0,
                    help="override the workload's global batch (e.g. the per-rank batch of an N-GPU run on one GPU)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-workloads", action="store_true", help="skip the short runs of the other configurations")
    ap.add_argument("--no-graph", action="store_true", help="launch the step kernel by kernel instead of as a CUDA graph")
    args = ap.parse_args()
    if args.global_batch > 0:
        b, kw, _, kind = WORKLOADS[args.workload]
        WORKLOADS[args.workload] = (b, kw, args.global_batch, kind)
    if args.impl == "reference":
        run_reference(args)
    elif WORKLOADS[args.workload][0] is None:
        run_linear(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
