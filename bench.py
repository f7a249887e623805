#!/usr/bin/env python
"""Headline benchmark: Llama-2-7B-architecture int4 greedy decode, tokens/s, on N B200s.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: batch 1, 128 synthetic prompt tokens fed one at a time, then greedy decode; seeded
random-init weights of the Llama-2-7B architecture (int4 g=128 linears, fp16 embeddings/norms/KV
cache).  A "step" is one token through the whole model.  N > 1 is tensor parallel (strong scaling:
the same token stream, weights split over the GPUs).

Timed region: K CUDA-graph replays bracketed by barrier + synchronize, CUDA events on the
launching stream, max over ranks; the region is repeated REPEATS times from the same state (prompt
re-fed each time, so every repeat covers the same positions) and the median is reported with
minimum and maximum, which also lets the clock sampler see several of its periods.  Every step
streams all weights (3.6 GB / N per GPU), far more than L2, so no explicit L2 flush is needed
between iterations.

Also reported on the same JSON line:
  e2e          the same K steps through LlamaInt4Decoder.step(): token id copied host->device,
               graph replay, chosen id copied device->host, every step;
  roofline     the W4A16 GEMV (dominant kernel): algorithmic bytes of the 128 GEMV launches of a
               step / their device time (the launches alone, replayed as a graph and timed with
               CUDA events), against the measured HBM copy bandwidth;
  cpu_baseline the reference's CPU runtime (c-mcpu thread pool, g++ -O2 -ffast-math JIT) on the
               same operator chain, timed on this box's host cores (rank 0, N=1 only).

--impl reference times only that CPU path.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_PROMPT = 128
METRIC = "llama2_7b_int4_decode_tokens_per_s"
UNIT = "tokens/s"

REPEATS = 10
# DRAM bytes (read + write) of one unsharded gate|up GEMV launch (K=4096, N=22016, one row) in an ncu
# capture of that kernel; algorithmic bytes of the same launch: 46,550,016.  A profiler figure quoted
# beside the run's own numbers, not something this script measures.
NCU_TRAFFIC_GATE_UP = 46535168 + 1280


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi in loop mode beside the run.  It needs a few hundred ms to come up, so it is started
    before the warm-up phase and only the samples stamped inside [mark_begin, mark_end] (host clock)
    are used; if the timed region was shorter than the sampling period, the samples closest to it."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc = index, None
        self.t0 = self.t1 = None

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        import datetime
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(parts[1]), float(parts[2]), [n for n, v in zip(names, parts[4:8]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        t0 = self.t0 if self.t0 is not None else float("-inf")
        t1 = self.t1 if self.t1 is not None else float("inf")
        inside = [r for r in rows if t0 <= r[0] <= t1]
        note = None
        if not inside and rows:  # timed region shorter than the sampling period: take the two nearest samples
            inside = sorted(rows, key=lambda r: min(abs(r[0] - t0), abs(r[0] - t1)))[:2]
            note = "no sample fell inside the timed region; nearest samples used"
        sm = [r[1] for r in inside]
        mx = [r[2] for r in inside]
        reasons = sorted({n for r in inside for n in r[3]})
        res = {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
               "samples": len(sm), "reasons": reasons}
        if note:
            res["note"] = note
        return res


# ---- reference arm: the reference's CPU runtime on the same operator chain -------------------------

def reference_layer_kernels(cfg, S):
    """Kernel-source modules + seeded inputs for one decoder layer as the sample chains them
    (samples/05_llama2_7b_int4.py:149-173), on the c-mcpu runtime."""
    import numpy as np
    from antares_b200 import packing
    from oracle import ref_kernels as rk, refrt
    d, f = cfg.dim, cfg.ffn
    mods = []

    def w4(name, K, N, seed):
        qw, sc = packing.synth_w4(K, N, seed)
        x = packing.synth_x(1, K, seed + 1)
        y = np.zeros((1, N), np.float16)
        mods.append((name, refrt.RefModule(rk.w4a16(1, K, N)), (x, qw, sc, y)))

    w4("vqk", d, 3 * d, 1)
    w4("o", d, d, 2)
    w4("gate", d, f, 3)
    w4("up", d, f, 4)
    w4("down", f, d, 5)
    rng = np.random.default_rng(0)
    x32 = rng.standard_normal(d).astype(np.float32)
    mods.append(("rmsnorm_att", refrt.RefModule(rk.rmsnorm_vsum_f32(d)),
                 (np.array([float((x32 * x32).sum())], np.float32), (1 + 0.1 * rng.standard_normal(d)).astype(np.float32), x32, np.zeros(d, np.float32))))
    mods.append(("rmsnorm_ffn", mods[-1][1], mods[-1][2]))
    xh = rng.standard_normal((1, cfg.n_heads, cfg.head_dim)).astype(np.float16)
    from antares_b200.llama import make_inv_freq
    rot = refrt.RefModule(rk.rotary(1, cfg.n_heads, cfg.head_dim))
    rot_args = (make_inv_freq(cfg.head_dim, cfg.rope_base), np.array([S - 1], np.int32), xh, np.zeros_like(xh))
    mods.append(("rotary_q", rot, rot_args))
    mods.append(("rotary_k", rot, rot_args))
    kc = rng.standard_normal((S, cfg.n_heads, cfg.head_dim)).astype(np.float16)
    vc = rng.standard_normal((S, cfg.n_heads, cfg.head_dim)).astype(np.float16)
    mods.append(("attention", refrt.RefModule(rk.attention(S, cfg.n_heads, cfg.head_dim, S)),
                 (np.array([cfg.head_dim ** -0.5], np.float32), kc, xh[0].copy(), vc, np.zeros((cfg.n_heads, cfg.head_dim), np.float16))))
    return mods


def run_reference(args, as_baseline=False):
    """Times the reference CPU path.  One step = one kernel of one decoder layer's chain (cycled), each
    timed by the reference evaluator's own protocol (one run, then min(1e4, 1/tpr) further runs,
    graph_evaluator/run_graph.cpp:214-236, capped here so that the whole arm stays bounded); a token is
    extrapolated as 32 layers + classifier.  Returns the JSON dict."""
    import numpy as np
    import torch
    from antares_b200.llama import LlamaConfig
    from oracle import refrt
    cfg = LlamaConfig()
    S = N_PROMPT + 128  # mid-run KV length of the workload
    use_ref = refrt.available()
    steps, warm = max(1, args.steps), max(0, args.warmup)
    budget_s, t_start = 240.0, time.perf_counter()
    times, executed = {}, 0
    if use_ref:
        mods = reference_layer_kernels(cfg, S)
        cores, kind = refrt.num_threads(), "reference"
        for i in range(warm + steps):
            name, m, a = mods[i % len(mods)]
            dt = m.time(*a, max_runs=3)           # the reference's protocol, at most 3 timed runs per step
            if i >= warm:
                times.setdefault(name, []).append(dt)
                executed += 1
            if time.perf_counter() - t_start > budget_s:
                break
        for name, m, a in mods:                   # a kernel the step budget never reached: one timing now
            if name not in times:
                times[name] = [m.time(*a, max_runs=1)]
    else:  # the reference headers were not compiled in: plain-C restatement
        from antares_b200 import packing
        from oracle import cport
        kind, cores = "port", os.cpu_count() or 1
        runners = []
        for name, K, N in (("vqk", cfg.dim, 3 * cfg.dim), ("o", cfg.dim, cfg.dim), ("gate", cfg.dim, cfg.ffn),
                           ("up", cfg.dim, cfg.ffn), ("down", cfg.ffn, cfg.dim)):
            qw, sc = packing.synth_w4(K, N, 1)
            x = packing.synth_x(1, K, 2)
            runners.append((name, (lambda x=x, qw=qw, sc=sc: cport.w4a16_gemm(x, qw, sc))))
        for name, fn in runners:
            fn()
        for i in range(warm + steps):
            name, fn = runners[i % len(runners)]
            t0 = time.perf_counter()
            fn()
            if i >= warm:
                times.setdefault(name, []).append(time.perf_counter() - t0)
                executed += 1
            if time.perf_counter() - t_start > budget_s:
                break
        for name, fn in runners:
            if name not in times:
                t0 = time.perf_counter()
                fn()
                times[name] = [time.perf_counter() - t0]
    # classifier: torch CPU matmul, as the sample does (line 176); fp32 like the sample
    torch.set_num_threads(cores)
    wc = torch.randn(cfg.vocab, cfg.dim)
    xc = torch.randn(1, cfg.dim)
    t_layer = sum(statistics.mean(v) for v in times.values())
    torch.matmul(xc, wc.t())
    t0 = time.perf_counter()
    for _ in range(3):
        torch.matmul(xc, wc.t())
    t_head = (time.perf_counter() - t0) / 3
    t_token = cfg.n_layers * t_layer + t_head
    sample = ("EXTRAPOLATED: one decoder layer's kernel chain (vqk, o, gate, up, down W4A16 GEMVs; rmsnorm x2, rotary x2, attention at "
              "S=%d) on the reference c-mcpu runtime, one kernel per step cycled over %d executed steps, each timed by the reference "
              "evaluator's protocol; token = %d layers x that chain + torch CPU classifier matmul" % (S, executed, cfg.n_layers))
    cb = {"value": 1.0 / t_token, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample}
    if as_baseline:
        return cb
    return {"impl": "reference", "metric": METRIC, "value": 1.0 / t_token, "unit": UNIT, "n_gpus": args.gpus,
            "steps": steps, "warmup": warm, "ms_per_step": 1e3 * t_token, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "llama2-7b-arch int4 g128 greedy decode, batch 1, %d prompt tokens; CPU arm: one layer x%d + classifier, extrapolated"
                                   % (N_PROMPT, cfg.n_layers),
                       "parallelism": "cpu x%d threads" % cores},
            "cpu_baseline": cb,
            "e2e": {"value": 1.0 / t_token, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


# ---- our arm -------------------------------------------------------------------------------------------

def gemv_roofline(dec, torch, peak_gbs, peak_kind):
    """Device time of the step's W4A16 GEMV launches alone (same weights, same order, as a graph)."""
    cfg = dec.cfg
    side = torch.cuda.Stream(device=dec.dev)
    n_launch, alg = 0, 0

    def enqueue():
        nonlocal n_launch, alg
        n_launch, alg = 0, 0
        dec._st = torch.cuda.current_stream().cuda_stream
        dec._n = dec._pi = 0
        for w in dec.layers:
            # the step's four projections with their fused prologues/epilogues (scratch buffers as outputs)
            for x, k, out, pro, epi, nw, K, N in ((dec.x, "vqk", dec.vqk, 1, 0, w["att_norm"], cfg.dim, 3 * dec.dl),
                                                  (dec.att, "o", dec.partial, 0, 2, None, dec.dl, cfg.dim),  # row-parallel: fp32 partial, no exchange
                                                  (dec.x, "gu", dec.gu, 1, 0, w["ffn_norm"], cfg.dim, 2 * dec.fl),
                                                  (dec.gu, "down", dec.partial, 2, 2, None, dec.fl, cfg.dim)):
                dec._proj(x, w[k + "_q"], w[k + "_s"], out, pro, epi, nw)
                n_launch += 1
                alg += K * N // 2 + (K // cfg.group) * N * 2 + K * 2 + N * 2

    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        enqueue()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            enqueue()
        for _ in range(3):
            g.replay()
        reps = 10
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        sec = e0.elapsed_time(e1) * 1e-3 / reps
    torch.cuda.current_stream().wait_stream(side)
    achieved = alg / sec / 1e9
    gate_up_alg = cfg.dim * 2 * dec.fl // 2 + (cfg.dim // cfg.group) * 2 * dec.fl * 2 + cfg.dim * 2 + 2 * dec.fl * 2
    if dec.world == 1:
        traffic = NCU_TRAFFIC_GATE_UP
        note = ("DRAM bytes of ONE unsharded gate|up launch from an ncu capture of that kernel, quoted, not measured by this run; "
                "algorithmic bytes of that launch: %d" % gate_up_alg)
    else:
        traffic = None
        note = "no ncu capture of the sharded launches (this rank's gate|up launch: %d algorithmic bytes)" % gate_up_alg
    return {"bound": "hbm", "kernel": "w4a16_gemv (decode, M=1)", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s",
            "frac": achieved / peak_gbs, "peak_kind": peak_kind, "traffic": traffic, "traffic_note": note,
            "launches": n_launch, "avg_launch_us": sec / n_launch * 1e6, "algorithmic_bytes_per_step": alg}


def extras_single_ops(torch, dev, peak_gbs, tensor_peak):
    """Operator-level figures next to the headline (rank 0, N=1): the W4A16 prefill GEMM (x fp16
    [2048, 4096], W 4096 -> 11008) on the tensor cores and the four decode GEMV shapes at batch 1, 8 and 16, each timed
    alone with CUDA events (GEMVs rotate through weight copies larger than L2)."""
    import numpy as np
    from antares_b200 import ops, packing
    out = {}
    M, K, N = 2048, 4096, 11008
    qw, sc = packing.synth_w4(K, N, 1)
    qd, sd = torch.from_numpy(qw).to(dev), torch.from_numpy(sc).to(dev)
    x = torch.from_numpy(packing.synth_x(M, K, 2)).to(dev)
    y = torch.empty((M, N), dtype=torch.float16, device=dev)
    for _ in range(3):
        ops.w4a16_gemm(x, qd, sd, y)
    ts = []
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops.w4a16_gemm(x, qd, sd, y)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ms = float(np.median(ts))
    tf = 2.0 * M * K * N / ms / 1e9
    out["prefill_gemm"] = {"shape": [M, K, N], "ms": ms, "tflops": tf, "peak_tflops": tensor_peak, "frac": tf / tensor_peak,
                           "kernel": "w4a16_gemm_tcgen05_kernel"}
    del qd, sd, x, y
    for M in (1, 8, 16):
        gemv = {}
        for name, (K, N) in (("o", (4096, 4096)), ("vqk", (4096, 12288)), ("gate_up", (4096, 22016)), ("down", (11008, 4096))):
            qw, sc = packing.synth_w4(K, N, 3)
            nbuf = int(300e6 // (qw.nbytes + sc.nbytes)) + 2
            qs = [torch.from_numpy(qw).to(dev) for _ in range(nbuf)]
            ss = [torch.from_numpy(sc).to(dev) for _ in range(nbuf)]
            x = torch.from_numpy(packing.synth_x(M, K, 4)).to(dev)
            y = torch.empty((M, N), dtype=torch.float16, device=dev)
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for i in range(3):
                    ops.w4a16_gemv(x, qs[i % nbuf], ss[i % nbuf], y)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for i in range(2 * nbuf):
                        ops.w4a16_gemv(x, qs[i % nbuf], ss[i % nbuf], y)
                g.replay()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / (2 * nbuf)
            torch.cuda.current_stream().wait_stream(side)
            alg = K * N // 2 + (K // 128) * N * 2 + M * K * 2 + M * N * 2
            gemv[name] = {"K": K, "N": N, "us": us, "GBs": alg / us / 1e3, "frac": alg / us / 1e3 / peak_gbs}
            del qs, ss, g
        out["gemv_m%d" % M] = gemv
    out["elementwise_reduction"] = extras_config1(torch, dev, peak_gbs)
    out["dispatch"] = extras_dispatch(torch, dev)
    return out


def _time_rotating(torch, dev, launch, nbuf):
    """Median-free quick timer: a graph of 2 * nbuf launches over nbuf distinct input sets (together larger than
    L2), replayed 3 times, best replay; microseconds per launch."""
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(3):
            launch(i % nbuf)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(2 * nbuf):
                launch(i % nbuf)
        g.replay()
        torch.cuda.synchronize()
        best = None
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (2 * nbuf)
            best = us if best is None else min(best, us)
    torch.cuda.current_stream().wait_stream(side)
    return best


def extras_config1(torch, dev, peak_gbs):
    """The element-wise / reduction operators at their benchmark shapes: sigmoid float32[4096000], RMSNorm fp16
    [2048, 4096] (eps 1e-6, weight N(1, 0.1)), RoPE fp16 [2048, 32, 128] (base 10000, position = row), row softmax
    fp16 [32, 4096] (scores N(0, 3)).  Each timed alone, inputs rotated through more than L2; bytes = input +
    output tensors; softmax moves 0.5 MB and is reported for its latency."""
    import numpy as np
    from antares_b200 import ops
    from antares_b200.llama import make_inv_freq
    rng = np.random.default_rng(0)
    res = {}

    def report(name, us, nbytes):
        res[name] = {"us": us, "GBs": nbytes / us / 1e3, "frac": nbytes / us / 1e3 / peak_gbs, "bytes": nbytes}

    nbuf = 10
    xs = [torch.from_numpy(rng.standard_normal(4096000).astype(np.float32)).to(dev) for _ in range(nbuf)]
    y = torch.empty_like(xs[0])
    report("sigmoid_f32_4096000", _time_rotating(torch, dev, lambda i: ops.sigmoid(xs[i], out=y), nbuf), 2 * 4096000 * 4)
    del xs, y
    xs = [torch.from_numpy(rng.standard_normal((2048, 4096)).astype(np.float16)).to(dev) for _ in range(nbuf)]
    w = torch.from_numpy((1 + 0.1 * rng.standard_normal(4096)).astype(np.float16)).to(dev)
    y = torch.empty_like(xs[0])
    report("rmsnorm_f16_2048x4096", _time_rotating(torch, dev, lambda i: ops.rmsnorm(xs[i], w, 1e-6, out=y), nbuf), 2 * 2048 * 4096 * 2 + 4096 * 2)
    del xs, y
    xs = [torch.from_numpy(rng.standard_normal((2048, 32, 128)).astype(np.float16)).to(dev) for _ in range(nbuf)]
    pos = torch.arange(2048, dtype=torch.int32, device=dev)
    inv = torch.from_numpy(make_inv_freq(128, 10000.0)).to(dev)
    y = torch.empty_like(xs[0])
    report("rope_f16_2048x32x128", _time_rotating(torch, dev, lambda i: ops.rope(xs[i], pos, inv, out=y), nbuf), 2 * 2048 * 32 * 128 * 2 + 2048 * 4)
    del xs, y
    xs = [torch.from_numpy((3 * rng.standard_normal((32, 4096))).astype(np.float16)).to(dev) for _ in range(nbuf)]
    y = torch.empty_like(xs[0])
    report("softmax_f16_32x4096", _time_rotating(torch, dev, lambda i: ops.softmax(xs[i], out=y), nbuf), 2 * 32 * 4096 * 2)
    res["softmax_f16_32x4096"]["note"] = "0.5 MB: latency-bound, read the microseconds"
    return res


def extras_dispatch(torch, dev):
    """Host cost of one operator call, the counterpart of the reference's per-call work in
    graph_evaluator/execute_module.hpp:321-393: (a) the Python route a sample script takes,
    autort.ops.<name>(x, qweight, scales, out=...); (b) the native route a C++ binding takes, ab200_forward on a
    key from ab200_inject.  Wall time per call while the launches queue up (nothing synchronised inside)."""
    import ctypes
    import numpy as np
    import autort
    from antares_b200 import _lib, packing
    from antares_b200.autort_api import W4A16_IR_SAMPLE
    K, N = 4096, 4096
    qw, sc = packing.synth_w4(K, N, 0)
    qd, sd = torch.from_numpy(qw).to(dev), torch.from_numpy(sc).to(dev)
    x = torch.from_numpy(packing.synth_x(1, K, 1)[0]).to(dev)
    y = torch.empty(N, dtype=torch.float16, device=dev)
    f = autort.export(ir=W4A16_IR_SAMPLE, inputs=["input0=float16[S:%d]" % K, "qweight=int32[L:%d, N:%d]" % (K // 8, N), "scales=float16[K:%d, N:%d]" % (K // 128, N)],
                      config="~N~:[256,8,32],~S~:[64,8]", name="bench_w4a16")
    for _ in range(20):
        f(x, qd, sd, out=y)
    torch.cuda.synchronize()
    n = 200
    t0 = time.perf_counter()
    for _ in range(n):
        f(x, qd, sd, out=y)
    py_us = (time.perf_counter() - t0) / n * 1e6
    torch.cuda.synchronize()
    src = ("// GLOBALS: input0:float16[%d], qweight:int32[%d, %d], scales:float16[%d, %d] -> my_result:float16[%d]\n"
           "// BACKEND: c-b200 (default)\n// CONFIG: \n// COMPUTE_V1: - einstein_v2(input_dict={}, extra_outputs=[], exprss=\"%s\")\n"
           % (K, K // 8, N, K // 128, N, N, W4A16_IR_SAMPLE.replace("\n", ";").replace('"', "`")))
    L = _lib.load()
    key = ctypes.c_int(-1)
    _lib.call("ab200_inject", src.encode(), ctypes.cast(ctypes.pointer(key), ctypes.c_void_p))
    args = (ctypes.c_void_p * 4)(x.data_ptr(), qd.data_ptr(), sd.data_ptr(), y.data_ptr())
    ns = ctypes.c_double(0)
    st = torch.cuda.current_stream().cuda_stream
    _lib.call("ab200_forward_host_ns", key.value, ctypes.cast(args, ctypes.c_void_p), 4, st, 20, ctypes.cast(ctypes.pointer(ns), ctypes.c_void_p))
    torch.cuda.synchronize()
    _lib.call("ab200_forward_host_ns", key.value, ctypes.cast(args, ctypes.c_void_p), 4, st, n, ctypes.cast(ctypes.pointer(ns), ctypes.c_void_p))
    torch.cuda.synchronize()
    return {"op": "W4A16 GEMV 4096x4096, one row", "python_autort_ops_us": py_us, "native_forward_us": ns.value / 1e3, "calls": n}


def run_ours(args):
    import torch
    from antares_b200 import parallel
    from antares_b200.llama import LlamaConfig, LlamaInt4Decoder, synth_prompt
    os.environ.setdefault("NCCL_DEBUG", "WARN")  # keep NCCL's version banner off stdout: one JSON line only
    rank, world, local_rank = parallel.init_from_env()
    if world != args.gpus:
        raise SystemExit("bench.py: --gpus %d but WORLD_SIZE=%d (launch N>1 with torch.distributed.run)" % (args.gpus, world))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    comm = None
    if world > 1:
        comm = parallel.TorchComm() if args.comm == "nccl" else parallel.PushComm(dev, 4096)
    K, W = args.steps, max(3, args.warmup)
    if args.pdl >= 0:
        from antares_b200 import ops as _ops
        _ops.set_option("pdl", args.pdl)
    cfg = LlamaConfig(max_seq=max(N_PROMPT + W + K + 8, 168))
    dec = LlamaInt4Decoder(cfg, dev, rank=rank, world=world, comm=comm, max_tokens=max(N_PROMPT + W + K + 8, 168),
                           prefetch=args.prefetch, tiled=not args.reference_layout, fused_allreduce=not args.separate_allreduce,
                           kv_page_rows=args.kv_page_rows)
    prompt = synth_prompt(cfg, N_PROMPT, 0)
    dec.prompt[:N_PROMPT].copy_(torch.from_numpy(prompt))
    dec.capture(N_PROMPT)

    def prefill_and_warm():
        dec.reset(torch.from_numpy(prompt).to(dev))
        for _ in range(N_PROMPT - 1 + W):  # prompt tokens go through the same step; then W warm-up tokens
            dec.graph.replay()

    def fence():
        torch.cuda.synchronize()
        if comm is not None:
            comm.barrier()
        torch.cuda.synchronize()

    from antares_b200 import ops as _ops

    def check_status(where):
        # a bounded device-side wait that ran out leaves a code here: such a run's numbers are void
        torch.cuda.synchronize()
        try:
            _ops.kernel_status()
        except Exception as e:  # noqa: BLE001
            raise SystemExit("bench.py: rank %d: %s after %s" % (rank, e, where))

    def timed(run_steps):
        """REPEATS x (re-feed the prompt, W warm-up tokens, then exactly K timed steps)."""
        secs = []
        for _ in range(args.repeats):
            prefill_and_warm()
            fence()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run_steps()
            e1.record()
            fence()
            sec = e0.elapsed_time(e1) * 1e-3
            if comm is not None:
                sec = comm.max_float(sec, dev)
            secs.append(sec)
        return secs

    # ---- device-timed run ---------------------------------------------------------------------------
    sampler = ClockSampler(local_rank)
    sampler.start()
    prefill_and_warm()
    fence()
    sampler.mark_begin()

    def replay_k():
        for _ in range(K):
            dec.graph.replay()

    secs = timed(replay_k)
    sampler.mark_end()
    clocks = sampler.stop()
    check_status("the device-timed run")
    sec = statistics.median(secs)
    tokens = dec.out_tokens[:N_PROMPT + W + K].cpu().numpy()

    # ---- end-to-end run through the public per-token call (host token in, host token out) ----------
    def step_k():
        tok = int(dec.token.item())
        for _ in range(K):
            tok = dec.step(tok)

    secs_e2e = timed(step_k)
    check_status("the end-to-end run")
    sec_e2e = statistics.median(secs_e2e)
    tokens_e2e = dec.out_tokens[:N_PROMPT + W + K].cpu().numpy()

    # ---- correctness of this run's numbers: last-step logits of the workload's first 32 generated tokens
    # against the values the CPU oracle stored for them, and bitwise agreement of the replicated residual stream
    logits_check = None
    gpath = os.path.join(ROOT, "tests", "golden")
    if os.path.exists(os.path.join(gpath, "llama_logits.npz")):
        import numpy as np
        g = json.load(open(os.path.join(gpath, "llama_tokens.json")))["p128_n32"]
        ref = np.load(os.path.join(gpath, "llama_logits.npz"))["p128_n32_pos158"]
        dec.reset(torch.from_numpy(prompt).to(dev))
        for _ in range(159):
            dec.graph.replay()
        torch.cuda.synchronize()
        got_tokens = dec.out_tokens[:160].cpu().numpy()
        if world > 1:
            full = torch.empty(cfg.vocab, dtype=torch.float32, device=dev)
            torch.distributed.all_gather_into_tensor(full, dec.logits_local)
            xs = [torch.empty_like(dec.x) for _ in range(world)]
            torch.distributed.all_gather(xs, dec.x)
            same_x = all(bool(torch.equal(xs[0], t)) for t in xs)
        else:
            full, same_x = dec.logits_local, True
        lg = full.cpu().numpy()
        logits_check = {"max_err_over_max_ref": float(np.abs(lg - ref).max() / np.abs(ref).max()),
                        "position": 158, "tokens_equal_oracle": bool((got_tokens == np.array(g["tokens"], np.int32)).all()),
                        "residual_stream_bitwise_equal_across_ranks": same_x}
        check_status("the logits check")

    peak, peak_kind = measured_peaks()
    roof = gemv_roofline(dec, torch, peak, peak_kind)
    step_bytes = statistics.mean(dec.step_bytes(p) for p in range(N_PROMPT + W, N_PROMPT + W + K))
    # time to first token for the 128-token prompt: the reference's way (token by token through
    # the decode step) and the batched prefill (tensor-core GEMMs over all prompt tokens); every rank takes part
    ttft = None
    if not args.no_extras:
        ttft = {}
        try:  # an extra: whatever goes wrong here (the same on every rank) must not cost the headline line
            for name in ("token_by_token", "batched_prefill"):
                best = None
                for _ in range(3):
                    fence()
                    t0 = time.perf_counter()
                    if name == "batched_prefill":
                        dec.prefill(prompt)
                    else:
                        dec.reset(torch.from_numpy(prompt).to(dev))
                        for _ in range(N_PROMPT):
                            dec.graph.replay()
                    fence()
                    dt = (time.perf_counter() - t0) * 1e3
                    best = dt if best is None else min(best, dt)
                ttft[name + "_ms"] = best
                ttft[name + "_first_token"] = int(dec.token.item())
            check_status("the time-to-first-token runs")
        except Exception as e:  # noqa: BLE001
            ttft = {"error": "%s: %s" % (type(e).__name__, e)}
    if rank != 0:
        return None
    line = {"metric": METRIC, "value": K / sec, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": 1e3 * sec / K, "ms_per_step_min": 1e3 * min(secs) / K, "ms_per_step_max": 1e3 * max(secs) / K, "repeats": args.repeats,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": "llama2-7b-arch int4 g128 greedy decode, batch 1, %d prompt tokens then %d timed tokens" % (N_PROMPT, K),
                       "parallelism": "tp%d" % world,
                       "allreduce": ("none" if world == 1 else ("nccl" if args.comm == "nccl" else ("push, fused into the O/down projections" if dec.fused_allreduce else "push, separate kernel"))), "l2": "each step streams %.2f GB of weights per GPU (> L2), no flush needed" % (step_bytes / 1e9),
                       "launcher": "cuda graph, 1 replay per token",
                       "weight_layout": "reference [K/8, N]" if args.reference_layout else "tile-major [N/128][K/8][128] (repacked at load)",
                       "kv_cache": ("paged, %d rows per page" % args.kv_page_rows) if args.kv_page_rows else "contiguous"},
            "e2e": {"value": K / sec_e2e, "unit": UNIT, "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
            "gpu_launches": dec.launches_per_step * K, "launches_per_step": dec.launches_per_step,
            "clocks": clocks, "roofline": roof,
            "step_hbm": {"bytes_per_step_per_gpu": step_bytes, "achieved_gbs": step_bytes / (sec / K) / 1e9,
                         "frac_of_peak": step_bytes / (sec / K) / 1e9 / peak},
            "logits_check": logits_check,
            "tokens_match_between_runs": bool((tokens == tokens_e2e).all()),
            "first_generated": [int(t) for t in tokens[N_PROMPT:N_PROMPT + 8]],
            "tokens_crc32": int(__import__("zlib").crc32(tokens.astype("int32").tobytes()))}
    if world == 1 and not args.no_extras:
        tensor_peak = 1642.0
        path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(path):
            with open(path) as f:
                tensor_peak = float(json.load(f).get("bf16_tflops", tensor_peak))
        del dec
        torch.cuda.empty_cache()
        line["extras"] = extras_single_ops(torch, dev, peak, tensor_peak)
        line["extras"]["time_to_first_token_128"] = ttft
    elif ttft is not None:
        line["extras"] = {"time_to_first_token_128": ttft}
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = run_reference(argparse.Namespace(steps=20, warmup=0, gpus=1), as_baseline=True)
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--repeats", type=int, default=REPEATS, help="how many times the K-step timed region is repeated (median reported)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kv-page-rows", type=int, default=0, help="KV cache in pages of this many rows (a power of two) behind a page table; 0 = contiguous (the default, as in the reference)")
    ap.add_argument("--no-extras", action="store_true", help="skip the operator-level figures (prefill GEMM, GEMV set)")
    ap.add_argument("--pdl", type=int, default=-1, help="programmatic dependent launch: 0 off, 1 release dependents at kernel start, 2 after the GEMV streaming loop")
    ap.add_argument("--reference-layout", action="store_true", help="keep the weights in the reference's [K/8, N] layout instead of tile-major")
    ap.add_argument("--prefetch", type=int, default=0, help="1: every projection kernel also pulls the next one's weights into L2 (measured neutral)")
    ap.add_argument("--separate-allreduce", action="store_true", help="tensor parallel: exchange in a kernel of its own instead of inside the O/down projections")
    ap.add_argument("--comm", default="push", choices=["push", "nccl"], help="all-reduce of row-parallel partials: one-shot NVLink push kernel or NCCL")
    args = ap.parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return 0
        print(json.dumps(run_reference(args)), flush=True)
        return 0
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(args.gpus),
               "--master-addr", "127.0.0.1", "--master-port", "29511", os.path.abspath(__file__)] + sys.argv[1:]
        return subprocess.call(cmd)
    line = run_ours(args)
    if line is not None:
        print(json.dumps(line), flush=True)
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
