#!/usr/bin/env python
"""Headline benchmark: Llama-2-7B-architecture int4 greedy decode, tokens/s, on N B200s.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE config 4): batch 1, 128 synthetic prompt tokens fed one at a time, then
greedy decode; seeded random-init weights of the 7B architecture (int4 g=128 linears, fp16
embeddings/norms/KV cache).  A "step" is one token through the whole model.  N > 1 is tensor
parallel (strong scaling: the same token stream, weights split over the GPUs).

Timed region: K CUDA-graph replays bracketed by barrier + synchronize, CUDA events on the
launching stream, max over ranks.  Every step streams all weights (3.6 GB / N per GPU), far more
than L2, so no explicit L2 flush is needed between iterations.

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

# dram__bytes_read.sum + dram__bytes_write.sum of one gate|up GEMV launch (K=4096, N=22016, M=1) from the
# ncu capture summarised in profiles/w4a16_gemv_scalar_gate_up_m1.md (algorithmic bytes: 46,550,016).
NCU_TRAFFIC_GATE_UP = 46535168 + 1280  # dram__bytes_read.sum + dram__bytes_write.sum of one gate|up launch (profiles/w4a16_gemv_scalar_gate_up_m1.md)


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
                 (np.array([float((x32 * x32).sum())], np.float32), np.ones(d, np.float32), x32, np.zeros(d, np.float32))))
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
    """Times the reference CPU path.  One step = one kernel of the layer chain (cycled), so that K
    steps stay bounded; a token = 32 layers + classifier.  Returns the JSON dict."""
    import numpy as np
    import torch
    from antares_b200.llama import LlamaConfig
    from oracle import refrt
    cfg = LlamaConfig()
    S = N_PROMPT + 128  # mid-run KV length of the workload
    use_ref = refrt.available()
    if use_ref:
        mods = reference_layer_kernels(cfg, S)
        cores, kind = refrt.num_threads(), "reference"
        runners = [(name, (lambda m=m, a=a: m(*a))) for name, m, a in mods]
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
    # classifier: torch CPU matmul, as the sample does (line 176); fp32 like the sample
    torch.set_num_threads(cores)
    wc = torch.randn(cfg.vocab, cfg.dim)
    xc = torch.randn(1, cfg.dim)
    times = {name: [] for name, _ in runners}
    first = {}
    for name, fn in runners:  # one untimed-for-the-mean pass of everything (JIT, page-in); kept as fallback
        t0 = time.perf_counter()
        fn()
        first[name] = time.perf_counter() - t0
    steps, warm = max(1, args.steps), max(0, args.warmup)
    budget_s, t_start = 240.0, time.perf_counter()
    executed = 0
    for i in range(warm + steps):
        name, fn = runners[i % len(runners)]
        t0 = time.perf_counter()
        fn()
        dt = time.perf_counter() - t0
        if i >= warm:
            times[name].append(dt)
            executed += 1
        if time.perf_counter() - t_start > budget_s:
            break
    t_layer = sum((statistics.mean(v) if v else first[n]) for n, v in times.items())
    torch.matmul(xc, wc.t())
    t0 = time.perf_counter()
    for _ in range(3):
        torch.matmul(xc, wc.t())
    t_head = (time.perf_counter() - t0) / 3
    t_token = cfg.n_layers * t_layer + t_head
    sample = ("one decoder layer's kernel chain (vqk, o, gate, up, down W4A16 GEMVs; rmsnorm x2, rotary x2, attention at "
              "S=%d) on the reference c-mcpu runtime, one kernel per step cycled over %d executed steps, x%d layers + "
              "torch CPU classifier matmul" % (S, executed, cfg.n_layers))
    cb = {"value": 1.0 / t_token, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample}
    if as_baseline:
        return cb
    return {"impl": "reference", "metric": METRIC, "value": 1.0 / t_token, "unit": UNIT, "n_gpus": args.gpus,
            "steps": steps, "warmup": warm, "ms_per_step": 1e3 * t_token, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "llama2-7b-arch int4 g128 greedy decode, batch 1, %d prompt tokens" % N_PROMPT,
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
                                                  (dec.att, "o", dec.partial, 0, 2, None, dec.dl, cfg.dim),
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
    return {"bound": "hbm", "kernel": "w4a16_gemv (decode, M=1)", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s",
            "frac": achieved / peak_gbs, "peak_kind": peak_kind,
            "traffic": NCU_TRAFFIC_GATE_UP, "traffic_note": "dram bytes of one gate|up launch (algorithmic %d B)" % gate_up_alg,
            "launches": n_launch, "avg_launch_us": sec / n_launch * 1e6, "algorithmic_bytes_per_step": alg}


def extras_single_ops(torch, dev, peak_gbs, tensor_peak):
    """Operator-level figures next to the headline (rank 0, N=1): the W4A16 prefill GEMM of BASELINE
    config 3 on the tensor cores and the four decode GEMV shapes of config 2 at batch 1, 8 and 16, each timed
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
    return out



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
    cfg = LlamaConfig(max_seq=N_PROMPT + W + K + 8)
    dec = LlamaInt4Decoder(cfg, dev, rank=rank, world=world, comm=comm, max_tokens=N_PROMPT + W + K + 8,
                           prefetch=args.prefetch, tiled=not args.reference_layout)
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

    # ---- device-timed run ---------------------------------------------------------------------------
    sampler = ClockSampler(local_rank)
    sampler.start()
    prefill_and_warm()
    fence()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.mark_begin()
    e0.record()
    for _ in range(K):
        dec.graph.replay()
    e1.record()
    fence()
    sampler.mark_end()
    clocks = sampler.stop()
    sec = e0.elapsed_time(e1) * 1e-3
    if comm is not None:
        sec = comm.max_float(sec, dev)
    tokens = dec.out_tokens[:N_PROMPT + W + K].cpu().numpy()

    # ---- end-to-end run through the public per-token call (host token in, host token out) ----------
    prefill_and_warm()
    fence()
    tok = int(dec.token.item())
    e0.record()
    for _ in range(K):
        tok = dec.step(tok)
    e1.record()
    fence()
    sec_e2e = e0.elapsed_time(e1) * 1e-3
    if comm is not None:
        sec_e2e = comm.max_float(sec_e2e, dev)
    tokens_e2e = dec.out_tokens[:N_PROMPT + W + K].cpu().numpy()

    peak, peak_kind = measured_peaks()
    roof = gemv_roofline(dec, torch, peak, peak_kind)
    step_bytes = statistics.mean(dec.step_bytes(p) for p in range(N_PROMPT + W, N_PROMPT + W + K))
    if rank != 0:
        return None
    line = {"metric": METRIC, "value": K / sec, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": 1e3 * sec / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": "llama2-7b-arch int4 g128 greedy decode, batch 1, %d prompt tokens then %d timed tokens" % (N_PROMPT, K),
                       "parallelism": "tp%d" % world, "allreduce": ("none" if world == 1 else args.comm), "l2": "each step streams %.2f GB of weights per GPU (> L2), no flush needed" % (step_bytes / 1e9),
                       "launcher": "cuda graph, 1 replay per token",
                       "weight_layout": "reference [K/8, N]" if args.reference_layout else "tile-major [N/128][K/8][128] (repacked at load)"},
            "e2e": {"value": K / sec_e2e, "unit": UNIT, "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
            "gpu_launches": dec.launches_per_step * K, "launches_per_step": dec.launches_per_step,
            "clocks": clocks, "roofline": roof,
            "step_hbm": {"bytes_per_step_per_gpu": step_bytes, "achieved_gbs": step_bytes / (sec / K) / 1e9,
                         "frac_of_peak": step_bytes / (sec / K) / 1e9 / peak},
            "tokens_match_between_runs": bool((tokens == tokens_e2e).all()),
            "first_generated": [int(t) for t in tokens[N_PROMPT:N_PROMPT + 8]],
            "tokens_crc32": int(__import__("zlib").crc32(tokens.astype("int32").tobytes()))}
    if world == 1 and not args.no_extras:
        tensor_peak = 1642.0
        path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(path):
            with open(path) as f:
                tensor_peak = float(json.load(f).get("bf16_tflops", tensor_peak))
        # time to first token for the 128-token prompt: the reference's way (token by token through
        # the decode step) and the batched prefill (tensor-core GEMMs over all prompt tokens)
        ttft = {}
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
        del dec
        torch.cuda.empty_cache()
        line["extras"] = extras_single_ops(torch, dev, peak, tensor_peak)
        line["extras"]["time_to_first_token_128"] = ttft
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = run_reference(argparse.Namespace(steps=20, warmup=0, gpus=1), as_baseline=True)
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the operator-level figures (prefill GEMM, GEMV set)")
    ap.add_argument("--pdl", type=int, default=-1, help="programmatic dependent launch: 0 off, 1 release dependents at kernel start, 2 after the GEMV streaming loop")
    ap.add_argument("--reference-layout", action="store_true", help="keep the weights in the reference's [K/8, N] layout instead of tile-major")
    ap.add_argument("--prefetch", type=int, default=0, help="1: every projection kernel also pulls the next one's weights into L2 (measured neutral)")
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
