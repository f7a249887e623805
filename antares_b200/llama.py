"""Llama-2-7B-architecture int4 greedy decode built from the antares_b200 operators.

Mirrors the reference's model script samples/05_llama2_7b_int4.py:146-207 (`forward`, decode
loop) with these B200-first differences:
  * one decode step = one CUDA graph (captured once, replayed per token); token id, position and
    the generated ids live in device memory, so the loop needs no host round trip
    (the reference syncs on `int(torch.argmax(logits))` every token, line 200);
  * the residual stream is fp32, projection inputs/outputs fp16, KV cache fp16;
  * five launches per layer: RMSNorm is fused into the V|Q|K and gate|up projections, RoPE and the
    cache update into the attention kernel, SiLU*up and the residual adds into the O/down projections;
  * tensor parallel over `world` GPUs: column-parallel V|Q|K and gate|up, row-parallel O and
    down with one all-reduce each, vocabulary-parallel classifier with an all-gather.
Weights are seeded synthetic stand-ins for the GPTQ checkpoint (same shapes and value ranges).
"""
import math
from dataclasses import dataclass

import numpy as np
import torch

from . import packing
from ._lib import call


@dataclass
class LlamaConfig:
    n_layers: int = 32
    dim: int = 4096
    n_heads: int = 32
    ffn: int = 11008
    vocab: int = 32000
    max_seq: int = 512
    eps: float = 1e-6
    rope_base: float = 10000.0
    group: int = 128

    @property
    def head_dim(self):
        return self.dim // self.n_heads


# projection ids for seeding: seed = 1000 * layer + id
_V, _Q, _K, _O, _GATE, _UP, _DOWN, _NORM = range(8)


def synth_layer(cfg, layer, centered=False, scale_mul=1.0):
    """Unsharded synthetic weights of one layer (numpy).  centered: zero-mean nibbles and scales times
    scale_mul (packing.synth_w4)."""
    d, f, g = cfg.dim, cfg.ffn, cfg.group
    s = 1000 * layer
    w = {}
    if centered:
        import functools
        synth = functools.partial(packing.synth_w4, centered=True, scale_mul=scale_mul)
        parts = [synth(d, d, s + i, g) for i in (_V, _Q, _K)]
        w["vqk_q"] = np.ascontiguousarray(np.concatenate([p[0] for p in parts], axis=1))
        w["vqk_s"] = np.ascontiguousarray(np.concatenate([p[1] for p in parts], axis=1))
        w["o_q"], w["o_s"] = synth(d, d, s + _O, g)
        w["gate_q"], w["gate_s"] = synth(d, f, s + _GATE, g)
        w["up_q"], w["up_s"] = synth(d, f, s + _UP, g)
        w["down_q"], w["down_s"] = synth(f, d, s + _DOWN, g)
        rng = np.random.default_rng(s + _NORM)
        w["att_norm"] = (1 + 0.1 * rng.standard_normal(d, dtype=np.float32)).astype(np.float16)
        w["ffn_norm"] = (1 + 0.1 * rng.standard_normal(d, dtype=np.float32)).astype(np.float16)
        return w
    parts = [packing.synth_w4(d, d, s + i, g) for i in (_V, _Q, _K)]
    w["vqk_q"] = np.ascontiguousarray(np.concatenate([p[0] for p in parts], axis=1))  # order V, Q, K (line 27)
    w["vqk_s"] = np.ascontiguousarray(np.concatenate([p[1] for p in parts], axis=1))
    w["o_q"], w["o_s"] = packing.synth_w4(d, d, s + _O, g)
    w["gate_q"], w["gate_s"] = packing.synth_w4(d, f, s + _GATE, g)
    w["up_q"], w["up_s"] = packing.synth_w4(d, f, s + _UP, g)
    w["down_q"], w["down_s"] = packing.synth_w4(f, d, s + _DOWN, g)
    rng = np.random.default_rng(s + _NORM)
    w["att_norm"] = (1 + 0.1 * rng.standard_normal(d, dtype=np.float32)).astype(np.float16)
    w["ffn_norm"] = (1 + 0.1 * rng.standard_normal(d, dtype=np.float32)).astype(np.float16)
    return w


def _f16(a_f32):
    # IEEE round-to-nearest-even like numpy's astype, but multithreaded (numpy's is scalar).
    return torch.from_numpy(a_f32).to(torch.float16).numpy()


def synth_globals(cfg):
    rng = np.random.default_rng(999983)
    def table():
        a = rng.standard_normal((cfg.vocab, cfg.dim), dtype=np.float32)
        a *= np.float32(0.02)
        return _f16(a)
    return {"embed": table(), "lm_head": table(),
            "final_norm": (1 + 0.1 * rng.standard_normal(cfg.dim, dtype=np.float32)).astype(np.float16)}


def synth_prompt(cfg, n, seed=0):
    return np.random.default_rng(seed).integers(3, cfg.vocab, size=n).astype(np.int32)


def make_inv_freq(head_dim, base):
    j = np.arange(0, head_dim, 2, dtype=np.float32)
    f = (1.0 / (np.float32(base) ** (j / np.float32(head_dim)))).astype(np.float32)
    return np.concatenate([f, f]).astype(np.float32)  # length head_dim, halves equal (lines 125-126)


def shard_layer(cfg, w, rank, world):
    """Per-rank slices of one layer's weights."""
    d, g = cfg.dim, cfg.group
    dl = d // world
    sl = slice(rank * dl, (rank + 1) * dl)
    out = {}
    out["vqk_q"] = np.ascontiguousarray(np.concatenate([w["vqk_q"][:, i * d:(i + 1) * d][:, sl] for i in range(3)], axis=1))
    out["vqk_s"] = np.ascontiguousarray(np.concatenate([w["vqk_s"][:, i * d:(i + 1) * d][:, sl] for i in range(3)], axis=1))
    out["o_q"] = np.ascontiguousarray(w["o_q"][rank * dl // 8:(rank + 1) * dl // 8])
    out["o_s"] = np.ascontiguousarray(w["o_s"][rank * dl // g:(rank + 1) * dl // g])
    k0, k1 = packing.row_shard_bounds(cfg.ffn, world, g)[rank]
    out["gu_q"] = np.ascontiguousarray(np.concatenate([w["gate_q"][:, k0:k1], w["up_q"][:, k0:k1]], axis=1))
    out["gu_s"] = np.ascontiguousarray(np.concatenate([w["gate_s"][:, k0:k1], w["up_s"][:, k0:k1]], axis=1))
    out["down_q"] = np.ascontiguousarray(w["down_q"][k0 // 8:k1 // 8])
    out["down_s"] = np.ascontiguousarray(w["down_s"][k0 // g:k1 // g])
    out["att_norm"], out["ffn_norm"] = w["att_norm"], w["ffn_norm"]
    return out


class SynthWeights:
    """Weight source for LlamaInt4Decoder(weights=...) / the oracle: the seeded synthetic model, optionally
    with zero-mean nibbles (whose greedy stream does not settle on one token)."""

    def __init__(self, cfg, centered=False, scale_mul=1.0):
        self.cfg, self.centered, self.scale_mul = cfg, bool(centered), float(scale_mul)

    def layer(self, l):
        return synth_layer(self.cfg, l, self.centered, self.scale_mul)

    def globals(self):
        return synth_globals(self.cfg)


class LlamaInt4Decoder:
    """Greedy decoder for one rank of a tensor-parallel group (world=1: the whole model).

    `comm` is None for world=1, otherwise an object with
      all_reduce_sum_(t_f32)  and  all_gather_into(out, t)   (see parallel.py).
    `weights` selects the checkpoint (gptq.GptqLlamaWeights); None = seeded synthetic weights.
    """

    def __init__(self, cfg, device, rank=0, world=1, comm=None, max_tokens=1024, prefetch=0, weights=None, tiled=True,
                 fused_allreduce=True, kv_page_rows=0, kv_page_table=None):
        assert cfg.dim % (world * cfg.group) == 0 and cfg.n_heads % world == 0 and cfg.vocab % world == 0
        self.cfg, self.dev, self.rank, self.world, self.comm = cfg, device, rank, world, comm
        self.hl = cfg.n_heads // world            # local heads
        self.dl = cfg.dim // world                # local attention width
        k0, k1 = packing.row_shard_bounds(cfg.ffn, world, cfg.group)[rank]
        self.fl = k1 - k0                         # local FFN width
        self.vl = cfg.vocab // world
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
        self.layers = []
        # `weights`: any object with layer(l) and globals() (e.g. gptq.GptqLlamaWeights); default: seeded synthetic weights
        for l in range(cfg.n_layers):
            full = weights.layer(l) if weights is not None else synth_layer(cfg, l)
            w = shard_layer(cfg, full, rank, world)
            if tiled:  # tile-major weights: what one CTA streams is one contiguous range of HBM
                for k in ("vqk", "o", "gu", "down"):
                    w[k + "_q"], w[k + "_s"] = packing.tile_weights(w[k + "_q"], w[k + "_s"])
            self.layers.append({k: t(v) for k, v in w.items()})
        gl = weights.globals() if weights is not None else synth_globals(cfg)
        self.embed = t(gl["embed"])
        self.lm_head = t(gl["lm_head"][rank * self.vl:(rank + 1) * self.vl])
        self.final_norm = t(gl["final_norm"])
        self.inv_freq = t(make_inv_freq(cfg.head_dim, cfg.rope_base))
        z = lambda *s, dt=torch.float16: torch.zeros(*s, dtype=dt, device=device)
        # KV cache: contiguous [layer, max_seq, dl], or paged: kv_page_rows (a power of two) rows per page and a
        # table logical page -> physical page (identity unless kv_page_table is given; the same table for every layer)
        self.kv_page_rows = int(kv_page_rows)
        self.page_table = None
        phys_rows = cfg.max_seq
        if self.kv_page_rows:
            n_pages = (cfg.max_seq + self.kv_page_rows - 1) // self.kv_page_rows
            table = np.arange(n_pages, dtype=np.int32) if kv_page_table is None else np.asarray(kv_page_table, np.int32)
            assert table.shape == (n_pages,) and sorted(table.tolist()) == list(range(n_pages)), "kv_page_table must be a permutation of the pages"
            self.page_table = torch.from_numpy(table).to(device)
            phys_rows = n_pages * self.kv_page_rows
        self.k_cache = z(cfg.n_layers, phys_rows, self.dl)
        self.v_cache = z(cfg.n_layers, phys_rows, self.dl)
        self.x = z(cfg.dim, dt=torch.float32)
        self.xb = z(cfg.dim)
        self.vqk = z(3 * self.dl)
        self.q = z(self.dl)
        self.att = z(self.dl)
        self.gu = z(2 * self.fl)
        self.h = z(self.fl)
        self.partial = z(cfg.dim, dt=torch.float32)
        self.logits_local = z(self.vl, dt=torch.float32)
        self.logits = self.logits_local if world == 1 else z(cfg.vocab, dt=torch.float32)
        self.token = torch.zeros(1, dtype=torch.int32, device=device)
        self.pos = torch.zeros(1, dtype=torch.int32, device=device)
        self.max_tokens = max_tokens
        self.prompt = torch.zeros(max_tokens, dtype=torch.int32, device=device)
        self.out_tokens = torch.zeros(max_tokens + 1, dtype=torch.int32, device=device)
        self.n_prompt = 0
        self.att_scale = 1.0 / math.sqrt(cfg.head_dim)
        self.graph = None
        self.graph_io = None
        self._ref_cache = {}
        self.tiled = bool(tiled)
        self.fused_allreduce = bool(fused_allreduce)  # tensor parallel: sum over ranks inside the O / down projection kernels
        self.launches_per_step = 0
        self._steps_left = 0   # host count of steps the cache and the token log still have room for
        self.gemv_impl_by_shape = {}
        self._prefill_graphs = {}  # prompt length -> (CUDA graph of the batched prompt pass, its buffers)
        self.prefetch = int(prefetch)   # 1: every projection kernel also pulls the next one's weights into L2
        self._plist = []
        for w in self.layers:
            for k in ("vqk", "o", "gu", "down"):
                self._plist.append((w[k + "_q"], w[k + "_s"]))
        self._pin_in = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._pin_out = torch.zeros(1, dtype=torch.int32).pin_memory()

    # -- one decode step, eager (enqueues every kernel on the current stream) --------------------
    def _proj(self, x, q, s, out, prologue=0, epilogue=0, norm_w=None):
        """One fused W4A16 projection launch (prologue 0 plain / 1 RMSNorm of the fp32 residual /
        2 SiLU(gate)*up; epilogue 0 fp16 / 1 residual += / 2 fp32 partial)."""
        if self.tiled:  # q: [N/128, K/8, 128]
            K, N = q.shape[1] * 8, q.shape[0] * q.shape[2]
            if self.gemv_impl_by_shape:  # tuning aid: kernel variant per projection shape, {(K, N): gemv_impl}
                call("ab200_set_option", b"gemv_impl", int(self.gemv_impl_by_shape.get((K, N), 0)))
            call("ab200_w4a16_gemv_tiled", x.data_ptr(), prologue, 0 if norm_w is None else norm_w.data_ptr(), self.cfg.eps,
                 q.data_ptr(), s.data_ptr(), out.data_ptr(), epilogue, 1, K, N, self.cfg.group, self._st)
        else:
            K, N = q.shape[0] * 8, q.shape[1]
            if self.prefetch == 1:
                # the projection kernel itself pulls the NEXT projection's weights into L2 while it streams
                nq, ns = self._plist[(self._pi + 1) % len(self._plist)]
                call("ab200_w4a16_gemv_prefetch_hint", nq.data_ptr(), nq.numel() * 4, ns.data_ptr(), ns.numel() * 2)
                self._pi += 1
            call("ab200_w4a16_gemv_fused", x.data_ptr(), prologue, 0 if norm_w is None else norm_w.data_ptr(), self.cfg.eps,
                 q.data_ptr(), s.data_ptr(), out.data_ptr(), epilogue, 1, K, N, self.cfg.group, 0, 0, self._st)
        self._n += 1

    def _row_parallel(self, x, q, s, prologue):
        """Row-parallel projection + residual: fused when alone, all-reduce of fp32 partials otherwise."""
        if self.world == 1:
            self._proj(x, q, s, self.x, prologue, 1)
        elif self.fused_allreduce and self.tiled and hasattr(self.comm, "gemv_all_reduce_residual_"):
            self.comm.gemv_all_reduce_residual_(self.x, x, q, s, prologue)  # projection + sum over ranks + residual: one kernel
            self._n += 1
        elif hasattr(self.comm, "all_reduce_residual_"):
            self._proj(x, q, s, self.partial, prologue, 2)
            self.comm.all_reduce_residual_(self.x, self.partial)   # push all-reduce + residual in one kernel
            self._n += 1
        else:
            self._proj(x, q, s, self.partial, prologue, 2)
            self.comm.all_reduce_sum_(self.partial)
            call("ab200_residual_add", self.x.data_ptr(), self.partial.data_ptr(), self.cfg.dim, self._st)
            self._n += 1

    def step_eager(self):
        cfg = self.cfg
        self._st = torch.cuda.current_stream().cuda_stream
        self._n = 0
        self._pi = 0
        st = self._st
        call("ab200_embed_lookup", self.embed.data_ptr(), self.token.data_ptr(), self.x.data_ptr(), cfg.dim, cfg.vocab, st)
        self._n += 1
        for l, w in enumerate(self.layers):
            self._proj(self.x, w["vqk_q"], w["vqk_s"], self.vqk, 1, 0, w["att_norm"])        # RMSNorm + V|Q|K
            if self.page_table is None:
                call("ab200_attention_fused", self.vqk.data_ptr(), self.inv_freq.data_ptr(), self.pos.data_ptr(),
                     self.k_cache[l].data_ptr(), self.v_cache[l].data_ptr(), self.att.data_ptr(), self.hl, cfg.head_dim,
                     self.dl, cfg.max_seq, self.att_scale, st)                              # RoPE + cache + attention
            else:
                call("ab200_attention_fused_paged", self.vqk.data_ptr(), self.inv_freq.data_ptr(), self.pos.data_ptr(),
                     self.k_cache[l].data_ptr(), self.v_cache[l].data_ptr(), self.att.data_ptr(), self.hl, cfg.head_dim,
                     self.dl, cfg.max_seq, self.att_scale, self.page_table.data_ptr(), self.kv_page_rows, st)
            self._n += 1
            self._row_parallel(self.att, w["o_q"], w["o_s"], 0)                               # O + residual
            self._proj(self.x, w["gu_q"], w["gu_s"], self.gu, 1, 0, w["ffn_norm"])           # RMSNorm + gate|up
            self._row_parallel(self.gu, w["down_q"], w["down_s"], 2)                          # SiLU*up + down + residual
        call("ab200_rmsnorm", self.x.data_ptr(), 1, self.final_norm.data_ptr(), self.xb.data_ptr(), 1, cfg.dim, cfg.eps, st)
        call("ab200_dense_gemv", self.xb.data_ptr(), self.lm_head.data_ptr(), self.logits_local.data_ptr(), cfg.dim, self.vl, st)
        self._n += 2
        if self.world > 1 and hasattr(self.comm, "greedy_next_"):
            # vocabulary-parallel argmax: candidates exchanged by peer stores, no gather of logits
            self.comm.greedy_next_(self.logits_local, self.rank * self.vl, self.prompt, self._n_prompt_capture,
                                   self.token, self.pos, self.out_tokens)
        else:
            if self.world > 1:
                self.comm.all_gather_into(self.logits, self.logits_local)
            call("ab200_greedy_next", self.logits.data_ptr(), cfg.vocab, self.prompt.data_ptr(), self._n_prompt_capture,
                 self.token.data_ptr(), self.pos.data_ptr(), self.out_tokens.data_ptr(), self.out_tokens.numel(), st)
        self._n += 1
        self.launches_per_step = self._n

    # -- batched prefill -------------------------------------------------------------------------------
    def _ref_layout(self, l, k):
        """Weights of projection k of layer l in the checkpoint's [K/8, N] layout (what the prefill GEMM
        takes); made once, on the device, from the tile-major copies the decode kernels stream."""
        key = (l, k)
        if key not in self._ref_cache:
            q, s = self.layers[l][k + "_q"], self.layers[l][k + "_s"]
            if self.tiled:
                q = q.permute(1, 0, 2).reshape(q.shape[1], -1).contiguous()
                s = s.permute(1, 0, 2).reshape(s.shape[1], -1).contiguous()
            self._ref_cache[key] = (q, s)
        return self._ref_cache[key]

    def prefill(self, prompt):
        """Runs the whole prompt through the model in one pass (every projection is one tensor-core
        GEMM over all prompt tokens, attention is causal over the freshly written cache rows) instead
        of token by token as the reference does (samples/05_llama2_7b_int4.py:194-200).  Leaves the
        decoder exactly where token-by-token feeding would: cache rows 0..T-1 filled, pos = T,
        token = the first generated token.  Returns that token (int).
        Tensor parallel: the column-parallel projections are GEMMs on the rank's shard, the row-parallel ones
        (O, down) produce fp16 partial sums that are added across ranks with one all-reduce each (on the
        process group, i.e. NCCL), the classifier is vocabulary-parallel as in the decode step; the pass runs
        eagerly (no graph) there."""
        cfg = self.cfg
        prompt = np.asarray(prompt, np.int32)
        T = int(len(prompt))
        assert 1 <= T <= cfg.max_seq and T <= self.max_tokens
        self.reset(torch.from_numpy(prompt).to(self.dev))
        cached = self._prefill_graphs.get(T)
        if self.world > 1:
            self._prefill_pass(T, self._prefill_buffers(T))
        elif cached is None:
            # first prompt of this length: run the pass eagerly, then record it as a CUDA graph over the same
            # buffers (352 launches at 32 layers: replayed, the pass is bound by the GPU, not by the host)
            bufs = self._prefill_buffers(T)
            self._prefill_pass(T, bufs)
            side = torch.cuda.Stream(device=self.dev)
            side.wait_stream(torch.cuda.current_stream())
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    self._prefill_pass(T, bufs)
            torch.cuda.current_stream().wait_stream(side)
            if len(self._prefill_graphs) >= 4:  # a few prompt lengths at most stay recorded
                self._prefill_graphs.pop(next(iter(self._prefill_graphs)))
            self._prefill_graphs[T] = (graph, bufs)
        else:
            cached[0].replay()
        self._steps_left = min(cfg.max_seq, self.max_tokens) - T
        return int(self.token.item())

    def _prefill_buffers(self, T):
        d, dl, f, dev = self.cfg.dim, self.dl, self.fl, self.dev
        h16 = lambda *shape: torch.empty(*shape, dtype=torch.float16, device=dev)
        return dict(x=torch.empty(T, d, dtype=torch.float32, device=dev), xb=h16(T, d), vqk=h16(T, 3 * dl), q=h16(T, dl), att=h16(T, dl),
                    o=h16(T, d), gu=h16(T, 2 * f), hh=h16(T, f))

    def _prefill_pass(self, T, b):
        """The launches of one batched prompt pass on torch's current stream; reads self.prompt[:T], pos = 0."""
        cfg = self.cfg
        st = torch.cuda.current_stream().cuda_stream
        toks = self.prompt[:T]
        d, f = cfg.dim, self.fl
        x, xb, vqk, q, att, o, gu, hh = b["x"], b["xb"], b["vqk"], b["q"], b["att"], b["o"], b["gu"], b["hh"]
        call("ab200_embed_rows", self.embed.data_ptr(), toks.data_ptr(), x.data_ptr(), T, d, cfg.vocab, st)

        def gemm(a, l, k, out):
            qw, sc = self._ref_layout(l, k)
            call("ab200_w4a16_gemm", a.data_ptr(), qw.data_ptr(), sc.data_ptr(), out.data_ptr(), T, qw.shape[0] * 8, qw.shape[1], cfg.group, 0, st)

        for l, w in enumerate(self.layers):
            call("ab200_rmsnorm", x.data_ptr(), 1, w["att_norm"].data_ptr(), xb.data_ptr(), T, d, cfg.eps, st)
            gemm(xb, l, "vqk", vqk)
            if self.page_table is None:
                call("ab200_rope_kv_store_rows", vqk.data_ptr(), self.inv_freq.data_ptr(), self.pos.data_ptr(), q.data_ptr(),
                     self.k_cache[l].data_ptr(), self.v_cache[l].data_ptr(), T, self.hl, cfg.head_dim, self.dl, cfg.max_seq, st)
                call("ab200_attention_prefill", q.data_ptr(), self.k_cache[l].data_ptr(), self.v_cache[l].data_ptr(), att.data_ptr(),
                     self.pos.data_ptr(), T, cfg.max_seq, self.hl, cfg.head_dim, self.dl, self.att_scale, st)
            else:
                pt, pr = self.page_table.data_ptr(), self.kv_page_rows
                call("ab200_rope_kv_store_rows_paged", vqk.data_ptr(), self.inv_freq.data_ptr(), self.pos.data_ptr(), q.data_ptr(),
                     self.k_cache[l].data_ptr(), self.v_cache[l].data_ptr(), T, self.hl, cfg.head_dim, self.dl, cfg.max_seq, pt, pr, st)
                call("ab200_attention_prefill_paged", q.data_ptr(), self.k_cache[l].data_ptr(), self.v_cache[l].data_ptr(), att.data_ptr(),
                     self.pos.data_ptr(), T, cfg.max_seq, self.hl, cfg.head_dim, self.dl, self.att_scale, pt, pr, st)
            gemm(att, l, "o", o)
            if self.world > 1:
                self.comm.all_reduce_sum_(o)
            call("ab200_residual_add_f16", x.data_ptr(), o.data_ptr(), T * d, st)
            call("ab200_rmsnorm", x.data_ptr(), 1, w["ffn_norm"].data_ptr(), xb.data_ptr(), T, d, cfg.eps, st)
            gemm(xb, l, "gu", gu)
            call("ab200_silu_mul_rows", gu.data_ptr(), hh.data_ptr(), T, f, st)
            gemm(hh, l, "down", o)
            if self.world > 1:
                self.comm.all_reduce_sum_(o)
            call("ab200_residual_add_f16", x.data_ptr(), o.data_ptr(), T * d, st)
        # classifier on the last token only, then the same bookkeeping as a decode step at pos = T - 1
        self.x.copy_(x[T - 1])
        self.pos.fill_(T - 1)
        call("ab200_rmsnorm", self.x.data_ptr(), 1, self.final_norm.data_ptr(), self.xb.data_ptr(), 1, d, cfg.eps, st)
        call("ab200_dense_gemv", self.xb.data_ptr(), self.lm_head.data_ptr(), self.logits_local.data_ptr(), d, self.vl, st)
        if self.world > 1 and hasattr(self.comm, "greedy_next_"):
            self.comm.greedy_next_(self.logits_local, self.rank * self.vl, self.prompt, T, self.token, self.pos, self.out_tokens)
        else:
            if self.world > 1:
                self.comm.all_gather_into(self.logits, self.logits_local)
            call("ab200_greedy_next", self.logits.data_ptr(), cfg.vocab, self.prompt.data_ptr(), T, self.token.data_ptr(), self.pos.data_ptr(),
                 self.out_tokens.data_ptr(), self.out_tokens.numel(), st)
        self.out_tokens[:T].copy_(toks)

    # -- graph ---------------------------------------------------------------------------------------
    def capture(self, n_prompt):
        """Captures one step as a CUDA graph.  n_prompt is baked into the graph (the argmax kernel
        forces prompt tokens while pos + 1 < n_prompt)."""
        self._n_prompt_capture = int(n_prompt)
        side = torch.cuda.Stream(device=self.dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.reset(self.prompt[:max(n_prompt, 1)].clone())
            for _ in range(2):  # warm-up outside capture (first-use attribute calls, NCCL setup)
                self.step_eager()
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                self.step_eager()
            # the same step between the copy of a host token id in and the copy of the chosen id out
            # (pinned host buffers), for step(): one launch per token instead of three stream operations
            self.graph_io = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph_io, stream=side):
                self.token.copy_(self._pin_in, non_blocking=True)
                self.step_eager()
                self._pin_out.copy_(self.token, non_blocking=True)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        return self

    def reset(self, prompt_dev):
        """Start a new sequence: pos = 0, token = prompt[0]."""
        n = int(prompt_dev.numel())
        assert 1 <= n <= self.max_tokens
        self.n_prompt = n
        self.prompt[:n].copy_(prompt_dev)
        self.token.copy_(self.prompt[:1])
        self.pos.zero_()
        self.out_tokens.zero_()
        self.out_tokens[:1].copy_(self.prompt[:1])
        self._steps_left = min(self.cfg.max_seq, self.max_tokens)

    def generate(self, prompt, n_new, batched_prefill=False):
        """Generates n_new tokens greedily after the prompt.  By default the prompt is fed token by
        token through the decode step (as the reference does, lines 194-200); with batched_prefill
        it goes through prefill() in one pass.  Returns all n_prompt + n_new token ids (numpy)."""
        prompt = np.asarray(prompt, np.int32)
        n_prompt = len(prompt)
        total = n_prompt + n_new
        assert total <= self.cfg.max_seq + 1 and total <= self.max_tokens
        if self.graph is None or self._n_prompt_capture != n_prompt:
            self.prompt[:n_prompt].copy_(torch.from_numpy(prompt))
            self.capture(n_prompt)
        if batched_prefill and n_new >= 1:
            self.prefill(prompt)                 # produces the first new token
            for _ in range(n_new - 1):
                self.graph.replay()
        else:
            self.reset(torch.from_numpy(prompt).to(self.dev))
            for _ in range(total - 1):
                self.graph.replay()
        torch.cuda.synchronize()
        return self.out_tokens[:total].cpu().numpy()

    def step(self, token):
        """Public per-token call with HOST token ids: copies the id in, runs one step, copies the
        chosen id out.  Position advances on the device; the host counts the steps taken since
        reset() / prefill() and raises once the KV cache (max_seq rows) or the token log
        (max_tokens + 1 ids) is full, instead of stepping past them."""
        if self.graph is None:
            raise RuntimeError("step(): call capture() first")
        if self._steps_left <= 0:
            raise IndexError("step(): the sequence has reached max_seq=%d / max_tokens=%d; reset() first" % (self.cfg.max_seq, self.max_tokens))
        self._steps_left -= 1
        self._pin_in[0] = int(token)
        self.graph_io.replay()
        torch.cuda.current_stream().synchronize()
        return int(self._pin_out[0])

    # bytes one step must move through HBM on this rank (the roofline numerator for decode)
    def step_bytes(self, pos):
        cfg, g = self.cfg, self.cfg.group
        def lin(K, N):
            return K * N // 2 + (K // g) * N * 2 + K * 2 + N * 2
        per_layer = lin(cfg.dim, 3 * self.dl) + lin(self.dl, cfg.dim) + lin(cfg.dim, 2 * self.fl) + lin(self.fl, cfg.dim)
        per_layer += 2 * (pos + 1) * self.dl * 2  # K and V rows read by attention
        return cfg.n_layers * per_layer + self.vl * cfg.dim * 2
