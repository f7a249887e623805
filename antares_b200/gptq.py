"""Loader for GPTQ int4 Llama checkpoints in the layout the reference's sample consumes
(samples/05_llama2_7b_int4.py:11-107: `TheBloke/Llama-2-7B-Chat-GPTQ`, `model.safetensors`), and the
sample's token <-> text helpers (lines 13-15, 178-189).

What the sample does with the checkpoint, and what this module does instead of doing it silently:
  * `qweight int32 [K/8, N]` and `scales fp16 [K/128, N]` are used as they are (lines 22-29, 41-49);
    V, Q, K are concatenated along N in that order (line 27), here also gate | up (one launch);
  * `qzeros` are DISCARDED and the zero-point is hard-coded to 8 (lines 34-40, 137).  Here they are
    checked: the checkpoint's packed zero-points must all be 7 (AutoGPTQ stores zero - 1, so 7 means
    8, the symmetric 4-bit case); anything else raises, because the kernels implement zero-point 8;
  * `g_idx` is discarded (lines 52-58), i.e. groups are assumed contiguous.  Here a `g_idx` that is
    not `arange(K) // group` (act-order checkpoints) raises;
  * `bias` tensors are discarded (lines 60-66).  Here a non-zero bias raises.

The checkpoint itself is not shipped (no network): tests write a small synthetic file in the same
key naming and read it back.
"""
import re

import numpy as np

_PROJ = {"q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj", "o": "self_attn.o_proj",
         "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj"}


class CheckpointError(ValueError):
    pass


def check_qzeros(qzeros, name):
    """Packed zero-points (int32, 8 nibbles per word, value = zero - 1) must all encode zero-point 8."""
    z = np.asarray(qzeros).view(np.uint32)
    if z.size and not np.all(z == np.uint32(0x77777777)):
        bad = z[z != np.uint32(0x77777777)].ravel()[0]
        raise CheckpointError("%s: zero-points other than 8 are not supported by the W4A16 operator "
                              "(found packed word 0x%08x; the operator's IR fixes the zero-point at 8)" % (name, int(bad)))


def check_g_idx(g_idx, K, group, name):
    g = np.asarray(g_idx).astype(np.int64).ravel()
    if g.size and not np.array_equal(g, np.arange(K, dtype=np.int64) // group):
        raise CheckpointError("%s: g_idx is not arange(K) // %d: act-order (desc_act) checkpoints are not supported" % (name, group))


def check_bias(bias, name):
    b = np.asarray(bias)
    if b.size and np.any(b.astype(np.float32) != 0):
        raise CheckpointError("%s: non-zero bias; the operator path has no bias term" % name)


class GptqLlamaWeights:
    """Weights of a GPTQ int4 Llama checkpoint in the form LlamaInt4Decoder(weights=...) takes:
    `layer(l)` -> dict of unsharded numpy arrays (vqk_q, vqk_s, o_q, o_s, gate_q, gate_s, up_q, up_s,
    down_q, down_s, att_norm, ffn_norm), `globals()` -> dict (embed, lm_head, final_norm)."""

    def __init__(self, path, cfg, validate=True):
        from safetensors import safe_open
        self.cfg, self.validate, self.path = cfg, validate, path
        self._f = safe_open(path, framework="np")
        self._keys = set(self._f.keys())
        need = "model.layers.%d.self_attn.q_proj.qweight" % (cfg.n_layers - 1)
        if need not in self._keys:
            raise CheckpointError("%s has no %s: not a GPTQ Llama checkpoint with %d layers" % (path, need, cfg.n_layers))

    def _get(self, key):
        if key not in self._keys:
            raise CheckpointError("%s: missing tensor %s" % (self.path, key))
        return self._f.get_tensor(key)

    def _proj(self, l, which, K, N):
        base = "model.layers.%d.%s" % (l, _PROJ[which])
        q = self._get(base + ".qweight")
        s = self._get(base + ".scales")
        g = self.cfg.group
        if q.dtype != np.int32 or q.shape != (K // 8, N):
            raise CheckpointError("%s.qweight: expected int32 %s, found %s %s" % (base, (K // 8, N), q.dtype, q.shape))
        if s.shape != (K // g, N):
            raise CheckpointError("%s.scales: expected %s, found %s (group size %d)" % (base, (K // g, N), s.shape, g))
        if self.validate:
            if base + ".qzeros" in self._keys:
                check_qzeros(self._f.get_tensor(base + ".qzeros"), base + ".qzeros")
            if base + ".g_idx" in self._keys:
                check_g_idx(self._f.get_tensor(base + ".g_idx"), K, g, base + ".g_idx")
            if base + ".bias" in self._keys:
                check_bias(self._f.get_tensor(base + ".bias"), base + ".bias")
        return np.ascontiguousarray(q), np.ascontiguousarray(s.astype(np.float16))

    def layer(self, l):
        d, f = self.cfg.dim, self.cfg.ffn
        w = {}
        parts = [self._proj(l, n, d, d) for n in ("v", "q", "k")]  # order V, Q, K (samples/05_llama2_7b_int4.py:27)
        w["vqk_q"] = np.ascontiguousarray(np.concatenate([p[0] for p in parts], axis=1))
        w["vqk_s"] = np.ascontiguousarray(np.concatenate([p[1] for p in parts], axis=1))
        w["o_q"], w["o_s"] = self._proj(l, "o", d, d)
        w["gate_q"], w["gate_s"] = self._proj(l, "gate", d, f)
        w["up_q"], w["up_s"] = self._proj(l, "up", d, f)
        w["down_q"], w["down_s"] = self._proj(l, "down", f, d)
        w["att_norm"] = self._get("model.layers.%d.input_layernorm.weight" % l).astype(np.float16)
        w["ffn_norm"] = self._get("model.layers.%d.post_attention_layernorm.weight" % l).astype(np.float16)
        return w

    def globals(self):
        c = self.cfg
        emb = self._get("model.embed_tokens.weight")
        head = self._get("lm_head.weight")
        if emb.shape != (c.vocab, c.dim) or head.shape != (c.vocab, c.dim):
            raise CheckpointError("embedding / lm_head shapes %s / %s do not match vocab %d x dim %d" % (emb.shape, head.shape, c.vocab, c.dim))
        return {"embed": np.ascontiguousarray(emb.astype(np.float16)), "lm_head": np.ascontiguousarray(head.astype(np.float16)),
                "final_norm": self._get("model.norm.weight").astype(np.float16)}


def write_gptq_checkpoint(path, cfg, layers, glob, qzero_word=0x77777777, act_order=False):
    """Writes numpy weights (the dicts of GptqLlamaWeights.layer / .globals, per layer) as a
    safetensors file with the checkpoint's key naming, including the qzeros / g_idx / bias tensors
    a GPTQ export carries.  Used by the tests and to export synthetic models."""
    from safetensors.numpy import save_file
    g, d, f = cfg.group, cfg.dim, cfg.ffn
    t = {"model.embed_tokens.weight": glob["embed"], "lm_head.weight": glob["lm_head"], "model.norm.weight": glob["final_norm"]}

    def put(l, which, q, s, K, N):
        base = "model.layers.%d.%s" % (l, _PROJ[which])
        t[base + ".qweight"] = np.ascontiguousarray(q)
        t[base + ".scales"] = np.ascontiguousarray(s)
        t[base + ".qzeros"] = np.full((K // g, N // 8), qzero_word, dtype=np.uint32).view(np.int32)
        gi = np.arange(K, dtype=np.int32) // g
        t[base + ".g_idx"] = gi[::-1].copy() if act_order else gi
        t[base + ".bias"] = np.zeros(N, dtype=np.float16)

    for l, w in enumerate(layers):
        for i, n in enumerate(("v", "q", "k")):
            put(l, n, w["vqk_q"][:, i * d:(i + 1) * d], w["vqk_s"][:, i * d:(i + 1) * d], d, d)
        put(l, "o", w["o_q"], w["o_s"], d, d)
        put(l, "gate", w["gate_q"], w["gate_s"], d, f)
        put(l, "up", w["up_q"], w["up_s"], d, f)
        put(l, "down", w["down_q"], w["down_s"], f, d)
        t["model.layers.%d.input_layernorm.weight" % l] = w["att_norm"]
        t["model.layers.%d.post_attention_layernorm.weight" % l] = w["ffn_norm"]
    save_file(t, path)


# ---- token <-> text, as the sample does it ------------------------------------------------------------

def load_vocab(path):
    """The sample's vocabulary file is a torch-saved list of 32000 pieces (line 11)."""
    import torch
    vocab = torch.load(path)
    return list(vocab), {w: i for i, w in enumerate(vocab)}


def encode_prompt(text, dictionary, bos=1):
    """Whitespace split, each word looked up with a leading space first (line 188)."""
    return [bos] + [dictionary[" " + w] if (" " + w) in dictionary else dictionary[w] for w in text.split()]


def decode_piece(prev, nxt, vocab, bos=1):
    """Text of token `nxt` following token `prev` (lines 178-184): the space after BOS is dropped,
    byte tokens `<0xNN>` become the character."""
    piece = vocab[nxt]
    if prev == bos and piece.startswith(" "):
        piece = piece[1:]
    if re.match(r"^<0x..>$", piece):
        piece = chr(int(piece[1:-1], 16))
    return piece
