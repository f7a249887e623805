"""CPU oracle of the Llama-2-7B-architecture int4 decode step (TEST INFRASTRUCTURE ONLY).

Follows samples/05_llama2_7b_int4.py:146-207 operator by operator, on the plain-C oracle
functions, unsharded, with the numeric contract the product uses: fp32 residual stream, fp16
projection inputs/outputs and KV cache, fp32 accumulation, fp32 logits, first-maximum argmax.
Weights come from the same seeded generator as the product (antares_b200.llama.synth_*).
"""
import numpy as np

from antares_b200 import llama as L
from . import cport


class OracleLlama:
    def __init__(self, cfg, weights=None):
        self.cfg = cfg
        if weights is None:
            weights = L.SynthWeights(cfg)
        self.layers = [weights.layer(l) for l in range(cfg.n_layers)]
        self.g = weights.globals()
        self.inv_freq = L.make_inv_freq(cfg.head_dim, cfg.rope_base)
        self.kc = np.zeros((cfg.n_layers, cfg.max_seq, cfg.dim), np.float16)
        self.vc = np.zeros((cfg.n_layers, cfg.max_seq, cfg.dim), np.float16)
        self.scale = 1.0 / np.sqrt(cfg.head_dim)

    def forward(self, token, pos):
        """Returns fp32 logits [vocab] (lines 146-177)."""
        cfg = self.cfg
        d, H, D = cfg.dim, cfg.n_heads, cfg.head_dim
        x = self.g["embed"][token].astype(np.float32)                      # line 147
        for l, w in enumerate(self.layers):
            xb = cport.rmsnorm(x.reshape(1, d), w["att_norm"], cfg.eps)    # line 150
            vqk = cport.w4a16_gemm(xb, w["vqk_q"], w["vqk_s"], cfg.group)[0]  # line 152, order V, Q, K
            v, q, k = vqk[:d], vqk[d:2 * d], vqk[2 * d:]
            p = np.array([pos], np.int32)
            q = cport.rope(q.reshape(1, H, D), p, self.inv_freq)[0]        # lines 157-158
            self.kc[l, pos] = cport.rope(k.reshape(1, H, D), p, self.inv_freq).reshape(d)
            self.vc[l, pos] = v
            att = cport.attention_decode(q, self.kc[l], self.vc[l], pos + 1, self.scale)  # line 165
            o = cport.w4a16_gemm(att.reshape(1, d), w["o_q"], w["o_s"], cfg.group)[0]     # line 167
            cport.residual_add(x, o)                                       # line 168
            xb = cport.rmsnorm(x.reshape(1, d), w["ffn_norm"], cfg.eps)    # line 169
            gate = cport.w4a16_gemm(xb, w["gate_q"], w["gate_s"], cfg.group)[0]
            up = cport.w4a16_gemm(xb, w["up_q"], w["up_s"], cfg.group)[0]
            h = cport.silu_mul(gate, up)                                   # line 171
            dn = cport.w4a16_gemm(h.reshape(1, cfg.ffn), w["down_q"], w["down_s"], cfg.group)[0]  # line 172
            cport.residual_add(x, dn)                                      # line 173
        xb = cport.rmsnorm(x.reshape(1, d), self.g["final_norm"], cfg.eps)[0]  # line 175
        return cport.dense_gemv_f16(xb, self.g["lm_head"])                # line 176

    def generate(self, prompt, n_new, return_logits=False):
        """Greedy decode with the prompt fed token by token (lines 187-207).  Returns all token
        ids, and optionally the logits of every step."""
        prompt = [int(t) for t in prompt]
        tokens = list(prompt)
        logits_all = []
        token = prompt[0]
        for pos in range(len(prompt) + n_new - 1):
            logits = self.forward(token, pos)
            if return_logits:
                logits_all.append(logits)
            nxt = prompt[pos + 1] if pos + 1 < len(prompt) else cport.argmax(logits)
            if pos + 1 >= len(prompt):
                tokens.append(nxt)
            token = nxt
        return (np.array(tokens, np.int32), logits_all) if return_logits else np.array(tokens, np.int32)
