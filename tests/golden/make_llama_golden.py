"""Generates tests/golden/llama_tokens.json with the CPU oracle (oracle/llama_oracle.py):
greedy token ids of the full 32-layer Llama-2-7B-architecture int4 model on seeded synthetic
weights, for (a) an 8-token prompt + 32 generated tokens and (b) the benchmark workload's
128-token prompt + its first 32 generated tokens.  Also records the smallest gap between the best
and second-best logit over the generated steps: a GPU run can only be expected to reproduce the
ids when that gap is well above the numerical tolerance.

  python tests/golden/make_llama_golden.py        (about 5 minutes on 8 cores)
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from antares_b200.llama import LlamaConfig, synth_prompt  # noqa: E402
from oracle.llama_oracle import OracleLlama  # noqa: E402


def run(model, n_prompt, n_new, seed):
    prompt = synth_prompt(model.cfg, n_prompt, seed)
    model.kc[:] = 0
    model.vc[:] = 0
    tokens, logits = model.generate(prompt, n_new, return_logits=True)
    gaps = []
    for lg in logits[n_prompt - 1:]:
        s = np.partition(lg, -2)[-2:]
        gaps.append(float(s[1] - s[0]))
    last = logits[-1]
    return dict(n_prompt=n_prompt, n_new=n_new, prompt_seed=seed, tokens=[int(t) for t in tokens],
                min_top2_gap=min(gaps), logit_std=float(last.std()),
                last_logits_head=[float(v) for v in last[:16]], last_logits_max=float(last.max()))


def main():
    cfg = LlamaConfig()
    model = OracleLlama(cfg)
    out = {"config": "32 layers, d=4096, 32 heads, ffn 11008, vocab 32000, g=128, eps 1e-6, seeds per antares_b200.llama"}
    out["p8_n32"] = run(model, 8, 32, 0)
    print(out["p8_n32"]["tokens"], out["p8_n32"]["min_top2_gap"], flush=True)
    out["p128_n32"] = run(model, 128, 32, 0)
    print(out["p128_n32"]["tokens"][128:], out["p128_n32"]["min_top2_gap"], flush=True)
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "llama_tokens.json"), "w") as f:
        json.dump(out, f, indent=1)


if __name__ == "__main__":
    main()
