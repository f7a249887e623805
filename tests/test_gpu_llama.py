"""GPU parity of the full decode step against the CPU oracle: logits within 1e-2 * max|ref| under
teacher forcing, and identical greedy token ids (the full-decode workload's correctness bar)."""
import json
import os

import numpy as np
import pytest
import torch

from antares_b200 import ops
from antares_b200.llama import LlamaConfig, LlamaInt4Decoder, synth_prompt
from oracle.llama_oracle import OracleLlama

pytestmark = pytest.mark.gpu
TOL = 1e-2


def test_two_layer_logits_and_tokens(cuda):
    cfg = LlamaConfig(n_layers=2, max_seq=64)
    prompt = synth_prompt(cfg, 5, 1)
    ref_tokens, ref_logits = OracleLlama(cfg).generate(prompt, 12, return_logits=True)
    dec = LlamaInt4Decoder(cfg, cuda)
    tokens = dec.generate(prompt, 12)
    assert list(tokens) == list(ref_tokens)
    # teacher-forced logits through the host-token API
    dec.reset(torch.from_numpy(prompt).to(cuda))
    for pos in range(len(ref_tokens) - 1):
        dec.step(int(ref_tokens[pos]))
        lg = dec.logits.cpu().numpy()
        ref = ref_logits[pos]
        assert np.abs(lg - ref).max() <= TOL * np.abs(ref).max(), "logits differ at position %d" % pos
    assert ops.kernel_status() == 0


def test_full_model_tokens_match_golden(cuda, golden_dir):
    """32 layers, 8-token prompt, 32 greedy tokens: ids equal to those the CPU oracle produced
    (tests/golden/llama_tokens.json), and bitwise repeatable across two runs."""
    g = json.load(open(os.path.join(golden_dir, "llama_tokens.json")))["p8_n32"]
    cfg = LlamaConfig(max_seq=64)
    prompt = synth_prompt(cfg, g["n_prompt"], g["prompt_seed"])
    assert list(prompt) == g["tokens"][:g["n_prompt"]]
    dec = LlamaInt4Decoder(cfg, cuda)
    tokens = dec.generate(prompt, g["n_new"])
    assert list(tokens) == g["tokens"], "greedy ids differ from the oracle's (min top-2 logit gap there: %g)" % g["min_top2_gap"]
    lg1 = dec.logits.clone()
    assert list(dec.generate(prompt, g["n_new"])) == g["tokens"]
    assert torch.equal(dec.logits, lg1)
    # last-step logits against the stored oracle values
    head = np.array(g["last_logits_head"], np.float32)
    assert np.abs(lg1[:16].cpu().numpy() - head).max() <= TOL * g["last_logits_max"]


def test_decoder_from_gptq_checkpoint_file(cuda, tmp_path):
    """The checkpoint route (safetensors file in the GPTQ key naming -> loader -> decoder) gives the
    same tokens and logits as the in-memory weights it was written from."""
    from antares_b200 import gptq
    from antares_b200.llama import synth_globals, synth_layer
    cfg = LlamaConfig(n_layers=2, max_seq=64)
    path = str(tmp_path / "model.safetensors")
    gptq.write_gptq_checkpoint(path, cfg, [synth_layer(cfg, l) for l in range(cfg.n_layers)], synth_globals(cfg))
    prompt = synth_prompt(cfg, 5, 1)
    ref = LlamaInt4Decoder(cfg, cuda)
    want = ref.generate(prompt, 10)
    want_logits = ref.logits.clone()
    dec = LlamaInt4Decoder(cfg, cuda, weights=gptq.GptqLlamaWeights(path, cfg))
    assert list(dec.generate(prompt, 10)) == list(want)
    assert torch.equal(dec.logits, want_logits)


def test_batched_prefill_matches_token_by_token(cuda):
    """The whole prompt through the tensor-core GEMM + causal attention leaves the decoder where
    feeding it token by token does: same generated tokens, next-token logits within tolerance, and
    the cache rows written by both routes agree."""
    cfg = LlamaConfig(n_layers=2, max_seq=192)
    prompt = synth_prompt(cfg, 130, 3)   # not a multiple of the GEMM's 256-row tile
    a = LlamaInt4Decoder(cfg, cuda)
    want = a.generate(prompt, 6)
    k_ref, v_ref = a.k_cache[:, :130].clone(), a.v_cache[:, :130].clone()
    b = LlamaInt4Decoder(cfg, cuda)
    got = b.generate(prompt, 6, batched_prefill=True)
    assert list(got) == list(want)
    # cache rows of layer 0 depend only on the embeddings: both routes must agree within tolerance there;
    # deeper layers see each other's rounding through softmax and are compared by their typical error
    for ref, new in ((k_ref, b.k_cache[:, :130]), (v_ref, b.v_cache[:, :130])):
        ref, new = ref.float(), new.float()
        assert float((new[0] - ref[0]).abs().max()) <= TOL * float(ref[0].abs().max())
        rel = (new - ref).abs().amax(dim=-1) / ref.abs().amax(dim=-1).clamp_min(1e-9)
        assert float(rel.median()) <= TOL
    # logits of the first generated token against the oracle (teacher-forced prompt)
    ref_tokens, ref_logits = OracleLlama(cfg).generate(prompt[:8], 1, return_logits=True)
    c = LlamaInt4Decoder(cfg, cuda)
    c.prefill(prompt[:8])
    lg = c.logits.cpu().numpy()
    assert np.abs(lg - ref_logits[7]).max() <= TOL * np.abs(ref_logits[7]).max()
    assert int(c.token.item()) == int(ref_tokens[8])
    # a second prompt of the same length replays the recorded pass: same result as a fresh decoder's first pass
    other = synth_prompt(cfg, 8, 5)
    first_tok, first_logits = c.prefill(other), c.logits.clone()
    c.prefill(prompt[:8])
    assert torch.equal(c.logits, torch.from_numpy(lg).to(cuda))
    fresh = LlamaInt4Decoder(cfg, cuda)
    assert fresh.prefill(other) == first_tok and torch.equal(fresh.logits, first_logits)
    assert ops.kernel_status() == 0


def test_paged_kv_cache_is_bitwise_the_contiguous_one(cuda):
    """A cache handed out in pages of 16 rows through a shuffled page table gives bit-identical logits and tokens,
    token by token and through the batched prompt pass, and its rows are the contiguous cache's rows, permuted."""
    cfg = LlamaConfig(n_layers=2, max_seq=96)
    prompt = synth_prompt(cfg, 37, 11)
    rows = 16
    table = np.random.default_rng(5).permutation(cfg.max_seq // rows).astype(np.int32)
    for batched in (False, True):
        flat = LlamaInt4Decoder(cfg, cuda)
        paged = LlamaInt4Decoder(cfg, cuda, kv_page_rows=rows, kv_page_table=table)
        want = flat.generate(prompt, 9, batched_prefill=batched)
        got = paged.generate(prompt, 9, batched_prefill=batched)
        assert list(got) == list(want)
        assert torch.equal(paged.logits, flat.logits)
        n = len(prompt) + 8                                # cache rows written: positions 0 .. n - 1
        s = torch.arange(n, device=cuda)
        phys = torch.from_numpy(table).to(cuda)[s // rows].long() * rows + s % rows
        assert torch.equal(paged.k_cache[:, phys], flat.k_cache[:, :n]) and torch.equal(paged.v_cache[:, phys], flat.v_cache[:, :n])
    assert ops.kernel_status() == 0


def test_paged_calls_reject_bad_page_tables(cuda):
    from antares_b200 import _lib
    cfg = LlamaConfig(n_layers=1, max_seq=64)
    dec = LlamaInt4Decoder(cfg, cuda, kv_page_rows=16)
    st = torch.cuda.current_stream().cuda_stream
    args = (dec.vqk.data_ptr(), dec.inv_freq.data_ptr(), dec.pos.data_ptr(), dec.k_cache[0].data_ptr(), dec.v_cache[0].data_ptr(),
            dec.att.data_ptr(), dec.hl, cfg.head_dim, dec.dl, cfg.max_seq, dec.att_scale)
    with pytest.raises(_lib.Ab200Error):
        _lib.call("ab200_attention_fused_paged", *args, dec.page_table.data_ptr(), 12, st)   # not a power of two
    with pytest.raises(_lib.Ab200Error):
        _lib.call("ab200_attention_fused_paged", *args, 0, 16, st)                           # no table
    with pytest.raises(AssertionError):
        LlamaInt4Decoder(cfg, cuda, kv_page_rows=16, kv_page_table=[0, 0, 1, 2])              # not a permutation


def _teacher_forced_logits(dec, tokens, positions, cuda):
    """Feeds `tokens` one by one through the host-token API and returns {position: logits} for the
    requested positions (logits after the token at that position went in)."""
    dec.reset(torch.from_numpy(np.asarray(tokens[:1], np.int32)).to(cuda))
    got = {}
    for pos in range(max(positions) + 1):
        dec.step(int(tokens[pos]))
        if pos in positions:
            got[pos] = dec.logits.cpu().numpy().copy()
    return got


def test_benchmark_workload_tokens_and_full_logits(cuda, golden_dir):
    """The benchmark's own workload at 32 layers: 128-token prompt + the first 32 greedy tokens equal
    the oracle's, and the full 32000-entry logits at three teacher-forced positions (early prompt, last
    prompt token, last generated step) are within 1e-2 * max|ref| of the oracle's."""
    g = json.load(open(os.path.join(golden_dir, "llama_tokens.json")))["p128_n32"]
    lg = np.load(os.path.join(golden_dir, "llama_logits.npz"))
    cfg = LlamaConfig(max_seq=192)
    prompt = synth_prompt(cfg, g["n_prompt"], g["prompt_seed"])
    assert list(prompt) == g["tokens"][:g["n_prompt"]]
    dec = LlamaInt4Decoder(cfg, cuda, max_tokens=192)
    tokens = dec.generate(prompt, g["n_new"])
    assert list(tokens) == g["tokens"], "greedy ids differ from the oracle's (min top-2 logit gap there: %g)" % g["min_top2_gap"]
    got = _teacher_forced_logits(dec, g["tokens"], set(g["logits_at"]), cuda)
    for pos in g["logits_at"]:
        ref = lg["p128_n32_pos%d" % pos]
        assert ref.shape == (cfg.vocab,)
        err = np.abs(got[pos] - ref).max() / np.abs(ref).max()
        assert err <= TOL, "position %d: max|err| = %.3g of max|ref|" % (pos, err)
    assert ops.kernel_status() == 0


def test_non_degenerate_stream_matches_the_oracle(cuda, golden_dir):
    """Test-only weights (zero-mean nibbles, scales times 0.25): the oracle's greedy stream keeps moving
    (16 distinct ids among the 32), so equal ids here say something about attention, the cache and
    position handling on generated steps.  The free-running ids must agree up to the first step whose
    top-2 logit gap in the oracle is inside the tolerance (after a legitimate near-tie the streams may
    part); under teacher forcing every step with a clear gap must pick the oracle's id, and the full
    logits at three positions must be within tolerance.  Tolerance: 2e-2 * max|ref| on this model - a
    deep stack without the benchmark weights' common offset amplifies rounding differences between any
    two implementations (measured with the oracle alone: noise of 5e-4 * max|y| on every projection
    output moves these logits by 1 %, the benchmark model's by 0.03 %)."""
    from antares_b200.llama import SynthWeights
    tol = 2e-2
    g = json.load(open(os.path.join(golden_dir, "llama_tokens.json")))["p8_n32_centered"]
    lg = np.load(os.path.join(golden_dir, "llama_logits.npz"))
    n_prompt, n_new = g["n_prompt"], g["n_new"]
    assert len(set(g["tokens"][n_prompt:])) >= 12
    cfg = LlamaConfig(max_seq=64)
    dec = LlamaInt4Decoder(cfg, cuda, weights=SynthWeights(cfg, centered=True, scale_mul=0.25))
    prompt = np.array(g["tokens"][:n_prompt], np.int32)
    tokens = list(dec.generate(prompt, n_new))
    # gaps[i] belongs to the step that chose token n_prompt + i; a choice is "clear" when the oracle's
    # top-2 gap exceeds twice the logit tolerance (both candidates may move by tol * max|ref|)
    margin = [2 * tol * m for m in g["logit_abs_max"]]
    clear = [gap > mg for gap, mg in zip(g["top2_gaps"], margin)]
    assert sum(clear) >= 12, "the golden stream needs enough clear choices to be a check"
    first_unclear = clear.index(False) if False in clear else n_new
    assert tokens[:n_prompt + first_unclear] == g["tokens"][:n_prompt + first_unclear]
    assert len(set(tokens[n_prompt:])) >= 8, "the GPU's own greedy stream must not settle on one id either"
    # teacher forcing over the whole golden stream
    dec.reset(torch.from_numpy(prompt).to(cuda))
    keep = set(g["logits_at"])
    for pos in range(n_prompt + n_new - 1):
        chosen = dec.step(int(g["tokens"][pos]))
        if pos >= n_prompt - 1 and clear[pos - (n_prompt - 1)]:
            assert chosen == g["tokens"][pos + 1], "position %d" % pos
        if pos in keep:
            ref = lg["p8_n32_centered_pos%d" % pos]
            err = np.abs(dec.logits.cpu().numpy() - ref).max() / np.abs(ref).max()
            assert err <= tol, "position %d: max|err| = %.3g of max|ref|" % (pos, err)
    assert ops.kernel_status() == 0


def test_step_past_the_limits_raises_and_writes_nothing(cuda):
    """step() counts steps on the host and refuses to run past the KV cache or the token log; a bare
    graph replay past the end (no host check) leaves the token log's tail and the position untouched."""
    cfg = LlamaConfig(n_layers=1, max_seq=6)
    dec = LlamaInt4Decoder(cfg, cuda, max_tokens=6)
    prompt = synth_prompt(cfg, 2, 1)
    dec.prompt[:2].copy_(torch.from_numpy(prompt))
    dec.capture(2)
    dec.reset(torch.from_numpy(prompt).to(cuda))
    tok = int(prompt[0])
    for _ in range(6):
        tok = dec.step(tok)
    with pytest.raises(IndexError):
        dec.step(tok)
    before = dec.out_tokens.clone()
    pos_before = int(dec.pos.item())
    assert pos_before == 6
    dec.graph.replay()   # what a caller without the host check would do
    torch.cuda.synchronize()
    assert torch.equal(dec.out_tokens, before) and int(dec.pos.item()) == pos_before
    assert ops.kernel_status() == 0
