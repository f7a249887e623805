"""CPU tests of the GPTQ checkpoint loader (samples/05_llama2_7b_int4.py:11-107 is the loading code
it replaces): a synthetic checkpoint in the checkpoint's key naming round-trips bit-exactly, and
the three things the sample silently discards (qzeros, g_idx, bias) are checked instead."""
import numpy as np
import pytest

from antares_b200 import gptq
from antares_b200.llama import LlamaConfig, synth_globals, synth_layer

CFG = LlamaConfig(dim=256, n_heads=2, ffn=384, vocab=512, n_layers=2, max_seq=64)


def _write(tmp_path, **kw):
    layers = [synth_layer(CFG, l) for l in range(CFG.n_layers)]
    glob = synth_globals(CFG)
    path = str(tmp_path / "model.safetensors")
    gptq.write_gptq_checkpoint(path, CFG, layers, glob, **kw)
    return path, layers, glob


def test_round_trip_is_bit_exact(tmp_path):
    path, layers, glob = _write(tmp_path)
    w = gptq.GptqLlamaWeights(path, CFG)
    for l in range(CFG.n_layers):
        got = w.layer(l)
        assert set(got) == set(layers[l])
        for k in got:
            assert got[k].dtype == layers[l][k].dtype and np.array_equal(got[k], layers[l][k]), (l, k)
    g = w.globals()
    for k in ("embed", "lm_head", "final_norm"):
        assert np.array_equal(g[k], glob[k])


def test_fused_order_is_v_q_k(tmp_path):
    """Line 27 of the sample concatenates V, Q, K in that order along N."""
    from safetensors import safe_open
    path, layers, _ = _write(tmp_path)
    with safe_open(path, framework="np") as f:
        v = f.get_tensor("model.layers.0.self_attn.v_proj.qweight")
        k = f.get_tensor("model.layers.0.self_attn.k_proj.qweight")
    fused = gptq.GptqLlamaWeights(path, CFG).layer(0)["vqk_q"]
    d = CFG.dim
    assert np.array_equal(fused[:, :d], v) and np.array_equal(fused[:, 2 * d:], k)


def test_asymmetric_zero_points_are_rejected(tmp_path):
    path, _, _ = _write(tmp_path, qzero_word=0x77777776)
    with pytest.raises(gptq.CheckpointError, match="zero-points other than 8"):
        gptq.GptqLlamaWeights(path, CFG).layer(0)
    gptq.GptqLlamaWeights(path, CFG, validate=False).layer(0)  # the sample's behaviour: ignore them


def test_act_order_is_rejected(tmp_path):
    path, _, _ = _write(tmp_path, act_order=True)
    with pytest.raises(gptq.CheckpointError, match="act-order"):
        gptq.GptqLlamaWeights(path, CFG).layer(0)


def test_wrong_layer_count_is_reported(tmp_path):
    path, _, _ = _write(tmp_path)
    with pytest.raises(gptq.CheckpointError, match="3 layers"):
        gptq.GptqLlamaWeights(path, LlamaConfig(dim=256, n_heads=2, ffn=384, vocab=512, n_layers=3, max_seq=64))


def test_token_text_helpers():
    vocab = ["<unk>", "<s>", "</s>", " How", " large", "is", "<0x0A>", " Ocean"]
    d = {w: i for i, w in enumerate(vocab)}
    assert gptq.encode_prompt("How large is Ocean", d) == [1, 3, 4, 5, 7]
    assert gptq.decode_piece(1, 3, vocab) == "How"        # the space after BOS is dropped
    assert gptq.decode_piece(3, 4, vocab) == " large"
    assert gptq.decode_piece(4, 6, vocab) == "\n"          # byte token
