"""CPU tests: the C oracle against the golden vectors produced by the reference's own CPU runtime,
and against an independent numpy restatement."""
import hashlib
import json
import os

import numpy as np
import pytest

from antares_b200 import packing
from oracle import cport

TOL = 1e-2  # outputs: max|err| <= TOL * max|ref|


def _load(golden_dir, name):
    return dict(np.load(os.path.join(golden_dir, name)))


def _close(a, b, tol=TOL):
    a, b = a.astype(np.float32), b.astype(np.float32)
    return np.abs(a - b).max() <= tol * np.abs(b).max()


@pytest.mark.parametrize("name", ["w4a16_f16_m1_k256_n64.npz", "w4a16_f16_m3_k512_n128.npz", "w4a16_f32_m2_k256_n64.npz"])
def test_w4a16_matches_reference_runtime(golden_dir, name):
    g = _load(golden_dir, name)
    w = cport.w4_dequant(g["qweight"], g["scales"])
    # dequantised weights: bit-exact
    assert np.array_equal(w.view(np.uint8), g["w"].view(np.uint8))
    y = cport.w4a16_gemm(g["x"], g["qweight"], g["scales"])
    assert _close(y, g["y"])
    if g["x"].dtype == np.float16:
        # same accumulation order as the reference kernel text -> identical fp16 results
        assert np.array_equal(y.view(np.uint16), g["y"].view(np.uint16))


def test_dequant_table_bit_exact(golden_dir):
    g = _load(golden_dir, "w4_dequant_table_f16.npz")
    assert np.array_equal(cport.w4_unpack(g["qweight"]), g["q"])
    assert np.array_equal(cport.w4_pack(g["q"]), g["qweight"])
    w = cport.w4_dequant(g["qweight"], g["scales"])
    assert np.array_equal(w.view(np.uint16), g["w"].view(np.uint16))
    assert np.array_equal(cport.np_w4_dequant(g["qweight"], g["scales"]).view(np.uint16), g["w"].view(np.uint16))


def test_pack_roundtrip_and_layout():
    rng = np.random.default_rng(3)
    q = rng.integers(0, 16, size=(64, 12), dtype=np.uint8)
    qw = packing.pack_w4(q)
    assert qw.dtype == np.int32 and qw.shape == (8, 12)
    assert np.array_equal(packing.unpack_w4(qw), q)
    assert np.array_equal(cport.w4_pack(q), qw)
    assert np.array_equal(cport.np_w4_unpack(qw), q)
    # lowest nibble = lowest k (samples/05_llama2_7b_int4.py:136)
    one = np.zeros((8, 1), np.uint8)
    one[0, 0] = 5
    one[7, 0] = 9
    assert packing.pack_w4(one).view(np.uint32)[0, 0] == (5 | (9 << 28))
    # negative words (top nibble >= 8) unpack through the arithmetic shift + mask
    neg = np.array([[-1]], np.int32)
    assert np.array_equal(cport.w4_unpack(neg), np.full((8, 1), 15, np.uint8))


def test_c0_digest(golden_dir):
    info = json.load(open(os.path.join(golden_dir, "c0_digest.json")))
    qw, sc = packing.synth_w4(4096, 4096, 0)
    x = packing.synth_x(1, 4096, 1)
    y = cport.w4a16_gemm(x, qw, sc)
    assert hashlib.sha256(y.tobytes()).hexdigest() == info["sha256"]
    assert abs(cport.digest(y) - info["digest_k0"]) <= 1e-5 * abs(info["digest_k0"])


def test_numpy_restatement_agrees():
    qw, sc = packing.synth_w4(512, 64, 5)
    x = packing.synth_x(4, 512, 6)
    assert _close(cport.w4a16_gemm(x, qw, sc), cport.np_w4a16_gemm(x, qw, sc), 2e-3)
    qw32, sc32 = packing.synth_w4(256, 32, 7, scales_dtype=np.float32)
    x32 = packing.synth_x(2, 256, 8, np.float32)
    assert _close(cport.w4a16_gemm(x32, qw32, sc32), cport.np_w4a16_gemm(x32, qw32, sc32), 1e-5)


def test_elementwise_against_reference_runtime(golden_dir):
    g = _load(golden_dir, "softmax_f16_8x256.npz")
    assert _close(cport.softmax(g["x"]), g["y"], 2e-3)
    g = _load(golden_dir, "sigmoid_f32_1000.npz")
    assert _close(cport.sigmoid(g["x"]), g["y"], 1e-6)
    g = _load(golden_dir, "rmsnorm_f16_4x512.npz")
    assert _close(cport.rmsnorm(g["x"], g["weight"]), g["y"], 2e-3)
    g = _load(golden_dir, "rope_f16_6x4x128.npz")
    assert _close(cport.rope(g["x"], g["pos"], g["inv_freq"]), g["y"], 2e-3)
    g = _load(golden_dir, "attention_f16_s37_h4.npz")
    S, H, D = g["k"].shape
    y = cport.attention_decode(g["q"], g["k"].reshape(S, H * D), g["v"].reshape(S, H * D), S, float(g["scale"][0]))
    assert _close(y, g["y"], 2e-3)


def test_softmax_sigmoid_edge_values():
    x = np.array([[-np.inf, 0.0, 1.0, 2.0, 3.0, 4.0, 5.0, 6.0]], np.float32)
    y = cport.softmax(x)
    assert y[0, 0] == 0 and abs(y.sum() - 1) < 1e-6
    s = cport.sigmoid(np.array([-100.0, 0.0, 100.0], np.float32))
    assert s[0] == 0.0 and s[1] == 0.5 and s[2] == 1.0


def test_row_shards_cover_k():
    for world in (1, 2, 4, 8):
        b = packing.row_shard_bounds(11008, world)
        assert b[0][0] == 0 and b[-1][1] == 11008
        assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))
        assert all(k0 % 128 == 0 and k1 > k0 for k0, k1 in b)
    qw, sc = packing.synth_w4(1024, 64, 9)
    x = packing.synth_x(1, 1024, 10).astype(np.float32)
    full = cport.np_w4a16_gemm(x, qw, sc.astype(np.float32))
    acc = np.zeros_like(full)
    for r in range(4):
        q_r, s_r, (k0, k1) = packing.shard_rows(qw, sc, r, 4)
        acc += cport.np_w4a16_gemm(x[:, k0:k1], q_r, s_r.astype(np.float32))
    assert np.allclose(acc, full, rtol=1e-4, atol=1e-4)
    cols = [cport.np_w4a16_gemm(x, *[a.astype(np.float32) if a.dtype == np.float16 else a for a in packing.shard_columns(qw, sc, r, 4)]) for r in range(4)]
    assert np.allclose(np.concatenate(cols, axis=1), full, rtol=1e-5, atol=1e-5)


def test_tile_major_repacking_is_a_pure_permutation():
    """packing.tile_weights: tile t holds columns 128 t .. 128 t + 127 of every packed row / scale row."""
    from antares_b200 import packing
    qw, sc = packing.synth_w4(256, 384, 1)
    qt, st = packing.tile_weights(qw, sc)
    assert qt.shape == (3, 32, 128) and st.shape == (3, 2, 128)
    for t in range(3):
        assert np.array_equal(qt[t], qw[:, t * 128:(t + 1) * 128]) and np.array_equal(st[t], sc[:, t * 128:(t + 1) * 128])
    with pytest.raises(ValueError):
        packing.tile_weights(qw[:, :100], sc[:, :100])
