"""Generates tests/golden/*.npz by running hand-restated kernel texts on the reference's own
c-mcpu runtime (oracle/refrt.py).  Needs the reference checkout (to build oracle/_ref) and g++.

  python tests/golden/make_golden.py

The fixtures hold inputs AND outputs, so the tests that read them need neither the reference nor
the same random generator.  `c0_digest.json` pins the full-size 4096x4096 fp16 case
(x fp16 [1,4096], W 4096x4096, g=128, seed 0) by the evaluator's digest formula
(graph_evaluator/run_graph.cpp:189-209) and a sha256 of the fp16 output bytes.
"""
import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from antares_b200 import packing  # noqa: E402
from oracle import cport, ref_kernels as rk, refrt  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def w4a16_case(M, K, N, seed, dtype):
    qw, sc = packing.synth_w4(K, N, seed, scales_dtype=dtype)
    x = packing.synth_x(M, K, seed + 1, dtype)
    y = np.zeros((M, N), dtype)
    refrt.RefModule(rk.w4a16(M, K, N, "float16" if dtype == np.float16 else "float32"))(x, qw, sc, y)
    w = np.zeros((K, N), dtype)
    refrt.RefModule(rk.w4_dequant(K, N, "float16" if dtype == np.float16 else "float32"))(qw, sc, w)
    return dict(x=x, qweight=qw, scales=sc, y=y, w=w)


def main():
    rng = np.random.default_rng(1234)
    np.savez_compressed(os.path.join(HERE, "w4a16_f16_m1_k256_n64.npz"), **w4a16_case(1, 256, 64, 11, np.float16))
    np.savez_compressed(os.path.join(HERE, "w4a16_f16_m3_k512_n128.npz"), **w4a16_case(3, 512, 128, 12, np.float16))
    np.savez_compressed(os.path.join(HERE, "w4a16_f32_m2_k256_n64.npz"), **w4a16_case(2, 256, 64, 13, np.float32))

    # every nibble value x a spread of scales: the bit-exact dequant table
    q = np.tile(np.arange(16, dtype=np.uint8).reshape(16, 1), (8, 64))  # [128, 64]
    q = q[rng.permutation(128)]
    qw = packing.pack_w4(q)
    sc = np.concatenate([np.linspace(0.001, 0.02, 60), [6.1e-5, 5.96e-8, 0.5, 65504.0 / 8]]).astype(np.float16).reshape(1, 64)
    w = np.zeros((128, 64), np.float16)
    refrt.RefModule(rk.w4_dequant(128, 64))(qw, sc, w)
    np.savez_compressed(os.path.join(HERE, "w4_dequant_table_f16.npz"), q=q, qweight=qw, scales=sc, w=w)

    x = (rng.standard_normal((8, 256)) * 3).astype(np.float16)
    y = np.zeros_like(x)
    refrt.RefModule(rk.softmax(8, 256))(x, y)
    np.savez_compressed(os.path.join(HERE, "softmax_f16_8x256.npz"), x=x, y=y)

    x = rng.standard_normal(1000).astype(np.float32) * 4
    y = np.zeros_like(x)
    refrt.RefModule(rk.sigmoid_f32(1000))(x, y)
    np.savez_compressed(os.path.join(HERE, "sigmoid_f32_1000.npz"), x=x, y=y)

    x = rng.standard_normal((4, 512)).astype(np.float16)
    wgt = (1 + 0.1 * rng.standard_normal(512)).astype(np.float16)
    y = np.zeros_like(x)
    refrt.RefModule(rk.rmsnorm_rows(4, 512))(wgt, x, y)
    np.savez_compressed(os.path.join(HERE, "rmsnorm_f16_4x512.npz"), x=x, weight=wgt, y=y)

    x = rng.standard_normal((6, 4, 128)).astype(np.float16)
    pos = np.array([0, 1, 2, 7, 100, 383], np.int32)
    inv_freq = cport.make_inv_freq(128)
    y = np.zeros_like(x)
    refrt.RefModule(rk.rotary(6, 4, 128))(inv_freq, pos, x, y)
    np.savez_compressed(os.path.join(HERE, "rope_f16_6x4x128.npz"), x=x, pos=pos, inv_freq=inv_freq, y=y)

    S, H, D = 37, 4, 128
    qv = rng.standard_normal((H, D)).astype(np.float16)
    kc = rng.standard_normal((S, H, D)).astype(np.float16)
    vc = rng.standard_normal((S, H, D)).astype(np.float16)
    att_f = np.array([1.0 / np.sqrt(D)], np.float32)
    y = np.zeros((H, D), np.float16)
    refrt.RefModule(rk.attention(S, H, D, S))(att_f, kc, qv, vc, y)
    np.savez_compressed(os.path.join(HERE, "attention_f16_s37_h4.npz"), q=qv, k=kc, v=vc, scale=att_f, y=y)

    # the 4096x4096 fp16 case at full size
    qw, sc = packing.synth_w4(4096, 4096, 0)
    x = packing.synth_x(1, 4096, 1)
    y = np.zeros((1, 4096), np.float16)
    refrt.RefModule(rk.w4a16(1, 4096, 4096))(x, qw, sc, y)
    info = dict(config="x fp16 [1,4096] seed 1; W 4096x4096 seed 0 (packing.synth_w4); g=128",
                digest_k0=cport.digest(y), sha256=hashlib.sha256(y.tobytes()).hexdigest(),
                max_abs=float(np.abs(y.astype(np.float32)).max()))
    with open(os.path.join(HERE, "c0_digest.json"), "w") as f:
        json.dump(info, f, indent=1)
    print(info)


if __name__ == "__main__":
    main()
