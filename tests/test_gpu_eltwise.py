"""GPU parity tests of the elementwise / reduction operators (the benchmark's element-wise / reduction shapes and the
golden vectors of the reference runtime).  Tolerance: max|err| <= 1e-2 * max|ref|."""
import os

import numpy as np
import pytest
import torch

from antares_b200 import ops
from oracle import cport

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _err(y, ref):
    y, ref = y.astype(np.float32), ref.astype(np.float32)
    return np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30)


def test_golden_elementwise(cuda, golden_dir):
    g = dict(np.load(os.path.join(golden_dir, "softmax_f16_8x256.npz")))
    assert _err(ops.softmax(_dev(g["x"], cuda)).cpu().numpy(), g["y"]) <= TOL
    g = dict(np.load(os.path.join(golden_dir, "sigmoid_f32_1000.npz")))
    assert _err(ops.sigmoid(_dev(g["x"], cuda)).cpu().numpy(), g["y"]) <= 1e-5
    g = dict(np.load(os.path.join(golden_dir, "rmsnorm_f16_4x512.npz")))
    assert _err(ops.rmsnorm(_dev(g["x"], cuda), _dev(g["weight"], cuda)).cpu().numpy(), g["y"]) <= TOL
    g = dict(np.load(os.path.join(golden_dir, "rope_f16_6x4x128.npz")))
    y = ops.rope(_dev(g["x"], cuda), _dev(g["pos"], cuda), _dev(g["inv_freq"], cuda)).cpu().numpy()
    assert _err(y, g["y"]) <= TOL
    g = dict(np.load(os.path.join(golden_dir, "attention_f16_s37_h4.npz")))
    S, H, D = g["k"].shape
    y = ops.attention_decode(_dev(g["q"], cuda), _dev(g["k"].reshape(S, H * D), cuda), _dev(g["v"].reshape(S, H * D), cuda),
                             torch.tensor([S], dtype=torch.int32, device=cuda), float(g["scale"][0])).cpu().numpy()
    assert _err(y, g["y"]) <= TOL


def test_config1_sigmoid(cuda):
    x = np.random.default_rng(0).standard_normal(4096000).astype(np.float32)
    y = ops.sigmoid(_dev(x, cuda)).cpu().numpy()
    assert _err(y, cport.sigmoid(x)) <= 1e-5
    x10 = torch.arange(0, 10, dtype=torch.float32, device=cuda)  # README.md:64-67: 10 elements into N:4096000
    assert torch.allclose(ops.sigmoid(x10), torch.sigmoid(x10), atol=1e-6)
    xh = x[:100003].astype(np.float16)[:100000]
    assert _err(ops.sigmoid(_dev(xh, cuda)).cpu().numpy(), cport.sigmoid(xh)) <= TOL


def test_config1_rmsnorm(cuda):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((2048, 4096)).astype(np.float16)
    w = (1 + 0.1 * rng.standard_normal(4096)).astype(np.float16)
    y = ops.rmsnorm(_dev(x, cuda), _dev(w, cuda), eps=1e-6).cpu().numpy()
    assert _err(y, cport.rmsnorm(x, w, 1e-6)) <= TOL
    x32 = x[:3].astype(np.float32) * 7
    assert _err(ops.rmsnorm(_dev(x32, cuda), _dev(w, cuda)).cpu().numpy(), cport.rmsnorm(x32, w)) <= TOL
    # the AutoRT call form: vsum computed by the caller (samples/05_llama2_7b_int4.py:128-131)
    v = x32[0]
    vsum = _dev(np.array([(v * v).sum()], np.float32), cuda)
    y = ops.rmsnorm_vsum(_dev(v, cuda), vsum, _dev(w.astype(np.float32), cuda), 1.0 / 4096).cpu().numpy()
    assert _err(y, cport.rmsnorm_vsum_f32(v, np.array([(v * v).sum()], np.float32), w.astype(np.float32), 1.0 / 4096)) <= 1e-5


def test_config1_rope(cuda):
    x = np.random.default_rng(2).standard_normal((2048, 32, 128)).astype(np.float16)
    pos = np.arange(2048, dtype=np.int32)
    inv_freq = cport.make_inv_freq(128)
    y = ops.rope(_dev(x, cuda), _dev(pos, cuda), _dev(inv_freq, cuda)).cpu().numpy()
    assert _err(y, cport.rope(x, pos, inv_freq)) <= TOL
    # rotation preserves the norm of each (j, j+D/2) pair
    n_in = np.hypot(x[..., :64].astype(np.float32), x[..., 64:].astype(np.float32))
    n_out = np.hypot(y[..., :64].astype(np.float32), y[..., 64:].astype(np.float32))
    assert np.abs(n_in - n_out).max() <= 1e-2 * n_in.max()


def test_config1_softmax(cuda):
    x = (np.random.default_rng(3).standard_normal((32, 4096)) * 3).astype(np.float16)
    y = ops.softmax(_dev(x, cuda)).cpu().numpy()
    assert _err(y, cport.softmax(x)) <= TOL
    assert np.abs(y.astype(np.float32).sum(-1) - 1).max() < 2e-2
    x32 = x.astype(np.float32)[:, :1024]
    assert _err(ops.softmax(_dev(x32, cuda)).cpu().numpy(), cport.softmax(x32)) <= 1e-5


@pytest.mark.parametrize("S", [1, 2, 17, 384, 1000])
def test_attention_decode(cuda, S):
    rng = np.random.default_rng(S)
    H, D, max_seq = 32, 128, 1024
    q = rng.standard_normal((H, D)).astype(np.float16)
    kc = rng.standard_normal((max_seq, H * D)).astype(np.float16)
    vc = rng.standard_normal((max_seq, H * D)).astype(np.float16)
    scale = 1.0 / np.sqrt(D)
    ref = cport.attention_decode(q, kc, vc, S, scale)
    y = ops.attention_decode(_dev(q, cuda), _dev(kc, cuda), _dev(vc, cuda), torch.tensor([S], dtype=torch.int32, device=cuda), scale)
    assert _err(y.cpu().numpy(), ref) <= TOL


@pytest.mark.parametrize("pos", [0, 1, 5, 130, 383])
@pytest.mark.parametrize("H", [32, 4])
def test_attention_fused_matches_unfused_chain(cuda, pos, H):
    """rope(q), rope(k) -> cache row pos, v -> cache row pos, attention over rows 0..pos, in one launch."""
    from antares_b200._lib import call
    rng = np.random.default_rng(pos + H)
    D, max_seq = 128, 512
    vqk = rng.standard_normal(3 * H * D).astype(np.float16)
    kc = rng.standard_normal((max_seq, H * D)).astype(np.float16)
    vc = rng.standard_normal((max_seq, H * D)).astype(np.float16)
    inv_freq = cport.make_inv_freq(D)
    p = np.array([pos], np.int32)
    q_r = cport.rope(vqk[H * D:2 * H * D].reshape(1, H, D), p, inv_freq)[0]
    kc_ref, vc_ref = kc.copy(), vc.copy()
    kc_ref[pos] = cport.rope(vqk[2 * H * D:].reshape(1, H, D), p, inv_freq).reshape(-1)
    vc_ref[pos] = vqk[:H * D]
    ref = cport.attention_decode(q_r, kc_ref, vc_ref, pos + 1, 1 / np.sqrt(D))
    kc_d, vc_d = _dev(kc, cuda), _dev(vc, cuda)
    out = torch.empty((H, D), dtype=torch.float16, device=cuda)
    vqk_d, invf_d, pos_d = _dev(vqk, cuda), _dev(inv_freq, cuda), torch.tensor([pos], dtype=torch.int32, device=cuda)
    call("ab200_attention_fused", vqk_d.data_ptr(), invf_d.data_ptr(), pos_d.data_ptr(), kc_d.data_ptr(), vc_d.data_ptr(), out.data_ptr(),
         H, D, H * D, max_seq, 1 / np.sqrt(D), torch.cuda.current_stream().cuda_stream)
    assert _err(out.cpu().numpy(), ref) <= TOL
    assert _err(kc_d[pos].cpu().numpy(), kc_ref[pos]) <= TOL and torch.equal(vc_d[pos].cpu(), torch.from_numpy(vc_ref[pos]))
    assert torch.equal(kc_d[pos + 1:].cpu(), torch.from_numpy(kc[pos + 1:])), "rows beyond pos must be untouched"


@pytest.mark.parametrize("S", [1, 37, 384])
def test_attention_against_the_reference_samples_open_statement(cuda, S):
    """The attention op itself ships closed in the reference, but its tiny-Llama sample states the same
    math in three open torch lines (samples/03_llama_tiny.py:93-98): scores = einsum('hm,shm->hs', q, K) *
    att_f; softmax over s; out = einsum('hs,shm->hm', att, V).  Expected values here are exactly those
    lines in fp32 on the CPU, for 32 heads of 128 and cache lengths 1, 37 and 384 (fp32 and fp16 operands)."""
    H, D = 32, 128
    rng = np.random.default_rng(500 + S)
    q = rng.standard_normal((H, D)).astype(np.float32)
    k = rng.standard_normal((S, H, D)).astype(np.float32)
    v = rng.standard_normal((S, H, D)).astype(np.float32)
    att_f = 1.0 / np.sqrt(D)
    for dt, tol in ((np.float32, 1e-4), (np.float16, 1e-2)):
        qd, kd, vd = q.astype(dt), k.astype(dt), v.astype(dt)
        tq, tk, tv = torch.from_numpy(qd).float(), torch.from_numpy(kd).float(), torch.from_numpy(vd).float()
        att = torch.einsum('hm,shm->hs', tq, tk) * att_f
        att = torch.nn.functional.softmax(att, dim=-1)
        ref = torch.einsum('hs,shm->hm', att, tv).numpy()
        y = ops.attention_decode(_dev(qd, cuda), _dev(kd.reshape(S, H * D), cuda), _dev(vd.reshape(S, H * D), cuda),
                                 torch.tensor([S], dtype=torch.int32, device=cuda), att_f)
        err = np.abs(y.float().cpu().numpy() - ref).max() / np.abs(ref).max()
        assert err <= tol, (dt, err)
