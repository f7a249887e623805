"""CPU tests (gloo, world size 2) of the tensor-parallel host logic: weight sharding, the
all-reduce of row-parallel partials and the all-gather of vocabulary shards reproduce the
unsharded result.  The per-shard arithmetic is done by the CPU oracle; no GPU is involved."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from antares_b200 import packing
from antares_b200.llama import LlamaConfig, shard_layer, synth_layer
from antares_b200.parallel import TorchComm


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_q):
    from oracle import cport
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        comm = TorchComm()
        assert (comm.rank, comm.world) == (rank, world)
        cfg = LlamaConfig(n_layers=1, dim=512, n_heads=4, ffn=1408, vocab=64, group=128)
        w = synth_layer(cfg, 0)
        sh = shard_layer(cfg, w, rank, world)
        d, dl = cfg.dim, cfg.dim // world
        k0, k1 = packing.row_shard_bounds(cfg.ffn, world, cfg.group)[rank]
        assert sh["vqk_q"].shape == (d // 8, 3 * dl) and sh["o_q"].shape == (dl // 8, d)
        assert sh["gu_q"].shape == (d // 8, 2 * (k1 - k0)) and sh["down_q"].shape == ((k1 - k0) // 8, d)
        rng = np.random.default_rng(5)
        x = rng.standard_normal((1, d)).astype(np.float16)
        # column-parallel V|Q|K: local columns are the rank's heads of each of V, Q, K
        full = cport.w4a16_gemm(x, w["vqk_q"], w["vqk_s"])[0]
        local = cport.w4a16_gemm(x, sh["vqk_q"], sh["vqk_s"])[0]
        want = np.concatenate([full[i * d + rank * dl:i * d + (rank + 1) * dl] for i in range(3)])
        assert np.array_equal(local, want)
        # row-parallel O: fp32 partials, all-reduce, equals the unsharded product
        a = rng.standard_normal((1, d)).astype(np.float16)
        part = cport.np_w4a16_gemm(a[:, rank * dl:(rank + 1) * dl].astype(np.float32), sh["o_q"], sh["o_s"].astype(np.float32))
        t = torch.from_numpy(part.copy())
        comm.all_reduce_sum_(t)
        ref = cport.np_w4a16_gemm(a.astype(np.float32), w["o_q"], w["o_s"].astype(np.float32))
        assert np.allclose(t.numpy(), ref, rtol=1e-4, atol=1e-3)
        # row-parallel down over uneven, group-aligned K shards
        h = rng.standard_normal((1, cfg.ffn)).astype(np.float32)
        part = cport.np_w4a16_gemm(h[:, k0:k1], sh["down_q"], sh["down_s"].astype(np.float32))
        t = torch.from_numpy(part.copy())
        comm.all_reduce_sum_(t)
        ref = cport.np_w4a16_gemm(h, w["down_q"], w["down_s"].astype(np.float32))
        assert np.allclose(t.numpy(), ref, rtol=1e-4, atol=1e-3)
        # vocabulary-parallel logits: all-gather in rank order
        vl = cfg.vocab // world
        logits = torch.arange(cfg.vocab, dtype=torch.float32)
        got = torch.empty(cfg.vocab)
        comm.all_gather_into(got, logits[rank * vl:(rank + 1) * vl].clone())
        assert torch.equal(got, logits)
        assert comm.max_float(float(rank), torch.device("cpu")) == world - 1
        comm.barrier()
        out_q.put((rank, "ok"))
    except Exception as e:  # report instead of hanging the parent
        out_q.put((rank, "FAIL: %r" % (e,)))
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_host_logic_world2():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_row_shard_bounds_cover_llama_ffn():
    for world in (1, 2, 4, 8):
        b = packing.row_shard_bounds(11008, world)
        assert b[0][0] == 0 and b[-1][1] == 11008 and all(x[1] == y[0] for x, y in zip(b, b[1:]))
        assert all((k1 - k0) % 128 == 0 for k0, k1 in b)
