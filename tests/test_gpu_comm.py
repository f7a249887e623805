"""GPU tests of the one-shot push all-reduce (csrc/comm.cu) on ONE GPU: all ranks run as the blocks
of a single cooperative launch over per-rank buffers, so the flag/epoch protocol is exercised
without needing several GPUs; and a wait that can never be satisfied runs out, reports through the
status word and leaves the context usable."""
import ctypes

import numpy as np
import pytest
import torch

from antares_b200 import _lib, ops
from antares_b200._lib import call

pytestmark = pytest.mark.gpu


def _alloc(world, n_max):
    p = ctypes.c_void_p()
    call("ab200_comm_alloc", world, n_max, ctypes.cast(ctypes.pointer(p), ctypes.c_void_p), None)
    return p.value


@pytest.mark.parametrize("world", [2, 4, 8])
def test_emulated_ranks_agree_bitwise_over_several_epochs(cuda, world):
    n, n_max = 4096, 4096
    bufs = [_alloc(world, n_max) for _ in range(world)]
    try:
        L = _lib.load()
        scratch = torch.zeros(int(L.ab200_comm_emulation_scratch_bytes()), dtype=torch.uint8, device=cuda)
        rng = np.random.default_rng(world)
        x0 = rng.standard_normal(n).astype(np.float32)
        xs = [torch.from_numpy(x0.copy()).to(cuda) for _ in range(world)]
        want = x0.copy()
        bufs_arr = (ctypes.c_void_p * world)(*bufs)
        for epoch in range(5):  # odd and even epochs use different slot sets
            parts_np = [rng.standard_normal(n).astype(np.float32) * 3 for _ in range(world)]
            parts = [torch.from_numpy(p).to(cuda) for p in parts_np]
            x_arr = (ctypes.c_void_p * world)(*[t.data_ptr() for t in xs])
            p_arr = (ctypes.c_void_p * world)(*[t.data_ptr() for t in parts])
            call("ab200_allreduce_residual_emulated", ctypes.cast(x_arr, ctypes.c_void_p), ctypes.cast(p_arr, ctypes.c_void_p), n,
                 ctypes.cast(bufs_arr, ctypes.c_void_p), world, n_max, scratch.data_ptr(), torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            s = np.zeros(n, np.float32)
            for p in parts_np:  # rank order, fp32
                s = s + p
            want = want + s.astype(np.float16).astype(np.float32)
            for r in range(world):
                assert torch.equal(xs[r], xs[0]), "ranks must hold bit-identical results"
            assert np.array_equal(xs[0].cpu().numpy(), want), "epoch %d" % epoch
        assert ops.kernel_status() == 0
    finally:
        for b in bufs:
            call("ab200_comm_free", b)


def test_wait_for_a_missing_peer_runs_out_and_is_reported(cuda):
    """Rank 0 of a 2-rank group whose peer never pushes: the bounded wait gives up, the status word
    names the peer, the kernel returns and later kernels run normally."""
    n = 1024
    bufs = [_alloc(2, n), _alloc(2, n)]
    ops.set_option("comm_wait_polls", 1 << 14)
    try:
        x = torch.zeros(n, device=cuda)
        part = torch.ones(n, device=cuda)
        bufs_arr = (ctypes.c_void_p * 2)(*bufs)
        call("ab200_allreduce_residual", x.data_ptr(), part.data_ptr(), n, ctypes.cast(bufs_arr, ctypes.c_void_p), 0, 2, n,
             torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        with pytest.raises(_lib.Ab200Error) as ei:
            ops.kernel_status()
        assert ei.value.code == _lib.ETIMEOUT and "site 101" in str(ei.value)
        assert ops.kernel_status() == 0                       # reading clears it
        assert float((torch.ones(8, device=cuda) * 2).sum()) == 16.0  # context still usable
    finally:
        ops.set_option("comm_wait_polls", 1 << 24)
        for b in bufs:
            call("ab200_comm_free", b)


@pytest.mark.parametrize("world", [2, 8])
def test_emulated_vocabulary_parallel_greedy_step(cuda, world):
    """Every rank holds a shard of the logits; after the candidate exchange all ranks pick the token
    torch.argmax picks on the gathered logits (lowest index on ties), advance the position and log
    the token - over several steps (both slot sets), with a tie placed across two shards."""
    vl = 1000
    bufs = [_alloc(world, 4) for _ in range(world)]
    try:
        L = _lib.load()
        scratch = torch.zeros(int(L.ab200_comm_emulation_scratch_bytes()), dtype=torch.uint8, device=cuda)
        rng = np.random.default_rng(world)
        tok = [torch.zeros(1, dtype=torch.int32, device=cuda) for _ in range(world)]
        pos = [torch.zeros(1, dtype=torch.int32, device=cuda) for _ in range(world)]
        outs = [torch.zeros(16, dtype=torch.int32, device=cuda) for _ in range(world)]
        prompt = torch.tensor([5, 6], dtype=torch.int32, device=cuda)  # position 1 is forced to prompt[1]
        P = ctypes.c_void_p
        arr = lambda xs: ctypes.cast((P * world)(*xs), P)
        n_arr = (ctypes.c_int * world)(*([vl] * world))
        off_arr = (ctypes.c_int * world)(*[r * vl for r in range(world)])
        want = []
        for step in range(5):
            full = rng.standard_normal(world * vl).astype(np.float32)
            if step == 2:  # the same maximum in the last shard and in shard 0: the lower index must win
                full[world * vl - 3] = 9.0
                full[17] = 9.0
            shards = [torch.from_numpy(full[r * vl:(r + 1) * vl].copy()).to(cuda) for r in range(world)]
            call("ab200_greedy_next_tp_emulated", arr([t.data_ptr() for t in shards]), ctypes.cast(n_arr, P), ctypes.cast(off_arr, P),
                 arr(bufs), world, 4, prompt.data_ptr(), 2, arr([t.data_ptr() for t in tok]), arr([t.data_ptr() for t in pos]),
                 arr([t.data_ptr() for t in outs]), scratch.data_ptr(), torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            expect = 6 if step == 0 else int(np.argmax(full))
            want.append(expect)
            for r in range(world):
                assert int(tok[r].item()) == expect and int(pos[r].item()) == step + 1, (step, r)
        assert want[2] == 17
        for r in range(world):
            assert outs[r][1:6].cpu().tolist() == want
        assert ops.kernel_status() == 0
    finally:
        for b in bufs:
            call("ab200_comm_free", b)
