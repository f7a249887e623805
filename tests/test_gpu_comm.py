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
                 arr([t.data_ptr() for t in outs]), 16, scratch.data_ptr(), torch.cuda.current_stream().cuda_stream)
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


def _tiled_dev(K, N, seed, cuda):
    from antares_b200 import packing
    qw, sc = packing.synth_w4(K, N, seed)
    qt, st = packing.tile_weights(qw, sc)
    return torch.from_numpy(qt).to(cuda), torch.from_numpy(st).to(cuda)


@pytest.mark.parametrize("world,prologue", [(2, 0), (4, 2), (8, 0)])
def test_emulated_fused_gemv_allreduce(cuda, world, prologue):
    """The row-parallel projection with the sum over ranks fused into its epilogue, all ranks as CTA
    ranges of one cooperative launch: uneven K shards (22 groups over the ranks), several exchanges in a
    row (both slot sets, the ticket that advances the epoch), every rank bit-identical, and equal to
    the rank-ordered fp32 sum of the per-rank projections computed by the same kernel alone."""
    from antares_b200 import packing
    K_total, N, n_max = 2816, 512, 512
    bounds = packing.row_shard_bounds(K_total, world)
    Ks = [k1 - k0 for k0, k1 in bounds]
    assert len(set(Ks)) > 1 or world == 2
    bufs = [_alloc(world, n_max) for _ in range(world)]
    ops.set_option("gemv_cluster", 2)  # same K split in the fused and the stand-alone launches: identical partial sums
    ops.set_option("gemv_impl", 5)     # and the same kernel (the bulk-copy ring GEMV carries the fused exchange)
    try:
        L = _lib.load()
        scratch = torch.zeros(int(L.ab200_w4a16_gemv_emulation_scratch_bytes()), dtype=torch.uint8, device=cuda)
        weights = [_tiled_dev(Ks[r], N, 900 + r, cuda) for r in range(world)]
        rng = np.random.default_rng(world)
        x0 = rng.standard_normal(N).astype(np.float32)
        xs = [torch.from_numpy(x0.copy()).to(cuda) for _ in range(world)]
        want = torch.from_numpy(x0.copy()).to(cuda)
        P = ctypes.c_void_p
        arr = lambda v: ctypes.cast((P * world)(*v), P)
        st = torch.cuda.current_stream().cuda_stream
        for step in range(4):
            width = 2 if prologue == 2 else 1
            acts = [torch.from_numpy(rng.standard_normal((1, width * Ks[r])).astype(np.float16)).to(cuda) for r in range(world)]
            k_arr = (ctypes.c_int * world)(*Ks)
            call("ab200_w4a16_gemv_tiled_allreduce_emulated", arr([a.data_ptr() for a in acts]), prologue,
                 arr([w[0].data_ptr() for w in weights]), arr([w[1].data_ptr() for w in weights]), arr([x.data_ptr() for x in xs]),
                 ctypes.cast(k_arr, P), N, arr(bufs), world, n_max, scratch.data_ptr(), st)
            torch.cuda.synchronize()
            total = torch.zeros(N, dtype=torch.float32, device=cuda)
            for r in range(world):  # rank order, fp32
                part = torch.empty((1, N), dtype=torch.float32, device=cuda)
                ops.w4a16_gemv_tiled(acts[r], weights[r][0], weights[r][1], part, prologue=prologue, epilogue=ops.EPI_F32)
                total = total + part[0]
            want = want + total.to(torch.float16).to(torch.float32)
            for r in range(world):
                assert torch.equal(xs[r], xs[0]), "ranks must hold bit-identical results (step %d)" % step
            assert torch.equal(xs[0], want), "step %d" % step
        assert ops.kernel_status() == 0
    finally:
        ops.set_option("gemv_cluster", 0)
        ops.set_option("gemv_impl", 0)
        for b in bufs:
            call("ab200_comm_free", b)


def test_fused_gemv_allreduce_missing_peer_times_out_then_stays_fast(cuda):
    """Rank 0 of a 2-rank group whose peer never pushes, through the fused projection: the bounded wait
    gives up and names the peer; while the status word is set a second exchange returns without
    waiting again (a timeout is sticky until the host reads it); afterwards the context is usable."""
    import time
    K, N = 512, 512
    bufs = [_alloc(2, N), _alloc(2, N)]
    ops.set_option("comm_wait_polls", 1 << 16)
    try:
        qt, st_ = _tiled_dev(K, N, 950, cuda)
        act = torch.ones((1, K), dtype=torch.float16, device=cuda)
        x = torch.zeros(N, device=cuda)
        bufs_arr = (ctypes.c_void_p * 2)(*bufs)
        stream = torch.cuda.current_stream().cuda_stream

        def exchange():
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            call("ab200_w4a16_gemv_tiled_allreduce", act.data_ptr(), 0, qt.data_ptr(), st_.data_ptr(), x.data_ptr(), K, N, 128,
                 ctypes.cast(bufs_arr, ctypes.c_void_p), 0, 2, N, stream)
            torch.cuda.synchronize()
            return time.perf_counter() - t0

        t_first = exchange()
        t_second = exchange()           # status still set: polls once
        assert t_second < max(0.25 * t_first, 2e-3), (t_first, t_second)
        with pytest.raises(_lib.Ab200Error) as ei:
            ops.kernel_status()
        assert ei.value.code == _lib.ETIMEOUT and "site 101" in str(ei.value)
        assert ops.kernel_status() == 0
        assert float((torch.ones(8, device=cuda) * 2).sum()) == 16.0
    finally:
        ops.set_option("comm_wait_polls", 1 << 24)
        for b in bufs:
            call("ab200_comm_free", b)


def test_greedy_next_never_writes_past_the_token_log(cuda):
    """The token log holds out_cap ids: a step too many stores nothing and leaves the position where
    it was (single-GPU kernel and the vocabulary-parallel one)."""
    logits = torch.zeros(100, device=cuda)
    logits[42] = 1.0
    tok = torch.zeros(1, dtype=torch.int32, device=cuda)
    pos = torch.zeros(1, dtype=torch.int32, device=cuda)
    log = torch.full((8,), -7, dtype=torch.int32, device=cuda)   # capacity 4 declared, 4 guard entries behind it
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(6):
        call("ab200_greedy_next", logits.data_ptr(), 100, None, 0, tok.data_ptr(), pos.data_ptr(), log.data_ptr(), 4, st)
    torch.cuda.synchronize()
    assert log.cpu().tolist() == [-7, 42, 42, 42, -7, -7, -7, -7]
    assert int(pos.item()) == 3 and int(tok.item()) == 42
    bufs = [_alloc(1, 4)]
    try:
        pos.zero_()
        log.fill_(-7)
        bufs_arr = (ctypes.c_void_p * 1)(*bufs)
        for _ in range(6):
            call("ab200_greedy_next_tp", logits.data_ptr(), 100, 0, ctypes.cast(bufs_arr, ctypes.c_void_p), 0, 1, 4, None, 0,
                 tok.data_ptr(), pos.data_ptr(), log.data_ptr(), 4, st)
        torch.cuda.synchronize()
        assert log.cpu().tolist() == [-7, 42, 42, 42, -7, -7, -7, -7]
        assert int(pos.item()) == 3
    finally:
        call("ab200_comm_free", bufs[0])
