"""Tensor-parallel plumbing: one process per GPU, torch.distributed over NCCL (NVLink / NVSwitch).

The reference has no tensor-parallel path for this model (its samples are single-device); its
only collectives are the TensorFlow plugin's NCCL calls (frameworks/tensorflow/communicate_ops.cc:
191-193: all-reduce, reduce-scatter, all-gather over flat tensors).  The decode step needs two of
them: sum all-reduce of the [dim] fp32 partials after the row-parallel projections, and an
all-gather of vocabulary-shard logits.
"""
import os

import torch
import torch.distributed as dist


def init_from_env(backend=None):
    """Joins the process group described by RANK / WORLD_SIZE / MASTER_* (as set by torchrun).
    Returns (rank, world, local_rank)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        kw = {}
        if backend == "nccl":
            torch.cuda.set_device(local_rank)
            kw["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kw)
    return rank, world, local_rank


class TorchComm:
    """Collectives the decoder needs, on a torch.distributed process group (NCCL on GPUs, gloo
    for the CPU tests).  Both calls are legal inside CUDA graph capture with NCCL."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

    def all_reduce_sum_(self, t):
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def all_gather_into(self, out, t):
        dist.all_gather_into_tensor(out, t, group=self.group)
        return out

    def barrier(self):
        dist.barrier(group=self.group)

    def max_float(self, v, device):
        t = torch.tensor([float(v)], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())


class PushComm(TorchComm):
    """TorchComm plus the one-shot push all-reduce over NVLink peer memory (csrc/comm.cu): every
    rank owns a receive buffer, maps its peers' buffers through CUDA IPC and the exchange is one
    kernel per rank (peer stores of (value, epoch) pairs, bounded wait, rank-ordered sum fused with the
    residual update).  torch.distributed is used only to swap the 64-byte IPC handles."""

    def __init__(self, device, n_max, group=None):
        super().__init__(group)
        self.device, self.n_max = device, int(n_max)
        torch.cuda.set_device(device)
        self._own, self._peers, self._bufs = self._make_buffers(self.n_max)
        # a second, tiny exchange buffer for the vocabulary-parallel greedy step
        self._own_g, self._peers_g, self._bufs_g = self._make_buffers(4)
        dist.barrier(group=group)

    def _make_buffers(self, n_max):
        import ctypes
        from ._lib import call
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        call("ab200_comm_alloc", self.world, n_max, ctypes.cast(ctypes.pointer(ptr), ctypes.c_void_p), ctypes.cast(handle, ctypes.c_void_p))
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=self.group)
        peers = []
        bufs = (ctypes.c_void_p * self.world)()
        for r, h in enumerate(handles):
            if r == self.rank:
                bufs[r] = ptr.value
            else:
                p = ctypes.c_void_p()
                hb = ctypes.create_string_buffer(h, 64)
                call("ab200_comm_open", ctypes.cast(hb, ctypes.c_void_p), ctypes.cast(ctypes.pointer(p), ctypes.c_void_p))
                bufs[r] = p.value
                peers.append(p.value)
        return ptr.value, peers, bufs

    def greedy_next_(self, logits_local, vocab_offset, prompt, n_prompt, token, pos, out_tokens):
        """Vocabulary-parallel argmax + loop bookkeeping in one kernel per rank, no NCCL."""
        import ctypes
        from ._lib import call
        call("ab200_greedy_next_tp", logits_local.data_ptr(), logits_local.numel(), int(vocab_offset),
             ctypes.cast(self._bufs_g, ctypes.c_void_p), self.rank, self.world, 4, prompt.data_ptr(), int(n_prompt),
             token.data_ptr(), pos.data_ptr(), out_tokens.data_ptr(), out_tokens.numel(), torch.cuda.current_stream().cuda_stream)

    def all_reduce_residual_(self, x_f32, partial_f32):
        """x += fp16_round(sum over ranks of partial): one kernel, no NCCL."""
        import ctypes
        from ._lib import call
        call("ab200_allreduce_residual", x_f32.data_ptr(), partial_f32.data_ptr(), x_f32.numel(),
             ctypes.cast(self._bufs, ctypes.c_void_p), self.rank, self.world, self.n_max, torch.cuda.current_stream().cuda_stream)
        return x_f32

    def gemv_all_reduce_residual_(self, x_f32, act, qweight_tiled, scales_tiled, prologue):
        """x += fp16_round(sum over ranks of act . W_rank): the row-parallel projection with the sum over
        ranks fused into its epilogue (one kernel per rank, no separate exchange kernel)."""
        import ctypes
        from ._lib import call
        K, N = qweight_tiled.shape[1] * 8, qweight_tiled.shape[0] * qweight_tiled.shape[2]
        call("ab200_w4a16_gemv_tiled_allreduce", act.data_ptr(), int(prologue), qweight_tiled.data_ptr(), scales_tiled.data_ptr(),
             x_f32.data_ptr(), K, N, 128, ctypes.cast(self._bufs, ctypes.c_void_p), self.rank, self.world, self.n_max,
             torch.cuda.current_stream().cuda_stream)
        return x_f32

    def close(self):
        from ._lib import call
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for p in self._peers + self._peers_g:
            call("ab200_comm_close", p)
        self._peers, self._peers_g = [], []
        for own in (self._own, self._own_g):
            if own:
                call("ab200_comm_free", own)
        self._own = self._own_g = None
