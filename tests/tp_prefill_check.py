"""Worker of tests/test_gpu_tp_prefill.py (run under torch.distributed.run, one rank per GPU): the batched prompt pass
on a tensor-parallel decoder gives the tokens of the token-by-token route and of a single-GPU decoder, and next-token
logits within tolerance of the single-GPU pass."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from antares_b200 import ops, parallel  # noqa: E402
from antares_b200.llama import LlamaConfig, LlamaInt4Decoder, synth_prompt  # noqa: E402

TOL = 1e-2


def main():
    rank, world, local_rank = parallel.init_from_env()
    assert world > 1
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    comm = parallel.PushComm(dev, 4096)
    cfg = LlamaConfig(n_layers=2, max_seq=96)
    prompt = synth_prompt(cfg, 40, 7)
    tp = LlamaInt4Decoder(cfg, dev, rank=rank, world=world, comm=comm)
    batched = tp.generate(prompt, 5, batched_prefill=True)
    tp.prefill(prompt)
    logits_tp = tp.logits_local.clone()  # this rank's vocabulary shard
    one_by_one = tp.generate(prompt, 5)
    single = LlamaInt4Decoder(cfg, dev)  # every rank builds the same single-GPU decoder on its own GPU
    want = single.generate(prompt, 5, batched_prefill=True)
    single.prefill(prompt)
    ref = single.logits.float()
    err = float((logits_tp.float() - ref[rank * tp.vl:(rank + 1) * tp.vl]).abs().max() / ref.abs().max())
    ok = list(batched) == list(want) and list(one_by_one) == list(want) and err <= TOL and ops.kernel_status() == 0
    flag = torch.tensor([1 if ok else 0], device=dev)
    torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN)
    if rank == 0:
        print("generated", [int(t) for t in batched[-5:]], [int(t) for t in one_by_one[-5:]], [int(t) for t in want[-5:]], "logit err", err)
        print("TP_PREFILL_OK" if int(flag.item()) == 1 else "TP_PREFILL_FAILED")
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
