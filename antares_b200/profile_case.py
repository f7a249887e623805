"""Small, bounded workloads for profilers (ncu): one operator shape launched a few times, or a few
decode steps of a shortened model.  Holds at most a few hundred MB on the device.

  python -m antares_b200.profile_case gemv K N M [--impl I] [--launches L]
  python -m antares_b200.profile_case gemm M K N [--launches L]
  python -m antares_b200.profile_case step [--layers L] [--pos P] [--steps S]
"""
import argparse

import numpy as np
import torch

from . import ops, packing
from .llama import LlamaConfig, LlamaInt4Decoder, synth_prompt


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemv", "gemm", "step"])
    ap.add_argument("dims", nargs="*", type=int)
    ap.add_argument("--impl", type=int, default=0)
    ap.add_argument("--launches", type=int, default=6)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--pos", type=int, default=256)
    ap.add_argument("--steps", type=int, default=3)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    if a.what == "gemv":
        K, N, M = a.dims
        qw_np, sc_np = packing.synth_w4(K, N, 1)
        nbuf = 4  # distinct weight copies so that consecutive launches do not hit L2
        qws = [torch.from_numpy(qw_np).to(dev) for _ in range(nbuf)]
        scs = [torch.from_numpy(sc_np).to(dev) for _ in range(nbuf)]
        x = torch.from_numpy(packing.synth_x(M, K, 2)).to(dev)
        out = torch.empty((M, N), dtype=torch.float16, device=dev)
        ops.set_option("gemv_impl", a.impl)
        for i in range(a.launches):
            ops.w4a16_gemv(x, qws[i % nbuf], scs[i % nbuf], out)
        torch.cuda.synchronize()
    elif a.what == "gemm":
        M, K, N = a.dims
        qw_np, sc_np = packing.synth_w4(K, N, 1)
        qw, sc = torch.from_numpy(qw_np).to(dev), torch.from_numpy(sc_np).to(dev)
        x = torch.from_numpy(packing.synth_x(M, K, 2)).to(dev)
        out = torch.empty((M, N), dtype=torch.float16, device=dev)
        for i in range(a.launches):
            ops.w4a16_gemm(x, qw, sc, out)
        torch.cuda.synchronize()
    else:
        cfg = LlamaConfig(n_layers=a.layers, max_seq=512)
        dec = LlamaInt4Decoder(cfg, dev)
        dec._n_prompt_capture = 1
        dec.reset(torch.from_numpy(synth_prompt(cfg, 1, 0)).to(dev))
        dec.pos.fill_(a.pos)
        for _ in range(a.steps):
            dec.step_eager()
        torch.cuda.synchronize()
    print("ok", ops.kernel_status())


if __name__ == "__main__":
    main()
