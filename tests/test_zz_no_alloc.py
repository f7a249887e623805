"""GPU test of ab200_w4a16_gemv_static, the W4A16 GEMV entry point for hosts that may not allocate
device memory (its split-K scratch is a fixed array inside the library).  Collected last on
purpose: a failure here cannot hide the result of any other test in a run that stops at the first
failure.  It must pass both on its own in a fresh process and after every other test has run."""
import ctypes

import numpy as np
import pytest
import torch

from antares_b200 import _lib, ops, packing
from oracle import cport

pytestmark = pytest.mark.gpu
TOL = 1e-2  # same bound as the other GEMV tests: max|err| <= TOL * max|ref|


def _dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _static_gemv(x, qw, sc, out, group=128):
    """Straight through the C ABI: plain device pointers, no torch types in the call."""
    L = _lib.load()
    M = x.shape[0]
    K, N = qw.shape[0] * 8, qw.shape[1]
    rc = L.ab200_w4a16_gemv_static(x.data_ptr(), qw.data_ptr(), sc.data_ptr(), out.data_ptr(), M, K, N, group,
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, L.ab200_last_error().decode()


@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (1, 11008, 4096), (4, 4096, 22016)])
def test_static_scratch_entry_matches_the_allocating_one_twice_in_a_row(cuda, M, K, N):
    qw_np, sc_np = packing.synth_w4(K, N, 77)
    qw, sc = _dev(qw_np, cuda), _dev(sc_np, cuda)
    for call_no in range(2):  # the second call finds the array as the first one left it
        x_np = packing.synth_x(M, K, 100 + call_no)
        x = _dev(x_np, cuda)
        want = ops.w4a16_gemv(x, qw, sc).float()
        got = torch.full((M, N), float("nan"), dtype=torch.float16, device=cuda)
        rc, msg = _static_gemv(x, qw, sc, got)
        assert rc == 0, msg
        torch.cuda.synchronize()
        err = (got.float() - want).abs().max().item()
        assert err <= TOL * want.abs().max().item(), "call %d: off by %g" % (call_no, err)
        ref = cport.w4a16_gemm(x_np, qw_np, sc_np).astype(np.float32)
        assert np.abs(got.float().cpu().numpy() - ref).max() <= TOL * np.abs(ref).max()


def test_static_scratch_entry_rejects_what_does_not_fit(cuda):
    # 4 rows x 36864 columns is cut into 4 K slices: 2.25 MiB of partial sums, more than the built-in 2 MiB
    qw_np, sc_np = packing.synth_w4(4096, 36864, 78)
    x = _dev(packing.synth_x(4, 4096, 79), cuda)
    out = torch.empty((4, 36864), dtype=torch.float16, device=cuda)
    rc, msg = _static_gemv(x, _dev(qw_np, cuda), _dev(sc_np, cuda), out)
    assert rc == _lib.EINVAL and "scratch" in msg
