"""The reference's own evaluator executable (graph_evaluator/run_graph.cpp, unmodified) driving this
library through the c-b200 HAL (include/c-b200/backend.hpp), next to the same evaluator on the
reference's CPU backend: both load a kernel-source file, fill inputs from <tensor>.npy
(run_graph.cpp:100-123), print the output digest `- K/0:` (:189-209) and the time per run `- TPR:`
(:214-236).  The reference cross-checks backends by comparing exactly these digests
(antares/antares_compiler.py:506-520)."""
import os
import re
import subprocess

import numpy as np
import pytest

from antares_b200 import packing
from oracle import build as obuild, cport, ref_kernels as rk

M, K, N = 1, 4096, 4096
TOL = 1e-2


def _run(exe, source, workdir, name):
    path = os.path.join(workdir, name)
    with open(path, "w") as f:
        f.write(source)
    out = subprocess.run([exe, path, "--value_absdir", workdir, "--dev", "0"], cwd=workdir, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    digest = float(re.search(r"- K/0: (\S+)", out.stdout).group(1))
    tpr = float(re.search(r"- TPR: (\S+)", out.stdout).group(1))
    return digest, tpr


def _inputs(workdir):
    qw, sc = packing.synth_w4(K, N, 0)
    x = packing.synth_x(M, K, 1)
    np.save(os.path.join(workdir, "input0.npy"), x)
    np.save(os.path.join(workdir, "qweight.npy"), qw)
    np.save(os.path.join(workdir, "scales.npy"), sc)
    return x, qw, sc


def _b200_source():
    ins = "input0:float16[%d, %d], qweight:int32[%d, %d], scales:float16[%d, %d]" % (M, K, K // 8, N, K // 128, N)
    outs = "my_result:float16[%d, %d]" % (M, N)
    return ("// GLOBALS: %s -> %s\n// BACKEND: c-b200 (default)\n// CONFIG: null\n"
            "// COMPUTE_V1: - einstein_v2(input_dict={}, extra_outputs=[], exprss=\"%s\")\n\n%s// LOCAL: template_op_kernel0 -- %s -> %s\n"
            % (ins, outs, rk.W4A16_IR, rk.SEP, ins, outs))


def _evaluators():
    mcpu, b200 = obuild.build_evaluators()
    if mcpu is None or b200 is None:
        pytest.skip("the reference's evaluator is not built (no reference checkout when oracle/_ref was made)")
    return mcpu, b200


def test_cpu_evaluator_digest_equals_the_oracles(tmp_path):
    mcpu, _ = _evaluators()
    x, qw, sc = _inputs(str(tmp_path))
    digest, tpr = _run(mcpu, rk.w4a16(M, K, N), str(tmp_path), "my_kernel_mcpu.cc")
    ref = cport.w4a16_gemm(x, qw, sc)
    assert abs(digest - cport.digest(ref)) <= 1e-6 * max(1.0, abs(digest))
    assert tpr > 0


@pytest.mark.gpu
def test_b200_hal_digest_agrees_with_the_cpu_backend(cuda, tmp_path):
    mcpu, b200 = _evaluators()
    x, qw, sc = _inputs(str(tmp_path))
    d_cpu, t_cpu = _run(mcpu, rk.w4a16(M, K, N), str(tmp_path), "my_kernel_mcpu.cc")
    d_gpu, t_gpu = _run(b200, _b200_source(), str(tmp_path), "my_kernel_b200.cc")
    max_abs = float(np.abs(cport.w4a16_gemm(x, qw, sc).astype(np.float32)).max())
    # the digest is a linear functional of the output with weights (i + 1) % 83: same bound as for the outputs
    assert abs(d_gpu - d_cpu) <= TOL * max_abs * 83 * N / 64, (d_gpu, d_cpu)
    assert 0 < t_gpu < 1e-3 and t_cpu > 0, (t_gpu, t_cpu)
