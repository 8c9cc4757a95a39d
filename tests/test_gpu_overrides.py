"""The alternative kernels and launch forms behind the RT_ATTN_* overrides, each against the same oracle checks as
the default path.

The library reads its overrides once per process (a launch costs no getenv), so a test cannot switch them with
monkeypatch: every override here gets a child pytest process that runs an existing GPU test file with the variable
set.  What runs under each override:
  RT_ATTN_DECODE_IMPL=simt           the CUDA-core decode kernel for every shape        (csrc/decode.cu)
  RT_ATTN_DECODE_FUSED_MERGE=0       the separate chunk-merge kernel everywhere          (csrc/decode.cu)
  RT_ATTN_DECODE_PUSH_IN_KERNEL=1    record delivery from inside the decode kernel       (csrc/decode_tc.cu)
  RT_ATTN_EXCHANGE_PDL=0             the row-exchange kernel under a plain launch        (csrc/decode.cu)
  RT_ATTN_MERGE_PDL=0                the chunk-merge kernel under a plain launch         (csrc/decode.cu)
  RT_ATTN_DECODE_PDL=0               the decode kernel under a plain launch              (csrc/decode_tc.cu)
  RT_ATTN_BACKWARD_IMPL=mma_sync     the mma.sync backward kernel                        (csrc/backward_tc.cu)
  RT_ATTN_PREFILL_F32_IMPL=rows      the warp-per-row exact f32 forward                  (csrc/prefill_simt.cu)
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_tests_with(var, value, target, select=None, timeout=900):
    env = dict(os.environ)
    env[var] = value
    cmd = [sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider", os.path.join("tests", target)]
    if select:
        cmd += ["-k", select]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, f"{var}={value} {target}\n{r.stdout[-3000:]}\n{r.stderr[-1000:]}"
    assert " passed" in r.stdout, r.stdout[-500:]


@pytest.mark.parametrize("var,value,target,select", [
    ("RT_ATTN_DECODE_IMPL", "simt", "test_gpu_decode.py", None),
    ("RT_ATTN_DECODE_FUSED_MERGE", "0", "test_gpu_decode.py", None),
    ("RT_ATTN_DECODE_PUSH_IN_KERNEL", "1", "test_gpu_decode.py", "exchange or push or peer or record"),
    ("RT_ATTN_EXCHANGE_PDL", "0", "test_gpu_decode.py", "exchange"),
    ("RT_ATTN_MERGE_PDL", "0", "test_gpu_decode.py", None),
    ("RT_ATTN_DECODE_PDL", "0", "test_gpu_decode.py", None),
    ("RT_ATTN_BACKWARD_IMPL", "mma_sync", "test_gpu_backward.py", None),
    ("RT_ATTN_PREFILL_F32_IMPL", "rows", "test_gpu_prefill_f32.py", None),
])
def test_override_passes_the_default_path_tests(var, value, target, select):
    run_tests_with(var, value, target, select)
