"""The library's run-time switches select alternative code paths that must give the same results (the reference tests
every MACSEEK_* switch the same way, tests/test_dec_fuse.mm:172-205).  They are read once per process, so each
combination runs the relevant GPU tests in a child process:
  MSB_IDX_LEGACY=1   FP8 index scoring on mma.sync instead of tcgen05
  MSB_TOPK_FUSED=0   top-k selection and read-out as two launches
  MSB_PDL=0          launches without programmatic stream serialization"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("env,files", [
    ({"MSB_IDX_LEGACY": "1"}, ["tests/test_attn_gpu.py"]),
    ({"MSB_TOPK_FUSED": "0"}, ["tests/test_attn_gpu.py"]),
    ({"MSB_PDL": "0"}, ["tests/test_decode_step_gpu.py", "tests/test_moe_gpu.py"]),
], ids=["idx-legacy", "topk-unfused", "no-pdl"])
def test_switch(env, files):
    e = dict(os.environ, **env)
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider"] + files,
                       cwd=ROOT, env=e, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0, r.stdout[-3000:]
