"""Tensor-parallel decode over 2 GPUs (one process per GPU, exchange inside the persistent kernel over peer memory)
against the CPU restatement of the full model.  Skipped on a box with fewer than two GPUs."""
import os
import subprocess
import sys

import pytest

import helix_b200 as hb

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _gpus():
    import ctypes as C
    n = C.c_int()
    return n.value if hb.lib().hx_device_count(C.byref(n)) == 0 else 0


@pytest.mark.parametrize("which", ["tiny", "wide2"])
def test_tp2_matches_full_model(which, tiny_file, tmp_path_factory):
    if _gpus() < 2:
        pytest.skip("needs two GPUs")
    if which == "tiny":
        path = tiny_file
    else:
        from conftest import make_model_file
        path = make_model_file(tmp_path_factory, dict(NL=2, DM=256, NH=8, NKV=2, DH=64, DFF=512, NV=512), 21, "wide2")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(HERE, "tp_worker.py"), path, "12", "12"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "TP-OK world=2" in r.stdout
