"""Tensor-parallel decode over 2, 4 and 8 GPUs (one process per GPU, exchange inside the persistent kernel over peer memory)
against the CPU restatement of the full model.  A case is skipped on a box with fewer GPUs than it needs."""
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


CASES = {
    # name: (world size, model shape or None for the shared tiny file)
    "tiny-tp2": (2, None),
    "wide-tp2": (2, dict(NL=2, DM=256, NH=8, NKV=2, DH=64, DFF=512, NV=512)),
    "wide-tp4": (4, dict(NL=2, DM=256, NH=8, NKV=4, DH=64, DFF=1024, NV=1024)),
    "wide-tp8": (8, dict(NL=2, DM=512, NH=16, NKV=8, DH=64, DFF=2048, NV=2048)),
}


@pytest.mark.parametrize("which", list(CASES))
def test_tp_matches_full_model(which, tiny_file, tmp_path_factory):
    world, shape = CASES[which]
    if _gpus() < world:
        pytest.skip("needs %d GPUs" % world)
    if shape is None:
        path = tiny_file
    else:
        from conftest import make_model_file
        path = make_model_file(tmp_path_factory, shape, 21, which)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(HERE, "tp_worker.py"), path, "12", "12"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-6000:]
    assert "TP-OK world=%d" % world in r.stdout and "TP-BATCH-OK world=%d" % world in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
