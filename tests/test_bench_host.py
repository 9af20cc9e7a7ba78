"""Host-side logic of the benchmark: the algorithmic byte count, the host-built HXGW v3 image of the
reference arm, and the replica sharding over ranks (world_size 2, gloo, CPU)."""
import os
import subprocess
import sys

import numpy as np

import oracle_lib as ol

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_algorithmic_bytes_qwen3_8b():
    import helix_b200 as hb
    w, kv, emb = bench.algorithmic_bytes_per_token(dict(hb.QWEN3_8B), 640)
    assert abs(w - 4.257e9) < 2e6            # 7.568 G weights x 0.5625 B
    assert kv == 294912 * 640 and emb == 16384


def test_host_built_image_is_a_valid_model():
    shape = dict(n_layers=2, d_model=128, n_heads=4, n_kv_heads=2, head_dim=32, d_ff=256, vocab=300)
    img = bench.synth_image_on_host(shape, seed=4)
    assert ol.oracle().orc_v3_validate(img.ctypes.data, img.nbytes) == 0
    v, cores = bench.cpu_decode_tok_s(img, 3, kv_cap=8)
    assert v > 0 and cores >= 1


def test_two_rank_reduction_over_gloo(tmp_path):
    # the multi-GPU path shards whole sequences over ranks and only reduces timings on the host
    script = tmp_path / "w.py"
    script.write_text(
        "import os, sys\n"
        f"sys.path.insert(0, {ROOT!r})\n"
        "import bench\n"
        "d = bench.dist_init(2)\n"
        "r = int(os.environ['RANK'])\n"
        "m = bench.all_max(d, 10.0 + r); s = bench.all_sum(d, 1.0 + r)\n"
        "assert m == 11.0 and s == 3.0, (m, s)\n"
        "d.barrier(); d.destroy_process_group()\n"
        "sys.stdout.write('rank-%d-ok\\n' % r); sys.stdout.flush()\n")
    import socket
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                       capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout + p.stderr
    assert "rank-0-ok" in p.stdout and "rank-1-ok" in p.stdout
