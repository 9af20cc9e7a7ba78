#!/usr/bin/env python
"""Captures the reference GPU worker's own logits as a fixture (run on a machine with a GPU).

Runs tests/test_ref_worker_gpu.py with HX_REF_WORKER_DUMP set, which makes the test save the last-row logits that
the unmodified reference worker (oracle/_ref/gpt2_infer + its own PTX, oracle/_ref/kovc/) computed for each small
model, then packs them with the recipe of their inputs into ref_worker_logits.npz next to this script (or into the
folder given as argument).  tests/test_oracle_golden.py rebuilds the same seeded models on the CPU and compares the
CPU restatement with these logits, so the restatement stays pinned where no GPU is present.

usage: python tests/golden/make_ref_worker_golden.py [<output folder>]
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "tests")); sys.path.insert(0, ROOT)


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else HERE
    import test_ref_worker_gpu as t
    with tempfile.TemporaryDirectory() as d:
        env = dict(os.environ, HX_REF_WORKER_DUMP=d)
        subprocess.check_call([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_ref_worker_gpu.py"), "-q", "-m", "gpu",
                               "-k", "prefill_logits and kovc"], env=env, cwd=ROOT)
        pack = dict(seed_w=t.SEED_W, seed_ids=t.SEED_IDS, n_prompt=t.N_PROMPT)
        for name, cfg in t.CFGS.items():
            pack["logits_" + name] = np.load(os.path.join(d, f"ref_worker_logits_{name}.npy"))
            pack["cfg_" + name] = np.array([cfg[k] for k in ("NL", "DM", "NH", "NKV", "DH", "DFF", "NV")], np.int32)
        np.savez_compressed(os.path.join(out_dir, "ref_worker_logits.npz"), **pack)
    print("wrote", os.path.join(out_dir, "ref_worker_logits.npz"))


if __name__ == "__main__":
    main()
