"""Generates the committed golden vectors from the REFERENCE's own code, compiled unmodified
(oracle/Makefile target `ref`: helixc/runtime/gpt2_pack.c through oracle/ref_wrap.c, and the gpt2_pack /
gpt2_infer binaries).  Run here, where the reference tree is present; the outputs travel as small files.

    python tests/golden/make_golden.py

Writes tests/golden/quant_golden.npz (inputs + the reference quantizer's words / micro / ts / scales
+ its host dequant), tests/golden/codec_golden.npz (encoder decisions on boundary values) and
tests/golden/v3_tiny.json (SHA-256 and size of the file `gpt2_pack --pack-qwen3` writes for a seeded
tiny checkpoint, plus the reference verifier's verdicts on receipts).
"""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as ol  # noqa: E402


def main():
    ref = ol.reference()
    assert ref is not None, "build the reference first: make -C oracle ref"
    rng = np.random.default_rng(20261125)
    cases = {}
    shapes = [(5, 100), (8, 112), (16, 256), (3, 7), (6, 1030), (4, 4096), (2, 113)]
    for i, (rows, K) in enumerate(shapes):
        scale = [0.02, 1.0, 37.5, 1e-6, 0.02, 0.02, 3.0][i]
        w = (scale * rng.standard_normal((rows, K))).astype(np.float32)
        if i == 1:      # the reference self-test pattern, gpt2_pack.c:398
            w = np.array([[((r * 37 + k * 13) % 101 - 50) * 0.043 for k in range(K)] for r in range(rows)], np.float32)
        if i == 2:      # exact ties and zeros
            w[0, :] = 0.0
            w[1, :16] = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0], np.float32) * 8
        W, mic, ts, sc = ol.quantize(w, ref, "ref_nvfp4_quantize")
        deq = np.zeros((rows, W.shape[1] * 7), np.float32)
        ref.ref_nvfp4_host_dequant(W, sc, deq, rows, W.shape[1] * 7)
        cases[f"w{i}"] = w
        cases[f"W{i}"] = W
        cases[f"mic{i}"] = mic
        cases[f"ts{i}"] = np.float32(ts)
        cases[f"sc{i}"] = sc
        cases[f"deq{i}"] = deq
    zero = np.zeros((2, 32), np.float32)
    W, mic, ts, sc = ol.quantize(zero, ref, "ref_nvfp4_quantize")
    cases.update(wz=zero, Wz=W, micz=mic, tsz=np.float32(ts), scz=sc, n=np.int32(len(shapes)))
    np.savez_compressed(os.path.join(HERE, "quant_golden.npz"), **cases)

    # encoder decisions around every decision boundary (+-2 ulp), from the reference's own encoders
    vals = []
    for c in range(0x7F):
        a, b = ref.ref_e4m3_decode(c), ref.ref_e4m3_decode(c + 1) if c + 1 < 0x7F else 512.0
        for base in (a, (a + b) / 2):
            f = np.float32(base)
            for _ in range(3):
                f = np.nextafter(f, np.float32(-1))
            for _ in range(7):
                vals.append(f)
                f = np.nextafter(f, np.float32(1e9))
    vals += [0.0, 1e-12, 1e-7, 447.9, 448.0, 448.1, 500.0, 1e20, 1e31, float("inf"), float("nan"), -1.0, -0.001, -448.0]
    vals = np.array(vals, np.float32)
    e4 = np.array([ref.ref_e4m3_encode(float(v)) for v in vals], np.int32)
    v2 = np.concatenate([np.arange(-8, 8, 0.0005, dtype=np.float64).astype(np.float32),
                         np.array([0, .25, .5, .75, 1, 1.25, 1.5, 1.75, 2, 2.5, 3, 3.5, 4, 5, 6, 7], np.float32),
                         -np.array([0, .25, .5, .75, 1, 1.25, 1.5, 1.75, 2, 2.5, 3, 3.5, 4, 5, 6, 7], np.float32),
                         np.array([np.nan, np.inf, -np.inf], np.float32)])
    e2 = np.array([ref.ref_e2m1_encode(float(v)) for v in v2], np.int8)
    e2r = np.array([ref.ref_e2m1_encode_ref(float(v)) for v in v2[:-3]], np.int8)
    d4 = np.array([ref.ref_e4m3_decode(c) for c in range(256)], np.float32)
    d2 = np.array([ref.ref_e2m1_decode(c) for c in range(16)], np.float32)
    np.savez_compressed(os.path.join(HERE, "codec_golden.npz"), e4m3_in=vals, e4m3_code=e4, e2m1_in=v2, e2m1_code=e2,
                        e2m1_code_search=e2r, e4m3_table=d4, e2m1_table=d2)

    # the reference packer on a seeded tiny Qwen3-shaped checkpoint
    cfg = dict(NL=2, DM=128, NH=4, NKV=2, DH=32, DFF=256, NV=300)
    T = ol.synth_tensors(cfg, seed=3)
    d = tempfile.mkdtemp()
    ol.write_safetensors(d + "/model.safetensors", T)
    ol.write_qwen3_config(d + "/config.json", cfg)
    p = subprocess.run([ol.REF_PACK, "--pack-qwen3", d, d + "/ref.weights"], capture_output=True, text=True)
    assert "PACK_QWEN3_OK" in p.stdout, p.stdout + p.stderr
    data = open(d + "/ref.weights", "rb").read()
    env = dict(os.environ, LD_LIBRARY_PATH=os.path.join(ol.ORACLE_DIR, "_ref", "cpu_stub"))
    kat = subprocess.run([ol.REF_INFER, "--sha256-selftest"], capture_output=True, text=True, env=env)
    out = dict(cfg=cfg, seed=3, size=len(data), sha256=ol.sha256_hex(data),
               pack_stdout=p.stdout.strip(), ref_sha_selftest=kat.stdout.strip())
    # cross-check of the oracle's SHA-256 with the system's
    import hashlib
    assert hashlib.sha256(data).hexdigest() == out["sha256"]
    json.dump(out, open(os.path.join(HERE, "v3_tiny.json"), "w"), indent=1)
    print("golden vectors written:", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    main()
