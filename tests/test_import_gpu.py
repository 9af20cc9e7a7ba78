"""The GPU importer (hx_pack_qwen3: safetensors checkpoint -> HXGW v3 NVFP4 file) against the reference's
pack_qwen3 (helixc/runtime/gpt2_pack.c:587-733): the file must be the same bytes.  Checked three ways: the
committed hash of the file the reference packer wrote for the seeded tiny checkpoint, the CPU restatement's writer
on the same tensors, and -- where the compiled reference packer is present -- the reference run on the very same
checkpoint directory (F32 single file, BF16 in shards)."""
import json
import os
import subprocess

import numpy as np
import pytest

import helix_b200 as hb
import oracle_lib as ol
from conftest import TINY

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_f32_single_file_matches_the_reference_packer(tmp_path):
    T = ol.synth_tensors(TINY, seed=3)
    d = str(tmp_path)
    ol.write_safetensors(d + "/model.safetensors", T)
    ol.write_qwen3_config(d + "/config.json", TINY)
    rep = hb.pack_qwen3(d, d + "/ours.weights")
    data = open(d + "/ours.weights", "rb").read()
    want = json.load(open(os.path.join(G, "v3_tiny.json")))          # written by the reference packer, hash committed
    assert len(data) == want["size"] == rep["bytes"]
    assert ol.sha256_hex(data) == want["sha256"]
    assert rep["tensors"] == 2 * 11 + 3 and rep["packed"] == 2 * 7 + 1
    assert rep["verified"] and rep["f32_exact"] and 0.05 < rep["worst_rms"] < 0.15      # the reference expects about 0.095
    ol.write_v3(d + "/oracle.weights", TINY, T)
    assert data == open(d + "/oracle.weights", "rb").read()


@pytest.mark.parametrize("cfg", [dict(NL=2, DM=256, NH=4, NKV=2, DH=128, DFF=640, NV=1500),      # q width != d_model
                                 dict(NL=3, DM=192, NH=6, NKV=2, DH=32, DFF=328, NV=1001)])      # K not a multiple of 112 or 16
def test_bf16_shards_match_the_reference_packer(tmp_path, cfg):
    T = ol.synth_tensors(cfg, seed=9)
    d = str(tmp_path)
    ol.write_sharded_checkpoint(d, cfg, T, n_shards=3, dtype="BF16")
    rep = hb.pack_qwen3(d, d + "/ours.weights")
    data = open(d + "/ours.weights", "rb").read()
    widened = {n: ol.from_bf16_bits(ol.to_bf16_bits(t)).reshape(t.shape) for n, t in T.items()}
    ol.write_v3(d + "/oracle.weights", cfg, widened)
    assert data == open(d + "/oracle.weights", "rb").read()
    assert rep["f32_exact"] and rep["worst_rms"] < 0.15
    if os.path.exists(ol.REF_PACK):
        p = subprocess.run([ol.REF_PACK, "--pack-qwen3", d, d + "/ref.weights"], capture_output=True, text=True)
        assert "PACK_QWEN3_OK" in p.stdout, p.stdout + p.stderr
        assert data == open(d + "/ref.weights", "rb").read()
        ref_worst = float(p.stdout.split("worst_rms=")[1].split()[0])
        assert abs(ref_worst - rep["worst_rms"]) < 2e-4              # the reference prints four decimals
    # the file loads and decodes like any other
    gm = hb.Model.load(d + "/ours.weights", kv_cap=32)
    om = ol.OracleModel(d + "/ours.weights", kv_cap=32)
    ids = np.random.default_rng(2).integers(0, cfg["NV"], 6).astype(np.int32)
    nx, lg = gm.prefill(ids, want_logits=True)
    lo = om.prefill(ids)
    gm.close(); om.close()
    assert float(np.max(np.abs(lg - lo))) < 2e-4 and nx == int(np.argmax(lo))


def test_importer_rejects_bad_checkpoints(tmp_path):
    T = ol.synth_tensors(TINY, seed=3)
    d = str(tmp_path)
    ol.write_qwen3_config(d + "/config.json", TINY)
    # a tensor is missing
    part = {n: t for n, t in T.items() if n != "model.layers.1.mlp.up_proj.weight"}
    ol.write_safetensors(d + "/model.safetensors", part)
    with pytest.raises(hb.HxError, match="lacks tensor"):
        hb.pack_qwen3(d, d + "/x.weights")
    # a shape that does not fit the config
    bad = dict(T); bad["model.norm.weight"] = np.ones(TINY["DM"] + 1, np.float32)
    ol.write_safetensors(d + "/model.safetensors", bad)
    with pytest.raises(hb.HxError, match="expected"):
        hb.pack_qwen3(d, d + "/x.weights")
    # a dtype the importer does not take (the reference exits on it too, gpt2_pack.c:195-197)
    ol.write_safetensors(d + "/model.safetensors", T)
    raw = open(d + "/model.safetensors", "rb").read()
    open(d + "/model.safetensors", "wb").write(raw.replace(b'"dtype":"F32"', b'"dtype":"F16"', 1))
    with pytest.raises(hb.HxError, match="F16"):
        hb.pack_qwen3(d, d + "/x.weights")
    # no checkpoint at all
    with pytest.raises(hb.HxError):
        hb.pack_qwen3(d + "/nowhere", d + "/x.weights")
