"""The C-ABI library loads without a GPU, exports every symbol include/helix_b200.h declares, and its
host-side pieces (codecs, SHA-256, receipt) agree with the checker.  No compute calls."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

import helix_b200 as hb
import oracle_lib as ol

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
G = os.path.join(ROOT, "tests", "golden")

ENTRY_NAMES = ["nvfp4_dequant", "nvfp4_dequant_tiled", "gemv_abt_nvfp4", "dequant_gemv_blockred", "dequant_gemv_warp",
               "fused_decode_attn", "softmax_causal_offset", "gpu_gemv_abt", "gpu_gemv_ab", "gpu_softmax_row",
               "gpu_softmax_causal", "gpu_rmsnorm_fwd_eps", "gpu_rope_rot", "gpu_silu_mul", "gpu_layernorm_fwd_eps",
               "gpu_add_bias_rowbcast", "gpu_gelu_stable", "vector_add", "gpu_scale_rt", "tiled_matmul", "tiled_matmul_abt"]


def declared_functions():
    src = open(os.path.join(ROOT, "include", "helix_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(hx_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    L = C.CDLL(hb.lib_path())
    names = declared_functions()
    assert len(names) >= 40
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/helix_b200.h but not exported"


def test_binding_covers_header():
    from helix_b200.lib import _SIGS
    assert set(declared_functions()) <= set(_SIGS) | {"hx_sha256"}


def test_kernel_image_has_every_reference_entry():
    blob = open(hb.fatbin_path(), "rb").read()
    for n in ENTRY_NAMES:
        assert n.encode() in blob, f"entry {n} missing from the kernel image"


def test_no_gpu_is_an_error_not_a_fallback():
    L = hb.lib()
    n = C.c_int(0)
    rc = L.hx_device_count(C.byref(n))
    if rc == 0 and n.value > 0:
        pytest.skip("a GPU is present")
    w = np.ones((2, 16), np.float32)
    with pytest.raises(hb.HxError):
        hb.quantize_host(w)
    with pytest.raises(hb.HxError):
        hb.Model.synth(dict(n_layers=1, d_model=64, n_heads=2, n_kv_heads=1, head_dim=32, d_ff=64, vocab=64), kv_cap=8)


def test_host_codecs_match_reference_golden():
    L = hb.lib()
    g = np.load(os.path.join(G, "codec_golden.npz"))
    for c in range(256):
        a, b = L.hx_e4m3_decode(c), float(g["e4m3_table"][c])
        assert (np.isnan(a) and np.isnan(b)) or a == b
    for c in range(16):
        assert L.hx_e2m1_decode(c) == float(g["e2m1_table"][c])
    got = np.array([L.hx_e4m3_encode(float(v)) for v in g["e4m3_in"]], np.int32)
    bad = np.nonzero(got != g["e4m3_code"])[0]
    assert len(bad) == 0, [(float(g["e4m3_in"][i]), int(got[i]), int(g["e4m3_code"][i])) for i in bad[:5]]
    got = np.array([L.hx_e2m1_encode(float(v)) for v in g["e2m1_in"]], np.int8)
    assert np.array_equal(got, g["e2m1_code"])


def test_closed_form_e4m3_encoder_equals_search_on_random_values():
    # the library finds the E4M3 code in closed form; the reference searches 254 codes
    L, o = hb.lib(), ol.oracle()
    rng = np.random.default_rng(9)
    v = np.concatenate([np.exp(rng.uniform(np.log(1e-6), np.log(600.0), 40000)), rng.uniform(0, 0.02, 5000),
                        rng.uniform(440, 460, 2000)]).astype(np.float32)
    for x in v:
        assert L.hx_e4m3_encode(float(x)) == o.orc_e4m3_encode(float(x)), float(x)


def test_sha256_and_kpad():
    L = hb.lib()
    buf = C.create_string_buffer(65)
    for msg in (b"", b"abc", b"abcdbcdecdefdefgefghfghighijhijkijkljklmklmnlmnomnopnopq", bytes(range(256)) * 777):
        assert L.hx_sha256_hex(msg, len(msg), buf) == 0
        assert buf.value.decode() == ol.sha256_hex(msg)
    for K, want in [(768, 784), (3072, 3136), (4096, 4144), (5120, 5152), (8192, 8288), (12288, 12320), (25600, 25648), (100, 112)]:
        assert L.hx_kpad(K) == want


def _write(path, arr):
    with open(path, "wb") as f:
        f.write(np.ascontiguousarray(arr).tobytes())


def test_receipt_roundtrip_and_named_rejects(tmp_path, tiny_file):
    L = hb.lib()
    rng = np.random.default_rng(2)
    nv = 300
    logits = rng.standard_normal(nv).astype(np.float32)
    oracle_logits = (logits + 1e-3 * rng.standard_normal(nv)).astype(np.float32)
    ids = np.array([5, 9, 200], np.int32)
    rc_path, orc_path = str(tmp_path / "r.receipt"), str(tmp_path / "oracle.bin")
    _write(orc_path, oracle_logits)
    assert L.hx_receipt_emit(rc_path.encode(), tiny_file.encode(), ids.ctypes.data, 3, logits.ctypes.data, nv,
                             oracle_logits.ctypes.data, 0.5, b"unit-test") == 0
    lg_path = rc_path + ".logits"
    assert L.hx_receipt_check(rc_path.encode(), tiny_file.encode(), lg_path.encode(), orc_path.encode()) == 0
    text = open(rc_path).read()
    assert text.startswith("HELIX_V16_RECEIPT\n") and f"argmax {int(np.argmax(logits))}\n" in text
    assert "ids 5 9 200\n" in text and "tier3_tau 0.5\n" in text

    def reject(receipt=rc_path, weights=tiny_file, lg=lg_path, orc=orc_path):
        rc = L.hx_receipt_check(receipt.encode(), weights.encode(), lg.encode(), orc.encode())
        assert rc != 0
        return L.hx_last_error().decode()

    # the reference's five named rejects (scripts/gpu_qwen3_receipt_check.sh)
    bad_w = str(tmp_path / "w.bad"); d = bytearray(open(tiny_file, "rb").read()); d[1000] ^= 1; open(bad_w, "wb").write(d)
    assert "REJECT=MODEL_HASH" in reject(weights=bad_w)
    bad_l = str(tmp_path / "l.bad"); l2 = logits.copy(); l2[7] += 1.0; _write(bad_l, l2)
    assert "REJECT=LOGITS_HASH" in reject(lg=bad_l)
    far = str(tmp_path / "far.bin"); _write(far, oracle_logits + 2.0)
    assert "REJECT=TIER3_ENVELOPE" in reject(orc=far)
    t2 = str(tmp_path / "t.receipt"); open(t2, "w").write(re.sub(r"argmax \d+", "argmax 1", text, count=1))
    assert "REJECT=ARGMAX" in reject(receipt=t2)
    t3 = str(tmp_path / "v.receipt"); open(t3, "w").write("HELIX_V16_RECEIPT\n")
    assert "REJECT=VACUITY" in reject(receipt=t3)
    # tau below the receipt's own max_abs
    t4 = str(tmp_path / "tau.receipt"); open(t4, "w").write(re.sub(r"tier3_tau \S+", "tier3_tau 1e-9", text))
    assert "REJECT=TIER3_ENVELOPE" in reject(receipt=t4)

    # the reference's own verifier accepts the receipt this library wrote
    if os.path.exists(ol.REF_INFER):
        env = dict(os.environ)
        stub = os.path.join(ol.ORACLE_DIR, "_ref", "cpu_stub")
        n = C.c_int(0)
        if L.hx_device_count(C.byref(n)) != 0 or n.value == 0:
            env["LD_LIBRARY_PATH"] = stub + ":" + env.get("LD_LIBRARY_PATH", "")
        p = subprocess.run([ol.REF_INFER, "--v3-receipt-check", rc_path, tiny_file, lg_path, orc_path],
                           capture_output=True, text=True, env=env)
        assert "RECEIPT_CHECK_PASS" in p.stdout, p.stdout + p.stderr
        p = subprocess.run([ol.REF_INFER, "--v3-receipt-check", rc_path, bad_w, lg_path, orc_path],
                           capture_output=True, text=True, env=env)
        assert "REJECT=MODEL_HASH" in p.stdout


def test_bad_files_are_rejected_before_any_device_work(tmp_path, tiny_file):
    L = hb.lib()
    h = C.c_void_p()
    assert L.hx_model_load(C.byref(h), b"/nonexistent/file", 16, 1, 0, 0, 1) == 3          # HX_ERR_IO
    data = bytearray(open(tiny_file, "rb").read())
    for name, mut in [("trunc", lambda d: d[:-5]), ("magic", lambda d: bytes([d[0] ^ 1]) + bytes(d[1:])),
                      ("drift", lambda d: bytes(d[:80]) + bytes([d[80] ^ 4]) + bytes(d[81:])),
                      ("short", lambda d: d[:40])]:
        p = str(tmp_path / name); open(p, "wb").write(bytes(mut(data)))
        assert L.hx_model_load(C.byref(h), p.encode(), 16, 1, 0, 0, 1) == 4, name       # HX_ERR_FORMAT


def test_argument_checks_of_the_wider_entry_points_need_no_device(tiny_file):
    """Shape and range checks come before any CUDA call: tensor-parallel shards, batch, GPT-2, no-alloc quantizer."""
    L = hb.lib()
    h = C.c_void_p()
    # TINY has 4 heads / 2 kv heads: a group of 3 ranks does not divide them, rank outside the group is refused
    assert L.hx_model_load(C.byref(h), tiny_file.encode(), 16, 1, 0, 0, 3) == 1           # HX_ERR_ARG
    assert b"divisible" in L.hx_last_error()
    assert L.hx_model_load(C.byref(h), tiny_file.encode(), 16, 1, 0, 2, 2) == 1
    assert L.hx_model_load(C.byref(h), tiny_file.encode(), 16, 0, 0, 0, 1) == 1           # batch 0
    from helix_b200.lib import HxConfig, HxGpt2Weights
    cfg = HxConfig(1, 2, 128, 4, 4, 32, 512, 300, 64, 0.0, 1e-5, 0)                       # arch 1 is not GPT-2
    one = (C.c_float * 4)()
    w = HxGpt2Weights(C.addressof(one), C.addressof(one), C.addressof(one), C.addressof(one), None)
    assert L.hx_model_gpt2(C.byref(h), C.byref(cfg), C.byref(w), 16) == 1                 # null layer table
    assert L.hx_quantize_nvfp4_noalloc(C.addressof(one), L.hx_noalloc_max_rows() + 1, 16, C.addressof(one), None, None, None, None) == 1
    assert L.hx_decode_batch(None, None, None, 1, None) == 1
