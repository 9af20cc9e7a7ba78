"""The CPU checker against the reference's own fixtures and against golden vectors produced by the
reference's code (tests/golden/make_golden.py).  No GPU."""
import json
import os

import numpy as np
import pytest

import oracle_lib as ol

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_codec_tables_reference_selftest():
    # cuda_launch.c:769-786: 16 E2M1 values, six E4M3 known answers, NaN sentinel
    o = ol.oracle()
    e2 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for c in range(16):
        want = -e2[c & 7] if c & 8 else e2[c & 7]
        assert o.orc_e2m1_decode(c) == want
    for code, val in zip([0x00, 0x01, 0x08, 0x38, 0x7E, 0x40], [0.0, 0.001953125, 0.015625, 1.0, 448.0, 2.0]):
        assert o.orc_e4m3_decode(code) == val
    assert np.isnan(o.orc_e4m3_decode(0x7F))


def test_codecs_against_reference_golden():
    o = ol.oracle()
    g = np.load(os.path.join(G, "codec_golden.npz"))
    for c in range(256):
        a, b = o.orc_e4m3_decode(c), float(g["e4m3_table"][c])
        assert (np.isnan(a) and np.isnan(b)) or a == b
    got = np.array([o.orc_e4m3_encode(float(v)) for v in g["e4m3_in"]], np.int32)
    assert np.array_equal(got, g["e4m3_code"])
    got = np.array([o.orc_e2m1_encode(float(v)) for v in g["e2m1_in"]], np.int8)
    assert np.array_equal(got, g["e2m1_code"])


def test_e2m1_threshold_equals_search():
    # gpt2_pack.c:320-332 (--e2m1-equiv): 32 033 points
    o = ol.oracle()
    g = np.load(os.path.join(G, "codec_golden.npz"))
    v = g["e2m1_in"][:-3]
    assert len(v) == 32000 + 32 + 1 - 1 or len(v) > 32000
    a = np.array([o.orc_e2m1_encode(float(x)) for x in v], np.int8)
    b = np.array([o.orc_e2m1_encode_ref(float(x)) for x in v], np.int8)
    assert np.array_equal(a, b)
    assert np.array_equal(b, g["e2m1_code_search"])


def test_quantizer_against_reference_golden():
    g = np.load(os.path.join(G, "quant_golden.npz"))
    for i in list(range(int(g["n"]))) + ["z"]:
        W, mic, ts, sc = ol.quantize(g[f"w{i}"])
        assert np.array_equal(W, g[f"W{i}"]), i
        assert np.array_equal(mic, g[f"mic{i}"]), i
        assert np.float32(ts) == g[f"ts{i}"], i
        assert np.array_equal(sc, g[f"sc{i}"]), i
        if i != "z":
            assert np.array_equal(ol.dequant_micro(W, mic, ts), g[f"deq{i}"]), i
    assert g["tsz"] == np.float32(1.0)          # all-zero tensor: ts guard


def test_format_selftest_pattern():
    # gpt2_pack.c:391-416: rows=5, K=100 -> Kpad 112, dequant equals decode(code)*eff, pad columns 0
    o = ol.oracle()
    w = np.array([[((r * 37 + k * 13) % 101 - 50) * 0.043 for k in range(100)] for r in range(5)], np.float32)
    W, mic, ts, sc = ol.quantize(w)
    assert W.shape == (5, 16) and mic.shape == (5, 7)
    deq = ol.dequant_micro(W, mic, ts)
    for r in range(5):
        for k in range(112):
            eff = sc[r, k // 16]
            orig = w[r, k] if k < 100 else 0.0
            code = o.orc_e2m1_encode(float(np.float32(orig) / eff)) if eff > 0 else 0
            assert deq[r, k] == np.float32(o.orc_e2m1_decode(code)) * eff
            if k >= 100:
                assert deq[r, k] == 0.0


@pytest.mark.skipif(ol.reference() is None, reason="reference not compiled here (make -C oracle ref)")
def test_quantizer_against_live_reference():
    rng = np.random.default_rng(5)
    for rows, K in [(9, 333), (4, 2048), (1, 16), (12, 112)]:
        w = (rng.standard_normal((rows, K)) * rng.choice([1e-3, 0.02, 5.0])).astype(np.float32)
        a = ol.quantize(w)
        b = ol.quantize(w, ol.reference(), "ref_nvfp4_quantize")
        for x, y in zip(a, b):
            assert np.array_equal(np.asarray(x), np.asarray(y))


def test_sha256_known_answers():
    # the three NIST vectors of the reference self-test, gpt2_infer.c:199-213
    assert ol.sha256_hex(b"") == "e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855"
    assert ol.sha256_hex(b"abc") == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"
    assert ol.sha256_hex(b"abcdbcdecdefdefgefghfghighijhijkijkljklmklmnlmnomnopnopq") == \
        "248d6a61d20638b8e5c026930c3e6039a33ce45964ff2167f6ecedd419db06c1"
    import hashlib
    blob = bytes(range(256)) * 1000 + b"x"
    assert ol.sha256_hex(blob) == hashlib.sha256(blob).hexdigest()


def test_v3_writer_matches_reference_packer(tiny_file):
    # the file gpt2_pack --pack-qwen3 wrote for the same seeded checkpoint (hash committed)
    want = json.load(open(os.path.join(G, "v3_tiny.json")))
    data = open(tiny_file, "rb").read()
    assert len(data) == want["size"]
    assert ol.sha256_hex(data) == want["sha256"]
    assert ol.oracle().orc_v3_validate(data, len(data)) == 0


def test_v3_validation_rejects_damage(tiny_file):
    data = bytearray(open(tiny_file, "rb").read())
    o = ol.oracle()
    assert o.orc_v3_validate(bytes(data[:-1]), len(data) - 1) != 0          # truncated
    bad = bytearray(data); bad[0] ^= 1
    assert o.orc_v3_validate(bytes(bad), len(bad)) != 0                     # magic
    bad = bytearray(data); bad[64 + 16] ^= 4
    assert o.orc_v3_validate(bytes(bad), len(bad)) != 0                     # descriptor drift


def test_pack_micro_layout():
    # gpt2_infer.c:2151-2161: 4 bytes per word, low byte first, zero tail
    mic = (np.arange(3 * 7, dtype=np.uint8).reshape(3, 7) * 5 + 0x30) & 0x7E
    dst = np.zeros((3, 2), np.int32)
    ol.oracle().orc_pack_micro(mic, 3, 7, dst)
    for r in range(3):
        for b in range(7):
            assert (int(dst[r, b // 4]) >> (8 * (b % 4))) & 0xFF == mic[r, b]
        assert int(dst[r, 1]) >> 24 == 0


def test_gemv_orders_agree():
    # cuda_launch.c:2069-2073 fixture: codes (r*5+k*7+3)%16, micro (r*3+bk*11+0x30)&0x7E, ts=1/3,
    # x[k]=((k%11)-5)*0.25; ascending order vs the warp order within rel 1e-3 (cuda_launch.c:2088)
    N, K = 64, 336
    codes = np.array([[(r * 5 + k * 7 + 3) % 16 for k in range(K)] for r in range(N)], np.int64)
    W = np.zeros((N, K // 7), np.int32)
    for j in range(7):
        W += (codes[:, j::7] << (4 * j)).astype(np.int32)
    mic = np.array([[(r * 3 + b * 11 + 0x30) & 0x7E for b in range(K // 16)] for r in range(N)], np.uint8)
    x = np.array([((k % 11) - 5) * 0.25 for k in range(K)], np.float32)
    ts = np.float32(1.0 / 3.0)
    y1 = np.zeros(N, np.float32); y2 = np.zeros(N, np.float32)
    ol.oracle().orc_gemv_packed(x, W, mic, ts, y1, N, K)
    ol.oracle().orc_gemv_packed_warp_order(x, W, mic, ts, y2, N, K)
    # independent numpy restatement of the fixture's own oracle loop
    e2 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float32)
    e4 = np.array([ol.oracle().orc_e4m3_decode(int(c)) for c in range(128)], np.float32)
    wd = e2[codes] * (e4[mic] * ts).repeat(16, axis=1)
    y3 = (wd.astype(np.float64) @ x.astype(np.float64)).astype(np.float32)
    for y in (y1, y2):
        assert np.max(np.abs(y - y3) / np.maximum(np.abs(y3), 1e-6)) < 1e-3


def test_model_ops_against_numpy():
    # llama_ops_parity.sh shapes: rmsnorm S x 576 (x*4), rope (S*9) x 64 theta 1e5, silu_mul (g*5), softmax 3 x 91
    o = ol.oracle()
    rng = np.random.default_rng(20260609)
    x = (rng.standard_normal((5, 576)) * 4).astype(np.float32); w = rng.standard_normal(576).astype(np.float32)
    y = np.zeros_like(x); o.orc_rmsnorm(x, y, w, 5, 576, 1e-5)
    ref = w * (x / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-5))
    assert np.max(np.abs(y - ref)) < 1e-4
    half = 32; S = 45
    cosT = np.zeros((S, half), np.float32); sinT = np.zeros((S, half), np.float32)
    o.orc_rope_tables(cosT, sinT, S, 64, 1e5)
    inv = 1e5 ** (-2.0 * np.arange(half) / 64); ang = np.arange(S)[:, None] * inv
    assert np.array_equal(cosT, np.cos(ang).astype(np.float32)) and np.array_equal(sinT, np.sin(ang).astype(np.float32))
    q = rng.standard_normal((S, 64)).astype(np.float32); q0 = q.copy()
    o.orc_rope_rot(q, cosT, sinT, S, half)
    rot = np.concatenate([-q0[:, half:], q0[:, :half]], 1)
    ref = q0 * np.concatenate([cosT, cosT], 1) + rot * np.concatenate([sinT, sinT], 1)
    assert np.max(np.abs(q - ref)) < 1e-5
    g = (rng.standard_normal(300) * 5).astype(np.float32); u = rng.standard_normal(300).astype(np.float32)
    y = np.zeros(300, np.float32); o.orc_silu_mul(g, u, y, 300)
    assert np.max(np.abs(y - g / (1 + np.exp(-g.astype(np.float64))) * u)) < 1e-4
    s = rng.standard_normal((3, 91)).astype(np.float32); p = np.zeros_like(s)
    o.orc_softmax_row(s, p, 3, 91)
    e = np.exp(s - s.max(-1, keepdims=True)); assert np.max(np.abs(p - e / e.sum(-1, keepdims=True))) < 1e-6
    xg = rng.standard_normal(257).astype(np.float32); yg = np.zeros_like(xg); o.orc_gelu(xg, yg, 257)
    ref = 0.5 * xg * (1 + np.tanh(0.7978845608 * (xg + 0.044715 * xg.astype(np.float64) ** 3)))
    assert np.max(np.abs(yg - ref)) < 1e-5
    assert o.orc_argmax(np.array([1, 5, 5, np.nan, 2], np.float32), 5) == 1


def test_decode_equals_online_attention_form(tiny_file):
    # the two attention forms of the reference (three-pass per head vs the fused online softmax) agree
    m = ol.OracleModel(tiny_file, kv_cap=32)
    ids = np.random.default_rng(1).integers(0, m.NV, 12)
    lg = m.prefill(ids)
    assert np.isfinite(lg).all() and lg.shape == (m.NV,)
    out = m.generate(ids, 5)
    m2 = ol.OracleModel(tiny_file, kv_cap=32)
    lg2 = m2.prefill(ids)
    assert np.array_equal(lg, lg2) and out[0] == int(np.argmax(lg))
    m.close(); m2.close()


def test_model_level_restatement_against_the_reference_gpu_worker():
    """ref_worker_logits.npz holds last-row logits computed by the UNMODIFIED reference worker (gpt2_infer.c with
    its own compiler's PTX) on a B200 for three small seeded models (tests/golden/make_ref_worker_golden.py).  The
    CPU restatement of the decode sequencing, run on the same seeded weights and prompt, must reproduce them."""
    import tempfile
    g = np.load(os.path.join(G, "ref_worker_logits.npz"))
    names = sorted(k[len("logits_"):] for k in g.files if k.startswith("logits_"))
    assert len(names) >= 3
    for name in names:
        NL, DM, NH, NKV, DH, DFF, NV = (int(v) for v in g["cfg_" + name])
        cfg = dict(NL=NL, DM=DM, NH=NH, NKV=NKV, DH=DH, DFF=DFF, NV=NV)
        with tempfile.TemporaryDirectory() as d:
            path = os.path.join(d, "m.weights")
            ol.write_v3(path, cfg, ol.synth_tensors(cfg, seed=int(g["seed_w"])))
            ids = np.random.default_rng(int(g["seed_ids"])).integers(0, NV, int(g["n_prompt"])).astype(np.int32)
            om = ol.OracleModel(path, kv_cap=64)
            lo = om.prefill(ids)
            om.close()
        want = g["logits_" + name]
        assert np.max(np.abs(lo - want)) < 2e-5, (name, float(np.max(np.abs(lo - want))))
        assert int(np.argmax(lo)) == int(np.argmax(want))
