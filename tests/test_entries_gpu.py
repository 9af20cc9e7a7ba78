"""The kernel-entry image launched like the reference's launchers launch their PTX: same entry names,
argument lists and grid/block shapes, checked with the fixtures and tolerances of the reference's
kernel gates (cuda_launch.c modes nvfp4, gemv_nvfp4, dgemv_blockred, dgemv_warp; gemv_ops_parity.sh;
llama_ops_parity.sh)."""
import numpy as np
import pytest

import helix_b200 as hb
import oracle_lib as ol

pytestmark = pytest.mark.gpu
DB = hb.DeviceBuffer


@pytest.fixture(scope="module")
def img():
    im = hb.KernelImage()
    yield im
    im.close()


def fixture_codes(rows, K):
    codes = np.array([[(r * 5 + k * 7 + 3) % 16 for k in range(K)] for r in range(rows)], np.int64)
    W = np.zeros((rows, K // 7), np.int32)
    for j in range(7):
        W += (codes[:, j::7] << (4 * j)).astype(np.int32)
    mic = np.array([[(r * 3 + b * 11 + 0x30) & 0x7E for b in range(K // 16)] for r in range(rows)], np.uint8)
    return codes, W, mic


def e4(mic):
    t = np.array([ol.oracle().orc_e4m3_decode(c) for c in range(128)], np.float32)
    return t[mic]


E2 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float32)


@pytest.mark.parametrize("entry,M,K", [("nvfp4_dequant", 8, 112), ("nvfp4_dequant", 5, 336), ("nvfp4_dequant_tiled", 8, 112),
                                       ("nvfp4_dequant_tiled", 3, 4144)])
def test_nvfp4_dequant_modes(img, entry, M, K):
    # cuda_launch.c:1990-2040: ts = 1/3, exact within abs 1e-5 or rel 1e-6; negative controls wflip / sflip
    codes, W, mic = fixture_codes(M, K)
    sc = (e4(mic) * np.float32(1.0 / 3.0)).astype(np.float32)
    ref = E2[codes] * sc.repeat(16, axis=1)
    dW, dS, dO = DB.from_array(W), DB.from_array(sc), DB(M * K * 4)

    def run():
        if entry == "nvfp4_dequant":
            img.launch(entry, (M,), (K,), [dW, dS, dO, M, K, 1])
        else:
            img.launch(entry, (M * K // 112,), (112,), [dW, dS, dO, 0, K, 112])
        return dO.to_array(np.float32).reshape(M, K)

    out = run()
    assert np.array_equal(out, ref)
    W2 = W.copy(); W2[0, 0] = W2[0, 0] - (W2[0, 0] & 15) + ((W2[0, 0] & 15) + 1) % 16
    dW.upload(W2); assert not np.array_equal(run(), ref)                     # wflip must trip
    dW.upload(W); sc2 = sc.copy(); sc2[0, 0] = sc2[0, 0] * 1.5 + 0.123
    dS.upload(sc2); assert not np.array_equal(run(), ref)                    # sflip must trip


@pytest.mark.parametrize("N,K", [(8, 112), (64, 112), (128, 4144), (64, 784)])
def test_fused_gemv_modes(img, N, K):
    codes, W, mic = fixture_codes(N, K)
    ts = np.float32(1.0 / 3.0)
    x = np.array([((k % 11) - 5) * 0.25 for k in range(K)], np.float32)
    yref = np.zeros(N, np.float32); ol.oracle().orc_gemv_packed(x, W, mic, ts, yref, N, K)
    ywarp = np.zeros(N, np.float32); ol.oracle().orc_gemv_packed_warp_order(x, W, mic, ts, ywarp, N, K)
    mst = (K // 16 + 3) // 4
    m4 = np.zeros((N, mst), np.int32); ol.oracle().orc_pack_micro(mic, N, K // 16, m4)
    sc = (e4(mic) * ts).astype(np.float32)
    dX, dW, dM, dT, dS, dY = DB.from_array(x), DB.from_array(W), DB.from_array(m4), DB.from_array(np.array([ts])), DB.from_array(sc), DB(N * 4)

    def rel(y):
        return np.max(np.abs(y - yref) / np.maximum(np.abs(yref), 1e-6))

    img.launch("dequant_gemv_warp", ((N + 7) // 8,), (32, 8), [dX, dW, dM, dT, dY, K])
    y = dY.to_array(np.float32)
    assert np.array_equal(y, ywarp) and rel(y) <= 1e-3
    dY.zero(); img.launch("dequant_gemv_blockred", (N,), (256,), [dX, dW, dM, dT, dY, K])
    assert rel(dY.to_array(np.float32)) <= 1e-3
    dY.zero(); img.launch("gemv_abt_nvfp4", (N,), (1,), [dX, dW, dS, dY, K])
    assert rel(dY.to_array(np.float32)) <= 1e-3
    # sflip negative control: bump block 0's micro byte (cuda_launch.c:2133)
    m4b = m4.copy(); m4b[0, 0] = (m4b[0, 0] & ~0xFF) | (0x18 if mic[0, 0] == 0x10 else 0x10)
    dM.upload(m4b); dY.zero(); img.launch("dequant_gemv_warp", ((N + 7) // 8,), (32, 8), [dX, dW, dM, dT, dY, K])
    assert rel(dY.to_array(np.float32)) > 1e-3


def test_unquantized_ops(img):
    # gemv_ops_parity.sh: gemv_abt N=113,K=960; gemv_ab T=37,N=64; softmax_row 3x91; max-abs 1e-4
    o = ol.oracle()
    rng = np.random.default_rng(20260610)
    x = rng.standard_normal(960).astype(np.float32); w = rng.standard_normal((113, 960)).astype(np.float32)
    dY = DB(113 * 4); img.launch("gpu_gemv_abt", (113,), (1,), [DB.from_array(x), DB.from_array(w), dY, 960])
    assert np.max(np.abs(dY.to_array(np.float32) - (w.astype(np.float64) @ x).astype(np.float32))) < 1e-4
    w2 = rng.standard_normal((128, 64)).astype(np.float32); x2 = rng.standard_normal(64).astype(np.float32)
    dY = DB(128 * 4); img.launch("gpu_gemv_abt", (1,), (128,), [DB.from_array(x2), DB.from_array(w2), dY, 64])
    assert np.max(np.abs(dY.to_array(np.float32) - (w2.astype(np.float64) @ x2))) < 1e-4
    p = rng.standard_normal(37).astype(np.float32); m = rng.standard_normal((37, 64)).astype(np.float32)
    dY = DB(64 * 4); img.launch("gpu_gemv_ab", (64,), (1,), [DB.from_array(p), DB.from_array(m), dY, 37, 64])
    assert np.max(np.abs(dY.to_array(np.float32) - (p.astype(np.float64) @ m))) < 1e-4
    s = rng.standard_normal((3, 91)).astype(np.float32); ref = np.zeros_like(s); o.orc_softmax_row(s, ref, 3, 91)
    dY = DB(s.nbytes); img.launch("gpu_softmax_row", (3,), (1,), [DB.from_array(s), dY, 91])
    assert np.max(np.abs(dY.to_array(np.float32).reshape(3, 91) - ref)) < 1e-6
    sq = rng.standard_normal((16, 16)).astype(np.float32); ref = np.zeros_like(sq); o.orc_softmax_causal_offset(sq, ref, 16, 16, 0)
    dY = DB(sq.nbytes); img.launch("gpu_softmax_causal", (16,), (1,), [DB.from_array(sq), dY, 16, 16])
    assert np.max(np.abs(dY.to_array(np.float32).reshape(16, 16) - ref)) < 1e-6
    so = rng.standard_normal((4, 24)).astype(np.float32); ref = np.zeros_like(so); o.orc_softmax_causal_offset(so, ref, 4, 24, 9)
    dY = DB(so.nbytes); img.launch("softmax_causal_offset", (4,), (1,), [DB.from_array(so), dY, 4, 24, 9])
    assert np.max(np.abs(dY.to_array(np.float32).reshape(4, 24) - ref)) < 1e-6


def test_llama_ops(img):
    # llama_ops_parity.sh: rmsnorm S x 576 (x*4), rope (S*9) x 64 theta=1e5, silu_mul (g*5); max-abs 1e-4
    o = ol.oracle()
    rng = np.random.default_rng(20260609)
    S = 7
    x = (rng.standard_normal((S, 576)) * 4).astype(np.float32); w = rng.standard_normal(576).astype(np.float32)
    ref = np.zeros_like(x); o.orc_rmsnorm(x, ref, w, S, 576, 1e-5)
    dY = DB(x.nbytes); img.launch("gpu_rmsnorm_fwd_eps", (S,), (1,), [DB.from_array(x), dY, DB.from_array(w), 576])
    assert np.max(np.abs(dY.to_array(np.float32).reshape(S, 576) - ref)) < 1e-4
    rows, half = S * 9, 32
    cosT = np.zeros((rows, half), np.float32); sinT = np.zeros((rows, half), np.float32)
    o.orc_rope_tables(cosT, sinT, rows, 64, 1e5)
    q = rng.standard_normal((rows, 64)).astype(np.float32); ref = q.copy(); o.orc_rope_rot(ref, cosT, sinT, rows, half)
    dQ = DB.from_array(q); img.launch("gpu_rope_rot", (rows,), (1,), [dQ, DB.from_array(cosT), DB.from_array(sinT), half])
    assert np.max(np.abs(dQ.to_array(np.float32).reshape(rows, 64) - ref)) < 1e-5
    n = 1536
    g = (rng.standard_normal(n) * 5).astype(np.float32); u = rng.standard_normal(n).astype(np.float32)
    ref = np.zeros(n, np.float32); o.orc_silu_mul(g, u, ref, n)
    dY = DB(n * 4); img.launch("gpu_silu_mul", (n,), (1,), [DB.from_array(g), DB.from_array(u), dY, n])
    assert np.max(np.abs(dY.to_array(np.float32) - ref)) < 1e-4
    gm = rng.standard_normal(576).astype(np.float32); bt = rng.standard_normal(576).astype(np.float32)
    ref = np.zeros_like(x); o.orc_layernorm(x, ref, gm, bt, S, 576, 1e-5)
    dY = DB(x.nbytes); img.launch("gpu_layernorm_fwd_eps", (S,), (1,), [DB.from_array(x), dY, DB.from_array(gm), DB.from_array(bt), 576])
    assert np.max(np.abs(dY.to_array(np.float32).reshape(S, 576) - ref)) < 1e-4
    ref = np.zeros(n, np.float32); o.orc_gelu(g, ref, n)
    dY = DB(n * 4); img.launch("gpu_gelu_stable", (n // 256,), (256,), [DB.from_array(g), dY, n])
    assert np.max(np.abs(dY.to_array(np.float32) - ref)) < 1e-5
    yb = rng.standard_normal(S * 576).astype(np.float32); dYb = DB.from_array(yb)
    img.launch("gpu_add_bias_rowbcast", ((S * 576 + 255) // 256,), (256,), [dYb, DB.from_array(bt), S * 576, 576])
    assert np.array_equal(dYb.to_array(np.float32), yb + np.tile(bt, S))
    a = rng.standard_normal(n).astype(np.float32); dC = DB(n * 4)
    img.launch("vector_add", (n // 256,), (256,), [DB.from_array(a), DB.from_array(g), dC, n])
    assert np.array_equal(dC.to_array(np.float32), a + g)
    dA = DB.from_array(a); img.launch("gpu_scale_rt", (n // 256,), (256,), [dA, DB.from_array(np.array([0.125], np.float32)), n])
    assert np.array_equal(dA.to_array(np.float32), a * np.float32(0.125))


def test_fused_decode_attn_and_matmuls(img):
    o = ol.oracle()
    rng = np.random.default_rng(4)
    NH, NKV, DH, T, cap, NLy = 8, 2, 64, 37, 48, 2
    q = rng.standard_normal(NH * DH).astype(np.float32)
    kc = rng.standard_normal(NLy * NKV * cap * DH).astype(np.float32); vc = rng.standard_normal(kc.size).astype(np.float32)
    scale = np.float32(1.0 / np.sqrt(np.float32(DH)))
    koff = 1 * NKV * cap * DH                       # layer 1
    ref = np.zeros(NH * DH, np.float32)
    o.orc_decode_attn_online(q, kc, vc, ref, scale, NH, T, DH, koff, NH // NKV, cap * DH)
    dO = DB(NH * DH * 4)
    img.launch("fused_decode_attn", (NH,), (DH,), [DB.from_array(q), DB.from_array(kc), DB.from_array(vc), dO,
                                                    DB.from_array(np.array([scale])), T, DH, koff, NH // NKV, cap * DH])
    assert np.max(np.abs(dO.to_array(np.float32) - ref)) < 1e-5
    M, K, N = 128, 72, 192
    a = rng.standard_normal((M, K)).astype(np.float32); b = rng.standard_normal((K, N)).astype(np.float32)
    bt = np.ascontiguousarray(b.T)
    dC = DB(M * N * 4); img.launch("tiled_matmul", (N // 64, M // 64), (16, 16), [DB.from_array(a), DB.from_array(b), dC, M, K, N])
    ref = a.astype(np.float64) @ b
    assert np.max(np.abs(dC.to_array(np.float32).reshape(M, N) - ref)) < 1e-4
    dC.zero(); img.launch("tiled_matmul_abt", (N // 64, M // 64), (16, 16), [DB.from_array(a), DB.from_array(bt), dC, M, K, N])
    assert np.max(np.abs(dC.to_array(np.float32).reshape(M, N) - ref)) < 1e-4
