"""GPU quantizer / dequantizer / layout converters against the CPU checker: bit-exact.
Runs through the C ABI (hx_quantize_nvfp4_host and the device-pointer calls)."""
import ctypes as C
import os

import numpy as np
import pytest

import helix_b200 as hb
from helix_b200.lib import check
import oracle_lib as ol

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def same(a, b):
    return np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1]) and np.float32(a[2]) == np.float32(b[3]) \
        and np.array_equal(a[3], b[2])


@pytest.mark.parametrize("rows,K,scale", [(5, 100, 0.043), (8, 112, 0.02), (1, 16, 1.0), (3, 7, 0.02), (17, 1030, 0.02),
                                          (33, 4097, 0.02), (64, 4096, 0.02), (2, 1792, 5.0), (2, 1793, 1e-3),
                                          (7, 3584, 0.02), (4, 12288, 0.02), (1, 25600, 0.02), (300, 768, 0.02)])
def test_quantizer_bit_exact(rows, K, scale):
    rng = np.random.default_rng(rows * 100003 + K)
    w = (scale * rng.standard_normal((rows, K))).astype(np.float32)
    assert same(ol.quantize(w), hb.quantize_host(w))


def test_quantizer_golden_from_reference():
    g = np.load(os.path.join(G, "quant_golden.npz"))
    for i in list(range(int(g["n"]))) + ["z"]:
        W, mic, sc, ts = hb.quantize_host(g[f"w{i}"])
        assert np.array_equal(W, g[f"W{i}"]) and np.array_equal(mic, g[f"mic{i}"]), i
        assert np.float32(ts) == g[f"ts{i}"] and np.array_equal(sc, g[f"sc{i}"]), i


def test_quantizer_edge_values():
    rng = np.random.default_rng(77)
    w = (0.02 * rng.standard_normal((6, 224))).astype(np.float32)
    w[0, :] = 0.0                                   # an all-zero row inside a non-zero tensor
    w[1, :16] = 0.0                                 # an all-zero block: eff == 0 -> codes 0
    w[2, 5] = 3.0                                   # an outlier that sets the tensor scale
    w[3, :8] = [1e-30, -1e-30, 1e-38, -1e-38, 1e-45, -1e-45, 0.0, -0.0]   # denormals
    assert same(ol.quantize(w), hb.quantize_host(w))
    # exact ties of the E2M1 thresholds and of E4M3 midpoints
    t = np.zeros((2, 32), np.float32)
    t[0, :16] = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    t[0, 16:] = t[0, :16] * 0.46875
    t[1, :] = np.linspace(-6, 6, 32)
    assert same(ol.quantize(t), hb.quantize_host(t))
    # all zero: ts guard gives 1.0, every code 0
    z = np.zeros((3, 48), np.float32)
    W, mic, sc, ts = hb.quantize_host(z)
    assert ts == 1.0 and not W.any() and not mic.any()
    # tiny amax: ts underflows to 0 in f32 and is replaced by 1.0, as in the reference
    tiny = np.full((1, 16), 1e-44, np.float32)
    assert same(ol.quantize(tiny), hb.quantize_host(tiny))
    big = (1e30 * rng.standard_normal((2, 64))).astype(np.float32)
    assert same(ol.quantize(big), hb.quantize_host(big))


def test_quantizer_nonfinite_inputs():
    rng = np.random.default_rng(78)
    w = (0.02 * rng.standard_normal((4, 64))).astype(np.float32)
    w[1, 3] = np.nan
    assert same(ol.quantize(w), hb.quantize_host(w))
    w[2, 9] = np.inf
    a, b = ol.quantize(w), hb.quantize_host(w)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_config1_full_size_bit_exact_and_roundtrip():
    """The single-matrix round trip: W 12288x4096 N(0,0.02) from a seed, x N(0,1); codes, scales and ts bit-exact,
    y = dequant(W) x within rel 1e-3 of the checker's ascending f32 GEMV (the reference's per-GEMV bar,
    cuda_launch.c:2088)."""
    rng = np.random.default_rng(1)
    w = (0.02 * rng.standard_normal((12288, 4096))).astype(np.float32)
    x = rng.standard_normal(4096).astype(np.float32)
    a = ol.quantize(w)
    b = hb.quantize_host(w)
    assert same(a, b)
    W, mic, ts, _ = a
    xp = np.zeros(W.shape[1] * 7, np.float32); xp[:4096] = x
    yref = np.zeros(12288, np.float32)
    ol.oracle().orc_gemv_packed(xp, W, mic, np.float32(ts), yref, 12288, W.shape[1] * 7)
    y = hb.roundtrip_host(w, x)
    rel = np.abs(y - yref) / np.maximum(np.abs(yref), 1e-6)
    assert np.max(np.abs(y - yref)) < 2e-5 and np.median(rel) < 1e-5
    # size-independent property: quantization is a projection -- dequant(quant(dequant(quant(W)))) is a fixed point
    deq = ol.dequant_micro(W[:64], mic[:64], ts)[:, :4096]
    W2, mic2, sc2, ts2 = hb.quantize_host(np.vstack([deq, w[np.argmax(np.abs(w).max(1))][None, :]]))
    assert np.array_equal(W2[:64], W[:64]) and np.array_equal(mic2[:64], mic[:64])


def test_device_pointer_calls_and_layouts():
    L = hb.lib()
    rng = np.random.default_rng(3)
    rows, K = 37, 1000
    w = (0.02 * rng.standard_normal((rows, K))).astype(np.float32)
    W, mic, ts, sc = ol.quantize(w)
    kp = W.shape[1] * 7
    dw = hb.DeviceBuffer.from_array(w)
    dW, dmic = hb.DeviceBuffer(W.nbytes), hb.DeviceBuffer(mic.nbytes)
    dsc, dts = hb.DeviceBuffer(sc.nbytes), hb.DeviceBuffer(4)
    check(L.hx_quantize_nvfp4(dw.ptr, rows, K, dW.ptr, dmic.ptr, dsc.ptr, dts.ptr, None))
    assert np.array_equal(dW.to_array(np.int32).reshape(W.shape), W)
    assert np.array_equal(dmic.to_array(np.uint8).reshape(mic.shape), mic)
    assert dts.to_array(np.float32)[0] == np.float32(ts)
    # dequant: bit-identical to v3_dequant_packed and to the collapsed-scale form
    dout = hb.DeviceBuffer(rows * kp * 4)
    check(L.hx_dequant_nvfp4(dW.ptr, dmic.ptr, dts.ptr, None, dout.ptr, rows, kp, None))
    ref = ol.dequant_micro(W, mic, ts)
    assert np.array_equal(dout.to_array(np.float32).reshape(rows, kp), ref)
    assert not ref[:, K:].any()
    check(L.hx_dequant_nvfp4(dW.ptr, None, None, dsc.ptr, dout.ptr, rows, kp, None))
    assert np.array_equal(dout.to_array(np.float32).reshape(rows, kp), ref)
    # micro re-layout
    mst = (kp // 16 + 3) // 4
    dm4 = hb.DeviceBuffer(rows * mst * 4)
    check(L.hx_pack_micro(dmic.ptr, rows, kp // 16, dm4.ptr, None))
    want = np.zeros((rows, mst), np.int32); ol.oracle().orc_pack_micro(mic, rows, kp // 16, want)
    assert np.array_equal(dm4.to_array(np.int32).reshape(rows, mst), want)
    # GEMV over the committed layout vs the checker in both summation orders
    x = np.zeros(kp, np.float32); x[:K] = rng.standard_normal(K)
    dx, dy = hb.DeviceBuffer.from_array(x), hb.DeviceBuffer(rows * 4)
    check(L.hx_gemv_nvfp4(dx.ptr, dW.ptr, dm4.ptr, dts.ptr, dy.ptr, rows, kp, None))
    y = dy.to_array(np.float32)
    y_warp = np.zeros(rows, np.float32); ol.oracle().orc_gemv_packed_warp_order(x, W, mic, np.float32(ts), y_warp, rows, kp)
    y_asc = np.zeros(rows, np.float32); ol.oracle().orc_gemv_packed(x, W, mic, np.float32(ts), y_asc, rows, kp)
    assert np.array_equal(y, y_warp)               # same lane order, same fma chain: bit-identical
    assert np.max(np.abs(y - y_asc) / np.maximum(np.abs(y_asc), 1e-6)) < 1e-3
    # dense decode layout carries the same codes and scales
    kd = L.hx_kd(K)
    dc, ds = hb.DeviceBuffer(rows * kd // 2), hb.DeviceBuffer(rows * kd // 16)
    check(L.hx_repack_d16(dW.ptr, dmic.ptr, rows, K, kp, dc.ptr, ds.ptr, None))
    codes = dc.to_array(np.uint8).reshape(rows, kd // 2)
    nib = np.stack([codes & 15, codes >> 4], -1).reshape(rows, kd)
    src = np.stack([(W >> (4 * j)) & 15 for j in range(7)], -1).reshape(rows, kp)
    assert np.array_equal(nib[:, :K], src[:, :K]) and not nib[:, K:].any()
    sc8 = ds.to_array(np.uint8).reshape(rows, kd // 16)
    nb = (K + 15) // 16
    assert np.array_equal(sc8[:, :nb], mic[:, :nb]) and not sc8[:, nb:].any()
    xd = np.zeros(kd, np.float32); xd[:K] = x[:K]
    dxd = hb.DeviceBuffer.from_array(xd)
    check(L.hx_gemv_d16(dxd.ptr, dc.ptr, ds.ptr, dts.ptr, dy.ptr, rows, kd, None))
    y2 = dy.to_array(np.float32)
    assert np.max(np.abs(y2 - y_asc) / np.maximum(np.abs(y_asc), 1e-6)) < 1e-3
    assert np.max(np.abs(y2 - y_asc)) < 1e-5
