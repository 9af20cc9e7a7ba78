"""hx_quantize_nvfp4_noalloc (scratch inside the library, no device allocation) against hx_quantize_nvfp4.

Kept in a file that sorts last so that it also runs after every other GPU test has used the device."""
import numpy as np
import pytest

import helix_b200 as hb
from helix_b200.lib import check
import oracle_lib as ol

pytestmark = pytest.mark.gpu


def _run(fn, w):
    rows, K = w.shape
    kp = hb.lib().hx_kpad(K)
    dw = hb.DeviceBuffer.from_array(w)
    dW, dmic = hb.DeviceBuffer(rows * (kp // 7) * 4), hb.DeviceBuffer(rows * (kp // 16))
    dsc, dts = hb.DeviceBuffer(rows * (kp // 16) * 4), hb.DeviceBuffer(4)
    check(fn(dw.ptr, rows, K, dW.ptr, dmic.ptr, dsc.ptr, dts.ptr, None))
    check(hb.lib().hx_sync())
    return dW.to_array(np.int32), dmic.to_array(np.uint8), dsc.to_array(np.float32), dts.to_array(np.float32)


@pytest.mark.parametrize("rows,K,seed", [(37, 1000, 1), (300, 4096, 2), (5000, 96, 3), (1, 2048, 4)])
def test_matches_allocating_entry_twice_in_a_row(rows, K, seed):
    L = hb.lib()
    rng = np.random.default_rng(seed)
    w = (0.05 * rng.standard_normal((rows, K))).astype(np.float32)
    w[rng.integers(0, rows), rng.integers(0, K)] = 3.5            # the tensor amax sits in one row
    want = _run(L.hx_quantize_nvfp4, w)
    for _ in range(2):                                              # the second call meets the first one's leftovers
        got = _run(L.hx_quantize_nvfp4_noalloc, w)
        for a, b in zip(got, want):
            assert np.array_equal(a.view(np.uint8), b.view(np.uint8))


def test_matches_the_cpu_checker_directly():
    """Independent of the allocating entry: codes, scale bytes and tensor scale against the CPU restatement."""
    rng = np.random.default_rng(12)
    w = (0.02 * rng.standard_normal((129, 1000))).astype(np.float32)
    W, mic, ts, sc = ol.quantize(w)
    gW, gmic, gsc, gts = _run(hb.lib().hx_quantize_nvfp4_noalloc, w)
    assert np.array_equal(gW, W.ravel()) and np.array_equal(gmic, mic.ravel())
    assert np.array_equal(gsc.view(np.uint32), sc.ravel().view(np.uint32)) and np.float32(gts[0]) == np.float32(ts)


def test_leftovers_of_a_larger_call_are_not_read():
    L = hb.lib()
    rng = np.random.default_rng(9)
    big = (10.0 * rng.standard_normal((4096, 128))).astype(np.float32)
    small = (0.01 * rng.standard_normal((16, 128))).astype(np.float32)
    _run(L.hx_quantize_nvfp4_noalloc, big)                          # leaves large row maxima behind
    got = _run(L.hx_quantize_nvfp4_noalloc, small)
    want = _run(L.hx_quantize_nvfp4, small)
    for a, b in zip(got, want):
        assert np.array_equal(a.view(np.uint8), b.view(np.uint8))


def test_all_zero_tensor_and_size_limit():
    L = hb.lib()
    z = np.zeros((8, 112), np.float32)
    got, want = _run(L.hx_quantize_nvfp4_noalloc, z), _run(L.hx_quantize_nvfp4, z)
    for a, b in zip(got, want):
        assert np.array_equal(a.view(np.uint8), b.view(np.uint8))
    assert got[3][0] == np.float32(1.0)
    too_many = L.hx_noalloc_max_rows() + 1
    d = hb.DeviceBuffer(64)
    rc = L.hx_quantize_nvfp4_noalloc(d.ptr, too_many, 16, d.ptr, d.ptr, d.ptr, d.ptr, None)   # refused before any launch
    assert rc == 1                                                  # HX_ERR_ARG
    assert b"exceed" in L.hx_last_error()
