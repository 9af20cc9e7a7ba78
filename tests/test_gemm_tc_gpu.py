"""hx_gemm_nvfp4_tc (tcgen05 block-scaled NVFP4 GEMM) against a float64 evaluation of the same codes.

Every product of two E2M1 values and two E4M3 scales is exact in f32 and the sums stay far below 2^24 ulps of
their terms for these sizes, so the comparison is to f32 rounding of the exact result."""
import numpy as np
import pytest

import helix_b200 as hb
from helix_b200.lib import check

pytestmark = pytest.mark.gpu

E2 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float64)


def e4m3(c):
    c = np.asarray(c); e = (c >> 3) & 15; m = c & 7
    return np.where(e == 0, (m / 8.0) * 2.0 ** -6, (1 + m / 8.0) * 2.0 ** (e.astype(np.float64) - 7))


def swizzle(by):
    """by [..., rows, 8 chunks, 16 B] -> chunk j stored at position j ^ (row & 7)."""
    out = np.empty_like(by)
    r = np.arange(by.shape[-3])
    for j in range(8):
        out[..., r, j ^ (r & 7), :] = by[..., r, j, :]
    return out


def scale_chunks(sp):
    """sp [128, K/16] scale bytes -> one 512-byte chunk per 64 columns: byte (row%32)*16 + (row/32)*4 + block."""
    return sp.reshape(4, 32, -1, 4).transpose(2, 1, 0, 3).reshape(-1, 512)


def pack_a(codes, sc):
    rows, K = codes.shape; nt = (rows + 127) // 128; kg = K // 256
    cp = np.zeros((nt * 128, K), np.uint8); cp[:rows] = codes
    sp = np.zeros((nt * 128, K // 16), np.uint8); sp[:rows] = sc
    by = (cp[:, 0::2] | (cp[:, 1::2] << 4)).reshape(nt, 128, kg, 8, 16).transpose(0, 2, 1, 3, 4)
    out = np.zeros((nt, kg, 18432), np.uint8)
    out[:, :, :16384] = swizzle(by).reshape(nt, kg, 16384)
    for t in range(nt):
        out[t, :, 16384:] = scale_chunks(sp[t * 128:(t + 1) * 128]).reshape(kg, 2048)
    return out


def pack_b(codes, sc):
    n, K = codes.shape; kg = K // 256
    by = (codes[:, 0::2] | (codes[:, 1::2] << 4)).reshape(n, kg, 8, 16).transpose(1, 0, 2, 3)
    out = np.zeros((kg, n * 128 + 2048), np.uint8)
    out[:, :n * 128] = swizzle(by).reshape(kg, n * 128)
    sp = np.zeros((128, K // 16), np.uint8); sp[:n] = sc
    out[:, n * 128:] = scale_chunks(sp).reshape(kg, 2048)
    return out


@pytest.mark.parametrize("rows,K,n,stage,seed", [(128, 256, 8, 4, 0), (128, 512, 8, 4, 1), (256, 1024, 16, 8, 2),
                                                   (300, 4096, 16, 8, 3), (128, 512, 128, 4, 4), (1000, 2048, 64, 4, 5)])
def test_gemm_matches_float64(rows, K, n, stage, seed):
    L = hb.lib()
    rng = np.random.default_rng(seed)
    ac = rng.integers(0, 16, (rows, K)).astype(np.uint8); asc = rng.integers(0x28, 0x48, (rows, K // 16)).astype(np.uint8)
    bc = rng.integers(0, 16, (n, K)).astype(np.uint8); bsc = rng.integers(0x30, 0x40, (n, K // 16)).astype(np.uint8)
    A = E2[ac] * np.repeat(e4m3(asc), 16, axis=1); B = E2[bc] * np.repeat(e4m3(bsc), 16, axis=1)
    ref = A @ B.T
    da, db = hb.DeviceBuffer.from_array(pack_a(ac, asc)), hb.DeviceBuffer.from_array(pack_b(bc, bsc))
    dy = hb.DeviceBuffer(((rows + 127) // 128) * 128 * n * 4).zero()
    check(L.hx_gemm_nvfp4_tc(da.ptr, rows, K, db.ptr, n, dy.ptr, stage, None))
    y = dy.to_array(np.float32)[:rows * n].reshape(rows, n)
    # f32 accumulation of exact products: a few ulps of the largest partial sum
    tol = 4 * np.finfo(np.float32).eps * np.abs(A) @ np.abs(B).T
    assert np.all(np.abs(y - ref) <= tol + 1e-30)


def test_gemm_argument_checks():
    L = hb.lib()
    d = hb.DeviceBuffer(1 << 16)
    assert L.hx_gemm_nvfp4_tc(d.ptr, 128, 200, d.ptr, 8, d.ptr, 4, None) == 1      # K not a multiple of 256
    assert L.hx_gemm_nvfp4_tc(d.ptr, 128, 256, d.ptr, 12, d.ptr, 4, None) == 1     # ncols not a multiple of 8
