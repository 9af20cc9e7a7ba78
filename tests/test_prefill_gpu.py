"""Batched prefill (chunks of 64 tokens = four groups of 16 through the tcgen05 GEMM in digit mode) against the fp32 CPU restatement
and against the token-by-token path of the same library."""
import os

import numpy as np
import pytest

import helix_b200 as hb
import oracle_lib as ol

pytestmark = pytest.mark.gpu
LOGIT_TOL = 2e-4


@pytest.mark.parametrize("which,T", [("tiny", 16), ("tiny", 37), ("ragged", 37), ("wide", 50), ("ragged", 5),
                                     ("tiny", 64), ("ragged", 70), ("wide", 150), ("tiny", 200), ("gqa4", 300)])
def test_batched_prefill_matches_checker_and_token_path(which, T, tiny_file, ragged_file, wide_file, gqa4_file):
    path = dict(tiny=tiny_file, ragged=ragged_file, wide=wide_file, gqa4=gqa4_file)[which]
    om = ol.OracleModel(path, kv_cap=T + 32)
    ids = np.random.default_rng(100 + T).integers(0, om.NV, T).astype(np.int32)
    lo = om.prefill(ids)
    want = om.generate(ids, 24)

    gm = hb.Model.load(path, kv_cap=T + 32)
    assert gm.engine().startswith("persistent-tcgen05")
    nx, lg = gm.prefill(ids, want_logits=True)
    assert np.max(np.abs(lo - lg)) < LOGIT_TOL
    assert nx == int(np.argmax(lo)) == int(want[0])
    cont, _ = gm.decode_loop(nx, T, 23)               # decode on top of the KV rows the batched prefill wrote
    assert np.array_equal(cont, want[1:])
    gm.close()

    os.environ["HX_PREFILL"] = "token"                # same library, prompt fed position by position
    try:
        tm = hb.Model.load(path, kv_cap=T + 32)
        nx2, lg2 = tm.prefill(ids, want_logits=True)
        tm.close()
    finally:
        del os.environ["HX_PREFILL"]
    assert nx2 == nx and np.max(np.abs(lg2 - lg)) < LOGIT_TOL
    om.close()


def test_prefill_throughput_reports(tiny_file):
    """generate() reports separate prefill and decode times; both paths leave the same tokens."""
    gm = hb.Model.load(tiny_file, kv_cap=128)
    ids = np.random.default_rng(3).integers(0, 300, 64).astype(np.int32)
    out, ms_p, ms_d = gm.generate(ids, 16)
    assert ms_p > 0 and ms_d > 0 and len(out) == 16
    gm.close()
