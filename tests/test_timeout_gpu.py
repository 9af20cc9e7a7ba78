"""A bounded device-side wait that runs out: the call returns HX_ERR_TIMEOUT, nothing faults or hangs, and the model
decodes correctly afterwards.

The failure is injected without touching the GPU's health: hx_model_debug_waits shortens the poll limit and makes the
decode kernel begin with a wait on a word that nothing ever writes.  The wait gives up, the kernel's roles leave
through their common exit (bulk copies drained, tensor memory freed), the host resets the launch counters."""
import numpy as np
import pytest

import helix_b200 as hb
import oracle_lib as ol

pytestmark = pytest.mark.gpu
HX_ERR_TIMEOUT = 8


@pytest.mark.parametrize("which", ["tiny", "wide"])
def test_wait_runs_out_then_the_model_recovers(which, tiny_file, wide_file):
    path = dict(tiny=tiny_file, wide=wide_file)[which]
    om = ol.OracleModel(path, kv_cap=32)
    gm = hb.Model.load(path, kv_cap=32)
    assert gm.engine() == "persistent-tcgen05-dataflow"
    ids = np.random.default_rng(3).integers(0, om.NV, 6)
    lo0 = om.decode(int(ids[0]), 0)
    nx, lg = gm.decode_step(int(ids[0]), 0, want_logits=True)
    assert np.max(np.abs(lg - lo0)) < 2e-4
    gm.debug_waits(wait_limit=20000, inject_stall=True)
    for _ in range(2):                                   # twice: the recovery itself leaves a clean state
        with pytest.raises(hb.HxError) as e:
            gm.decode_step(int(ids[1]), 1)
        assert e.value.code == HX_ERR_TIMEOUT
    gm.debug_waits()                                     # default limit, no injection
    for pos in range(1, 6):
        lo = om.decode(int(ids[pos]), pos)
        nx, lg = gm.decode_step(int(ids[pos]), pos, want_logits=True)
        assert np.max(np.abs(lg - lo)) < 2e-4, pos
        assert nx == int(np.argmax(lo))
    om.close(); gm.close()
