"""The tensor-pipe probe (hx_probe_mxf4_rate): the block-scaled FP4 MMA issues at a rate that does not depend on N,
which is what makes the N = 16 decode formulation stream at about the HBM rate and no faster."""
import pytest

import helix_b200 as hb

pytestmark = pytest.mark.gpu


def test_mma_issue_rate_is_flat_in_n():
    c16, t16 = hb.probe_mxf4_rate(16)
    c256, t256 = hb.probe_mxf4_rate(256)
    c16s, _ = hb.probe_mxf4_rate(16, True)
    print(f"M128 x N x K64 mxf4nvf4: N=16 {c16:.0f} clk, N=256 {c256:.0f} clk ({t256:.0f} TFLOP/s over all SMs), N=16 with scale copies {c16s:.0f} clk")
    assert 64 < c16 < 600 and 64 < c256 < 600
    assert c256 < 2.0 * c16                      # sixteen times the columns for (about) the same cycles
    assert c16s >= c16 * 0.95                    # the scale copies are not free
    assert t256 > 16 * t16 * 0.5
    with pytest.raises(hb.HxError):
        hb.probe_mxf4_rate(20)
