"""The numpy mixer checker against vectors recorded from the upstream
``causallsso.model.SolveDelta`` module in FP64 (tests/golden/make_mixer_golden.py).

Tolerance 5e-6 relative: the upstream CPU branch rounds gate pre-activations
to FP32 (causallsso/model.py:383-394,433-438); everything else is FP64."""
import numpy as np
import pytest

from tests.helpers import max_rel
from tests.mixer_helpers import load_mixer_golden, oracle_from_golden

CASES = ["mixer_small", "mixer_small_state", "mixer_noconv_bias", "mixer_masks_state"]
TOL = 5e-6


@pytest.mark.parametrize("name", CASES)
def test_mixer_oracle_matches_upstream(name):
    g = load_mixer_golden(name)
    orc = oracle_from_golden(g)
    stateful = "in_C0" in g
    out, fin, conv_T = orc.forward(
        g["in_x"], conv_state=g.get("in_conv0"),
        operator_state=(g["in_C0"], g["in_S0"]) if stateful else None,
        valid_mask=g.get("valid_mask"), reset_mask=g.get("reset_mask"))
    assert max_rel(out, g["out"]) < TOL
    if stateful:
        assert max_rel(fin[0], g["C_T"]) < TOL
        assert max_rel(fin[1], g["S_T"]) < TOL
        assert max_rel(conv_T, g["conv_T"]) < TOL
    dx, pg, dconv0, (dC0, dS0) = orc.backward(g["dout"], dC_T=g.get("dC_T"), dS_T=g.get("dS_T"),
                                               dconv_T=g.get("dconv_T"))
    assert max_rel(dx, g["grad_x"]) < TOL
    if stateful:
        assert max_rel(dC0, g["grad_C0"]) < TOL
        assert max_rel(dS0, g["grad_S0"]) < TOL
        assert max_rel(dconv0, g["grad_conv0"]) < TOL
    names = [k[len("pgrad_"):] for k in g if k.startswith("pgrad_")]
    assert names
    for pname in names:
        assert pname in pg, pname
        assert max_rel(pg[pname], g["pgrad_" + pname]) < TOL, pname
