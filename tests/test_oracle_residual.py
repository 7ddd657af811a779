"""Residual blocks with ShakeDrop: the CPU restatement (oracle/fc_residual.py)
against the committed fixture of the compiled reference and, where oracle/_ref
is built, against the compiled reference on other shapes."""
import pytest

import configs
import fc_residual
import golden_io
import ref_binding
import util

TOL_L2 = 2e-6
# Updated weights: the Adam first step lr*g/(|g|+eps) magnifies rounding of
# gradients that are of the order of eps (parity).
TOL_PARAMS = 1e-4


def _check(got, want):
    for key, (l2, mx) in util.compare(got, want).items():
        tol = TOL_PARAMS if key.startswith("params") else TOL_L2
        assert l2 <= tol, f"{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"


@pytest.mark.parametrize("name", sorted(golden_io.NOISY_CASES))
def test_residual_restatement_matches_golden(name):
    cfg, steps, X, Y, draws, p0, want = golden_io.load_noisy(name)
    model = util.build(fc_residual.ResidualOracleModel(), cfg, params=p0)
    _check(util.trace_noisy(model, cfg, steps, X, Y, draws), want)


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("cfg", [configs.residual_mlp(32, 2, 10, 8, p_last=0.0),
                                 configs.residual_mlp(40, 4, 5, 24)], ids=lambda c: c["name"])
def test_residual_restatement_matches_compiled_reference(cfg):
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    p0 = ref.get_array("parameters")
    want = util.trace_noisy(ref, cfg, steps=5)
    got = util.trace_noisy(util.build(fc_residual.ResidualOracleModel(), cfg, params=p0), cfg, steps=5)
    _check(got, want)
