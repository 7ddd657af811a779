"""IndRNN stacks: the CPU restatement (oracle/fc_indrnn.py) against the committed
fixtures of the compiled reference and, where oracle/_ref is built, against the
compiled reference on other shapes, sequence lengths and thread modes."""
import numpy as np
import pytest

import configs
import fc_indrnn
import golden_io
import ref_binding
import util
from enums import ACTIVATION, OPTIMIZER

TOL_L2 = 5e-6  # fp32 rounding carried through T steps of the recurrence and its reverse walk
# Updated weights: the first Adam-family step lr*g/(|g|+eps) magnifies rounding
# of gradients that are of the order of eps.
TOL_PARAMS = 1e-4


def _check(got, want):
    for key, (l2, mx) in util.compare(got, want).items():
        tol = TOL_PARAMS if key.startswith("params") else TOL_L2
        assert l2 <= tol, f"{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"


@pytest.mark.parametrize("name", sorted(golden_io.RECURRENT_CASES))
def test_indrnn_restatement_matches_golden(name):
    cfg, steps, X, Y, masks, p0, want = golden_io.load(name)
    got = util.trace(util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0), cfg, steps, X, Y, masks)
    _check(got, want)


def _cases():
    rnn = configs.indrnn_stack
    mid = rnn(n_in=7, hidden=12, depth=3, n_out=4, seq_w=9, batch=6, af=ACTIVATION.SELU, optimizer=OPTIMIZER.AMSGRAD)
    mid["time_delays"] = 4  # an error on the last five steps
    return [rnn(n_in=6, hidden=8, depth=1, n_out=3, seq_w=2, batch=5),
            rnn(n_in=12, hidden=20, depth=2, n_out=8, seq_w=24, batch=10, af=ACTIVATION.ELU),
            rnn(n_in=5, hidden=10, depth=2, n_out=5, seq_w=16, batch=4, norm=False, optimizer=OPTIMIZER.NOSADAM),
            mid]


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("mp", [False, True], ids=["serial", "openmp"])
@pytest.mark.parametrize("cfg", _cases(), ids=lambda c: f"{c['name']}_d{c['time_delays']}")
def test_indrnn_restatement_matches_compiled_reference(cfg, mp):
    cfg = dict(cfg, mp=mp)
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    configs.set_recurrent_uniform(ref, cfg)
    p0 = ref.get_array("parameters")
    want = util.trace(ref, cfg, steps=5)
    got = util.trace(util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0), cfg, steps=5)
    _check(got, want)


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
def test_recurrent_weights_are_clamped_like_the_reference():
    """Recurrent weights outside +-2^(1/T) come back inside after one update
    (v1/ops/constraints/constraint.cpp L:245-289)."""
    cfg = configs.indrnn_stack(n_in=6, hidden=8, depth=2, n_out=5, seq_w=4, batch=5)
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    p0 = ref.get_array("parameters")
    for _, s in configs.recurrent_slices(cfg):
        p0[s] = np.linspace(-1.5, 1.5, s.stop - s.start, dtype=np.float32)
    ref.set_array("parameters", p0)
    want = util.trace(ref, cfg, steps=2)
    got = util.trace(util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0), cfg, steps=2)
    bound = np.float32(2.0) ** np.float32(0.25)
    for _, s in configs.recurrent_slices(cfg):
        assert np.abs(want["params1"][s]).max() <= bound * (1 + 1e-6)
        assert np.isclose(np.abs(got["params1"][s]).max(), bound, rtol=1e-6)
    _check(got, want)


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
def test_clip_gradient_widens_the_recurrent_bound_like_the_reference():
    """The default bound is clip(clip_gradient, 2, 10)^(1/T)
    (v1/ops/constraints/constraint.cpp L:64-95); setting the norm re-derives it
    (v1/ops/constraints/clip_gradient.cpp L:34-73), also while clipping is off."""
    cfg = configs.indrnn_stack(n_in=6, hidden=8, depth=2, n_out=5, seq_w=4, batch=5)
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    ref.set_clip_gradient(False, 5.0)
    p0 = ref.get_array("parameters")
    for _, s in configs.recurrent_slices(cfg):
        p0[s] = np.linspace(-2.5, 2.5, s.stop - s.start, dtype=np.float32)
    ref.set_array("parameters", p0)
    want = util.trace(ref, cfg, steps=2)
    ora = util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0)
    ora.set_clip_gradient(False, 5.0)
    got = util.trace(ora, cfg, steps=2)
    bound = np.float32(5.0) ** np.float32(0.25)
    for _, s in configs.recurrent_slices(cfg):
        assert np.isclose(np.abs(want["params1"][s]).max(), bound, rtol=1e-6)
        assert np.isclose(np.abs(got["params1"][s]).max(), bound, rtol=1e-6)
    _check(got, want)


def test_parameter_layout():
    """An IndRNN layer's u follows its W; gamma starts at 0.1 for IndRNN layers."""
    cfg = configs.indrnn_stack(n_in=6, hidden=8, depth=2, n_out=5, seq_w=4, batch=3)
    m = util.build(fc_indrnn.IndRnnOracleModel(), cfg)
    assert m.size("total_weights") == 6 * 8 + 8 + 8 * 8 + 8 + 8 * 5
    assert m.size("total_bias") == 8 + 8 + 5
    assert m.size("total_normalized_units") == 6 + 8 + 8 + 5
    assert [(i, s.start, s.stop) for i, s in configs.recurrent_slices(cfg)] == [(1, 48, 56), (2, 120, 128)]
    g0 = m.size("total_weights") + m.size("total_bias")
    gamma = m.get_array("parameters")[g0:g0 + 27]
    assert np.allclose(gamma[:6], 1) and np.allclose(gamma[6:22], 0.1) and np.allclose(gamma[22:], 1)
