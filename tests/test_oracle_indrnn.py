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
def test_uout_in_a_time_stepped_model_like_the_reference():
    """UOut on IndRNN layers against the compiled reference, which draws its
    noise itself: layer by layer, inside a layer time step by time step, row by
    row (the serial order), replayed from the same seed."""
    from enums import LAYER_DROPOUT
    T, B, H = 4, 5, 8
    cfg = dict(configs.indrnn_stack(n_in=6, hidden=H, depth=2, n_out=5, seq_w=T, batch=B,
                                    dropout=(LAYER_DROPOUT.UOUT, 0.3)), mp=False)
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    configs.set_recurrent_uniform(ref, cfg)
    p0 = ref.get_array("parameters")
    ora = util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0)
    X, Y = configs.synthetic_batch(cfg)
    for step in range(3):
        ref.seed_uout(100 + step)
        noise = ref_binding.uout_draws(100 + step, [0.3, 0.3], T * B, [H, H])
        ora.set_uout_noise(1, noise[0])
        ora.set_uout_noise(2, noise[1])
        want = util.trace(ref, cfg, 1, X, Y)
        got = util.trace(ora, cfg, 1, X, Y)
        _check(got, want)


def _softmax_case(delay):
    cfg = configs.indrnn_stack(n_in=6, hidden=10, depth=2, n_out=5, seq_w=4, batch=7, optimizer=OPTIMIZER.ADAM)
    cfg["layers"][-1]["af"] = ACTIVATION.SOFTMAX
    from enums import LOSS_FN
    return dict(cfg, loss=LOSS_FN.CROSS_ENTROPY, targets="onehot", time_delays=delay)


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("delay", [0, 2], ids=["all_steps", "last_two"])
def test_softmax_output_reads_the_target_of_time_step_0_like_the_reference(delay):
    """With a softmax output the reference takes the error of every time step
    against the target of time step 0 (v1/learner/compute_error_mp.cpp
    L:237-247) while its loss reads the step's own target."""
    cfg = _softmax_case(delay)
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    configs.set_recurrent_uniform(ref, cfg)
    p0 = ref.get_array("parameters")
    want = util.trace(ref, cfg, steps=3)
    got = util.trace(util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0), cfg, steps=3)
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
def test_recurrent_bounds_set_by_hand_like_the_reference():
    """Bounds set per layer (Set__Regularization__Constraint_Recurrent_Weight,
    v1/ops/constraints/constraint.cpp L:143-243): one layer with its own interval,
    one with the clamp taken off (0 / 0)."""
    cfg = configs.indrnn_stack(n_in=6, hidden=8, depth=2, n_out=5, seq_w=4, batch=5)
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    p0 = ref.get_array("parameters")
    for _, s in configs.recurrent_slices(cfg):
        p0[s] = np.linspace(-1.5, 1.5, s.stop - s.start, dtype=np.float32)
    ref.set_array("parameters", p0)
    ref.set_constraint_recurrent_weight(1, -0.5, 0.75)
    ref.set_constraint_recurrent_weight(2, 0.0, 0.0)
    want = util.trace(ref, cfg, steps=2)
    ora = util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0)
    ora.set_constraint_recurrent_weight(1, -0.5, 0.75)
    ora.set_constraint_recurrent_weight(2, 0.0, 0.0)
    got = util.trace(ora, cfg, steps=2)
    (_, s1), (_, s2) = configs.recurrent_slices(cfg)
    for t in (want, got):
        assert t["params1"][s1].min() == np.float32(-0.5) and t["params1"][s1].max() == np.float32(0.75)
        assert np.abs(t["params1"][s2]).max() > 1.4  # not clamped
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


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("kind", [2, 3], ids=["plain", "inverted"])
@pytest.mark.parametrize("norm", [True, False], ids=["brn", "no_norm"])
def test_bernoulli_dropout_through_time_matches_compiled_reference(kind, norm):
    """Bernoulli dropout in a time-stepped model: flags mask[t * units + u] on
    the stored output of step t, which the recurrence of step t + 1 reads
    (fwp_mp.cpp L:1228-1262, L:4842-4868); nothing in the backward pass."""
    cfg = configs.indrnn_stack(n_in=6, hidden=8, depth=2, n_out=5, seq_w=4, batch=5, norm=norm, dropout=(kind, 0.7))
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    p0 = ref.get_array("parameters")
    want = util.trace(ref, cfg, steps=3)
    got = util.trace(util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0), cfg, steps=3)
    _check(got, want)
    # Inference: the plain form scales by the keep probability, the inverted form does nothing.
    ora = util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0)
    util.copy_trained_state(ref, ora, cfg)
    X, _ = configs.synthetic_batch(dict(cfg, data_seed=5))
    out = []
    for m in (ref, ora):
        m.train_begin(5)
        m.set_propagation(0)
        m.forward_pass(5, X)
        out.append(m.get_layer_outputs(3, 5).reshape(-1))
    assert util.rel_l2(out[1], out[0]) <= TOL_L2


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("kind", [2, 3], ids=["plain", "inverted"])
def test_dropout_on_the_inputs_through_time_matches_compiled_reference(kind):
    """Dropout on the input layer of a time-stepped model: the batch's copy is
    masked per time step and unit as it is assigned (assign_inputs_rec_mp,
    v1/learner/assign_inputs.cpp L:219-266); at inference the plain form scales
    by the keep probability."""
    cfg = configs.indrnn_stack(n_in=6, hidden=8, depth=2, n_out=5, seq_w=4, batch=5)
    cfg["layers"][0] = dict(cfg["layers"][0], dropout=(kind, 0.6))
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    p0 = ref.get_array("parameters")
    want = util.trace(ref, cfg, steps=3)
    got = util.trace(util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0), cfg, steps=3)
    _check(got, want)
    ora = util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0)
    util.copy_trained_state(ref, ora, cfg)
    X, _ = configs.synthetic_batch(dict(cfg, data_seed=5))
    out = []
    for m in (ref, ora):
        m.train_begin(5)
        m.set_propagation(0)
        m.forward_pass(5, X)
        out.append(m.get_layer_outputs(3, 5).reshape(-1))
    assert util.rel_l2(out[1], out[0]) <= TOL_L2


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


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("delay", [3, 0], ids=["last_step", "all_steps"])
def test_indrnn_evaluation_pass_matches_compiled_reference(delay):
    """Inference through time: every time step normalised by its own running
    averages, loss and accuracy over the steps t >= n_time_delay
    (compute_loss_rec_mp, v1/learner/compute_loss_mp.cpp L:115-205)."""
    cfg = configs.indrnn_stack(n_in=6, hidden=8, depth=2, n_out=5, seq_w=4, batch=5)
    cfg = dict(cfg, time_delays=delay)
    B, last = cfg["batch"], len(cfg["layers"]) - 1
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    ora = util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=ref.get_array("parameters"))
    Xe, Ye = configs.synthetic_batch(dict(cfg, data_seed=5))
    out = []
    util.trace(ref, cfg, steps=3)   # move the running averages away from their start
    util.copy_trained_state(ref, ora, cfg)
    for m in (ref, ora):
        m.set_propagation(0)
        m.set_accu_fn(3)   # DISTANCE
        m.set_accu_var(0.6)
        m.reset_loss()
        m.forward_pass(B, Xe)
        m.compute_loss(B, Ye)
        out.append((m.get_loss(), m.get_accu(B), m.get_layer_outputs(last, B).reshape(-1)))
    (lr, ar, qr), (lo, ao, qo) = out
    assert abs(lr - lo) <= 1e-5 * abs(lr) and ar == ao
    assert util.rel_l2(qo, qr) <= 5e-6
