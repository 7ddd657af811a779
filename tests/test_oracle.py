"""The CPU restatement (oracle/fc_step.py) against the reference: the committed
golden fixtures the compiled reference produced, and, where oracle/_ref is
built, the compiled reference itself on larger seeded workloads."""
import numpy as np
import pytest

import configs
import fc_step
import golden_io
import ref_binding
import util
from enums import ACTIVATION, LAYER_DROPOUT, LAYER_NORM, OPTIMIZER

# L2-relative bound for every compared tensor.  The restatement differs from the
# reference only in summation order (blocked dot vs sequential loop).
TOL_L2 = 2e-6


@pytest.mark.parametrize("name", sorted(golden_io.CASES))
def test_oracle_matches_golden(name):
    cfg, steps, X, Y, masks, p0, want = golden_io.load(name)
    got = util.trace(util.build(fc_step.OracleModel(), cfg, params=p0), cfg, steps, X, Y, masks)
    for key, (l2, mx) in util.compare(got, want).items():
        assert l2 <= TOL_L2, f"{name}/{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("cfg", [
    configs.mlp_softmax(),
    configs.deep_brn_mlp(64, 128, 3, 32, 64),
    configs.deep_brn_mlp(64, 128, 3, 32, 64, af=ACTIVATION.ELU, optimizer=OPTIMIZER.ADABOUND),
    configs.deep_brn_mlp(64, 128, 3, 32, 64, af=ACTIVATION.ISRLU, optimizer=OPTIMIZER.NOSADAM,
                         dropout=LAYER_DROPOUT.BERNOULLI_INVERTED),
    configs.deep_brn_mlp(64, 128, 3, 32, 64, af=ACTIVATION.RELU, optimizer=OPTIMIZER.AMSGRAD, dropout=None),
], ids=lambda c: f"{c['name']}-opt{c['optimizer']}-af{c['layers'][1].get('af')}")
def test_oracle_matches_compiled_reference(cfg):
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    p0 = ref.get_array("parameters")
    want = util.trace(ref, cfg, steps=20)
    got = util.trace(util.build(fc_step.OracleModel(), cfg, params=p0), cfg, steps=20)
    for key, (l2, mx) in util.compare(got, want).items():
        assert l2 <= TOL_L2, f"{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("rule", [OPTIMIZER.ADAM, OPTIMIZER.AMSGRAD, OPTIMIZER.ADABOUND, OPTIMIZER.AMSBOUND,
                                  OPTIMIZER.NOSADAM])
def test_flat_optimizer_sweep(rule):
    """Optimizer-only workload: flat vector, p ~ N(0, 0.02), g ~ N(0, 1e-3),
    zero moments, 10 steps, against the reference's own update loops."""
    rng = np.random.default_rng(5)
    n = 100_003
    p = (0.02 * rng.standard_normal(n)).astype(np.float32)
    g = (1e-3 * rng.standard_normal(n)).astype(np.float32)
    hp = dict(adam_learning_rate=1e-3, adam_beta1=0.9, adam_beta2=0.999, adam_epsilon=1e-8, adam_gamma=0.1,
              learning_rate_final=0.1, learning_gamma=1e-3)
    pr, m, v, vh = p.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros(n, np.float32)
    secs = ref_binding.optimizer_sweep(rule, pr, g, m, v, vh, 10, [1e-3, 0.9, 0.999, 1e-8, 0.1, 0.1, 1e-3])
    assert secs >= 0
    po, mo, vo, vho = p.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros(n, np.float32)
    state = {}
    for _ in range(10):
        gg = g.copy()
        fc_step.optimizer_update(rule, fc_step.optimizer_scalars(rule, hp, state), po, gg, mo, vo, vho)
    assert util.rel_l2(po - p, pr - p) <= 1e-5
    assert util.rel_l2(mo, m) <= 1e-6 and util.rel_l2(vo, v) <= 1e-6


def test_softmax_cross_entropy_known_answer():
    """Closed form for one row: delta = (q - onehot) / rows when the softmax
    Jacobian is contracted with the cross-entropy derivative (the identity the
    reference's own gradient test exercises on a 3-weight network,
    test/deep-learning/array_grad_adept_test.cpp L:149-237)."""
    z = np.array([[0.4 + 0.5 * 1.3, 0.4 + 0.5 * -5.3, 0.4 + 0.5 * 4.3]], np.float32)
    q = fc_step.softmax(z)
    y = np.array([[0.0, 0.0, 1.0]], np.float32)
    total, delta = fc_step.loss_and_delta(fc_step.LOSS_CROSS_ENTROPY, fc_step.AF_SOFTMAX, z, q, y)
    np.testing.assert_allclose(delta, (q - y), rtol=2e-6, atol=1e-7)
    np.testing.assert_allclose(total, -np.log(q[0, 2]), rtol=1e-6)


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("optimizer", [1, 2, 4, 5, 9], ids=["adabound", "adam", "amsbound", "amsgrad", "nosadam"])
def test_weight_decay_matches_compiled_reference(optimizer):
    """Decoupled, normalised weight decay on the weights only
    (v1/optimizers/adam.cpp L:130-147, v1/learner/train.cpp L:278-283,
    v1/learner/indexing.cpp L:58-81)."""
    cfg = configs.deep_brn_mlp(20, 32, 2, 12, 24, optimizer=optimizer)
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    ref.set_weight_decay(0.01)
    p0 = ref.get_array("parameters")
    want = util.trace(ref, cfg, steps=4)
    ora = util.build(fc_step.OracleModel(), cfg, params=p0)
    ora.set_weight_decay(0.01)
    got = util.trace(ora, cfg, steps=4)
    for key, (l2, mx) in util.compare(got, want).items():
        assert l2 <= TOL_L2, f"{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"
    plain = util.trace(util.build(fc_step.OracleModel(), cfg, params=p0), cfg, steps=4)
    assert util.rel_l2(plain["params_last"], want["params_last"]) > 1e-4   # the decay is not a no-op
    # The un-normalised form, use_normalized_weight_decay = false.  training_size is
    # 4 batches here so that the two forms differ.
    raw = dict(cfg, hparams=dict(cfg["hparams"], use_normalized_weight_decay=0))
    out = []
    for model in (util.build(ref_binding.RefModel(), raw, params=p0), util.build(fc_step.OracleModel(), raw, params=p0),
                  util.build(fc_step.OracleModel(), cfg, params=p0)):
        model.set_weight_decay(0.01)
        B = cfg["batch"]
        X, Y = configs.synthetic_batch(cfg)
        model.train_begin(B)
        for li, mk in configs.dropout_masks(cfg).items():
            model.set_dropout_mask(li, mk)
        model.reset_loss()
        model.forward_pass(B, X); model.compute_error(B, Y); model.backward_pass(B)
        model.update_derivatives(B); model.merge_derivatives(); model.update_weights(B, 4 * B)
        out.append(model.get_array("parameters"))
    assert util.rel_l2(out[1], out[0]) <= TOL_L2
    assert util.rel_l2(out[2] - p0, out[0] - p0) > 1e-3


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("mp", [True, False], ids=["openmp", "serial"])
def test_plain_batch_normalization_matches_compiled_reference(mp):
    """LAYER_NORM::BATCH_NORMALIZATION (fwp_mp.cpp L:4493-4603, bwp_mp.cpp
    L:1265-1385): the renormalization path with r = 1 and d = 0, although the
    model's r and d maxima are set to other values."""
    cfg = configs.deep_brn_mlp(20, 32, 2, 12, 24)
    layers = [dict(l, norm=LAYER_NORM.BATCH_NORMALIZATION) if l.get("norm") else l for l in cfg["layers"]]
    cfg = dict(cfg, layers=layers, mp=mp)
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    p0 = ref.get_array("parameters")
    want = util.trace(ref, cfg, steps=4)
    got = util.trace(util.build(fc_step.OracleModel(), cfg, params=p0), cfg, steps=4)
    for key, (l2, mx) in util.compare(got, want).items():
        assert l2 <= TOL_L2, f"{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"
    brn_cfg = configs.deep_brn_mlp(20, 32, 2, 12, 24)
    renorm = util.trace(util.build(fc_step.OracleModel(), brn_cfg, params=p0), brn_cfg, steps=4)
    assert util.rel_l2(renorm["params_last"], want["params_last"]) > 1e-5   # not the same as renormalization


GD_FORMS = {"plain": dict(learning_momentum=0.0), "momentum": dict(learning_momentum=0.9),
            "nesterov": dict(learning_momentum=0.9, use_nesterov=1)}


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("form", sorted(GD_FORMS))
@pytest.mark.parametrize("decay", [0.0, 0.01], ids=["no_decay", "decay"])
def test_gradient_descent_matches_compiled_reference(form, decay):
    """The three forms of Model::Update_Parameter__Gradient_Descent
    (v1/optimizers/gradient_descent.cpp L:24-130, gradient_descent_momentum.cpp
    L:66-107, nesterov_accelerated_gradient.cpp L:66-109), with and without
    weight decay."""
    cfg = configs.deep_brn_mlp(20, 32, 2, 12, 24, optimizer=OPTIMIZER.GD)
    cfg = dict(cfg, hparams=dict(learning_rate=0.05, **GD_FORMS[form]))
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    ora = util.build(fc_step.OracleModel(), cfg, params=ref.get_array("parameters"))
    if decay:
        ref.set_weight_decay(decay)
        ora.set_weight_decay(decay)
    want = util.trace(ref, cfg, steps=4)
    got = util.trace(ora, cfg, steps=4)
    for key, (l2, mx) in util.compare(got, want).items():
        assert l2 <= TOL_L2, f"{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
def test_gradient_clipping_matches_compiled_reference():
    """Clipping by the Euclidean norm of the whole gradient vector between the
    merge and the optimizer (v1/ops/constraints/euclidean.cpp L:48-71,
    v1/learner/model.cpp L:4742-4743).  Adam-family steps barely depend on
    the gradient's scale, so the clipped gradient itself is compared as well:
    the factor is max / norm of the gradients of the unclipped first step."""
    cfg = configs.deep_brn_mlp(20, 32, 2, 12, 24)
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    p0 = ref.get_array("parameters")
    plain = util.trace(util.build(fc_step.OracleModel(), cfg, params=p0), cfg, steps=4)
    norm = float(np.sqrt(np.sum(plain["grads"].astype(np.float64) ** 2)))
    limit = norm / 50.0
    ref.set_clip_gradient(True, limit)
    want = util.trace(ref, cfg, steps=4)
    ora = util.build(fc_step.OracleModel(), cfg, params=p0)
    ora.set_clip_gradient(True, limit)
    got = util.trace(ora, cfg, steps=4)
    for key, (l2, mx) in util.compare(got, want).items():
        assert l2 <= TOL_L2, f"{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"
    assert util.rel_l2(plain["params_last"], want["params_last"]) > 1e-4   # the clipping is not a no-op
    # A norm above the gradient's leaves the step as it was.
    loose = util.build(fc_step.OracleModel(), cfg, params=p0)
    loose.set_clip_gradient(True, norm * 1e3)
    assert np.array_equal(util.trace(loose, cfg, steps=1)["params1"], plain["params1"])


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
def test_uout_matches_compiled_reference():
    """UOut, A += A * U(-beta, beta) per element (v1/learner/fwp_mp.cpp
    L:4959-4985): the restatement receives the draws the serial reference makes
    after its generator is reseeded, replayed through the reference's own
    Dist::Real."""
    cfg = dict(configs.deep_brn_mlp(20, 32, 2, 12, 24, dropout=LAYER_DROPOUT.UOUT, keep=0.3), mp=False)
    B = cfg["batch"]
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    ora = util.build(fc_step.OracleModel(), cfg, params=ref.get_array("parameters"))
    X, Y = configs.synthetic_batch(cfg)
    ref.train_begin(B)
    for step in range(4):
        ref.seed_uout(100 + step)
        noise = ref_binding.uout_draws(100 + step, [0.3, 0.3], B, [32, 32])
        ora.set_uout_noise(1, noise[0])
        ora.set_uout_noise(2, noise[1])
        assert abs(ref.train_step(B, X, Y) - ora.train_step(B, X, Y)) <= 1e-6
        assert util.rel_l2(ora.get_layer_outputs(2, B), ref.get_layer_outputs(2, B).reshape(B, -1)) <= TOL_L2
        assert util.rel_l2(ora.get_array("parameters"), ref.get_array("parameters")) <= TOL_L2


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("mp", [False, True], ids=["serial", "openmp"])
@pytest.mark.parametrize("case", ["brn_bernoulli_distance", "softmax_accuracy", "brn_inverted_distance"])
def test_evaluation_pass_matches_compiled_reference(case, mp):
    """Driver::evalt: forward pass in inference mode (running averages, dropout
    scaling), loss and accuracy without an error (drivers/driver.cpp L:60-105)."""
    cfg, fn = {
        "brn_bernoulli_distance": (configs.deep_brn_mlp(20, 32, 2, 12, 24), fc_step.ACCU_DISTANCE),
        "softmax_accuracy": (configs.mlp_softmax(36, 24, 10, 16), fc_step.ACCU_CROSS_ENTROPY),
        "brn_inverted_distance": (configs.deep_brn_mlp(20, 32, 2, 12, 24, dropout=LAYER_DROPOUT.BERNOULLI_INVERTED),
                                  fc_step.ACCU_DISTANCE),
    }[case]
    cfg = dict(cfg, mp=mp)
    B, last = cfg["batch"], len(cfg["layers"]) - 1
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    ora = util.build(fc_step.OracleModel(), cfg, params=ref.get_array("parameters"))
    X, Y = configs.synthetic_batch(cfg)
    Xe, Ye = configs.synthetic_batch(dict(cfg, data_seed=5))
    out = []
    for m in (ref, ora):
        m.train_begin(B)
        for li, mk in configs.dropout_masks(cfg).items():
            m.set_dropout_mask(li, mk)
        for _ in range(3):
            m.train_step(B, X, Y)   # move the running averages away from their start
        m.set_propagation(0)
        m.set_accu_fn(fn)
        m.reset_loss()
        m.forward_pass(B, Xe)
        m.compute_loss(B, Ye)
        out.append((m.get_loss(), m.get_accu(B), m.get_layer_outputs(last, B).reshape(B, -1)))
    (lr, ar, qr), (lo, ao, qo) = out
    assert abs(lr - lo) <= 1e-6 * abs(lr) and ar == ao
    assert util.rel_l2(qo, qr) <= TOL_L2


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("kind", [2, 3], ids=["bernoulli", "inverted"])
def test_input_layer_dropout_matches_compiled_reference(kind):
    """Dropout on the input layer acts on the batch as it is assigned
    (Model::assign_inputs_fwp_mp, v1/learner/assign_inputs.cpp L:94-130): masked
    in training, the plain kind scaled by its keep probability at inference."""
    cfg = configs.deep_brn_mlp(20, 32, 2, 12, 24)
    layers = [dict(l) for l in cfg["layers"]]
    layers[0]["dropout"] = (kind, 0.8)
    cfg = dict(cfg, layers=layers)
    masks = configs.dropout_masks(cfg)
    assert 0 in masks and not masks[0].all()
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    p0 = ref.get_array("parameters")
    want = util.trace(ref, cfg, 3, masks=masks)
    ora = util.build(fc_step.OracleModel(), cfg, params=p0)
    got = util.trace(ora, cfg, 3, masks=masks)
    for key, (l2, mx) in util.compare(got, want).items():
        # A running mean is a sum of values of both signs: its relative error is
        # that of the batch means times their cancellation.
        tol = 3 * TOL_L2 if key.startswith("mean_average") else TOL_L2
        assert l2 <= tol, f"{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"
    nomask = util.trace(util.build(fc_step.OracleModel(), cfg, params=p0), cfg, 1,
                        masks={k: v for k, v in masks.items() if k != 0})
    assert util.rel_l2(nomask["act1"], want["act1"]) > 1e-2   # the input mask is not a no-op
    # Inference from the trained state.
    B, last = cfg["batch"], len(cfg["layers"]) - 1
    Xe, Ye = configs.synthetic_batch(dict(cfg, data_seed=5))
    util.copy_trained_state(ref, ora, cfg)
    outs = []
    for m in (ref, ora):
        m.set_propagation(0)
        m.reset_loss()
        m.forward_pass(B, Xe)
        outs.append(m.get_layer_outputs(last, B).reshape(B, -1))
        m.set_propagation(1)
    assert util.rel_l2(outs[1], outs[0]) <= TOL_L2


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("mp", [True, False], ids=["openmp", "serial"])
def test_l2_regularization_has_no_effect_in_the_reference(mp):
    """Model::set_l2 stores its value, but the update's call of the L2 routine
    passes (batch_size, 0, total_weights) where the routine takes (start, end,
    batch_size) (v1/learner/model.cpp L:4717-4719, L:4804-4806; l2.cpp L:79-104):
    the loop covers no element.  A run with l2 = 0.1 equals a run without, bit
    for bit; the drop-in therefore keeps the value and leaves the gradient alone."""
    cfg = dict(configs.deep_brn_mlp(20, 32, 2, 12, 24), mp=mp)
    plain = util.build(ref_binding.RefModel(), cfg, seed=0)
    p0 = plain.get_array("parameters")
    want = util.trace(plain, cfg, steps=3)
    with_l2 = util.build(ref_binding.RefModel(), cfg, params=p0)
    with_l2.set_l2(0.1)
    got = util.trace(with_l2, cfg, steps=3)
    assert np.array_equal(got["params_last"], want["params_last"])
    assert np.array_equal(got["grads"], want["grads"])
    ora = util.build(fc_step.OracleModel(), cfg, params=p0)
    ora.set_l2(0.1)
    assert util.rel_l2(util.trace(ora, cfg, steps=3)["params_last"], want["params_last"]) <= TOL_L2
