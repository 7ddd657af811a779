"""Whole-step parity on the GPU through the Model entry points of the C ABI
(forward_pass, compute_error, backward_pass, update_derivatives,
update_weights): against the committed golden fixtures of the reference, the
CPU restatement, and, where it has been built, the compiled reference."""
import numpy as np
import pytest

import configs
import dlb200
import fc_step
import golden_io
import ref_binding
import util
from enums import ACTIVATION, LAYER_DROPOUT, LAYER_NORM, OPTIMIZER

pytestmark = pytest.mark.gpu

# rel-err (L2) bars of the drop-in: activations, errors, gradients and updated
# weights after one step; parameters after many steps.  The many-step bar is
# widened to the reference's own serial-vs-threaded drift where that is larger.
TOL_1 = 1e-5
TOL_N = 1e-4
# Element-wise worst case of the updated weights: an Adam-family first step is
# lr * g / (|g| + eps), so weights whose gradient is of the order of eps move by
# an amount that any change of summation order shifts.  The reference differs
# from itself (one thread vs many) by this much.
TOL_1_MAX = 2e-4


def gpu_model(ctx, cfg, params):
    return util.build(dlb200.Model(ctx), cfg, params=params)


@pytest.mark.parametrize("name", sorted(golden_io.CASES))
def test_model_matches_golden(gpu_ctx, name):
    cfg, steps, X, Y, masks, p0, want = golden_io.load(name)
    got = util.trace(gpu_model(gpu_ctx, cfg, p0), cfg, steps, X, Y, masks)
    assert gpu_ctx.sync() == 0
    for key, (l2, mx) in util.compare(got, want).items():
        assert l2 <= TOL_1, f"{name}/{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"


CASES = [
    configs.mlp_softmax(),                                   # 784-256-10, batch 128
    configs.deep_brn_mlp(256, 512, 2, 256, 256),             # reduced deep MLP, tensor-core tiles
    configs.deep_brn_mlp(96, 160, 2, 40, 200, af=ACTIVATION.ELU, optimizer=OPTIMIZER.ADABOUND,
                         dropout=LAYER_DROPOUT.BERNOULLI_INVERTED),
    configs.deep_brn_mlp(130, 70, 3, 9, 33, af=ACTIVATION.ISRLU, optimizer=OPTIMIZER.NOSADAM),   # ragged
]


# (Inverted dropout is left to the entry-point test: the reference's ISRLU
# derivative (q / x)^3 on the scaled activation q jumps from 1 / keep^3 to 1 at 0.)
@pytest.mark.parametrize("dropout", [LAYER_DROPOUT.BERNOULLI, None], ids=["bernoulli", "no_dropout"])
def test_layers_without_normalization_use_the_product_epilogues(gpu_ctx, dropout):
    """A stack without normalization at tensor-core sizes: from the second step
    on bias, activation, dropout and the planes of A come out of the forward
    product's epilogue and the activation derivative out of the input-gradient
    product's (fewer launches than the first step, whose plane buffers have no
    scale to predict from); every step agrees with the restatement."""
    # ISRLU: a continuous derivative, so that no pre-activation of the 786 432 can
    # sit on a jump where two correct sums take different branches.
    cfg = configs.deep_brn_mlp(256, 512, 3, 256, 512, af=ACTIVATION.ISRLU, optimizer=OPTIMIZER.ADAM,
                               dropout=dropout, norm=False)
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    ora = util.build(fc_step.OracleModel(), cfg)
    p0, seed = ora.get_array("parameters"), 0
    nw = ora.size("total_weights")
    p0[:nw] = (np.random.default_rng(0).standard_normal(nw) / np.sqrt(512)).astype(np.float32)
    want = util.trace(util.build(fc_step.OracleModel(), cfg, params=p0), cfg, 1, X, Y, masks)
    # The same first step after a step that primed the plane buffers: the
    # parameters are put back, so the traced step runs the epilogues.
    model = gpu_model(gpu_ctx, cfg, p0)
    for li, mk in masks.items():
        model.set_dropout_mask(li, mk)
    B = cfg["batch"]
    counts = []
    for _ in range(2):
        before = gpu_ctx.launch_count()
        model.train_step(B, X, Y)
        counts.append(gpu_ctx.launch_count() - before)
    assert counts[1] < counts[0], f"launches per step {counts}: the second step did not fuse"
    for name in ("first_moment", "second_moment", "second_moment_hat"):
        model.set_array(name, np.zeros_like(p0))
    model.set_hparam("optimizer_time_step", 0.0)
    model.set_array("parameters", p0)
    got = util.trace(model, cfg, 1, X, Y, masks)
    assert gpu_ctx.sync() == 0
    for key, (l2, mx) in util.compare(got, want).items():
        assert l2 <= TOL_1, f"{key} (weight seed {seed}): rel_l2 {l2:.2e} (rel_max {mx:.2e})"


@pytest.mark.parametrize("cfg", CASES, ids=lambda c: c["name"])
def test_model_one_step_vs_restatement(gpu_ctx, cfg):
    """Activations, errors, gradients, running statistics and updated weights
    after one step.  The weights are drawn from the first seed for
    which no hidden pre-activation sits on a jump of the activation's
    derivative: there the branch x < 0 is decided by the last bits of a long
    sum and two correct implementations may differ (see util.near_kink)."""
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    p0, seed = util.kink_free_parameters(cfg, fc_step.OracleModel, X, masks,
                                         scale=1.0 / np.sqrt(cfg["layers"][1]["units"]))
    want = util.trace(util.build(fc_step.OracleModel(), cfg, params=p0), cfg, 1, X, Y, masks)
    got = util.trace(gpu_model(gpu_ctx, cfg, p0), cfg, 1, X, Y, masks)
    assert gpu_ctx.sync() == 0
    for key, (l2, mx) in util.compare(got, want).items():
        assert l2 <= TOL_1, f"{key} (weight seed {seed}): rel_l2 {l2:.2e} (rel_max {mx:.2e})"
    # Two more steps: a pre-activation may now meet a jump (the serial and the
    # threaded reference then part by up to 4e-4 on the running means of this
    # workload), so only the scale of the agreement is checked here; the
    # 100-step test below measures it against the reference's own drift.
    want3 = util.trace(util.build(fc_step.OracleModel(), cfg, params=p0), cfg, 3, X, Y, masks)
    got3 = util.trace(gpu_model(gpu_ctx, cfg, p0), cfg, 3, X, Y, masks)
    assert util.rel_l2(got3["params_last"], want3["params_last"]) <= 1e-3
    assert util.rel_l2(got3["losses"], want3["losses"]) <= 1e-4
    assert util.rel_max(got["params1"], want["params1"]) <= TOL_1_MAX


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("cfg", CASES[:2], ids=lambda c: c["name"])
def test_model_100_steps_vs_compiled_reference(gpu_ctx, cfg):
    serial = util.build(ref_binding.RefModel(), dict(cfg, mp=False), seed=0)
    p0 = serial.get_array("parameters")
    ws = util.trace(serial, dict(cfg, mp=False), steps=100)
    want = util.trace(util.build(ref_binding.RefModel(), cfg, params=p0), cfg, steps=100)
    got = util.trace(gpu_model(gpu_ctx, cfg, p0), cfg, steps=100)
    assert gpu_ctx.sync() == 0
    drift1 = util.rel_l2(ws["params1"], want["params1"])
    drift100 = util.rel_l2(ws["params_last"], want["params_last"])
    cmp = util.compare(got, want)
    print({k: f"{v[0]:.2e}" for k, v in cmp.items()}, f"reference self-drift {drift1:.2e} / {drift100:.2e}")
    for key in [k for k in cmp if k.startswith(("act", "delta", "grads"))]:
        assert cmp[key][0] <= TOL_1, f"{key}: {cmp[key][0]:.2e}"
    assert cmp["params1"][0] <= max(TOL_1, 3 * drift1)
    assert cmp["params_last"][0] <= max(TOL_N, 3 * drift100)
    assert util.rel_l2(got["losses"], want["losses"]) <= TOL_N


def test_glorot_uniform_draw_matches_reference_generator(gpu_ctx):
    """Same std::mt19937 stream and draw order as the reference: the fixture's
    initial parameters were drawn by the reference from seed 0."""
    cfg, _, _, _, _, p0, _ = golden_io.load("mlp_softmax_adam")
    m = util.build(dlb200.Model(gpu_ctx), cfg, seed=0)
    assert util.rel_max(m.get_array("parameters"), p0) <= 1e-6


def test_row_pointer_inputs_and_device_inputs_agree(gpu_ctx):
    cfg = configs.deep_brn_mlp(64, 128, 2, 32, 96)
    X, Y = configs.synthetic_batch(cfg)
    B = cfg["batch"]
    a = util.build(dlb200.Model(gpu_ctx), cfg, seed=3)
    b = util.build(dlb200.Model(gpu_ctx), cfg, seed=3)
    a.forward_pass(B, X); a.compute_error(B, Y); a.backward_pass(B); a.update_derivatives(B)
    a.merge_derivatives(); a.update_weights(B, B)
    b.train_step_device(B, gpu_ctx.array(X), gpu_ctx.array(Y))
    assert np.array_equal(a.get_array("parameters"), b.get_array("parameters"))


def test_staged_batches_train_like_train_step(gpu_ctx):
    """Batches copied one step ahead on the copy stream give the same weights,
    bit for bit, and the same losses as the same batches passed to train_step; the
    third stage without a step in between is refused, and so is a step with
    nothing staged."""
    cfg = configs.deep_brn_mlp(64, 128, 2, 32, 96)
    B = cfg["batch"]
    batches = []
    for step in range(5):
        pair = []
        for host in configs.synthetic_batch(cfg, step=step):
            buf = dlb200.pinned_empty(host.shape)
            buf[...] = host
            pair.append(buf)
        batches.append(tuple(pair))
    a = util.build(dlb200.Model(gpu_ctx), cfg, seed=3)
    b = util.build(dlb200.Model(gpu_ctx), cfg, seed=3)
    want = [a.train_step(B, X, Y) for X, Y in batches]
    with pytest.raises(dlb200.DlbError):
        b.train_step_staged()
    got = []
    b.stage_batch(B, *batches[0])
    for i in range(len(batches)):
        if i + 1 < len(batches):
            b.stage_batch(B, *batches[i + 1])
            if i == 0:
                with pytest.raises(dlb200.DlbError):
                    b.stage_batch(B, *batches[2])
        got.append(b.train_step_staged())
    # The loss is summed with double-precision atomic adds, whose order is free.
    np.testing.assert_allclose(got, want, rtol=1e-12)
    assert np.array_equal(a.get_array("parameters"), b.get_array("parameters"))
    assert gpu_ctx.sync() == 0


def test_minibatch_epoch_trains_like_the_batches_one_by_one(gpu_ctx):
    """The mini-batch loop (DL::v1::MiniBatch): 330 rows in batches of 100 are
    three batches, the last of 129: Set__Desired_Data_Per_Batch takes the
    remainder from (330 / 100 - 3) * 100 in double, which is 29.99...; an epoch
    through it gives, bit for bit, the weights of the same batches passed to
    train_step with the data set's size as training size, the mean of their
    losses, and one epoch more on the clock of the normalised weight decay."""
    cfg = configs.deep_brn_mlp(64, 128, 2, 32, 100)
    N = 330
    X, Y = configs.synthetic_batch(cfg, batch=N)
    a = util.build(dlb200.Model(gpu_ctx), cfg, seed=3)
    b = util.build(dlb200.Model(gpu_ctx), cfg, seed=3)
    for m in (a, b):
        m.set_weight_decay(1e-3)
    mb = dlb200.MiniBatch(b, X, Y, 100)
    last = 100 + int((N / 100 - 3) * 100)
    assert last == 129 and (mb.n_batch, mb.per_batch, mb.last_batch) == (3, 100, last)
    a.set_training_size(N)
    for epoch in range(2):
        want = [a.train_step(hi - lo, X[lo:hi], Y[lo:hi]) for lo, hi in ((0, 100), (100, 200), (200, 200 + last))]
        a.set_hparam("epoch_time_step", a.get_hparam("epoch_time_step") + 1.0)
        got = mb.train()
        np.testing.assert_allclose(got, np.mean(want), rtol=1e-12)
        assert np.array_equal(a.get_array("parameters"), b.get_array("parameters"))
        assert 0.0 <= mb.accuracy() <= 100.0
    assert b.get_hparam("epoch_time_step") == 3.0
    assert gpu_ctx.sync() == 0
    # Shuffled: the reference's Fisher-Yates pass; a permutation fixed by the seed.
    m1, m2 = dlb200.MiniBatch(b, X, Y, 100, use_shuffle=True, seed=7), dlb200.MiniBatch(b, X, Y, 100, use_shuffle=True, seed=7)
    assert np.array_equal(m1.order(), np.arange(N))
    m1.shuffle()
    m2.shuffle()
    assert np.array_equal(m1.order(), m2.order())
    assert np.array_equal(np.sort(m1.order()), np.arange(N)) and not np.array_equal(m1.order(), np.arange(N))
    before = m1.order()
    loss = m1.train()      # shuffles again, then trains
    assert np.isfinite(loss) and not np.array_equal(m1.order(), before)
    m1.set_shuffle(False)
    assert np.array_equal(m1.order(), np.arange(N))
    # Refused as in the reference: a batch larger than the data set, fewer than two batches.
    with pytest.raises(dlb200.DlbError):
        dlb200.MiniBatch(b, X, Y, N + 1)
    with pytest.raises(dlb200.DlbError):
        dlb200.MiniBatch(b, X, Y, 200)
    assert dlb200.MiniBatch(b, X, Y, 100, max_batches=2).last_batch == 100 + int((N / 100 - 2) * 100)


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("case", ["brn_bernoulli_distance", "softmax_accuracy"])
def test_training_accuracy_against_the_compiled_reference(gpu_ctx, case):
    """Model::compute_error keeps the accuracy counter of the training pass; here
    it is kept on request.  Three training steps each on the compiled reference
    and on the GPU, the accuracy of every step read where the reference's loop
    reads it (after the merge of the threads' counters)."""
    cfg, fn = {
        "brn_bernoulli_distance": (configs.deep_brn_mlp(64, 128, 2, 32, 96), fc_step.ACCU_DISTANCE),
        "softmax_accuracy": (configs.mlp_softmax(96, 128, 10, 128), fc_step.ACCU_CROSS_ENTROPY),
    }[case]
    B = cfg["batch"]
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    gpu = gpu_model(gpu_ctx, cfg, ref.get_array("parameters"))
    gpu.set_training_accuracy(True)
    seen = []
    for m in (ref, gpu):
        m.train_begin(B)
        m.set_accu_fn(fn)
        for li, mk in masks.items():
            m.set_dropout_mask(li, mk)
        acc = []
        for _ in range(3):
            m.reset_loss()
            m.forward_pass(B, X)
            m.compute_error(B, Y)
            m.backward_pass(B)
            m.update_derivatives(B)
            m.merge_derivatives()     # the reference adds its threads' counters up here
            acc.append(m.get_accu(B))
            m.update_weights(B, B)
        seen.append(acc)
    assert gpu_ctx.sync() == 0
    one_trial = 100.0 / (B * (1 if fn == fc_step.ACCU_CROSS_ENTROPY else cfg["layers"][-1]["units"]))
    print(case, seen)
    assert any(a > 0 for a in seen[0])
    for a_ref, a_gpu in zip(*seen):
        assert abs(a_ref - a_gpu) <= 2 * one_trial
    # Off (the default): a training step leaves the counter alone.
    gpu.set_training_accuracy(False)
    gpu.reset_loss()
    gpu.forward_pass(B, X)
    gpu.compute_error(B, Y)
    assert gpu.get_accu(B) == 0.0


def test_minibatch_epoch_with_batches_gathered_by_the_kept_host_threads(gpu_ctx):
    """Batches above 1 MB are gathered by the model's host threads: the same
    weights, bit for bit, as the batches passed one by one."""
    cfg = configs.deep_brn_mlp(1024, 256, 1, 512, 200)
    N = 660
    X, Y = configs.synthetic_batch(cfg, batch=N)
    a = util.build(dlb200.Model(gpu_ctx), cfg, seed=4)
    b = util.build(dlb200.Model(gpu_ctx), cfg, seed=4)
    mb = dlb200.MiniBatch(b, X, Y, 200, use_shuffle=True, seed=11)
    assert (mb.n_batch, mb.last_batch) == (3, 200 + int((N / 200 - 3) * 200))
    a.set_training_size(N)
    for epoch in range(2):
        got = mb.train()                 # shuffles, then trains
        order = mb.order()
        bounds = ((0, 200), (200, 400), (400, 400 + mb.last_batch))
        want = [a.train_step(hi - lo, X[order[lo:hi]], Y[order[lo:hi]]) for lo, hi in bounds]
        a.set_hparam("epoch_time_step", a.get_hparam("epoch_time_step") + 1.0)
        np.testing.assert_allclose(got, np.mean(want), rtol=1e-12)
        assert np.array_equal(a.get_array("parameters"), b.get_array("parameters"))
    assert gpu_ctx.sync() == 0


def test_unsupported_configurations_are_refused(gpu_ctx):
    m = dlb200.Model(gpu_ctx)
    m.compile([3, 3, 3], [8, 8, 4])
    with pytest.raises(dlb200.DlbError):
        m.set_layer_activation_function(1, 18)       # SIGMOID: outside the path
    with pytest.raises(dlb200.DlbError):
        m.Set__Layer_Normalization(2, 2)             # not on the output layer
    with pytest.raises(dlb200.DlbError):
        m.set_dropout(2, 2, 0.5)                     # not on the output layer
    with pytest.raises(dlb200.DlbError):
        m.set_optimizer(7)                           # iRPROP-
    with pytest.raises(dlb200.DlbError):
        m.forward_pass(4, np.zeros((4, 8), np.float32))   # activations never set (reference default: sigmoid)


@pytest.mark.parametrize("optimizer", [OPTIMIZER.ADAM, OPTIMIZER.AMSBOUND], ids=["adam", "amsbound"])
def test_weight_decay(gpu_ctx, optimizer):
    """Decoupled, normalised weight decay on the weights only, against the CPU
    restatement (itself pinned to the compiled reference)."""
    cfg = configs.deep_brn_mlp(64, 128, 2, 32, 96, optimizer=optimizer)
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    p0, seed = util.kink_free_parameters(cfg, fc_step.OracleModel, X, masks, scale=1.0 / np.sqrt(128))
    ora = util.build(fc_step.OracleModel(), cfg, params=p0)
    ora.set_weight_decay(0.05)
    want = util.trace(ora, cfg, 1, X, Y, masks)
    mod = gpu_model(gpu_ctx, cfg, p0)
    mod.set_weight_decay(0.05)
    got = util.trace(mod, cfg, 1, X, Y, masks)
    assert gpu_ctx.sync() == 0
    for key, (l2, mx) in util.compare(got, want).items():
        assert l2 <= TOL_1, f"{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"
    nw = mod.size("total_weights")
    moved = np.abs(got["params1"][:nw] - p0[:nw]).mean()
    plain = util.trace(gpu_model(gpu_ctx, cfg, p0), cfg, 1, X, Y, masks)
    assert np.abs(plain["params1"][:nw] - got["params1"][:nw]).mean() > 0.01 * moved
    with pytest.raises(dlb200.DlbError):
        mod.set_weight_decay(1.5)


def test_weight_decay_without_normalisation(gpu_ctx):
    """use_normalized_weight_decay = false: the decay enters as it is, whatever
    the ratio of batch to training size."""
    cfg = configs.deep_brn_mlp(64, 128, 2, 32, 96, optimizer=OPTIMIZER.ADAM)
    cfg = dict(cfg, hparams=dict(cfg["hparams"], use_normalized_weight_decay=0))
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    B = cfg["batch"]
    p0, seed = util.kink_free_parameters(cfg, fc_step.OracleModel, X, masks, scale=1.0 / np.sqrt(128))
    out = []
    for model in (util.build(fc_step.OracleModel(), cfg, params=p0), gpu_model(gpu_ctx, cfg, p0)):
        model.set_weight_decay(0.05)
        model.train_begin(B)
        for li, mk in masks.items():
            model.set_dropout_mask(li, mk)
        model.reset_loss()
        model.forward_pass(B, X); model.compute_error(B, Y); model.backward_pass(B)
        model.update_derivatives(B); model.merge_derivatives(); model.update_weights(B, 16 * B)
        out.append(model.get_array("parameters"))
    assert gpu_ctx.sync() == 0
    assert util.rel_l2(out[1], out[0]) <= TOL_1
    assert util.rel_l2(out[1] - p0, out[0] - p0) <= 1e-3


def test_plain_batch_normalization(gpu_ctx):
    """LAYER_NORM::BATCH_NORMALIZATION: r = 1, d = 0 whatever the model's maxima,
    against the CPU restatement (itself pinned to the compiled reference)."""
    cfg = configs.deep_brn_mlp(64, 128, 2, 32, 96)
    layers = [dict(l, norm=LAYER_NORM.BATCH_NORMALIZATION) if l.get("norm") else l for l in cfg["layers"]]
    cfg = dict(cfg, layers=layers)
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    p0, seed = util.kink_free_parameters(cfg, fc_step.OracleModel, X, masks, scale=1.0 / np.sqrt(128))
    want = util.trace(util.build(fc_step.OracleModel(), cfg, params=p0), cfg, 1, X, Y, masks)
    mod = gpu_model(gpu_ctx, cfg, p0)
    got = util.trace(mod, cfg, 1, X, Y, masks)
    assert gpu_ctx.sync() == 0
    for key, (l2, mx) in util.compare(got, want).items():
        assert l2 <= TOL_1, f"{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"
    assert np.all(mod.get_layer_norm(1, "r_correction", 128) == 1) and not mod.get_layer_norm(1, "d_correction", 128).any()


@pytest.mark.parametrize("form", ["plain", "momentum", "nesterov"])
def test_gradient_descent(gpu_ctx, form):
    """Gradient descent, with momentum and in the Nesterov form, with weight
    decay, against the CPU restatement (itself pinned to the compiled
    reference)."""
    extra = {"plain": dict(learning_momentum=0.0), "momentum": dict(learning_momentum=0.9),
             "nesterov": dict(learning_momentum=0.9, use_nesterov=1)}[form]
    cfg = configs.deep_brn_mlp(64, 128, 2, 32, 96, optimizer=OPTIMIZER.GD)
    cfg = dict(cfg, hparams=dict(learning_rate=0.05, **extra))
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    p0, seed = util.kink_free_parameters(cfg, fc_step.OracleModel, X, masks, scale=1.0 / np.sqrt(128))
    ora = util.build(fc_step.OracleModel(), cfg, params=p0)
    ora.set_weight_decay(0.05)
    want = util.trace(ora, cfg, 2, X, Y, masks)
    mod = gpu_model(gpu_ctx, cfg, p0)
    mod.set_weight_decay(0.05)
    got = util.trace(mod, cfg, 2, X, Y, masks)
    assert gpu_ctx.sync() == 0
    assert util.rel_l2(got["params1"], want["params1"]) <= TOL_1
    assert util.rel_l2(got["params_last"], want["params_last"]) <= TOL_N
    assert util.rel_l2(got["params_last"] - p0, want["params_last"] - p0) <= 1e-3   # the movement itself


def test_gradient_clipping(gpu_ctx):
    """Clipping by the norm of the whole gradient vector before the optimizer,
    against the CPU restatement (itself pinned to the compiled reference); a
    norm above the gradient's leaves the step bit for bit as it was."""
    cfg = configs.deep_brn_mlp(64, 128, 2, 32, 96, optimizer=OPTIMIZER.ADAM)
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    p0, seed = util.kink_free_parameters(cfg, fc_step.OracleModel, X, masks, scale=1.0 / np.sqrt(128))
    plain = util.trace(gpu_model(gpu_ctx, cfg, p0), cfg, 1, X, Y, masks)
    norm = float(np.sqrt(np.sum(plain["grads"].astype(np.float64) ** 2)))
    ora = util.build(fc_step.OracleModel(), cfg, params=p0)
    ora.set_clip_gradient(True, norm / 50)
    want = util.trace(ora, cfg, 2, X, Y, masks)
    mod = gpu_model(gpu_ctx, cfg, p0)
    mod.set_clip_gradient(True, norm / 50)
    got = util.trace(mod, cfg, 2, X, Y, masks)
    assert gpu_ctx.sync() == 0
    assert util.rel_l2(got["params1"], want["params1"]) <= TOL_1
    assert util.rel_l2(got["params_last"], want["params_last"]) <= TOL_N
    loose = gpu_model(gpu_ctx, cfg, p0)
    loose.set_clip_gradient(True, norm * 1e3)
    assert np.array_equal(util.trace(loose, cfg, 1, X, Y, masks)["params1"], plain["params1"])
    with pytest.raises(dlb200.DlbError):
        mod.set_clip_gradient(True, 0.0)


@pytest.mark.parametrize("n", [1, 5, 4096, 1000003])
def test_clip_gradient_kernel(gpu_ctx, n):
    """g *= max / |g| when |g| >= max, untouched otherwise; odd sizes and a
    start that is not 16-byte aligned."""
    rng = np.random.default_rng(n)
    g = rng.standard_normal(n + 1).astype(np.float32)
    norm = float(np.sqrt(np.sum(g[1:].astype(np.float64) ** 2)))
    for limit, clipped in ((norm * 0.25, True), (norm * 4, False)):
        d = gpu_ctx.array(g)
        dlb200.check(gpu_ctx.L.dlb_clip_gradient(gpu_ctx.h, d.offset(1), n, limit), "clip")
        out = d.get()
        assert gpu_ctx.sync() == 0
        assert out[0] == g[0]
        if clipped:
            f = np.float32(np.float32(limit) / np.float32(norm))
            assert util.rel_l2(out[1:], g[1:] * f) <= 1e-6
        else:
            assert np.array_equal(out[1:], g[1:])


def test_uout_dropout(gpu_ctx):
    """UOut inside the Model: the draws are an input of the step."""
    cfg = configs.deep_brn_mlp(64, 128, 2, 32, 96, dropout=LAYER_DROPOUT.UOUT, keep=0.25)
    B = cfg["batch"]
    X, Y = configs.synthetic_batch(cfg)
    rng = np.random.default_rng(8)
    noise = {li: rng.uniform(-0.25, 0.25, (B, 128)).astype(np.float32) for li in (1, 2)}

    def prepare(model):
        for li, nz in noise.items():
            model.set_uout_noise(li, nz)

    p0, seed = util.kink_free_parameters(cfg, fc_step.OracleModel, X, {}, scale=1.0 / np.sqrt(128), prepare=prepare)
    ora = util.build(fc_step.OracleModel(), cfg, params=p0)
    mod = gpu_model(gpu_ctx, cfg, p0)
    with pytest.raises(dlb200.DlbError):
        gpu_model(gpu_ctx, cfg, p0).forward_pass(B, X)   # no draws yet (on a model of its own: the
                                                         # refused pass has already moved running averages)
    prepare(ora)
    prepare(mod)
    want = util.trace(ora, cfg, 1, X, Y, {})
    got = util.trace(mod, cfg, 1, X, Y, {})
    assert gpu_ctx.sync() == 0
    for key, (l2, mx) in util.compare(got, want).items():
        assert l2 <= TOL_1, f"{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"
    plain = util.trace(gpu_model(gpu_ctx, dict(cfg, layers=[dict(l, dropout=None) for l in cfg["layers"]]), p0),
                       cfg, 1, X, Y, {})
    assert util.rel_l2(plain["act2"], got["act2"]) > 1e-2   # the noise is applied


@pytest.mark.parametrize("case", ["brn_bernoulli_distance", "softmax_accuracy"])
def test_evaluation_pass(gpu_ctx, case):
    """Inference forward (running averages, dropout scaling) and the loss /
    accuracy pass, against the CPU restatement (itself pinned to the compiled
    reference's Driver::evalt sequence)."""
    cfg, fn = {
        "brn_bernoulli_distance": (configs.deep_brn_mlp(64, 128, 2, 32, 96), fc_step.ACCU_DISTANCE),
        "softmax_accuracy": (configs.mlp_softmax(96, 128, 10, 128), fc_step.ACCU_CROSS_ENTROPY),
    }[case]
    B, last = cfg["batch"], len(cfg["layers"]) - 1
    X, Y = configs.synthetic_batch(cfg)
    Xe, Ye = configs.synthetic_batch(dict(cfg, data_seed=5))
    masks = configs.dropout_masks(cfg)
    p0, _ = util.kink_free_parameters(cfg, fc_step.OracleModel, X, masks, scale=1.0 / np.sqrt(128))
    out = []
    for m in (util.build(fc_step.OracleModel(), cfg, params=p0), gpu_model(gpu_ctx, cfg, p0)):
        m.train_begin(B)
        for li, mk in masks.items():
            m.set_dropout_mask(li, mk)
        m.train_step(B, X, Y)
        m.set_propagation(0)
        m.set_accu_fn(fn)
        m.reset_loss()
        m.forward_pass(B, Xe)
        m.compute_loss(B, Ye)
        out.append((m.get_loss(), m.get_accu(B), m.get_layer_outputs(last, B).reshape(B, -1)))
        m.set_propagation(1)
    (lo, ao, qo), (lg, ag, qg) = out
    assert gpu_ctx.sync() == 0
    assert util.rel_l2(qg, qo) <= TOL_1
    assert abs(lg - lo) <= 1e-5 * abs(lo)
    assert abs(ag - ao) <= 100.0 * 2 / (B * (1 if fn == fc_step.ACCU_CROSS_ENTROPY else qo.shape[1]))


@pytest.mark.parametrize("kind", [LAYER_DROPOUT.BERNOULLI, LAYER_DROPOUT.BERNOULLI_INVERTED],
                         ids=["bernoulli", "inverted"])
def test_input_layer_dropout(gpu_ctx, kind):
    """Dropout on the input layer (the reference applies it to the batch as it is
    assigned, v1/learner/assign_inputs.cpp L:94-130) in training and at
    inference, against the CPU restatement; it travels through a checkpoint."""
    cfg = configs.deep_brn_mlp(64, 128, 2, 32, 96)
    layers = [dict(l) for l in cfg["layers"]]
    layers[0]["dropout"] = (kind, 0.8)
    cfg = dict(cfg, layers=layers)
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    p0, seed = util.kink_free_parameters(cfg, fc_step.OracleModel, X, masks, scale=1.0 / np.sqrt(128))
    ora = util.build(fc_step.OracleModel(), cfg, params=p0)
    mod = gpu_model(gpu_ctx, cfg, p0)
    want = util.trace(ora, cfg, 1, X, Y, masks)
    got = util.trace(mod, cfg, 1, X, Y, masks)
    assert gpu_ctx.sync() == 0
    for key, (l2, mx) in util.compare(got, want).items():
        assert l2 <= TOL_1, f"{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"
    unmasked = util.trace(gpu_model(gpu_ctx, cfg, p0), cfg, 1, X, Y, {k: v for k, v in masks.items() if k})
    assert util.rel_l2(unmasked["act1"], got["act1"]) > 1e-2
    B, last = cfg["batch"], len(cfg["layers"]) - 1
    util.copy_trained_state(mod, ora, cfg)
    outs = []
    for m in (ora, mod):
        m.set_propagation(0)
        m.forward_pass(B, X)
        outs.append(m.get_layer_outputs(last, B).reshape(B, -1))
        m.set_propagation(1)
    assert util.rel_l2(outs[1], outs[0]) <= TOL_1
    assert mod.layer_info(0)["dropout"] == kind


def test_operand_form_can_change_under_a_live_model(gpu_ctx):
    """A model that has trained under one operand form keeps training correctly
    after dlb_ctx_set_gemm_kind: its weight planes are split again in the new
    form instead of being read as the other form's planes."""
    cfg = configs.deep_brn_mlp(256, 512, 2, 256, 256)
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    B = cfg["batch"]
    before = gpu_ctx.gemm_kind()
    try:
        for first, second in ((1, 0), (0, 1)):
            gpu_ctx.set_gemm_kind(first)
            live = util.build(dlb200.Model(gpu_ctx), cfg, seed=5)
            for li, mk in masks.items():
                live.set_dropout_mask(li, mk)
            live.train_step(B, X, Y)
            state = live.get_array("parameters")
            gpu_ctx.set_gemm_kind(second)
            fresh = util.build(dlb200.Model(gpu_ctx), cfg, params=state)
            for li, mk in masks.items():
                fresh.set_dropout_mask(li, mk)
            util.copy_trained_state(live, fresh, cfg)
            live.forward_pass(B, X)
            fresh.forward_pass(B, X)
            last = len(cfg["layers"]) - 1
            a, b = live.get_layer_outputs(last, B), fresh.get_layer_outputs(last, B)
            assert gpu_ctx.sync() == 0
            assert np.array_equal(a, b), f"{first}->{second}: rel_l2 {util.rel_l2(a, b):.2e}"
    finally:
        gpu_ctx.set_gemm_kind(before)


def test_training_size_enters_the_normalised_weight_decay(gpu_ctx):
    """The one-call steps pass dlb_model_set_training_size to the update: with a
    training set of 8 batches the decay is weight_decay * sqrt(1 / 8), as
    update_weights(batch, 8 * batch) gives (v1/learner/train.cpp L:278-283)."""
    cfg = configs.deep_brn_mlp(64, 128, 2, 32, 96, optimizer=OPTIMIZER.ADAM)
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    B = cfg["batch"]
    models = []
    for _ in range(3):
        m = util.build(dlb200.Model(gpu_ctx), cfg, seed=11)
        m.set_weight_decay(0.05)
        for li, mk in masks.items():
            m.set_dropout_mask(li, mk)
        models.append(m)
    one_call, by_hand, whole_set = models
    one_call.set_training_size(8 * B)
    one_call.train_step(B, X, Y)
    by_hand.forward_pass(B, X); by_hand.compute_error(B, Y); by_hand.backward_pass(B)
    by_hand.update_derivatives(B); by_hand.merge_derivatives(); by_hand.update_weights(B, 8 * B)
    whole_set.train_step(B, X, Y)
    assert gpu_ctx.sync() == 0
    a, b, c = (m.get_array("parameters") for m in models)
    assert np.array_equal(a, b)
    assert not np.array_equal(a, c)


def test_staged_steps_with_a_lagged_loss(gpu_ctx):
    """With a loss lag of one step a staged step returns the loss of the step
    before (NaN at first) and the host never waits for the step it has just
    enqueued; weights and losses are those of the in-order loop."""
    cfg = configs.deep_brn_mlp(64, 128, 2, 32, 96)
    B = cfg["batch"]
    batches = []
    for step in range(4):
        pair = []
        for host in configs.synthetic_batch(cfg, step=step):
            buf = dlb200.pinned_empty(host.shape)
            buf[...] = host
            pair.append(buf)
        batches.append(tuple(pair))
    a = util.build(dlb200.Model(gpu_ctx), cfg, seed=3)
    b = util.build(dlb200.Model(gpu_ctx), cfg, seed=3)
    want = [a.train_step(B, X, Y) for X, Y in batches]
    b.set_loss_lag(1)
    got = []
    for X, Y in batches:
        b.stage_batch(B, X, Y)
        got.append(b.train_step_staged())
    got.append(b.get_loss())
    assert np.isnan(got[0])
    np.testing.assert_allclose(got[1:], want, rtol=1e-12)
    assert np.array_equal(a.get_array("parameters"), b.get_array("parameters"))
    with pytest.raises(dlb200.DlbError):
        b.set_loss_lag(2)
    assert gpu_ctx.sync() == 0
