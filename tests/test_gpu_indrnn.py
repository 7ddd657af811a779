"""IndRNN stacks on the GPU, through the Model entry points of the C ABI and
through the time-batched kernels directly: against the committed fixtures of the
compiled reference and against the CPU restatement on shapes whose products run
on the tensor-core kernel."""
import numpy as np
import pytest

import configs
import dlb200
import fc_indrnn
import fc_step
import golden_io
import util
from enums import ACTIVATION, LAYER_DROPOUT

pytestmark = pytest.mark.gpu

TOL_1 = 1e-5       # activations, errors, gradients after one step (rel_l2)
TOL_PARAMS = 1e-4  # updated weights: the first Adam-family step magnifies gradients of the order of eps


def _check(got, want, skip=()):
    for key, (l2, mx) in util.compare(got, want).items():
        if key in skip:
            continue
        tol = TOL_PARAMS if key.startswith("params") else TOL_1
        assert l2 <= tol, f"{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"


@pytest.mark.parametrize("name", sorted(golden_io.RECURRENT_CASES))
def test_indrnn_model_matches_golden(gpu_ctx, name):
    cfg, steps, X, Y, masks, p0, want = golden_io.load(name)
    got = util.trace(util.build(dlb200.Model(gpu_ctx), cfg, params=p0), cfg, steps, X, Y, masks)
    assert gpu_ctx.sync() == 0
    _check(got, want)


def _kink_free(cfg, X, band=2e-6, tries=64):
    """Seeded weights (recurrent weights from U(0, 1)) for which no hidden
    pre-activation lies within `band` of a derivative jump."""
    scale = 1.0 / np.sqrt(cfg["layers"][1]["units"])
    for seed in range(tries):
        ora = util.build(fc_indrnn.IndRnnOracleModel(), cfg)
        rng = np.random.default_rng(seed)
        p0 = ora.get_array("parameters")
        nw = ora.size("total_weights")
        p0[:nw] = (rng.standard_normal(nw) * scale).astype(np.float32)
        for _, s in configs.recurrent_slices(cfg):
            p0[s] = rng.uniform(0, 1, s.stop - s.start).astype(np.float32)
        ora.set_array("parameters", p0)
        if util.near_kink(ora, cfg, X, configs.dropout_masks(cfg), band) == 0:
            return p0
    raise AssertionError("no kink-free seed found")


@pytest.mark.parametrize("cfg", [
    configs.indrnn_stack(n_in=64, hidden=128, depth=2, n_out=32, seq_w=8, batch=32),
    configs.indrnn_stack(n_in=128, hidden=128, depth=2, n_out=64, seq_w=4, batch=64, af=ACTIVATION.SELU),
    configs.indrnn_stack(n_in=64, hidden=128, depth=2, n_out=64, seq_w=6, batch=48, norm=False),
], ids=lambda c: c["name"])
def test_indrnn_model_vs_restatement_tensor_core_shape(gpu_ctx, cfg):
    X, Y = configs.synthetic_batch(cfg)
    p0 = _kink_free(cfg, X)
    want = util.trace(util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0), cfg, 1, X, Y)
    got = util.trace(util.build(dlb200.Model(gpu_ctx), cfg, params=p0), cfg, 1, X, Y)
    assert gpu_ctx.sync() == 0
    _check(got, want)
    # Later steps may meet a derivative jump; only the scale of the agreement is checked.
    want = util.trace(util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0), cfg, 3, X, Y)
    got = util.trace(util.build(dlb200.Model(gpu_ctx), cfg, params=p0), cfg, 3, X, Y)
    assert gpu_ctx.sync() == 0
    assert util.rel_l2(got["params_last"], want["params_last"]) <= 1e-3
    assert util.rel_l2(got["losses"], want["losses"]) <= 1e-4


def test_clip_gradient_sets_the_recurrent_bound(gpu_ctx):
    """Recurrent weights come back into +-clip(clip_gradient, 2, 10)^(1/T) after
    the update, with clipping on (norm 5: the gradient is scaled as well) and
    off (norm 5 only widens the bound)."""
    cfg = configs.indrnn_stack(n_in=64, hidden=128, depth=2, n_out=32, seq_w=4, batch=32)
    X, Y = configs.synthetic_batch(cfg)
    p0 = _kink_free(cfg, X)
    for _, s in configs.recurrent_slices(cfg):
        p0[s] = np.linspace(-2.5, 2.5, s.stop - s.start, dtype=np.float32)
    for use in (False, True):
        ora = util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0)
        ora.set_clip_gradient(use, 5.0)
        want = util.trace(ora, cfg, 1, X, Y)
        mod = util.build(dlb200.Model(gpu_ctx), cfg, params=p0)
        mod.set_clip_gradient(use, 5.0)
        got = util.trace(mod, cfg, 1, X, Y)
        assert gpu_ctx.sync() == 0
        bound = np.float32(5.0) ** np.float32(0.25)
        for _, s in configs.recurrent_slices(cfg):
            assert np.isclose(np.abs(got["params1"][s]).max(), bound, rtol=1e-6)
        assert util.rel_l2(got["params1"], want["params1"]) <= 1e-5


@pytest.mark.parametrize("delay", [0, 2], ids=["all_steps", "last_two"])
def test_softmax_output_in_a_time_stepped_model(gpu_ctx, delay):
    """Softmax + cross-entropy on the time steps t >= delay: the error against
    the target of time step 0, the loss against the step's own target, as the
    reference has them (pinned in tests/test_oracle_indrnn.py)."""
    from enums import LOSS_FN, OPTIMIZER
    cfg = configs.indrnn_stack(n_in=64, hidden=128, depth=2, n_out=32, seq_w=4, batch=32, optimizer=OPTIMIZER.ADAM)
    cfg["layers"][-1]["af"] = ACTIVATION.SOFTMAX
    cfg = dict(cfg, loss=LOSS_FN.CROSS_ENTROPY, targets="onehot", time_delays=delay)
    X, Y = configs.synthetic_batch(cfg)
    p0 = _kink_free(cfg, X)
    want = util.trace(util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0), cfg, 1, X, Y)
    got = util.trace(util.build(dlb200.Model(gpu_ctx), cfg, params=p0), cfg, 1, X, Y)
    assert gpu_ctx.sync() == 0
    _check(got, want)


def test_recurrent_bounds_set_by_hand(gpu_ctx, tmp_path):
    """Per-layer bounds of the recurrent weights: one layer with its own interval,
    one with the clamp off; the bounds survive a save / load, and a default bound
    keeps following set_clip_gradient."""
    cfg = configs.indrnn_stack(n_in=64, hidden=128, depth=2, n_out=32, seq_w=4, batch=32)
    X, Y = configs.synthetic_batch(cfg)
    p0 = _kink_free(cfg, X)
    for _, s in configs.recurrent_slices(cfg):
        p0[s] = np.linspace(-1.5, 1.5, s.stop - s.start, dtype=np.float32)
    ora = util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0)
    mod = util.build(dlb200.Model(gpu_ctx), cfg, params=p0)
    for m in (ora, mod):
        m.set_constraint_recurrent_weight(1, -0.5, 0.75)
        m.set_constraint_recurrent_weight(2, 0.0, 0.0)
    want = util.trace(ora, cfg, 1, X, Y)
    got = util.trace(mod, cfg, 1, X, Y)
    assert gpu_ctx.sync() == 0
    (_, s1), (_, s2) = configs.recurrent_slices(cfg)
    assert got["params1"][s1].min() == np.float32(-0.5) and got["params1"][s1].max() == np.float32(0.75)
    assert np.abs(got["params1"][s2]).max() > 1.4
    assert util.rel_l2(got["params1"], want["params1"]) <= 1e-5
    # The bounds are part of the parameter file.
    a, b = str(tmp_path / "m.net"), str(tmp_path / "m.nn")
    mod.save(a, b)
    back = dlb200.Model(gpu_ctx)
    back.load(a, b)
    assert back.get_constraint_recurrent_weight(1) == (np.float32(-0.5), np.float32(0.75))
    assert back.get_constraint_recurrent_weight(2) == (0.0, 0.0)
    # A layer back on the default follows the gradient norm again.
    back.set_constraint_recurrent_weight_default(1)
    back.set_clip_gradient(False, 5.0)
    lo, hi = back.get_constraint_recurrent_weight(1)
    assert np.isclose(hi, np.float32(5.0) ** np.float32(0.25), rtol=1e-6) and lo == -hi
    # What is refused: layers without recurrent weights, inverted intervals.
    with pytest.raises(dlb200.DlbError):
        back.set_constraint_recurrent_weight(len(cfg["layers"]) - 1, -1.0, 1.0)
    with pytest.raises(dlb200.DlbError):
        back.set_constraint_recurrent_weight(1, 1.0, -1.0)


@pytest.mark.parametrize("delay", [7, 0], ids=["last_step", "all_steps"])
def test_indrnn_evaluation_pass(gpu_ctx, delay):
    """Inference through time (each time step's own running averages), loss and
    accuracy over the steps t >= n_time_delay, against the CPU restatement from
    the same trained state."""
    cfg = dict(configs.indrnn_stack(n_in=64, hidden=128, depth=2, n_out=32, seq_w=8, batch=32), time_delays=delay)
    B, last = cfg["batch"], len(cfg["layers"]) - 1
    X, Y = configs.synthetic_batch(cfg)
    Xe, Ye = configs.synthetic_batch(dict(cfg, data_seed=5))
    p0 = _kink_free(cfg, X)
    ora = util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0)
    mod = util.build(dlb200.Model(gpu_ctx), cfg, params=p0)
    util.trace(mod, cfg, 2, X, Y)
    util.copy_trained_state(mod, ora, cfg)
    out = []
    for m in (ora, mod):
        m.train_begin(B)
        m.set_propagation(0)
        m.set_accu_fn(3)   # DISTANCE
        m.set_accu_var(0.6)
        m.reset_loss()
        m.forward_pass(B, Xe)
        m.compute_loss(B, Ye)
        out.append((m.get_loss(), m.get_accu(B), m.get_layer_outputs(last, B).reshape(-1)))
        m.set_propagation(1)
    (lo, ao, qo), (lg, ag, qg) = out
    assert gpu_ctx.sync() == 0
    assert util.rel_l2(qg, qo) <= 1e-5
    assert abs(lg - lo) <= 1e-5 * abs(lo)
    trials = B * (8 - delay) * 32
    assert abs(ag - ao) <= 100.0 * 3 / trials


def test_glorot_and_recurrent_initialisation_match_the_fixture_layout(gpu_ctx):
    cfg = configs.indrnn_stack(n_in=6, hidden=8, depth=2, n_out=5, seq_w=4, batch=3)
    m = util.build(dlb200.Model(gpu_ctx), cfg, seed=0)
    o = util.build(fc_indrnn.IndRnnOracleModel(), cfg)
    for name in ("total_parameters", "total_weights", "total_bias", "total_normalized_units"):
        assert m.size(name) == o.size(name)
    p = m.get_array("parameters")
    T = 4.0
    lo, hi = 0.5 ** (1 / T), 2.0 ** (1 / T)
    (l1, s1), (l2, s2) = configs.recurrent_slices(cfg)
    assert (p[s1] >= 0).all() and (p[s1] <= hi).all()
    assert (p[s2] >= lo * (1 - 1e-6)).all() and (p[s2] <= hi).all()   # top layer: long-term memory range
    g0 = m.size("total_weights") + m.size("total_bias")
    assert np.allclose(p[g0 + 6:g0 + 22], 0.1) and np.allclose(p[g0:g0 + 6], 1.0)


def _brn_state(rng, T, n):
    mean = rng.standard_normal((T, n)).astype(np.float32) * 0.1
    sigma = (0.5 + rng.random((T, n))).astype(np.float32)
    r = (0.8 + 0.4 * rng.random((T, n))).astype(np.float32)
    d = (rng.standard_normal((T, n)) * 0.1).astype(np.float32)
    gamma = (0.5 + rng.random(n)).astype(np.float32)
    beta = (rng.standard_normal(n) * 0.1).astype(np.float32)
    return mean, sigma, r, d, gamma, beta


@pytest.mark.parametrize("T,B,n", [(5, 16, 128), (7, 9, 10), (1, 8, 32), (6, 40, 256), (3, 5, 132), (2, 3, 384)])
@pytest.mark.parametrize("af", [ACTIVATION.RELU, ACTIVATION.ELU])
def test_time_kernels(gpu_ctx, T, B, n, af):
    """Forward walk, reverse walk, sums and apply against numpy on one layer."""
    ctx, L = gpu_ctx, gpu_ctx.L
    rng = np.random.default_rng(T * 100 + n)
    Z = rng.standard_normal((T, B, n)).astype(np.float32)
    mean, sigma, r, d, gamma, beta = _brn_state(rng, T, n)
    u_rec = rng.uniform(0, 1, n).astype(np.float32)
    dev = {k: ctx.array(v) for k, v in dict(mean=mean, sigma=sigma, r=r, d=d, gamma=gamma, beta=beta).items()}
    ma, sa = ctx.array(np.zeros((T, n), np.float32)), ctx.array(np.ones((T, n), np.float32))
    ua = dlb200.BrnUnitArrays(dev["mean"].ptr, dev["sigma"].ptr, ma.ptr, sa.ptr, dev["r"].ptr, dev["d"].ptr,
                              dev["gamma"].ptr, dev["beta"].ptr)
    import ctypes as C
    Zd, ud = ctx.array(Z), ctx.array(u_rec)
    A, A_lo = ctx.empty((T, B, n)), ctx.empty((T, B, n))
    dlb200.check(L.dlb_indrnn_forward(ctx.h, Zd.ptr, C.byref(ua), ud.ptr, af, A.ptr, A_lo.ptr, T, B, n))
    # numpy
    f32 = np.float32
    xh = ((Z - mean[:, None]) / sigma[:, None] * r[:, None] + d[:, None]).astype(f32)
    y = (gamma * xh + beta).astype(f32)
    pre = np.empty_like(y)
    h = np.empty_like(y)
    for t in range(T):
        pre[t] = y[t] if t == 0 else (y[t] + u_rec * h[t - 1]).astype(f32)
        h[t] = fc_step.af_fire(af, pre[t])
    got_h = A.get()
    assert util.rel_l2(got_h, h) <= 1e-6
    if ctx.gemm_kind() == 0:   # TF32 residual plane
        hi = got_h.view(np.uint32) & np.uint32(0xFFFFE000)
        assert np.allclose(hi.view(np.float32) + A_lo.get(), got_h, rtol=0, atol=1e-6 * np.abs(got_h).max())
    else:                      # fp16 planes of s * h, s = 2^(14 - floor(log2 max|h|))
        planes = A_lo.get().ravel().view(np.float16).astype(np.float64)
        s = 2.0 ** (14 - np.floor(np.log2(np.abs(got_h).max())))
        both = (planes[:got_h.size] + planes[got_h.size:]) / s
        assert np.allclose(both, got_h.ravel(), rtol=2.0 ** -21, atol=2.0 ** -38 * np.abs(got_h).max())
        # A second call on the same buffers: the walk writes the planes itself where
        # the width allows, with the scale predicted from the first call (two
        # octaves lower); the activations are the same bits either way.
        dlb200.check(L.dlb_indrnn_forward(ctx.h, Zd.ptr, C.byref(ua), ud.ptr, af, A.ptr, A_lo.ptr, T, B, n))
        assert np.array_equal(A.get(), got_h)
        planes = A_lo.get().ravel().view(np.float16).astype(np.float64)
        s2 = s / 4 if n % 128 == 0 else s
        both = (planes[:got_h.size] + planes[got_h.size:]) / s2
        assert np.allclose(both, got_h.ravel(), rtol=2.0 ** -21, atol=2.0 ** -36 * np.abs(got_h).max())
    # reverse walk
    dA = rng.standard_normal((T, B, n)).astype(np.float32)
    E = ctx.array(dA)
    dlb200.check(L.dlb_indrnn_backward_walk(ctx.h, E.ptr, Zd.ptr, A.ptr, C.byref(ua), ud.ptr, af, T, B, n))
    daf = np.empty_like(dA)
    for t in range(T - 1, -1, -1):
        fp = fc_step.af_derive(af, pre[t], h[t])
        dd = (dA[t] * fp).astype(f32)
        daf[t] = dd if t == T - 1 else (dd + u_rec * fp * daf[t + 1]).astype(f32)
    got_e = E.get()
    kink = np.abs(pre) < 1e-6
    assert util.rel_l2(np.where(kink, 0, got_e), np.where(kink, 0, daf)) <= 2e-6
    # sums
    sums = ctx.empty((5, T, n), dtype=np.float64)
    dlb200.check(L.dlb_indrnn_backward_sums(ctx.h, E.ptr, Zd.ptr, A.ptr, C.byref(ua), 1, T, B, n, sums.ptr))
    e = got_e.astype(np.float64)
    want = np.zeros((5, T, n))
    want[0] = (e * xh).sum(1)
    want[1] = e.sum(1)
    eh = e * gamma
    want[2] = (eh * (-r / sigma)[:, None]).sum(1)
    want[3] = (eh * (Z - mean[:, None]) * (-r / (sigma * sigma))[:, None]).sum(1)
    want[4, 1:] = (got_h[:-1].astype(np.float64) * e[1:]).sum(1)
    got_s = sums.get()
    for s in range(5):
        assert np.allclose(got_s[s], want[s], rtol=2e-5, atol=2e-5 * np.abs(want[s]).max() + 1e-12), s
    # fold over time
    out = ctx.array(np.ones(n, np.float32))
    dlb200.check(L.dlb_time_fold(ctx.h, sums.offset(4 * T * n), T, n, out.ptr))
    assert np.allclose(out.get(), 1 + got_s[4].sum(0), rtol=1e-6, atol=1e-6)
    # apply
    delta_lo = ctx.empty((T, B, n))
    dlb200.check(L.dlb_brn_time_backward_apply(ctx.h, E.ptr, delta_lo.ptr, Zd.ptr, C.byref(ua), sums.ptr, B, T, B, n))
    N = f32(B)
    dx = (got_e * gamma * (r / sigma)[:, None]).astype(f32)
    dx = dx + got_s[3].astype(f32)[:, None] * ((Z - mean[:, None]) / (N * sigma[:, None]))
    dx = dx + got_s[2].astype(f32)[:, None] * (f32(1) / N)
    got_dx = E.get()
    assert util.rel_l2(got_dx, dx) <= 2e-6
    if ctx.gemm_kind() != 0:
        # The apply again on the same buffers (its own output as the error this
        # time): the planes it now writes itself hold what it wrote to the tensor.
        dlb200.check(L.dlb_brn_time_backward_apply(ctx.h, E.ptr, delta_lo.ptr, Zd.ptr, C.byref(ua), sums.ptr, B, T, B, n))
        again = E.get()
        planes = delta_lo.get().ravel().view(np.float16).astype(np.float64)
        ratio = (planes[:again.size] + planes[again.size:]) / np.where(again.ravel() == 0, 1, again.ravel())
        live = np.abs(again.ravel()) > 2.0 ** -10 * np.abs(again).max()
        scale = np.median(ratio[live])
        assert scale == 2.0 ** np.round(np.log2(scale))
        assert np.allclose(ratio[live], scale, rtol=2.0 ** -20, atol=0)
    assert ctx.sync() == 0


@pytest.mark.parametrize("T,B,n", [(4, 8, 64), (3, 5, 7)])
def test_time_major_sums_and_clamp(gpu_ctx, T, B, n):
    ctx, L = gpu_ctx, gpu_ctx.L
    rng = np.random.default_rng(T + n)
    x = rng.standard_normal((B, T * n)).astype(np.float32)
    out, lo = ctx.empty((T, B, n)), ctx.empty((T, B, n))
    xd = ctx.array(x)   # kept alive: a temporary would be freed before the kernel reads it
    dlb200.check(L.dlb_time_major(ctx.h, xd.ptr, out.ptr, lo.ptr, B, T, n))
    want = x.reshape(B, T, n).transpose(1, 0, 2)
    assert np.array_equal(out.get(), want)
    sums = ctx.empty((2, T, n), dtype=np.float64)
    dlb200.check(L.dlb_brn_time_forward_sums(ctx.h, out.ptr, T, B, n, sums.ptr))
    got = sums.get()
    assert np.allclose(got[0], want.astype(np.float64).sum(1), rtol=1e-5, atol=1e-5)
    assert np.allclose(got[1], (want.astype(np.float64) ** 2).sum(1), rtol=1e-5, atol=1e-5)
    u = ctx.array(np.linspace(-2, 2, n).astype(np.float32))
    dlb200.check(L.dlb_indrnn_clamp(ctx.h, u.ptr, n, -1.25, 1.25))
    assert np.array_equal(u.get(), np.clip(np.linspace(-2, 2, n).astype(np.float32), -1.25, 1.25))
    assert ctx.sync() == 0


@pytest.mark.parametrize("kind", [LAYER_DROPOUT.BERNOULLI, LAYER_DROPOUT.BERNOULLI_INVERTED], ids=["plain", "inverted"])
@pytest.mark.parametrize("norm", [True, False], ids=["brn", "no_norm"])
def test_bernoulli_dropout_through_time(gpu_ctx, kind, norm):
    """A mask per time step on the stored outputs (the recurrence reads the masked
    value), training and inference, against the CPU restatement (itself pinned
    to the compiled reference)."""
    cfg = configs.indrnn_stack(n_in=64, hidden=128, depth=2, n_out=32, seq_w=6, batch=32, norm=norm,
                               dropout=(kind, 0.7))
    B, last = cfg["batch"], len(cfg["layers"]) - 1
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    p0 = _kink_free(cfg, X)
    ora = util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0)
    mod = util.build(dlb200.Model(gpu_ctx), cfg, params=p0)
    want = util.trace(ora, cfg, 1, X, Y, masks)
    got = util.trace(mod, cfg, 1, X, Y, masks)
    assert gpu_ctx.sync() == 0
    _check(got, want)
    assert not got["act1"].reshape(6, B, 128)[:, :, masks[1].reshape(6, 128)[0] == 0][0].any()
    util.copy_trained_state(mod, ora, cfg)
    out = []
    for m in (ora, mod):
        m.set_propagation(0)
        m.forward_pass(B, X)
        out.append(m.get_layer_outputs(last, B).reshape(-1))
    assert util.rel_l2(out[1], out[0]) <= 1e-5


@pytest.mark.parametrize("kind", [2, 3], ids=["plain", "inverted"])
def test_dropout_on_the_inputs_of_a_time_stepped_model(gpu_ctx, kind):
    """The input layer's Bernoulli dropout masks the model's copy of the batch per
    time step and unit (training), or scales it by the keep probability
    (inference, plain kind), against the CPU restatement (pinned to the compiled
    reference)."""
    cfg = configs.indrnn_stack(n_in=64, hidden=128, depth=2, n_out=32, seq_w=6, batch=32)
    cfg["layers"][0] = dict(cfg["layers"][0], dropout=(kind, 0.6))
    B, last = cfg["batch"], len(cfg["layers"]) - 1
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    assert 0 in masks and not masks[0].all()
    p0 = _kink_free(cfg, X)
    ora = util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0)
    mod = util.build(dlb200.Model(gpu_ctx), cfg, params=p0)
    want = util.trace(ora, cfg, 2, X, Y, masks)
    got = util.trace(mod, cfg, 2, X, Y, masks)
    assert gpu_ctx.sync() == 0
    for key in ("act1", "act3", "delta1", "grads", "params1", "losses"):
        assert util.rel_l2(got[key], want[key]) <= (1e-4 if key == "params1" else 2e-5), key
    util.copy_trained_state(mod, ora, cfg)
    out = []
    for m in (ora, mod):
        m.set_propagation(0)
        m.forward_pass(B, X)
        out.append(m.get_layer_outputs(last, B).reshape(-1))
    assert util.rel_l2(out[1], out[0]) <= 1e-5


def test_uout_in_a_time_stepped_model(gpu_ctx):
    """UOut on IndRNN layers: the output of a time step becomes h + h * draw before
    the next step's recurrence reads it; draws [seq_w * rows, units] are inputs of
    the step (the restatement is pinned to the compiled reference with the
    reference's own draws in tests/test_oracle_indrnn.py).  Without draws the step
    is refused."""
    T, B, H = 4, 32, 128
    cfg = configs.indrnn_stack(n_in=64, hidden=H, depth=2, n_out=32, seq_w=T, batch=B,
                               dropout=(LAYER_DROPOUT.UOUT, 0.25))
    X, Y = configs.synthetic_batch(cfg)
    p0 = _kink_free(configs.indrnn_stack(n_in=64, hidden=H, depth=2, n_out=32, seq_w=T, batch=B), X)
    rng = np.random.default_rng(5)
    noise = {li: ((rng.random((T * B, H)) * 2 - 1) * 0.25).astype(np.float32) for li in (1, 2)}
    out = []
    for model in (util.build(fc_indrnn.IndRnnOracleModel(), cfg, params=p0),
                  util.build(dlb200.Model(gpu_ctx), cfg, params=p0)):
        for li, nz in noise.items():
            model.set_uout_noise(li, nz)
        out.append(util.trace(model, cfg, 1, X, Y))
    assert gpu_ctx.sync() == 0
    _check(out[1], out[0])
    bare = util.build(dlb200.Model(gpu_ctx), cfg, params=p0)
    with pytest.raises(dlb200.DlbError):
        bare.forward_pass(B, X)


def test_indrnn_100_steps_vs_compiled_reference(gpu_ctx):
    """An unpicked weight seed, 100 steps: every tensor of the first step and the
    weights after 100 steps agree with the compiled reference (OpenMP mode) to the
    bar, or to three times what the reference's own serial and OpenMP modes differ
    by on the same tensor where a branch of the ReLU derivative or the order of its
    sums decides."""
    import ref_binding
    if not ref_binding.available():
        pytest.skip("oracle/_ref not built on this machine")
    cfg = configs.indrnn_stack(n_in=64, hidden=128, depth=2, n_out=32, seq_w=8, batch=32)
    serial = util.build(ref_binding.RefModel(), dict(cfg, mp=False), seed=0)
    configs.set_recurrent_uniform(serial, cfg)
    p0 = serial.get_array("parameters")
    ws = util.trace(serial, dict(cfg, mp=False), steps=100)
    want = util.trace(util.build(ref_binding.RefModel(), dict(cfg, mp=True), params=p0), cfg, steps=100)
    got = util.trace(util.build(dlb200.Model(gpu_ctx), cfg, params=p0), cfg, steps=100)
    assert gpu_ctx.sync() == 0
    drift = {k: v[0] for k, v in util.compare(ws, want).items()}
    cmp = util.compare(got, want)
    print({k: f"{v[0]:.2e} (reference against itself {drift[k]:.2e})" for k, v in cmp.items()})
    for key, (l2, _) in cmp.items():
        if key.startswith("mean_average"):
            continue   # running means of units centred on zero: no scale for a relative error
        base = 1e-4 if key in ("params_last", "losses") else (TOL_PARAMS if key.startswith("params") else TOL_1)
        assert l2 <= max(base, 3 * drift[key]), f"{key}: {l2:.2e}, reference against itself {drift[key]:.2e}"
