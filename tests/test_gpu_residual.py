"""Residual blocks with ShakeDrop on the GPU, through the Model entry points of
the C ABI: against the committed fixture of the compiled reference and against
the CPU restatement on a shape whose products run on the tensor-core kernel."""
import numpy as np
import pytest

import configs
import dlb200
import fc_residual
import golden_io
import ref_binding
import util

pytestmark = pytest.mark.gpu

TOL_1 = 1e-5       # activations, errors, gradients after one step (rel_l2)
TOL_PARAMS = 1e-4  # updated weights: Adam's first step magnifies gradients of the order of eps


def _check(got, want, skip=()):
    for key, (l2, mx) in util.compare(got, want).items():
        if key in skip:
            continue
        tol = TOL_PARAMS if key.startswith("params") else TOL_1
        assert l2 <= tol, f"{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"


@pytest.mark.parametrize("name", sorted(golden_io.NOISY_CASES))
def test_residual_model_matches_golden(gpu_ctx, name):
    cfg, steps, X, Y, draws, p0, want = golden_io.load_noisy(name)
    model = util.build(dlb200.Model(gpu_ctx), cfg, params=p0)
    got = util.trace_noisy(model, cfg, steps, X, Y, draws)
    assert gpu_ctx.sync() == 0
    _check(got, want)


@pytest.mark.skipif(not ref_binding.available(), reason="ShakeDrop draws come from oracle/_ref")
def test_residual_model_vs_restatement_tensor_core_shape(gpu_ctx):
    cfg = configs.residual_mlp(width=256, blocks=2, n_out=10, batch=256)
    X, Y = configs.synthetic_batch(cfg)
    draws = [util.shakedrop_step_draws(cfg, s) for s in range(3)]

    def prepare(model):
        util.set_step_noise(model, cfg, 0, draws[0])

    p0, seed = util.kink_free_parameters(cfg, fc_residual.ResidualOracleModel, X, {}, scale=1.0 / 16,
                                         prepare=prepare)
    want = util.trace_noisy(util.build(fc_residual.ResidualOracleModel(), cfg, params=p0), cfg, 1, X, Y, draws)
    got = util.trace_noisy(util.build(dlb200.Model(gpu_ctx), cfg, params=p0), cfg, 1, X, Y, draws)
    assert gpu_ctx.sync() == 0
    _check(got, want)
    # Later steps may meet a derivative jump; only the scale of the agreement is checked.
    want = util.trace_noisy(util.build(fc_residual.ResidualOracleModel(), cfg, params=p0), cfg, 3, X, Y, draws)
    got = util.trace_noisy(util.build(dlb200.Model(gpu_ctx), cfg, params=p0), cfg, 3, X, Y, draws)
    assert gpu_ctx.sync() == 0
    assert util.rel_l2(got["params_last"], want["params_last"]) <= 1e-3
    assert util.rel_l2(got["losses"], want["losses"]) <= 1e-4


@pytest.mark.skipif(not ref_binding.available(), reason="ShakeDrop draws come from oracle/_ref")
def test_residual_evaluation_pass(gpu_ctx):
    """Inference through residual blocks (running averages, block output of a
    ShakeDrop layer times 1 - p), loss and accuracy, against the CPU restatement
    from the same trained state."""
    cfg = configs.residual_mlp(width=256, blocks=2, n_out=10, batch=256)
    B, last = cfg["batch"], len(cfg["layers"]) - 1
    X, Y = configs.synthetic_batch(cfg)
    Xe, Ye = configs.synthetic_batch(dict(cfg, data_seed=5))
    draws = [util.shakedrop_step_draws(cfg, s) for s in range(2)]
    mod = util.build(dlb200.Model(gpu_ctx), cfg, seed=4)   # Glorot draws of the library
    ora = util.build(fc_residual.ResidualOracleModel(), cfg, params=mod.get_array("parameters"))
    util.trace_noisy(mod, cfg, 2, X, Y, draws)
    util.copy_trained_state(mod, ora, cfg)
    out = []
    for m in (ora, mod):
        m.train_begin(B)
        m.set_propagation(0)
        m.set_accu_fn(1)   # CROSS_ENTROPY
        m.reset_loss()
        m.forward_pass(B, Xe)
        m.compute_loss(B, Ye)
        out.append((m.get_loss(), m.get_accu(B), m.get_layer_outputs(last, B).reshape(B, -1)))
        m.set_propagation(1)
    (lo, ao, qo), (lg, ag, qg) = out
    assert gpu_ctx.sync() == 0
    assert util.rel_l2(qg, qo) <= 1e-5
    assert abs(lg - lo) <= 1e-5 * abs(lo)
    assert abs(ag - ao) <= 100.0 * 2 / B
    # Training goes on from the same state afterwards.
    util.trace_noisy(mod, cfg, 1, X, Y, draws)
    assert gpu_ctx.sync() == 0


def test_residual_kernels(gpu_ctx):
    ctx, L = gpu_ctx, gpu_ctx.L
    rng = np.random.default_rng(9)
    for rows, width in ((64, 128), (33, 10)):
        x = rng.standard_normal((rows, width), dtype=np.float32)
        block = rng.standard_normal((rows, width), dtype=np.float32)
        mask = (rng.random(rows) < 0.5).astype(np.uint8)
        noise = (rng.random((rows, width)) * 2 - 1).astype(np.float32)
        xd, bd, md, nd = ctx.array(x), ctx.array(block), ctx.array(mask), ctx.array(noise)
        out, lo = ctx.empty((rows, width)), ctx.empty((rows, width))
        dlb200.check(L.dlb_residual_forward(ctx.h, xd.ptr, bd.ptr, md.ptr, nd.ptr, out.ptr, lo.ptr, rows, width))
        pert = np.where(mask[:, None] != 0, block * noise, block)
        assert np.array_equal(bd.get(), pert)            # perturbed in place
        assert np.array_equal(out.get(), x + pert)
        d = rng.standard_normal((rows, width), dtype=np.float32)
        dd, delta = ctx.array(d), ctx.empty((rows, width))
        dlb200.check(L.dlb_shakedrop_backward(ctx.h, dd.ptr, md.ptr, nd.ptr, delta.ptr, None, rows, width))
        assert np.array_equal(delta.get(), np.where(mask[:, None] != 0, d * noise, d))
        dlb200.check(L.dlb_shakedrop_backward(ctx.h, dd.ptr, None, None, delta.ptr, None, rows, width))
        assert np.array_equal(delta.get(), d)
    assert ctx.sync() == 0


@pytest.mark.skipif(not ref_binding.available(), reason="ShakeDrop draws come from oracle/_ref")
@pytest.mark.parametrize("width,block_width", [(128, 192), (192, 128), (130, 136)])
def test_blocks_of_another_width_than_the_shortcut(gpu_ctx, width, block_width):
    """The zero-padded shortcut: the residual output is as wide as the wider of
    shortcut and block, the narrower one enters from column pad on, and each
    reads its window of the error on the way back."""
    cfg = configs.residual_mlp(width=width, blocks=2, n_out=10, batch=128, block_width=block_width)
    X, Y = configs.synthetic_batch(cfg)
    draws = [util.shakedrop_step_draws(cfg, s) for s in range(2)]

    def prepare(model):
        util.set_step_noise(model, cfg, 0, draws[0])

    p0, seed = util.kink_free_parameters(cfg, fc_residual.ResidualOracleModel, X, {}, scale=1.0 / 12,
                                         prepare=prepare)
    want = util.trace_noisy(util.build(fc_residual.ResidualOracleModel(), cfg, params=p0), cfg, 1, X, Y, draws)
    mod = util.build(dlb200.Model(gpu_ctx), cfg, params=p0)
    got = util.trace_noisy(mod, cfg, 1, X, Y, draws)
    assert gpu_ctx.sync() == 0
    _check(got, want)
    assert mod.layer_info(1)["n_out"] == max(width, block_width)


@pytest.mark.parametrize("delay", [0, 2], ids=["all_steps", "last_step"])
@pytest.mark.parametrize("width,block_width", [(256, 256), (128, 192)], ids=["equal", "padded"])
def test_residual_blocks_in_a_time_stepped_model(gpu_ctx, delay, width, block_width):
    """Residual blocks of FC layers with seq_w = 3: statistics, Bernoulli masks
    and ShakeDrop flags of their own per time step, the products over all
    T * rows rows at once; against the CPU restatement (which is pinned to the
    compiled reference in tests/test_oracle_residual.py), ShakeDrop noise as
    arrays of seq_w * rows rows given to both."""
    import fc_residual_time
    from enums import ACTIVATION, LAYER, LAYER_DROPOUT, MODEL
    T, B = 3, 128
    cfg = configs.residual_mlp(width=width, blocks=2, n_out=10, batch=B, block_width=block_width)
    cfg = dict(cfg, model_type=MODEL.RECURRENT, seq_w=T, time_delays=delay)
    for l in cfg["layers"]:
        if l["type"] == LAYER.FULLY_CONNECTED and l.get("norm"):
            l["af"] = ACTIVATION.ISRLU     # a continuous derivative: no branch for two correct sums to differ on
            l["dropout"] = (LAYER_DROPOUT.BERNOULLI, 0.8)
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    rng = np.random.default_rng(11)
    noise = {}
    for li, p in configs.shakedrop_layers(cfg):
        noise[li] = ((rng.random(T * B) < max(p, 0.3)).astype(np.uint8),
                     (rng.random((T * B, block_width)) * 2 - 1).astype(np.float32),
                     rng.random((T * B, block_width)).astype(np.float32))
    ora = util.build(fc_residual_time.ResidualTimeOracleModel(), cfg)
    p0 = ora.get_array("parameters")
    nw = ora.size("total_weights")
    p0[:nw] = (np.random.default_rng(0).standard_normal(nw) / np.sqrt(width)).astype(np.float32)

    def run(model):
        for li, (mk, fw, bw) in noise.items():
            model.set_shakedrop_noise(li, mk, fw, bw)
        return util.trace(model, cfg, 1, X, Y, masks)

    want = run(util.build(fc_residual_time.ResidualTimeOracleModel(), cfg, params=p0))
    got = run(util.build(dlb200.Model(gpu_ctx), cfg, params=p0))
    assert gpu_ctx.sync() == 0
    residual = {f"delta{li}" for li, l in enumerate(cfg["layers"]) if l["type"] == LAYER.RESIDUAL}
    _check(got, want, skip=residual)


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
def test_residual_100_steps_vs_compiled_reference(gpu_ctx):
    """An unpicked weight seed, 100 steps of a residual stack (ShakeDrop with
    probability 0, so that the reference's serial and OpenMP modes see the same
    model): every tensor of the first step and the weights after 100 steps agree
    with the OpenMP reference to the bar, or to three times what the reference's
    two modes differ by on the same tensor."""
    cfg = configs.residual_mlp(width=64, blocks=2, n_out=10, batch=64, p_last=1.0)
    serial = util.build(ref_binding.RefModel(), dict(cfg, mp=False), seed=0)
    p0 = serial.get_array("parameters")
    X, Y = configs.synthetic_batch(cfg)
    noise = {li: (np.zeros(64, np.uint8), np.zeros((64, 64), np.float32), np.zeros((64, 64), np.float32))
             for li, _ in configs.shakedrop_layers(cfg)}
    ws = util.trace(serial, dict(cfg, mp=False), 100, X, Y)
    want = util.trace(util.build(ref_binding.RefModel(), dict(cfg, mp=True), params=p0), cfg, 100, X, Y)
    model = util.build(dlb200.Model(gpu_ctx), cfg, params=p0)
    for li, (mk, fw, bw) in noise.items():
        model.set_shakedrop_noise(li, mk, fw, bw)
    got = util.trace(model, cfg, 100, X, Y)
    assert gpu_ctx.sync() == 0
    skip = {f"delta{li}" for li, l in enumerate(cfg["layers"]) if l["type"] == 9}
    drift = {k: v[0] for k, v in util.compare(ws, want).items()}
    cmp = util.compare(got, want)
    print({k: f"{v[0]:.2e} (reference against itself {drift[k]:.2e})" for k, v in cmp.items() if k not in skip})
    for key, (l2, _) in cmp.items():
        if key in skip or key.startswith("mean_average"):
            continue   # (running means of units centred on zero have no scale for a relative error)
        base = 1e-4 if key in ("params_last", "losses") else (TOL_PARAMS if key.startswith("params") else TOL_1)
        assert l2 <= max(base, 3 * drift[key]), f"{key}: {l2:.2e}, reference against itself {drift[key]:.2e}"
