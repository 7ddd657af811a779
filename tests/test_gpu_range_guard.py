"""Range guard of the 3xFP16 operand form.

The fp16 planes of a tensor share one power-of-two scale, so a row or column
whose every element is far below the tensor's largest keeps fewer than fp32's
bits.  The splits record the largest |x| of every row and column; a tensor with
a non-zero row (column) maximum below 2^-21 of its own maximum has its row
(column) flag set, a value beyond the scale predicted from its previous split
sets the overflow flag.  A product looks at the overflow flag and at the flag of
each operand's free dimension (small lines along the contraction are added to
the large ones and cost nothing); with a flag set the tensor-core kernel skips
the product and an fp32 CUDA-core kernel computes it.
Checked here with the library's default settings, through the C ABI:

* operands whose rows (or columns) span 2^-20 .. 2^20: every row and column of
  the three FC products is within 1e-5 of the float64 product in its own norm,
  the product that has the spread lines on its output side ran on the fp32
  kernel and the one that sums over them stayed on the tensor cores;
* operands spread over 2^-9 .. 2^9 stay on the tensor cores and meet the same bar;
* error tensors taken from a model after 100 training steps are not flagged and
  their products meet the bar row by row;
* a tensor that grows a hundredfold between two splits of the same buffer
  (beyond the headroom of the predicted scale) has its planes written a second
  time with its own scale and its products stay on the tensor cores;
* a classifier that has learnt most of its batch: the errors of the examples it
  gets right are 2^-20 and less of the largest error; inside a model those rows
  are not guarded (they reach the weights only through sums over the batch),
  the input-gradient products stay on the tensor cores and the weights are those
  of a run with every row guarded.
"""
import numpy as np
import pytest

import configs
import dlb200
import enums
import util
from dlb200 import check

pytestmark = pytest.mark.gpu

ROW_BAR = 1e-5


def _split(ctx, host):
    dev = ctx.array(host)
    planes = ctx.empty(host.shape)
    check(ctx.L.dlb_split_planes_2d(ctx.h, dev.ptr, planes.ptr, host.shape[0], host.shape[1]), "dlb_split_planes_2d")
    return dev, planes


def _products(ctx, x, w, d):
    """forward x w^T, input gradient d w, weight gradient d^T x on the device and in float64."""
    L = ctx.L
    B, I = x.shape
    H = w.shape[0]
    (xd, xl), (wd, wl), (dd, dl) = _split(ctx, x), _split(ctx, w), _split(ctx, d)
    z, dx, dw = ctx.empty((B, H)), ctx.empty((B, I)), ctx.empty((H, I))
    check(L.dlb_fc_forward(ctx.h, xd.ptr, xl.ptr, wd.ptr, wl.ptr, None, z.ptr, B, I, H), "forward")
    check(L.dlb_fc_backward_input(ctx.h, dd.ptr, dl.ptr, wd.ptr, wl.ptr, dx.ptr, B, I, H), "input gradient")
    check(L.dlb_fc_weight_gradient(ctx.h, dd.ptr, dl.ptr, xd.ptr, xl.ptr, dw.ptr, None, B, I, H, 0), "weight gradient")
    got = (z.get(), dx.get(), dw.get())
    assert ctx.sync() == 0
    x64, w64, d64 = (a.astype(np.float64) for a in (x, w, d))
    return got, (x64 @ w64.T, d64 @ w64, d64.T @ x64)


def _worst_lines(got, want):
    return max(util.rowwise_rel_l2(got, want), util.rowwise_rel_l2(got.T, want.T))


def _operands(rng, B=512, I=1024, H=1024):
    x = rng.standard_normal((B, I), dtype=np.float32)
    w = (rng.standard_normal((H, I), dtype=np.float32) / 32).astype(np.float32)
    d = (rng.standard_normal((B, H), dtype=np.float32) * 1e-4).astype(np.float32)
    return x, w, d


def _spread(rng, n, log2_span):
    return np.exp2(rng.uniform(-log2_span, log2_span, n)).astype(np.float32)


@pytest.mark.parametrize("which", ["x_rows", "d_rows", "w_rows", "d_columns", "x_columns"])
def test_lines_spanning_forty_octaves(gpu_ctx, which):
    assert gpu_ctx.gemm_kind() == 1, "the guard belongs to the default (3xFP16) form"
    rng = np.random.default_rng(3)
    x, w, d = _operands(rng)
    if which == "x_rows":
        x *= _spread(rng, x.shape[0], 20)[:, None]
    elif which == "d_rows":
        d *= _spread(rng, d.shape[0], 20)[:, None]
    elif which == "w_rows":
        w *= _spread(rng, w.shape[0], 20)[:, None]
    elif which == "d_columns":
        d *= _spread(rng, d.shape[1], 20)[None, :]
    else:
        x *= _spread(rng, x.shape[1], 20)[None, :]
    flagged0, fell0 = gpu_ctx.guard_counters()
    got, want = _products(gpu_ctx, x, w, d)
    flagged1, fell1 = gpu_ctx.guard_counters()
    for name, g, t in zip(("forward", "input gradient", "weight gradient"), got, want):
        worst = _worst_lines(g, t)
        print(f"{which} {name}: worst row or column {worst:.2e}, rel_l2 {util.rel_l2(g, t):.2e}")
        assert worst <= ROW_BAR, f"{which} {name}: {worst:.2e}"
    assert flagged1 - flagged0 == 1, "exactly the spread operand is flagged"
    assert fell1 - fell0 == 1, "of the two products that read it, the one with the spread lines on its output side"


def test_moderate_spread_stays_on_the_tensor_cores(gpu_ctx):
    rng = np.random.default_rng(4)
    x, w, d = _operands(rng)
    x *= _spread(rng, x.shape[0], 9)[:, None]
    d *= _spread(rng, d.shape[1], 9)[None, :]
    before = gpu_ctx.guard_counters()
    got, want = _products(gpu_ctx, x, w, d)
    assert gpu_ctx.guard_counters() == before
    for name, g, t in zip(("forward", "input gradient", "weight gradient"), got, want):
        worst = _worst_lines(g, t)
        print(f"{name}: worst row or column {worst:.2e}")
        assert worst <= ROW_BAR, f"{name}: {worst:.2e}"


def test_error_tensors_of_a_trained_model(gpu_ctx):
    """Errors and activations after 100 steps of the reduced deep MLP: nothing is
    flagged during training, and the products of the trained tensors meet the
    row bar."""
    cfg = configs.deep_brn_mlp(256, 512, 2, 256, 256)
    X, Y = configs.synthetic_batch(cfg)
    B = cfg["batch"]
    model = util.build(dlb200.Model(gpu_ctx), cfg, seed=2)
    for li, mk in configs.dropout_masks(cfg).items():
        model.set_dropout_mask(li, mk)
    before = gpu_ctx.guard_counters()
    for _ in range(100):
        model.train_step(B, X, Y)
    model.forward_pass(B, X)
    model.compute_error(B, Y)
    model.backward_pass(B)
    assert gpu_ctx.sync() == 0
    assert gpu_ctx.guard_counters() == before, "no operand of an ordinary training run is flagged"
    p = model.get_array("parameters")
    for li in (2, 3):
        info = model.layer_info(li)
        fan_in = model.layer_info(li - 1)["n_out"]
        w = p[info["first_connection"]:info["first_connection"] + info["n_out"] * fan_in].reshape(info["n_out"], fan_in)
        x = model.get_layer_outputs(li - 1, B).reshape(B, -1)
        d = model.get_layer_errors(li, B).reshape(B, -1)
        spans = []
        for t in (x, d, w):
            for axis in (0, 1):
                line = np.abs(t).max(axis=axis)
                line = line[line > 0]
                spans.append(float(np.log2(line.max() / line.min())))
        got, want = _products(gpu_ctx, x, w, d)
        for name, g, t in zip(("forward", "input gradient", "weight gradient"), got, want):
            worst = _worst_lines(g, t)
            print(f"layer {li} {name}: worst row or column {worst:.2e}; largest line span 2^{max(spans):.1f}")
            assert worst <= ROW_BAR, f"layer {li} {name}: {worst:.2e}"
    assert gpu_ctx.guard_counters() == before


def test_growth_beyond_the_predicted_scale(gpu_ctx):
    """The second and later splits of a buffer use the scale predicted from the
    split before (one pass instead of two).  A tensor that has outgrown the
    headroom of that scale is split a second time by the check behind the split,
    with the scale of its own maximum: nothing is flagged."""
    ctx, L = gpu_ctx, gpu_ctx.L
    rng = np.random.default_rng(5)
    B, I, H = 256, 512, 256
    x = rng.standard_normal((B, I), dtype=np.float32)
    w = (rng.standard_normal((H, I), dtype=np.float32) / 16).astype(np.float32)
    wd, wl = _split(ctx, w)
    xd, xl = ctx.array(x), ctx.empty(x.shape)
    z = ctx.empty((B, H))
    want = x.astype(np.float64) @ w.astype(np.float64).T
    fell, again = [], []
    for factor in (1.0, 1.5, 100.0, 1.0):
        xd.set(x * np.float32(factor))
        before, r0 = ctx.guard_counters()[1], ctx.guard_resplits()
        check(L.dlb_split_planes_2d(ctx.h, xd.ptr, xl.ptr, B, I), "split")
        check(L.dlb_fc_forward(ctx.h, xd.ptr, xl.ptr, wd.ptr, wl.ptr, None, z.ptr, B, I, H), "forward")
        got = z.get()
        assert ctx.sync() == 0
        fell.append(ctx.guard_counters()[1] - before)
        again.append(ctx.guard_resplits() - r0)
        assert util.rowwise_rel_l2(got, want * factor) <= ROW_BAR, f"factor {factor}"
    assert fell == [0, 0, 0, 0], fell
    assert again == [0, 0, 1, 0], again


def test_producer_written_planes_outgrowing_their_scale_are_split_again(gpu_ctx):
    """A product whose epilogue writes the planes of the activation uses the
    scale predicted from that tensor's previous split.  When the tensor has grown
    a hundredfold the check behind the product writes the planes a second time
    with the tensor's own scale: the next product stays on the tensor cores and
    is right row by row."""
    ctx, L = gpu_ctx, gpu_ctx.L
    rng = np.random.default_rng(6)
    B, I, H = 256, 512, 512
    x0 = rng.standard_normal((B, I), dtype=np.float32)
    w1 = (rng.standard_normal((H, I), dtype=np.float32) / 16).astype(np.float32)
    w2 = (rng.standard_normal((I, H), dtype=np.float32) / 16).astype(np.float32)
    (w1d, w1l), (w2d, w2l) = _split(ctx, w1), _split(ctx, w2)
    xd, xl = ctx.array(x0), ctx.empty(x0.shape)
    z, a, al, out = ctx.empty((B, H)), ctx.empty((B, H)), ctx.empty((B, H)), ctx.empty((B, I))
    resplit, fell = [], []
    for factor in (1.0, 1.0, 100.0, 1.0):
        xd.set(x0 * np.float32(factor))
        check(L.dlb_split_planes_2d(ctx.h, xd.ptr, xl.ptr, B, I), "split")
        assert ctx.sync() == 0
        f0, r0 = ctx.guard_counters()[1], ctx.guard_resplits()
        # a = x w1^T (linear activation, no dropout) with its planes, then a w2^T
        check(L.dlb_fc_forward_activation(ctx.h, xd.ptr, xl.ptr, w1d.ptr, w1l.ptr, None, z.ptr, enums.ACTIVATION.LINEAR,
                                          None, a.ptr, al.ptr, B, I, H), "forward + activation")
        check(L.dlb_fc_forward(ctx.h, a.ptr, al.ptr, w2d.ptr, w2l.ptr, None, out.ptr, B, H, I), "forward")
        got = out.get()
        assert ctx.sync() == 0
        fell.append(ctx.guard_counters()[1] - f0)
        resplit.append(ctx.guard_resplits() - r0)
        a64 = (x0.astype(np.float64) * factor) @ w1.astype(np.float64).T
        want = a64.astype(np.float32).astype(np.float64) @ w2.astype(np.float64).T
        assert util.rowwise_rel_l2(got, want) <= ROW_BAR, f"factor {factor}"
    assert resplit == [0, 0, 1, 0], resplit
    assert fell == [0, 0, 0, 0], fell


def test_errors_of_a_classifier_that_has_learnt_its_batch(gpu_ctx):
    # With this learning rate the softmax saturates within a few steps: the rows
    # of most examples are then 2^-21 .. 2^-100 of the largest, in the output
    # error and in the hidden layer's.  (The logits are in the tens by then, so
    # the weights are no longer comparable with another implementation's to
    # 1e-5: a rounding of the logit moves exp(logit) by the logit's size times
    # as much.  The library is compared with itself, guard strict and not.)
    cfg = configs.mlp_softmax(512, 1024, 64, 256)
    cfg["hparams"] = dict(cfg["hparams"], adam_learning_rate=1e-2)
    X, Y = configs.synthetic_batch(cfg)
    B, steps = cfg["batch"], 6
    p0 = util.build(dlb200.Model(gpu_ctx), cfg, seed=0).get_array("parameters")
    runs = {}
    try:
        for name, strict in (("default", False), ("strict", True)):
            gpu_ctx.set_guard_strict(strict)
            model = util.build(dlb200.Model(gpu_ctx), cfg, params=p0)
            model.train_begin(B)
            before = gpu_ctx.guard_counters()
            for _ in range(steps):
                model.train_step(B, X, Y)
            assert gpu_ctx.sync() == 0
            flagged, fell = (a - b for a, b in zip(gpu_ctx.guard_counters(), before))
            model.reset_loss()
            model.forward_pass(B, X)
            model.compute_error(B, Y)
            model.backward_pass(B)
            rows = np.abs(model.get_layer_errors(2, B).reshape(B, -1)).max(axis=1)
            small = int((rows < rows.max() * 2.0 ** -21).sum())
            print(f"{name}: loss {model.get_loss():.3g}; {small} of {B} error rows below 2^-21 of the largest; "
                  f"{flagged} tensors flagged, {fell} products on the fp32 kernel in {steps} steps")
            runs[name] = (model.get_array("parameters"), small, fell)
    finally:
        gpu_ctx.set_guard_strict(False)
    # The case is the one meant.
    assert runs["default"][1] >= B // 4
    # Guarded, the small rows send the input-gradient product of every step to the
    # fp32 kernel; exempt, what is left are the products whose output rows are
    # small columns of an error (a class or a unit with only small errors).
    assert runs["default"][2] < runs["strict"][2]
    assert runs["default"][2] <= 2 * steps
    # ... and the weights do not notice beyond what a change of kernel costs: the
    # guarded run forms whole input-gradient products on the fp32 kernel, every
    # row of which then differs in its last bits, and the saturated model carries
    # such differences forward (the reference's serial and OpenMP builds are 2e-6
    # apart after these six steps and 4e-5 after eleven).
    apart = util.rel_l2(runs["default"][0], runs["strict"][0])
    print(f"weights after {steps} steps, exempt against strict: {apart:.1e}")
    assert apart <= 1e-5
