"""Range guard of the 3xFP16 operand form.

The fp16 planes of a tensor share one power-of-two scale, so a row or column
whose every element is far below the tensor's largest keeps fewer than fp32's
bits.  The splits record the largest |x| of every row and column; a tensor with
a non-zero line maximum below 2^-21 of its own maximum (or with a value beyond
the scale predicted from its previous split) is flagged, the tensor-core kernel
skips the products that read it and an fp32 CUDA-core kernel computes them.
Checked here with the library's default settings, through the C ABI:

* operands whose rows (or columns) span 2^-20 .. 2^20: every row and column of
  the three FC products is within 1e-5 of the float64 product in its own norm,
  and the counters show that the guard acted;
* operands spread over 2^-9 .. 2^9 stay on the tensor cores and meet the same bar;
* error tensors taken from a model after 100 training steps are not flagged and
  their products meet the bar row by row;
* a tensor that grows a hundredfold between two splits of the same buffer
  (beyond the headroom of the predicted scale) is caught for that split and
  back on the tensor cores at the next.
"""
import numpy as np
import pytest

import configs
import dlb200
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
    assert fell1 - fell0 == 2, "the two products that read it ran on the fp32 kernel"


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
    split before (one pass instead of two).  A tensor that outgrows its headroom
    is flagged for that split only."""
    ctx, L = gpu_ctx, gpu_ctx.L
    rng = np.random.default_rng(5)
    B, I, H = 256, 512, 256
    x = rng.standard_normal((B, I), dtype=np.float32)
    w = (rng.standard_normal((H, I), dtype=np.float32) / 16).astype(np.float32)
    wd, wl = _split(ctx, w)
    xd, xl = ctx.array(x), ctx.empty(x.shape)
    z = ctx.empty((B, H))
    want = x.astype(np.float64) @ w.astype(np.float64).T
    fell = []
    for factor in (1.0, 1.5, 100.0, 1.0):
        xd.set(x * np.float32(factor))
        before = ctx.guard_counters()[1]
        check(L.dlb_split_planes_2d(ctx.h, xd.ptr, xl.ptr, B, I), "split")
        check(L.dlb_fc_forward(ctx.h, xd.ptr, xl.ptr, wd.ptr, wl.ptr, None, z.ptr, B, I, H), "forward")
        got = z.get()
        assert ctx.sync() == 0
        fell.append(ctx.guard_counters()[1] - before)
        assert util.rowwise_rel_l2(got, want * factor) <= ROW_BAR, f"factor {factor}"
    assert fell == [0, 0, 1, 0], fell
