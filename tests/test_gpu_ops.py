"""Per-kernel parity on the GPU, through the C ABI, against the CPU restatement
(oracle/fc_step.py) on seeded inputs; integer/flag work bit-exact, floating
point within the tolerance written beside each check."""
import ctypes as C

import numpy as np
import pytest

import dlb200
import fc_step
import util
from dlb200 import check

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5     # rel-err bar for activations and gradients after one step
GEMM_TOL = 2e-6    # rel_l2 of a 3xTF32 product against the float64 product


def _fc(ctx, kind, A, Bm, rows, n_in, n_out, tensor_core, bias=None, accumulate=None):
    L = ctx.L
    ctx.set_tensor_core(tensor_core)
    a, b = ctx.array(A), ctx.array(Bm)
    if kind == "fwd":
        out = ctx.zeros((rows, n_out))
        bz = ctx.array(bias) if bias is not None else None
        check(L.dlb_fc_forward(ctx.h, a.ptr, None, b.ptr, None, bz.ptr if bz else None, out.ptr, rows, n_in, n_out))
    elif kind == "dx":
        out = ctx.zeros((rows, n_in))
        check(L.dlb_fc_backward_input(ctx.h, a.ptr, None, b.ptr, None, out.ptr, rows, n_in, n_out))
    else:
        out = ctx.array(accumulate) if accumulate is not None else ctx.zeros((n_out, n_in))
        db = ctx.zeros(n_out) if bias is not None else None
        check(L.dlb_fc_weight_gradient(ctx.h, a.ptr, None, b.ptr, None, out.ptr, db.ptr if db else None, rows,
                                       n_in, n_out, 1 if accumulate is not None else 0))
        assert ctx.sync() == 0
        ctx.set_tensor_core(1)
        return out.get(), (db.get() if db else None)
    assert ctx.sync() == 0
    ctx.set_tensor_core(1)
    return out.get()


def _operands(kind, rows, n_in, n_out, rng):
    if kind == "fwd":
        return rng.standard_normal((rows, n_in), dtype=np.float32), rng.standard_normal((n_out, n_in), dtype=np.float32)
    if kind == "dx":
        return rng.standard_normal((rows, n_out), dtype=np.float32), rng.standard_normal((n_out, n_in), dtype=np.float32)
    return rng.standard_normal((rows, n_out), dtype=np.float32), rng.standard_normal((rows, n_in), dtype=np.float32)


def _exact(kind, A, Bm):
    A, Bm = A.astype(np.float64), Bm.astype(np.float64)
    return A @ Bm.T if kind == "fwd" else (A @ Bm if kind == "dx" else A.T @ Bm)


# rows, n_in, n_out: aligned tiles, k tails (784), partial m/n tiles, and
# shapes only the CUDA-core kernel can take (row pitch not a multiple of 16 B).
SHAPES = [(128, 64, 256), (256, 512, 512), (384, 784, 256), (200, 96, 160), (512, 1024, 1024), (128, 256, 10),
          (37, 19, 7), (1, 4, 4)]


@pytest.mark.parametrize("kind", ["fwd", "dx", "dw"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("tensor_core", [1, 2, 0], ids=["tcgen05-f16x3", "tcgen05-tf32x3", "cuda-core"])
def test_fc_products(gpu_ctx, kind, shape, tensor_core):
    rows, n_in, n_out = shape
    rng = np.random.default_rng(hash((kind, shape)) % 2**32)
    A, Bm = _operands(kind, rows, n_in, n_out, rng)
    want = _exact(kind, A, Bm)
    gpu_ctx.set_gemm_kind(0 if tensor_core == 2 else 1)
    try:
        got = _fc(gpu_ctx, kind, A, Bm, rows, n_in, n_out, min(tensor_core, 1))
    finally:
        gpu_ctx.set_gemm_kind(1)
    if kind == "dw":
        got = got[0]
    assert util.rel_l2(got, want) <= GEMM_TOL
    assert util.rel_max(got, want) <= 5 * GEMM_TOL


def test_fc_forward_bias_and_gradient_accumulate(gpu_ctx):
    rng = np.random.default_rng(3)
    rows, n_in, n_out = 256, 128, 384
    X, W = _operands("fwd", rows, n_in, n_out, rng)
    bias = rng.standard_normal(n_out, dtype=np.float32)
    got = _fc(gpu_ctx, "fwd", X, W, rows, n_in, n_out, 1, bias=bias)
    assert util.rel_l2(got, _exact("fwd", X, W) + bias) <= GEMM_TOL
    delta = rng.standard_normal((rows, n_out), dtype=np.float32)
    start = rng.standard_normal((n_out, n_in), dtype=np.float32)
    dW, db = _fc(gpu_ctx, "dw", delta, X, rows, n_in, n_out, 1, bias=bias, accumulate=start)
    assert util.rel_l2(dW, start + _exact("dw", delta, X)) <= GEMM_TOL
    assert util.rel_l2(db, delta.astype(np.float64).sum(0)) <= GEMM_TOL


def test_weight_gradient_with_output_rows_that_are_no_multiple_of_64(gpu_ctx):
    """1000 classes: TMA cannot tile the mn-contiguous error [rows, 1000] as the
    A operand of delta^T X.  The library makes planes of the error for this
    product, k contiguous and with a scale per class, and the product stays on
    the tensor cores (one tensor-core launch on record, nothing on the fp32
    kernel) within the bar of the other products, row by row as well, although
    every seventh class has errors 2^-30 of the others'."""
    ctx, L = gpu_ctx, gpu_ctx.L
    rng = np.random.default_rng(8)
    rows, n_in, n_out = 1024, 2048, 1000
    q = rng.random((rows, n_out), dtype=np.float32)
    q /= q.sum(axis=1, keepdims=True)
    y = np.zeros((rows, n_out), np.float32)
    y[np.arange(rows), rng.integers(0, n_out, rows)] = 1.0
    delta = ((q - y) / rows).astype(np.float32)
    delta[:, ::7] *= np.float32(2.0 ** -30)
    X = rng.standard_normal((rows, n_in), dtype=np.float32)
    d, x = ctx.array(delta), ctx.array(X)
    dp, xp = ctx.empty(delta.shape), ctx.empty(X.shape)
    check(L.dlb_split_planes_2d(ctx.h, d.ptr, dp.ptr, rows, n_out), "split")
    check(L.dlb_split_planes_2d(ctx.h, x.ptr, xp.ptr, rows, n_in), "split")
    out = ctx.empty((n_out, n_in))
    ctx.gemm_profile(True)
    ctx.gemm_profile_read()
    fell = ctx.guard_counters()[1]
    check(L.dlb_fc_weight_gradient(ctx.h, d.ptr, dp.ptr, x.ptr, xp.ptr, out.ptr, None, rows, n_in, n_out, 0), "dw")
    assert ctx.sync() == 0
    launches, _, _ = ctx.gemm_profile_read()
    ctx.gemm_profile(False)
    assert ctx.guard_counters()[1] == fell
    want = delta.astype(np.float64).T @ X.astype(np.float64)
    got = out.get()
    assert launches == 1, "the product ran on the tensor cores"
    assert util.rel_l2(got, want) <= GEMM_TOL
    assert util.rowwise_rel_l2(got, want) <= 1e-5


@pytest.mark.parametrize("kind", ["fwd", "dx", "dw"])
def test_products_whose_last_wave_is_split_along_k(gpu_ctx, kind):
    """160 output tiles on 148 SMs: the 12 tiles of the last wave are each
    computed by two CTAs (one per half of k) that add into a zeroed output.  The
    output buffer starts with garbage, the result must not depend on it, must
    be the same bits on every run, and bias goes in exactly once."""
    L = gpu_ctx.L
    rng = np.random.default_rng(21)
    if kind == "dw":
        rows, n_in, n_out = 1024, 2560, 2048   # output [n_out, n_in]: 16 x 10 tiles
    elif kind == "dx":
        rows, n_in, n_out = 2048, 2560, 1024   # output [rows, n_in]
    else:
        rows, n_in, n_out = 2048, 1024, 2560   # output [rows, n_out]
    A, Bm = _operands(kind, rows, n_in, n_out, rng)
    want = _exact(kind, A, Bm)
    bias = rng.standard_normal(n_out, dtype=np.float32) if kind == "fwd" else None
    if bias is not None:
        want = want + bias
    a, b = gpu_ctx.array(A), gpu_ctx.array(Bm)
    bz = gpu_ctx.array(bias) if bias is not None else None
    runs = []
    for fill in (7.5, -3.25):
        out = gpu_ctx.array(np.full(want.shape, fill, np.float32))
        if kind == "fwd":
            check(L.dlb_fc_forward(gpu_ctx.h, a.ptr, None, b.ptr, None, bz.ptr, out.ptr, rows, n_in, n_out))
        elif kind == "dx":
            check(L.dlb_fc_backward_input(gpu_ctx.h, a.ptr, None, b.ptr, None, out.ptr, rows, n_in, n_out))
        else:
            check(L.dlb_fc_weight_gradient(gpu_ctx.h, a.ptr, None, b.ptr, None, out.ptr, None, rows, n_in, n_out, 0))
        assert gpu_ctx.sync() == 0
        runs.append(out.get())
    assert np.array_equal(runs[0], runs[1])
    assert util.rel_l2(runs[0], want) <= GEMM_TOL
    assert util.rel_max(runs[0], want) <= 5 * GEMM_TOL


@pytest.mark.parametrize("gemm_kind", [1, 0], ids=["f16x3", "tf32x3"])
def test_products_with_caller_kept_plane_buffers(gpu_ctx, gemm_kind):
    """Plane buffers written by dlb_split_planes (and by a producing entry
    point) are what the products read; operands of very different magnitude
    (errors ~1e-7, weights ~1e-2) keep fp32-faithful precision."""
    L = gpu_ctx.L
    rng = np.random.default_rng(5)
    rows, n_in, n_out = 512, 384, 640
    delta = (rng.standard_normal((rows, n_out)) * 1e-7).astype(np.float32)
    W = (rng.standard_normal((n_out, n_in)) * 0.02).astype(np.float32)
    X = rng.standard_normal((rows, n_in), dtype=np.float32)
    gpu_ctx.set_gemm_kind(gemm_kind)
    try:
        d, w, x = gpu_ctx.array(delta), gpu_ctx.array(W), gpu_ctx.array(X)
        dp, wp, xp = gpu_ctx.empty(delta.shape), gpu_ctx.empty(W.shape), gpu_ctx.empty(X.shape)
        for t, p in ((d, dp), (w, wp), (x, xp)):
            check(L.dlb_split_planes(gpu_ctx.h, t.ptr, p.ptr, t.size))
        z = gpu_ctx.empty((rows, n_out))
        check(L.dlb_fc_forward(gpu_ctx.h, x.ptr, xp.ptr, w.ptr, wp.ptr, None, z.ptr, rows, n_in, n_out))
        dx = gpu_ctx.empty((rows, n_in))
        check(L.dlb_fc_backward_input(gpu_ctx.h, d.ptr, dp.ptr, w.ptr, wp.ptr, dx.ptr, rows, n_in, n_out))
        dw = gpu_ctx.empty((n_out, n_in))
        check(L.dlb_fc_weight_gradient(gpu_ctx.h, d.ptr, dp.ptr, x.ptr, xp.ptr, dw.ptr, None, rows, n_in, n_out, 0))
        # a sub-view of the rows, as the time-stepped model uses for the last steps
        half = rows // 2
        dx2 = gpu_ctx.empty((half, n_in))
        check(L.dlb_fc_backward_input(gpu_ctx.h, d.offset(half * n_out), dp.offset(half * n_out), w.ptr, wp.ptr,
                                      dx2.ptr, half, n_in, n_out))
        assert gpu_ctx.sync() == 0
        assert util.rel_l2(z.get(), _exact("fwd", X, W)) <= GEMM_TOL
        assert util.rel_l2(dx.get(), _exact("dx", delta, W)) <= GEMM_TOL
        assert util.rel_l2(dw.get(), _exact("dw", delta, X)) <= GEMM_TOL
        assert util.rel_l2(dx2.get(), _exact("dx", delta[half:], W)) <= GEMM_TOL
    finally:
        gpu_ctx.set_gemm_kind(1)


@pytest.mark.parametrize("af", [fc_step.AF_LEAKY_RELU, fc_step.AF_SELU, fc_step.AF_ISRLU])
@pytest.mark.parametrize("dropout", [fc_step.DROPOUT_NONE, fc_step.DROPOUT_BERNOULLI, fc_step.DROPOUT_BERNOULLI_INVERTED,
                                     fc_step.DROPOUT_UOUT])
@pytest.mark.parametrize("shape", [(512, 384, 640), (300, 200, 520)], ids=["whole_tiles", "ragged"])
def test_fc_forward_with_activation_in_the_epilogue(gpu_ctx, af, dropout, shape):
    """Bias, activation, dropout and the planes of A formed in the product's
    epilogue (second call: the first split of A's buffer has no scale to predict
    from and takes the two-kernel path) against the two kernels one after the
    other and against float64; the planes written by the epilogue are what the
    next product reads."""
    ctx, L = gpu_ctx, gpu_ctx.L
    rows, n_in, n_out = shape
    rng = np.random.default_rng(af + 7 * dropout)
    X = rng.standard_normal((rows, n_in), dtype=np.float32)
    W = (rng.standard_normal((n_out, n_in)) * 0.05).astype(np.float32)
    W2 = (rng.standard_normal((256, n_out)) * 0.05).astype(np.float32)
    bias = rng.standard_normal(n_out).astype(np.float32)
    mask = (rng.random(n_out) < 0.8).astype(np.uint8)
    noise = ((rng.random((rows, n_out)) * 2 - 1) * 0.1).astype(np.float32)
    x, w, w2, b, md, nd = (ctx.array(t) for t in (X, W, W2, bias, mask, noise))
    xp, wp, w2p = ctx.empty(X.shape), ctx.empty(W.shape), ctx.empty(W2.shape)
    check(L.dlb_split_planes_2d(ctx.h, x.ptr, xp.ptr, rows, n_in))
    check(L.dlb_split_planes_2d(ctx.h, w.ptr, wp.ptr, n_out, n_in))
    check(L.dlb_split_planes_2d(ctx.h, w2.ptr, w2p.ptr, 256, n_out))
    dp = dlb200.DropoutDesc(dropout, 0.8, md.ptr, nd.ptr)
    dpp = C.byref(dp) if dropout else None
    # the two kernels
    z0, a0, a0p = ctx.empty((rows, n_out)), ctx.empty((rows, n_out)), ctx.empty((rows, n_out))
    check(L.dlb_fc_forward(ctx.h, x.ptr, xp.ptr, w.ptr, wp.ptr, b.ptr, z0.ptr, rows, n_in, n_out))
    check(L.dlb_activation_forward(ctx.h, z0.ptr, None, af, dpp, a0.ptr, a0p.ptr, rows, n_out))
    # one call, twice: the second one runs the epilogue
    z1, a1, a1p = ctx.empty((rows, n_out)), ctx.empty((rows, n_out)), ctx.empty((rows, n_out))
    launches = []
    for _ in range(2):
        before = ctx.launch_count()
        check(L.dlb_fc_forward_activation(ctx.h, x.ptr, xp.ptr, w.ptr, wp.ptr, b.ptr, z1.ptr, af, dpp, a1.ptr, a1p.ptr,
                                          rows, n_in, n_out))
        launches.append(ctx.launch_count() - before)
    nxt = ctx.empty((rows, 256))
    check(L.dlb_fc_forward(ctx.h, a1.ptr, a1p.ptr, w2.ptr, w2p.ptr, None, nxt.ptr, rows, n_out, 256))
    assert ctx.sync() == 0
    assert launches[1] < launches[0], "the second call did not take the fused path"
    assert np.array_equal(z1.get(), z0.get())
    assert np.array_equal(a1.get(), a0.get())
    Zx = X.astype(np.float64) @ W.T.astype(np.float64) + bias
    assert util.rel_l2(z1.get(), Zx) <= GEMM_TOL
    want = fc_step.apply_dropout(fc_step.af_fire(af, z1.get()), dropout, 0.8, mask, noise)
    assert util.rel_max(a1.get(), want) <= F32_TOL
    assert util.rel_l2(nxt.get(), a1.get().astype(np.float64) @ W2.T.astype(np.float64)) <= GEMM_TOL


@pytest.mark.parametrize("af", [fc_step.AF_LEAKY_RELU, fc_step.AF_SELU, fc_step.AF_ISRLU])
@pytest.mark.parametrize("shape", [(512, 640, 384), (300, 520, 200)], ids=["whole_tiles", "ragged"])
def test_fc_backward_input_with_the_derivative_in_the_epilogue(gpu_ctx, af, shape):
    """dX = (delta W) f'(Z, A) of the layer below formed in the product's
    epilogue, with the planes of dX, against the three kernels one after the
    other and against float64."""
    ctx, L = gpu_ctx, gpu_ctx.L
    rows, n_in, n_out = shape
    rng = np.random.default_rng(af)
    delta = (rng.standard_normal((rows, n_out)) * 1e-3).astype(np.float32)
    W = (rng.standard_normal((n_out, n_in)) * 0.05).astype(np.float32)
    Zb = rng.standard_normal((rows, n_in), dtype=np.float32)
    Ab = fc_step.af_fire(af, Zb)
    W0 = (rng.standard_normal((n_in, 256)) * 0.05).astype(np.float32)   # the layer below's own weights
    d, w, zb, ab, w0 = (ctx.array(t) for t in (delta, W, Zb, Ab, W0))
    dpl, wp, w0p = ctx.empty(delta.shape), ctx.empty(W.shape), ctx.empty(W0.shape)
    check(L.dlb_split_planes_2d(ctx.h, d.ptr, dpl.ptr, rows, n_out))
    check(L.dlb_split_planes_2d(ctx.h, w.ptr, wp.ptr, n_out, n_in))
    check(L.dlb_split_planes_2d(ctx.h, w0.ptr, w0p.ptr, n_in, 256))
    e0, e0p = ctx.empty((rows, n_in)), ctx.empty((rows, n_in))
    check(L.dlb_fc_backward_input(ctx.h, d.ptr, dpl.ptr, w.ptr, wp.ptr, e0.ptr, rows, n_in, n_out))
    check(L.dlb_activation_backward(ctx.h, e0.ptr, zb.ptr, ab.ptr, None, af, rows, n_in, None))
    e1, e1p = ctx.empty((rows, n_in)), ctx.empty((rows, n_in))
    launches = []
    for _ in range(2):
        before = ctx.launch_count()
        check(L.dlb_fc_backward_input_derivative(ctx.h, d.ptr, dpl.ptr, w.ptr, wp.ptr, zb.ptr, ab.ptr, af, e1.ptr,
                                                 e1p.ptr, rows, n_in, n_out))
        launches.append(ctx.launch_count() - before)
    # the planes of e1 feed the next product down
    nxt = ctx.empty((rows, 256))
    check(L.dlb_fc_backward_input(ctx.h, e1.ptr, e1p.ptr, w0.ptr, w0p.ptr, nxt.ptr, rows, 256, n_in))
    assert ctx.sync() == 0
    assert launches[1] < launches[0], "the second call did not take the fused path"
    assert np.array_equal(e1.get(), e0.get())
    want = (delta.astype(np.float64) @ W.astype(np.float64)) * fc_step.af_derive(af, Zb, Ab)
    assert util.rel_l2(e1.get(), want) <= GEMM_TOL
    assert util.rel_l2(nxt.get(), e1.get().astype(np.float64) @ W0.astype(np.float64)) <= GEMM_TOL


def test_large_k_accumulation_stays_fp32_faithful(gpu_ctx):
    """k = 4096: the chunked drain keeps the tensor core's truncating
    accumulation from growing with k; the product is as close to the exact one
    as an fp32 FMA loop."""
    rng = np.random.default_rng(11)
    X, W = _operands("fwd", 256, 4096, 256, rng)
    want = _exact("fwd", X, W)
    tc = util.rel_l2(_fc(gpu_ctx, "fwd", X, W, 256, 4096, 256, 1), want)
    fma = util.rel_l2(_fc(gpu_ctx, "fwd", X, W, 256, 4096, 256, 0), want)
    assert tc <= GEMM_TOL and tc <= 3 * fma + 1e-7


def test_split_tf32_is_exact_residual(gpu_ctx):
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(100_003) * 10.0 ** rng.integers(-6, 6, 100_003)).astype(np.float32)
    xd, lo = gpu_ctx.array(x), gpu_ctx.empty(x.shape)
    check(gpu_ctx.L.dlb_split_tf32(gpu_ctx.h, xd.ptr, lo.ptr, x.size))
    got = lo.get()
    hi = (x.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)
    resid = x - hi                                   # exact in fp32
    assert (got.view(np.uint32) & np.uint32(0x1FFF)).max() == 0   # a TF32 value
    assert np.all(np.abs(got - resid) <= np.abs(resid) * 2.0 ** -11 + 1e-45)


def _brn_arrays(ctx, n, rng, gamma=None, beta=None):
    host = dict(mean=np.zeros(n, np.float32), sigma=np.ones(n, np.float32),
                mean_average=(0.1 * rng.standard_normal(n)).astype(np.float32),
                sigma_average=(1 + 0.1 * rng.random(n)).astype(np.float32),
                r=np.ones(n, np.float32), d=np.zeros(n, np.float32),
                gamma=gamma if gamma is not None else (1 + 0.2 * rng.standard_normal(n)).astype(np.float32),
                beta=beta if beta is not None else (0.1 * rng.standard_normal(n)).astype(np.float32))
    dev = {k: ctx.array(v) for k, v in host.items()}
    u = dlb200.BrnUnitArrays(**{k: dev[k].ptr for k in dev})
    return host, dev, u


@pytest.mark.parametrize("rows,n", [(512, 256), (300, 130), (64, 7), (4096, 1024)])
def test_batch_renorm_forward(gpu_ctx, rows, n):
    ctx, L = gpu_ctx, gpu_ctx.L
    rng = np.random.default_rng(rows * 131 + n)
    Z = (rng.standard_normal((rows, n)) * 2 + 0.5).astype(np.float32)
    host, dev, u = _brn_arrays(ctx, n, rng)
    zd, sums = ctx.array(Z), ctx.zeros(2 * n, np.float64)
    check(L.dlb_brn_forward_sums(ctx.h, zd.ptr, rows, n, sums.ptr))
    check(L.dlb_brn_forward_finalize(ctx.h, sums.ptr, rows, n, 0.99, 1e-5, 3.0, 5.0, C.byref(u)))
    s = sums.get()
    np.testing.assert_allclose(s[:n], Z.astype(np.float64).sum(0), rtol=1e-6, atol=1e-4)
    np.testing.assert_allclose(s[n:], (Z.astype(np.float64) ** 2).sum(0), rtol=1e-6)
    state = dict(mean_average=host["mean_average"].copy(), variance_average=host["sigma_average"].copy(),
                 gamma=host["gamma"], beta=host["beta"])
    x_hat, y = fc_step.brn_forward(Z, state, dict(momentum=0.99, eps=1e-5, r_max=3.0, d_max=5.0))
    for mine, theirs in (("mean", "mean"), ("sigma", "variance"), ("mean_average", "mean_average"),
                         ("sigma_average", "variance_average"), ("r", "r")):
        assert util.rel_max(dev[mine].get(), state[theirs]) <= F32_TOL, mine
    # d = (mean - running mean) / running sigma is a difference of nearly equal
    # numbers added to a normalised value of order 1: absolute bound.
    assert np.abs(dev["d"].get() - state["d"]).max() <= 1e-6
    # normalise + SELU + Bernoulli mask, and the residual plane of the result
    mask = (rng.random(n) < 0.9).astype(np.uint8)
    md, A, Alo = ctx.array(mask), ctx.empty((rows, n)), ctx.empty((rows, n))
    dp = dlb200.DropoutDesc(fc_step.DROPOUT_BERNOULLI, 0.9, md.ptr, None)
    check(L.dlb_activation_forward(ctx.h, zd.ptr, C.byref(u), fc_step.AF_SELU, C.byref(dp), A.ptr, Alo.ptr, rows, n))
    want = fc_step.apply_dropout(fc_step.af_fire(fc_step.AF_SELU, y), fc_step.DROPOUT_BERNOULLI, 0.9, mask)
    got = A.get()
    assert util.rel_max(got, want) <= F32_TOL
    assert np.array_equal(got[:, mask == 0], np.zeros_like(got[:, mask == 0]))   # dropped units: exact zeros
    if ctx.gemm_kind() == 0:   # TF32 residual plane
        hi = (got.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)
        assert np.all(np.abs(Alo.get() - (got - hi)) <= np.abs(got - hi) * 2.0 ** -11 + 1e-45)
    else:                      # fp16 planes of s * A, s = 2^(14 - floor(log2 max|A|))
        planes = Alo.get().ravel().view(np.float16).astype(np.float64)
        s = 2.0 ** (14 - np.floor(np.log2(np.abs(got).max())))
        assert np.abs(planes[:got.size]).max() < 2.0 ** 15
        both = (planes[:got.size] + planes[got.size:]) / s
        assert np.allclose(both, got.ravel(), rtol=2.0 ** -21, atol=2.0 ** -38 * np.abs(got).max())


@pytest.mark.parametrize("af", [fc_step.AF_RELU, fc_step.AF_LEAKY_RELU, fc_step.AF_ELU, fc_step.AF_SELU,
                                fc_step.AF_ISRLU, fc_step.AF_LINEAR])
@pytest.mark.parametrize("dropout", [fc_step.DROPOUT_NONE, fc_step.DROPOUT_BERNOULLI_INVERTED, fc_step.DROPOUT_UOUT])
def test_activation_forward_without_norm(gpu_ctx, af, dropout):
    ctx, L = gpu_ctx, gpu_ctx.L
    rng = np.random.default_rng(af * 10 + dropout)
    rows, n = 129, 67
    Z = (rng.standard_normal((rows, n)) * 2).astype(np.float32)
    mask = (rng.random(n) < 0.8).astype(np.uint8)
    noise = ((rng.random((rows, n)) * 2 - 1) * 0.1).astype(np.float32)
    zd, md, nd, A = ctx.array(Z), ctx.array(mask), ctx.array(noise), ctx.empty((rows, n))
    dp = dlb200.DropoutDesc(dropout, 0.8, md.ptr, nd.ptr)
    check(L.dlb_activation_forward(ctx.h, zd.ptr, None, af, C.byref(dp) if dropout else None, A.ptr, None, rows, n))
    want = fc_step.apply_dropout(fc_step.af_fire(af, Z), dropout, 0.8, mask, noise)
    assert util.rel_max(A.get(), want) <= F32_TOL


@pytest.mark.parametrize("af", [fc_step.AF_RELU, fc_step.AF_LEAKY_RELU, fc_step.AF_ELU, fc_step.AF_SELU,
                                fc_step.AF_ISRLU])
@pytest.mark.parametrize("rows,n", [(256, 128), (100, 37)])
def test_batch_renorm_backward(gpu_ctx, af, rows, n):
    ctx, L = gpu_ctx, gpu_ctx.L
    rng = np.random.default_rng(af * 1000 + rows + n)
    Z = (rng.standard_normal((rows, n)) * 1.5 + 0.3).astype(np.float32)
    host, dev, u = _brn_arrays(ctx, n, rng)
    zd, sums = ctx.array(Z), ctx.zeros(2 * n, np.float64)
    check(L.dlb_brn_forward_sums(ctx.h, zd.ptr, rows, n, sums.ptr))
    check(L.dlb_brn_forward_finalize(ctx.h, sums.ptr, rows, n, 0.99, 1e-5, 3.0, 5.0, C.byref(u)))
    mask = (rng.random(n) < 0.9).astype(np.uint8)
    md, A = ctx.array(mask), ctx.empty((rows, n))
    dp = dlb200.DropoutDesc(fc_step.DROPOUT_BERNOULLI, 0.9, md.ptr, None)
    check(L.dlb_activation_forward(ctx.h, zd.ptr, C.byref(u), af, C.byref(dp), A.ptr, None, rows, n))
    dA = rng.standard_normal((rows, n), dtype=np.float32)
    dd, dlo, bs = ctx.array(dA), ctx.empty((rows, n)), ctx.zeros(4 * n, np.float64)
    check(L.dlb_activation_backward(ctx.h, dd.ptr, zd.ptr, A.ptr, C.byref(u), af, rows, n, bs.ptr))
    check(L.dlb_brn_backward_apply(ctx.h, dd.ptr, dlo.ptr, zd.ptr, C.byref(u), bs.ptr, rows, rows, n))
    dg, db = ctx.zeros(n), ctx.zeros(n)
    check(L.dlb_brn_backward_param_grads(ctx.h, bs.ptr, n, dg.ptr, db.ptr, 0))
    # restatement
    state = dict(mean_average=host["mean_average"].copy(), variance_average=host["sigma_average"].copy(),
                 gamma=host["gamma"], beta=host["beta"])
    x_hat, y = fc_step.brn_forward(Z, state, dict(momentum=0.99, eps=1e-5, r_max=3.0, d_max=5.0))
    a = fc_step.apply_dropout(fc_step.af_fire(af, y), fc_step.DROPOUT_BERNOULLI, 0.9, mask)
    e = (dA * fc_step.af_derive(af, y, a)).astype(np.float32)
    dx, wg, wb = fc_step.brn_backward(e, Z, x_hat, state)
    assert util.rel_l2(dd.get(), dx) <= F32_TOL
    assert util.rel_l2(dg.get(), wg) <= F32_TOL and util.rel_l2(db.get(), wb) <= F32_TOL


def test_softmax_and_cross_entropy_delta(gpu_ctx):
    ctx, L = gpu_ctx, gpu_ctx.L
    rng = np.random.default_rng(2)
    for rows, n in ((128, 10), (77, 1000), (5, 3)):
        Z = (rng.standard_normal((rows, n)) * 3).astype(np.float32)
        Y = np.zeros((rows, n), np.float32)
        Y[np.arange(rows), rng.integers(0, n, rows)] = 1
        zd, yd, Q, D = ctx.array(Z), ctx.array(Y), ctx.empty((rows, n)), ctx.empty((rows, n))
        loss = ctx.zeros(1, np.float64)
        check(L.dlb_softmax_forward(ctx.h, zd.ptr, Q.ptr, rows, n))
        check(L.dlb_loss_delta(ctx.h, fc_step.LOSS_CROSS_ENTROPY, fc_step.AF_SOFTMAX, zd.ptr, Q.ptr, yd.ptr, D.ptr,
                               None, rows, n, rows, loss.ptr))
        q = fc_step.softmax(Z)
        total, delta = fc_step.loss_and_delta(fc_step.LOSS_CROSS_ENTROPY, fc_step.AF_SOFTMAX, Z, q, Y)
        assert util.rel_max(Q.get(), q) <= F32_TOL
        assert util.rel_max(D.get(), delta) <= F32_TOL
        np.testing.assert_allclose(loss.get()[0], total, rtol=1e-6)


def test_mse_delta(gpu_ctx):
    ctx, L = gpu_ctx, gpu_ctx.L
    rng = np.random.default_rng(4)
    rows, n = 333, 41
    pre = rng.standard_normal((rows, n), dtype=np.float32)
    Y = rng.standard_normal((rows, n), dtype=np.float32)
    pd, yd, D, loss = ctx.array(pre), ctx.array(Y), ctx.empty((rows, n)), ctx.zeros(1, np.float64)
    check(L.dlb_loss_delta(ctx.h, fc_step.LOSS_MSE, fc_step.AF_LINEAR, pd.ptr, pd.ptr, yd.ptr, D.ptr, None, rows, n,
                           2 * rows, loss.ptr))
    total, delta = fc_step.loss_and_delta(fc_step.LOSS_MSE, fc_step.AF_LINEAR, pre, pre, Y, global_rows=2 * rows)
    assert util.rel_max(D.get(), delta) <= 1e-6
    np.testing.assert_allclose(loss.get()[0], total, rtol=1e-9)


@pytest.mark.parametrize("rule", [fc_step.OPT_ADAM, fc_step.OPT_AMSGRAD, fc_step.OPT_ADABOUND,
                                  fc_step.OPT_AMSBOUND, fc_step.OPT_NOSADAM, fc_step.OPT_ADAMAX])
@pytest.mark.parametrize("n", [1_000_003, 4096, 5])
def test_optimizer_sweep(gpu_ctx, rule, n):
    """Flat-vector sweep: p ~ N(0, 0.02), g ~ N(0, 1e-3) refilled each step,
    zero moments, 10 steps.  AdaMax has no reference implementation; its
    expected values come from the published rule only."""
    ctx, L = gpu_ctx, gpu_ctx.L
    rng = np.random.default_rng(rule * 7 + n % 97)
    p = (0.02 * rng.standard_normal(n)).astype(np.float32)
    g = (1e-3 * rng.standard_normal(n)).astype(np.float32)
    hp = dict(adam_learning_rate=1e-3, adam_beta1=0.9, adam_beta2=0.999, adam_epsilon=1e-8, adam_gamma=0.1,
              learning_rate_final=0.1, learning_gamma=1e-3)
    pd, gd, m, v, vh = ctx.array(p), ctx.array(g), ctx.zeros(n), ctx.zeros(n), ctx.zeros(n)
    hyper = (C.c_float * 8)(1e-3, 0.9, 0.999, 1e-8, 0.1, 0.1, 1e-3, 1.0)
    t, prev = C.c_float(0), C.c_float(0)
    po, mo, vo, vho, state = p.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros(n, np.float32), {}
    for step in range(10):
        k = dlb200.OptimizerScalars()
        check(L.dlb_optimizer_prepare(rule, hyper, C.byref(t), C.byref(prev), C.byref(k)))
        if step:
            gd.set(g)
        check(L.dlb_optimizer_step(ctx.h, rule, C.byref(k), pd.ptr, gd.ptr, m.ptr, v.ptr, vh.ptr, None, n))
        gg = g.copy()
        fc_step.optimizer_update(rule, fc_step.optimizer_scalars(rule, hp, state), po, gg, mo, vo, vho)
    assert ctx.sync() == 0
    assert not gd.get().any()                       # gradient zeroed after use
    assert util.rel_l2(pd.get() - p, po - p) <= F32_TOL
    assert util.rel_l2(m.get(), mo) <= 1e-6 and util.rel_l2(v.get(), vo) <= 1e-6
    if rule in (fc_step.OPT_AMSGRAD, fc_step.OPT_AMSBOUND):
        assert util.rel_l2(vh.get(), vho) <= 1e-6


@pytest.mark.parametrize("form", ["plain", "momentum", "nesterov"])
@pytest.mark.parametrize("n", [1_000_003, 5])
def test_gradient_descent_sweep(gpu_ctx, form, n):
    """The three gradient-descent forms over a flat vector with weight decay,
    10 steps; plain descent takes no moment arrays at all."""
    ctx, L = gpu_ctx, gpu_ctx.L
    rng = np.random.default_rng(n % 89)
    p = (0.02 * rng.standard_normal(n)).astype(np.float32)
    g = (1e-3 * rng.standard_normal(n)).astype(np.float32)
    mask = (rng.random(n) < 0.7).astype(np.float32)
    mom, nag = {"plain": (0.0, 0), "momentum": (0.9, 0), "nesterov": (0.9, 1)}[form]
    hp = dict(learning_rate=0.05, learning_momentum=mom, use_nesterov=nag)
    pd, gd, m, md = ctx.array(p), ctx.array(g), ctx.zeros(n), ctx.array(mask)
    hyper = (C.c_float * 8)(0.05, mom, nag, 0, 0, 0, 0, 0)
    t, prev = C.c_float(0), C.c_float(0)
    po, mo, state = p.copy(), np.zeros(n, np.float32), {}
    for step in range(10):
        k = dlb200.OptimizerScalars()
        check(L.dlb_optimizer_prepare(6, hyper, C.byref(t), C.byref(prev), C.byref(k)))
        k.weight_decay = 0.01
        if step:
            gd.set(g)
        check(L.dlb_optimizer_step(ctx.h, 6, C.byref(k), pd.ptr, gd.ptr, m.ptr if mom else None, None, None,
                                   md.ptr, n))
        fc_step.optimizer_update(6, fc_step.optimizer_scalars(6, hp, state), po, g.copy(), mo, None, None,
                                 wd=0.01, mask=mask)
    assert ctx.sync() == 0 and t.value == 10
    assert not gd.get().any()
    assert util.rel_l2(pd.get() - p, po - p) <= F32_TOL
    if mom:
        assert util.rel_l2(m.get(), mo) <= 1e-6


def test_bad_arguments_are_refused(gpu_ctx):
    ctx, L = gpu_ctx, gpu_ctx.L
    x = ctx.zeros(16)
    assert L.dlb_fc_forward(ctx.h, None, None, x.ptr, None, None, x.ptr, 1, 4, 4) == 1
    assert L.dlb_fc_forward(ctx.h, x.ptr, None, x.ptr, None, None, x.ptr, 0, 4, 4) == 1
    k = dlb200.OptimizerScalars()
    assert L.dlb_optimizer_step(ctx.h, 7, C.byref(k), x.ptr, x.ptr, x.ptr, x.ptr, None, None, 16) == 3
    assert L.dlb_optimizer_step(ctx.h, 5, C.byref(k), x.ptr, x.ptr, x.ptr, x.ptr, None, None, 16) == 1
    assert L.dlb_loss_delta(ctx.h, 3, 11, x.ptr, x.ptr, x.ptr, x.ptr, None, 4, 4, 4, x.ptr) == 3
    assert b"invalid" in L.dlb_status_string(1)
    assert ctx.sync() == 0


# ---- peer-memory exchange of the batch-renormalization sums -----------------

@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("n", [1, 7, 256, 8192, 32768])
def test_peer_exchange_emulated_ranks(gpu_ctx, world, n):
    """Every emulated rank ends with the sum of all ranks' vectors, added in
    rank order (so bit-identical on all ranks and to the same loop on the
    host), over three exchanges back to back on the same buffers (both inbox
    halves and the flag sequence are reused)."""
    rng = np.random.default_rng(world * 100003 + n)
    v = rng.standard_normal((world, n)) * np.exp(rng.uniform(-20, 20, (world, n)))
    out = gpu_ctx.peer_exchange_emulated(v, rounds=3)
    want = np.zeros(n)
    for r in range(world):
        want = want + v[r] * 3.0
    for r in range(world):
        assert np.array_equal(out[r], want), r
    assert gpu_ctx.sync() == 0


def test_peer_exchange_gives_up_on_an_absent_rank(gpu_ctx):
    """A rank that never delivers: the others' bounded waits run out, the call
    reports the timeout, and the context works afterwards."""
    v = np.arange(4 * 600, dtype=np.float64).reshape(4, 600)
    with pytest.raises(dlb200.DlbError, match="gave up waiting"):
        gpu_ctx.peer_exchange_emulated(v, absent=2, wait_ms=200)
    assert gpu_ctx.sync() == 0
    out = gpu_ctx.peer_exchange_emulated(v)
    assert np.array_equal(out[3], v.sum(axis=0))
