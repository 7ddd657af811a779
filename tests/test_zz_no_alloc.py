"""dlb_brn_forward_sums_noalloc: the batch-renormalization sums for callers
that may not allocate device memory (code inside a stream capture, a host
callback or a latency-critical loop, or a process whose framework allocator
owns the whole GPU).  It keeps its partial sums in an array built into the
library instead of the context's growable scratch arena.

Checked here, through the C ABI: two calls in a row on different inputs give
the sums of the allocating entry point (the array is shared between calls and
keeps the previous call's contents, so the second call must not be disturbed
by the first), a request beyond the built-in capacity is refused with a
message instead of being launched, and so is a null argument.

The file name sorts last so that, in a run that stops at the first failure,
every other test has already run."""
import numpy as np
import pytest

import dlb200
from dlb200 import check

pytestmark = pytest.mark.gpu

NOALLOC_SCRATCH_DOUBLES = 1 << 20


def _sums_both_ways(ctx, Z):
    L = ctx.L
    rows, n = Z.shape
    zd = ctx.array(Z)
    want, got = ctx.zeros(2 * n, np.float64), ctx.zeros(2 * n, np.float64)
    check(L.dlb_brn_forward_sums(ctx.h, zd.ptr, rows, n, want.ptr), "dlb_brn_forward_sums")
    check(L.dlb_brn_forward_sums_noalloc(zd.ptr, rows, n, got.ptr, ctx.stream), "dlb_brn_forward_sums_noalloc")
    assert ctx.sync() == 0
    return got.get(), want.get()


def test_two_calls_in_a_row_match_the_allocating_entry_point(gpu_ctx):
    rng = np.random.default_rng(42)
    # Second call is smaller than the first: stale partial sums of the first
    # call stay in the shared array and must not leak into the second result.
    for rows, n in ((1024, 768), (200, 132), (333, 7)):
        Z = (rng.standard_normal((rows, n)) * 3 + 1).astype(np.float32)
        got, want = _sums_both_ways(gpu_ctx, Z)
        exact = np.concatenate([Z.astype(np.float64).sum(0), (Z.astype(np.float64) ** 2).sum(0)])
        # Same tolerance as the sums check of test_gpu_ops.test_batch_renorm_forward.
        np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-4)
        np.testing.assert_allclose(got, exact, rtol=1e-6, atol=1e-4)
        # Both entry points cut the rows into the same chunks and add the
        # chunks in the same order: the sums agree to the last bit.
        assert np.array_equal(got, want)


def test_calls_take_no_device_memory(gpu_ctx):
    """After the first call on the device (which looks the array's address up),
    further calls leave the free device memory where it was: nothing is
    allocated, by the entry point or on its behalf."""
    L = gpu_ctx.L
    rng = np.random.default_rng(7)
    Z = rng.standard_normal((512, 256)).astype(np.float32)
    zd = gpu_ctx.array(Z)
    out = gpu_ctx.zeros(2 * 256, np.float64)
    check(L.dlb_brn_forward_sums_noalloc(zd.ptr, 512, 256, out.ptr, gpu_ctx.stream), "first call")
    assert gpu_ctx.sync() == 0
    free0, _ = dlb200.device_mem_info()
    for rows in (512, 64, 300):
        check(L.dlb_brn_forward_sums_noalloc(zd.ptr, rows, 256, out.ptr, gpu_ctx.stream), "later call")
    assert gpu_ctx.sync() == 0
    free1, _ = dlb200.device_mem_info()
    assert free1 == free0


def test_request_beyond_the_built_in_scratch_is_refused(gpu_ctx):
    L = gpu_ctx.L
    # One chunk of rows already needs 2 * n_units doubles.
    n = NOALLOC_SCRATCH_DOUBLES // 2 + 4
    z = gpu_ctx.zeros((8, n))
    out = gpu_ctx.zeros(2 * n, np.float64)
    assert L.dlb_brn_forward_sums_noalloc(z.ptr, 8, n, out.ptr, gpu_ctx.stream) == 1
    msg = L.dlb_last_error().decode()
    assert "built-in" in msg and str(NOALLOC_SCRATCH_DOUBLES) in msg
    assert L.dlb_brn_forward_sums_noalloc(None, 8, 8, out.ptr, gpu_ctx.stream) == 1
    assert gpu_ctx.sync() == 0
