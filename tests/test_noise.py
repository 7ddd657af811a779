"""The counter-based generator behind the device-side noise: the CPU
restatement against the published known-answer vectors of Philox4x32-10, its
indexing rules, and (on a GPU) the device generator bit for bit against it."""
import ctypes as C

import numpy as np
import pytest

import configs
import dlb200
import fc_residual
import fc_step
import philox
import util
from enums import LAYER_DROPOUT

# Known-answer vectors distributed with the generator's reference
# implementation (counter, key) -> output.
KAT = [
    ((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
    ((0xffffffff,) * 4, (0xffffffff,) * 2, (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
    ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
     (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1)),
]


def test_restatement_matches_known_answer_vectors():
    for ctr, key, want in KAT:
        got = philox.philox4x32_10(np.array([ctr], np.uint64), key)[0]
        assert tuple(int(v) for v in got) == want


def test_a_slice_of_a_draw_is_the_draw_of_the_slice():
    whole = philox.words(1000, seed=(5 << 32) | 9, stream=6, step=3)
    for first, n in ((0, 1), (1, 5), (3, 4), (250, 333), (997, 3)):
        assert np.array_equal(philox.words(n, (5 << 32) | 9, 6, 3, first), whole[first:first + n])
    assert not np.array_equal(philox.words(1000, (5 << 32) | 9, 7, 3), whole)   # another stream
    assert not np.array_equal(philox.words(1000, (5 << 32) | 9, 6, 4), whole)   # another step
    u = philox.uniform(200000, -0.25, 0.25, 1, 0, 0)
    assert u.min() >= -0.25 and u.max() < 0.25 and abs(u.mean()) < 2e-3
    assert abs(philox.bernoulli(200000, 0.9, 1, 0, 0).mean() - 0.9) < 3e-3


@pytest.mark.gpu
@pytest.mark.parametrize("n,first", [(1, 0), (7, 0), (5, 3), (4096, 2), (100003, 1234567891234)])
def test_device_generator_matches_restatement(gpu_ctx, n, first):
    ctx, L = gpu_ctx, gpu_ctx.L
    seed = (0xDEADBEEF << 32) | 0x1234567
    u = ctx.empty(n)
    dlb200.check(L.dlb_noise_uniform(ctx.h, u.ptr, n, -0.3, 0.7, seed, 5, 2, first), "uniform")
    b = ctx.zeros(n, np.uint8)
    dlb200.check(L.dlb_noise_bernoulli(ctx.h, b.ptr, n, 0.4, seed, 6, 2, first), "bernoulli")
    assert ctx.sync() == 0
    assert np.array_equal(u.get(), philox.uniform(n, -0.3, 0.7, seed, 5, 2, first))
    assert np.array_equal(b.get(), philox.bernoulli(n, 0.4, seed, 6, 2, first))


@pytest.mark.gpu
def test_model_draws_uout_and_bernoulli_noise_on_the_device(gpu_ctx):
    """draw_noise + a step equals the CPU restatement's step on the same arrays,
    rebuilt on the host from (seed, 4 * layer + kind, step); a shard that starts
    at row 32 draws rows 32.. of the same arrays."""
    seed, step = 77, 4
    for kind, value in ((LAYER_DROPOUT.UOUT, 0.25), (LAYER_DROPOUT.BERNOULLI, 0.8)):
        cfg = configs.deep_brn_mlp(64, 128, 2, 32, 96, dropout=kind, keep=value)
        B = cfg["batch"]
        X, Y = configs.synthetic_batch(cfg)

        def prepare(model, rows=B, first=0):
            for li in (1, 2):
                if kind == LAYER_DROPOUT.UOUT:
                    model.set_uout_noise(li, philox.uniform(rows * 128, -value, value, seed, 4 * li + 1, step,
                                                            first * 128).reshape(rows, 128))
                else:
                    model.set_dropout_mask(li, philox.bernoulli(128, value, seed, 4 * li, step))

        p0, _ = util.kink_free_parameters(cfg, fc_step.OracleModel, X, {}, scale=1.0 / np.sqrt(128), prepare=prepare)
        ora = util.build(fc_step.OracleModel(), cfg, params=p0)
        prepare(ora)
        want = util.trace(ora, cfg, 1, X, Y, {})
        mod = util.build(dlb200.Model(gpu_ctx), cfg, params=p0)
        mod.draw_noise(B, seed, step)
        got = util.trace(mod, cfg, 1, X, Y, {})
        assert gpu_ctx.sync() == 0
        for key, (l2, mx) in util.compare(got, want).items():
            assert l2 <= 1e-5, f"{kind} {key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"
        # The second third of the rows as a shard of its own.
        sub = dict(cfg, batch=32)
        ora = util.build(fc_step.OracleModel(), sub, params=p0)
        prepare(ora, 32, 32)
        want = util.trace(ora, sub, 1, X[32:64], Y[32:64], {})
        mod = util.build(dlb200.Model(gpu_ctx), sub, params=p0)
        mod.draw_noise(32, seed, step, first_row=32)
        got = util.trace(mod, sub, 1, X[32:64], Y[32:64], {})
        assert util.rel_l2(got["act2"], want["act2"]) <= 1e-5


@pytest.mark.gpu
def test_model_draws_shakedrop_noise_on_the_device(gpu_ctx):
    seed, step = 11, 0
    cfg = configs.residual_mlp(width=256, blocks=2, n_out=10, batch=256)
    B = cfg["batch"]
    X, Y = configs.synthetic_batch(cfg)
    mod = util.build(dlb200.Model(gpu_ctx), cfg, seed=4)
    p0 = mod.get_array("parameters")
    ora = util.build(fc_residual.ResidualOracleModel(), cfg, params=p0)
    for li, p in configs.shakedrop_layers(cfg):
        ora.set_shakedrop_noise(li, philox.bernoulli(B, p, seed, 4 * li, step),
                                philox.uniform(B * 256, -1, 1, seed, 4 * li + 1, step).reshape(B, 256),
                                philox.uniform(B * 256, 0, 1, seed, 4 * li + 2, step).reshape(B, 256))
    mod.draw_noise(B, seed, step)
    out = []
    for m in (ora, mod):
        m.train_begin(B)
        m.reset_loss()
        m.forward_pass(B, X)
        m.compute_error(B, Y)
        m.backward_pass(B)
        m.update_derivatives(B)
        m.merge_derivatives()
        out.append((m.get_loss(), m.get_array("derivatives")))
    assert gpu_ctx.sync() == 0
    assert abs(out[0][0] - out[1][0]) <= 1e-5 * abs(out[0][0])
    assert util.rel_l2(out[1][1], out[0][1]) <= 2e-5
