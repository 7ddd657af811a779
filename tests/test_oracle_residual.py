"""Residual blocks with ShakeDrop: the CPU restatement (oracle/fc_residual.py)
against the committed fixture of the compiled reference and, where oracle/_ref
is built, against the compiled reference on other shapes."""
import pytest

import configs
import fc_residual
import fc_step
import golden_io
import ref_binding
import util

TOL_L2 = 2e-6
# Updated weights: the Adam first step lr*g/(|g|+eps) magnifies rounding of
# gradients that are of the order of eps.
TOL_PARAMS = 1e-4


def _check(got, want):
    for key, (l2, mx) in util.compare(got, want).items():
        tol = TOL_PARAMS if key.startswith("params") else TOL_L2
        assert l2 <= tol, f"{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"


@pytest.mark.parametrize("name", sorted(golden_io.NOISY_CASES))
def test_residual_restatement_matches_golden(name):
    cfg, steps, X, Y, draws, p0, want = golden_io.load_noisy(name)
    model = util.build(fc_residual.ResidualOracleModel(), cfg, params=p0)
    _check(util.trace_noisy(model, cfg, steps, X, Y, draws), want)


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("cfg", [configs.residual_mlp(32, 2, 10, 8, p_last=0.0),
                                 configs.residual_mlp(40, 4, 5, 24),
                                 # blocks wider / narrower than the shortcut, an odd difference:
                                 # the zero-padded shortcut (fwp_mp.cpp L:5058-5123, bwp_mp.cpp L:1078-1140)
                                 configs.residual_mlp(8, 2, 5, 12, block_width=12),
                                 configs.residual_mlp(12, 2, 5, 12, block_width=8),
                                 configs.residual_mlp(9, 2, 5, 12, block_width=12)], ids=lambda c: c["name"])
def test_residual_restatement_matches_compiled_reference(cfg):
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    p0 = ref.get_array("parameters")
    want = util.trace_noisy(ref, cfg, steps=5)
    got = util.trace_noisy(util.build(fc_residual.ResidualOracleModel(), cfg, params=p0), cfg, steps=5)
    _check(got, want)


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
def test_residual_evaluation_pass_matches_compiled_reference():
    """Inference through residual blocks: running averages in the blocks and in
    the residual layer's own normalization where it has one, the block output of
    a ShakeDrop layer times 1 - p (v1/learner/fwp_mp.cpp L:3876-3897), then the
    loss and the accuracy without an error."""
    cfg = configs.residual_mlp(40, 4, 5, 24)
    B, last = cfg["batch"], len(cfg["layers"]) - 1
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    ora = util.build(fc_residual.ResidualOracleModel(), cfg, params=ref.get_array("parameters"))
    Xe, Ye = configs.synthetic_batch(dict(cfg, data_seed=5))
    out = []
    util.trace_noisy(ref, cfg, steps=3)   # move the running averages away from their start
    util.copy_trained_state(ref, ora, cfg)
    for m in (ref, ora):
        m.set_propagation(0)
        m.set_accu_fn(fc_step.ACCU_CROSS_ENTROPY)
        m.reset_loss()
        m.forward_pass(B, Xe)
        m.compute_loss(B, Ye)
        out.append((m.get_loss(), m.get_accu(B), m.get_layer_outputs(last, B).reshape(B, -1)))
    (lr, ar, qr), (lo, ao, qo) = out
    assert abs(lr - lo) <= 1e-5 * abs(lr) and ar == ao
    assert util.rel_l2(qo, qr) <= TOL_L2


@pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("delay", [0, 2], ids=["all_steps", "last_step"])
def test_residual_blocks_in_a_time_stepped_model_match_compiled_reference(delay):
    """Residual blocks of FC layers with seq_w = 3 (oracle/fc_residual_time.py):
    statistics of their own per time step, gradients summed over the steps, the
    softmax error against the target of time step 0."""
    import fc_residual_time
    from enums import LAYER, MODEL
    cfg = configs.residual_mlp(width=8, blocks=2, n_out=5, batch=6)
    cfg = dict(cfg, model_type=MODEL.RECURRENT, seq_w=3, time_delays=delay, mp=True)
    for l in cfg["layers"]:
        if l["type"] == LAYER.RESIDUAL:
            l.pop("dropout", None)   # the replay of ShakeDrop draws covers feed-forward models
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    p0 = ref.get_array("parameters")
    X, Y = configs.synthetic_batch(cfg)
    want = util.trace_noisy(ref, cfg, 3, X, Y)
    got = util.trace_noisy(util.build(fc_residual_time.ResidualTimeOracleModel(), cfg, params=p0), cfg, 3, X, Y)
    _check(got, want)
