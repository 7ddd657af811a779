"""LSTM layers on the GPU, through the Model entry points of the C ABI: against
the committed fixtures of the compiled reference and against the CPU restatement
(oracle/fc_lstm.py, pinned to those fixtures) on shapes whose products run on the
tensor-core kernels."""
import numpy as np
import pytest

import configs
import dlb200
import fc_lstm
import golden_io
import util
from enums import ACTIVATION, LAYER

pytestmark = pytest.mark.gpu

TOL_1 = 1e-5       # activations, errors, gradients after one step (rel_l2)
TOL_PARAMS = 1e-4  # updated weights: Adam's first step magnifies gradients of the order of eps


def _check(got, want, cfg):
    skip = {f"delta{i}" for i, l in enumerate(cfg["layers"]) if l["type"] == LAYER.LSTM}
    for key, (l2, mx) in util.compare(got, want).items():
        if key in skip:
            continue
        tol = TOL_PARAMS if key.startswith("params") else TOL_1
        assert l2 <= tol, f"{key}: rel_l2 {l2:.2e} (rel_max {mx:.2e})"


@pytest.mark.parametrize("name", sorted(golden_io.LSTM_CASES))
def test_lstm_model_matches_golden(gpu_ctx, name):
    cfg, steps, X, Y, masks, p0, want = golden_io.load(name)
    got = util.trace(util.build(dlb200.Model(gpu_ctx), cfg, params=p0), cfg, steps, X, Y, masks)
    assert gpu_ctx.sync() == 0
    _check(got, want, cfg)


def _random_parameters(cfg, seed=0):
    ora = util.build(fc_lstm.LstmOracleModel(), cfg)
    p0 = ora.get_array("parameters")
    rng = np.random.default_rng(seed)
    nw = ora.size("total_weights")
    p0[:nw] = (rng.standard_normal(nw) * 0.08).astype(np.float32)
    p0[nw:] = (rng.standard_normal(p0.size - nw) * 0.1).astype(np.float32)
    return p0


@pytest.mark.parametrize("cfg", [
    configs.lstm_stack(n_in=64, blocks=64, cells=2, depth=1, n_out=128, seq_w=6, batch=64),
    configs.lstm_stack(n_in=96, blocks=128, cells=1, depth=2, n_out=128, seq_w=4, batch=128, hidden_fc=128),
    configs.lstm_stack(n_in=40, blocks=24, cells=3, depth=1, n_out=72, seq_w=5, batch=33),      # ragged
], ids=lambda c: c["name"])
def test_lstm_model_vs_restatement(gpu_ctx, cfg):
    """One step on shapes whose products (input sums over T * rows rows, the
    recurrent sums of a step, the two weight gradients) are tensor-core sized; then
    three steps for the scale of the agreement."""
    X, Y = configs.synthetic_batch(cfg)
    p0 = _random_parameters(cfg)
    want = util.trace(util.build(fc_lstm.LstmOracleModel(), cfg, params=p0), cfg, 1, X, Y)
    got = util.trace(util.build(dlb200.Model(gpu_ctx), cfg, params=p0), cfg, 1, X, Y)
    assert gpu_ctx.sync() == 0
    _check(got, want, cfg)
    want = util.trace(util.build(fc_lstm.LstmOracleModel(), cfg, params=p0), cfg, 3, X, Y)
    got = util.trace(util.build(dlb200.Model(gpu_ctx), cfg, params=p0), cfg, 3, X, Y)
    assert gpu_ctx.sync() == 0
    assert util.rel_l2(got["params_last"], want["params_last"]) <= 1e-4
    assert util.rel_l2(got["losses"], want["losses"]) <= 1e-5


def test_lstm_last_step_error_and_one_call_steps(gpu_ctx):
    """An error on the last time step only; train_step (one call) gives the weights
    of the entry points called one by one."""
    cfg = configs.lstm_stack(n_in=32, blocks=32, cells=2, depth=1, n_out=64, seq_w=5, batch=48)
    cfg["time_delays"] = 4
    X, Y = configs.synthetic_batch(cfg)
    p0 = _random_parameters(cfg, 3)
    want = util.trace(util.build(fc_lstm.LstmOracleModel(), cfg, params=p0), cfg, 2, X, Y)
    got = util.trace(util.build(dlb200.Model(gpu_ctx), cfg, params=p0), cfg, 2, X, Y)
    _check(got, want, cfg)
    one = util.build(dlb200.Model(gpu_ctx), cfg, params=p0)
    for _ in range(2):
        one.train_step(cfg["batch"], X, Y)
    assert gpu_ctx.sync() == 0
    assert util.rel_l2(one.get_array("parameters"), got["params_last"]) <= 1e-6


def test_unsupported_lstm_forms_are_refused(gpu_ctx):
    m = dlb200.Model(gpu_ctx)
    with pytest.raises(dlb200.DlbError):
        m.compile([3, 7, 3], [4, 3, 8], seq_w=3, model_type=4)            # no cells per block
    m = dlb200.Model(gpu_ctx)
    m.compile([3, 7, 3], [4, 3, 8], seq_w=3, model_type=4, layer_units2=[0, 2, 0])
    m.set_layer_activation_function(2, ACTIVATION.LINEAR)
    m.Set__Layer_Normalization(1, 2)
    with pytest.raises(dlb200.DlbError):
        m.forward_pass(2, np.zeros((2, 12), np.float32))
    # The layer after an LSTM layer narrower than the LSTM layer has cells: the
    # reference's bias indices would leave its parameter vector.
    m = dlb200.Model(gpu_ctx)
    m.compile([3, 7, 3], [4, 3, 2], seq_w=3, model_type=4, layer_units2=[0, 2, 0])
    m.set_layer_activation_function(2, ACTIVATION.LINEAR)
    with pytest.raises(dlb200.DlbError):
        m.forward_pass(2, np.zeros((2, 12), np.float32))
