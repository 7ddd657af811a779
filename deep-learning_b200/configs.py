"""Workload descriptions for the fully-connected training step, their seeded
synthetic inputs, and one builder that drives any object exposing the
reference's ``Model`` setter names (the CUDA-backed ``Model`` of this package,
or the reference checker used by the tests).

A workload is a plain dict:
  layers      list of dicts: type, units, af, norm, dropout=(kind, value)
  seq_w       time steps (1 = feed-forward)
  time_delays value for ``set_seq_w`` (error only for t >= time_delays)
  loss, optimizer, hparams, brn(r_max, d_max, momentum, eps), batch, seed
"""
from __future__ import annotations

import numpy as np

from enums import ACTIVATION, LAYER, LAYER_DROPOUT, LAYER_NORM, LOSS_FN, MODEL, OPTIMIZER


def mlp_softmax(n_in=784, hidden=256, n_out=10, batch=128):
    """MNIST-shaped two-layer MLP: Leaky ReLU hidden layer, softmax
    cross-entropy output, Adam."""
    return dict(
        name=f"mlp_{n_in}-{hidden}-{n_out}_b{batch}",
        model_type=MODEL.FEEDFORWARD, seq_w=1, time_delays=0,
        layers=[
            dict(type=LAYER.FULLY_CONNECTED, units=n_in),
            dict(type=LAYER.FULLY_CONNECTED, units=hidden, af=ACTIVATION.LEAKY_RELU),
            dict(type=LAYER.FULLY_CONNECTED, units=n_out, af=ACTIVATION.SOFTMAX),
        ],
        loss=LOSS_FN.CROSS_ENTROPY, optimizer=OPTIMIZER.ADAM,
        hparams=dict(adam_learning_rate=1e-3, adam_beta1=0.9, adam_beta2=0.999, adam_epsilon=1e-8),
        batch=batch, weight_seed=0, data_seed=0, inputs="uniform", targets="onehot",
    )


def deep_brn_mlp(n_in=1024, hidden=4096, depth=4, n_out=1024, batch=4096,
                 af=ACTIVATION.SELU, optimizer=OPTIMIZER.AMSBOUND, keep=0.9,
                 dropout=LAYER_DROPOUT.BERNOULLI, norm=True):
    """Deep MLP: every hidden layer is FC + batch renorm (r_max 3, d_max 5,
    momentum 0.99, eps 1e-5) + SELU + Bernoulli dropout (keep 0.9); linear
    output, MSE, AMSBound (final_lr 0.1, gamma 1e-3).  norm=False: the same stack
    with bias instead of normalization."""
    layers = [dict(type=LAYER.FULLY_CONNECTED, units=n_in)]
    for _ in range(depth):
        layers.append(dict(type=LAYER.FULLY_CONNECTED, units=hidden, af=af,
                           norm=LAYER_NORM.BATCH_RENORMALIZATION if norm else None,
                           dropout=(dropout, keep) if dropout else None))
    layers.append(dict(type=LAYER.FULLY_CONNECTED, units=n_out, af=ACTIVATION.LINEAR))
    return dict(
        name=("brn_mlp_" if norm else "plain_mlp_") + f"{n_in}-{depth}x{hidden}-{n_out}_b{batch}",
        model_type=MODEL.FEEDFORWARD, seq_w=1, time_delays=0, layers=layers,
        loss=LOSS_FN.MSE, optimizer=optimizer,
        hparams=dict(adam_learning_rate=1e-3, adam_beta1=0.9, adam_beta2=0.999, adam_epsilon=1e-8,
                     learning_rate_final=0.1, learning_gamma=1e-3, adam_gamma=0.1),
        brn=dict(r_max=3.0, d_max=5.0, momentum=0.99, eps=1e-5),
        batch=batch, weight_seed=0, data_seed=0, mask_seed=1, inputs="normal", targets="normal",
    )


def residual_mlp(width=8192, blocks=16, n_out=1000, batch=8192, p_last=0.5, optimizer=OPTIMIZER.ADAM,
                 block_width=None):
    """Residual MLP: `blocks` blocks of width `width`, each FC - batch renorm -
    ELU - FC with a ShakeDrop skip, softmax cross-entropy over n_out classes,
    Adam.  In the reference's layer list a block is a RESIDUAL layer of depth 2
    followed by its two FC layers, the second carrying the normalization and
    the activation (pre-activation order).  The paper's keep probability decays
    linearly to p_last; the reference's ShakeDrop value is the probability that
    a row IS perturbed, hence (l / blocks) * (1 - p_last) for block l.
    `block_width` (default: width) is the width of the layers inside the blocks;
    where it differs from the shortcut's, the reference pads the narrower one
    with zeros (the residual output is as wide as the wider one)."""
    inner = block_width or width
    layers = [dict(type=LAYER.FULLY_CONNECTED, units=width)]
    for b in range(1, blocks + 1):
        layers.append(dict(type=LAYER.RESIDUAL, units=2,
                           dropout=(LAYER_DROPOUT.SHAKEDROP, (b / blocks) * (1.0 - p_last))))
        layers.append(dict(type=LAYER.FULLY_CONNECTED, units=inner, af=ACTIVATION.ELU))
        layers.append(dict(type=LAYER.FULLY_CONNECTED, units=inner, af=ACTIVATION.ELU,
                           norm=LAYER_NORM.BATCH_RENORMALIZATION))
    layers.append(dict(type=LAYER.FULLY_CONNECTED, units=n_out, af=ACTIVATION.SOFTMAX))
    return dict(
        name=f"residual_mlp_{blocks}x{width}" + (f"({inner})" if inner != width else "") + f"-{n_out}_b{batch}",
        model_type=MODEL.FEEDFORWARD, seq_w=1, time_delays=0, layers=layers,
        loss=LOSS_FN.CROSS_ENTROPY, optimizer=optimizer,
        hparams=dict(adam_learning_rate=1e-3, adam_beta1=0.9, adam_beta2=0.999, adam_epsilon=1e-8),
        brn=dict(r_max=3.0, d_max=5.0, momentum=0.99, eps=1e-5),
        batch=batch, weight_seed=0, data_seed=0, shakedrop_seed=2, inputs="normal", targets="onehot", mp=False,
    )


def indrnn_stack(n_in=512, hidden=2048, depth=4, n_out=512, seq_w=256, batch=1024,
                 af=ACTIVATION.RELU, optimizer=OPTIMIZER.ADABOUND, norm=True, dropout=None):
    """IndRNN stack: `depth` independently recurrent layers of width `hidden`
    with ReLU recurrence and batch renormalization (statistics per time step),
    a linear output layer, MSE on the last time step only (time_delays =
    seq_w - 1), AdaBound.  The recurrent weights are drawn from U(0, 1) by
    `set_recurrent_uniform` after the Glorot initialisation."""
    layers = [dict(type=LAYER.FULLY_CONNECTED, units=n_in)]
    for _ in range(depth):
        layers.append(dict(type=LAYER.FULLY_CONNECTED_INDEPENDENTLY_RECURRENT, units=hidden, af=af,
                           norm=LAYER_NORM.BATCH_RENORMALIZATION if norm else None, dropout=dropout))
    layers.append(dict(type=LAYER.FULLY_CONNECTED, units=n_out, af=ACTIVATION.LINEAR))
    return dict(
        name=f"indrnn_{n_in}-{depth}x{hidden}-{n_out}_T{seq_w}_b{batch}",
        model_type=MODEL.RECURRENT, seq_w=seq_w, time_delays=seq_w - 1, layers=layers,
        loss=LOSS_FN.MSE, optimizer=optimizer,
        hparams=dict(adam_learning_rate=1e-3, adam_beta1=0.9, adam_beta2=0.999, adam_epsilon=1e-8,
                     learning_rate_final=0.1, learning_gamma=1e-3, adam_gamma=0.1),
        brn=dict(r_max=3.0, d_max=5.0, momentum=0.99, eps=1e-5),
        batch=batch, weight_seed=0, data_seed=0, recurrent_seed=3, inputs="normal", targets="normal",
    )


def lstm_stack(n_in=16, blocks=8, cells=2, depth=1, n_out=8, seq_w=4, batch=8, optimizer=OPTIMIZER.ADAM,
               hidden_fc=None, af=ACTIVATION.LINEAR):
    """`depth` LSTM layers of `blocks` memory blocks with `cells` cells each
    (peephole connections, tanh / sigmoid as the reference fixes them), optionally
    a fully connected layer of `hidden_fc` units in front, a fully connected
    output layer with activation `af`, MSE on every time step, Adam."""
    layers = [dict(type=LAYER.FULLY_CONNECTED, units=n_in)]
    if hidden_fc:
        layers.append(dict(type=LAYER.FULLY_CONNECTED, units=hidden_fc, af=ACTIVATION.ISRLU))
    for _ in range(depth):
        layers.append(dict(type=LAYER.LSTM, units=blocks, cells=cells))
    layers.append(dict(type=LAYER.FULLY_CONNECTED, units=n_out, af=af))
    return dict(
        name=f"lstm_{n_in}-{depth}x{blocks}x{cells}-{n_out}_T{seq_w}_b{batch}",
        model_type=MODEL.RECURRENT, seq_w=seq_w, time_delays=0, layers=layers,
        loss=LOSS_FN.MSE, optimizer=optimizer,
        hparams=dict(adam_learning_rate=1e-3, adam_beta1=0.9, adam_beta2=0.999, adam_epsilon=1e-8),
        batch=batch, weight_seed=0, data_seed=0, inputs="normal", targets="normal", mp=False,
    )


def recurrent_slices(cfg):
    """[(layer index, slice of the flat parameter vector)] of the recurrent
    weights: an IndRNN layer's u[units] follows its W[units, fan_in]
    (v1/learner/connections_prepare.cpp L:46-81)."""
    out, w = [], 0
    layers = cfg["layers"]
    for i in range(1, len(layers)):
        w += layers[i]["units"] * layers[i - 1]["units"]
        if layers[i]["type"] == LAYER.FULLY_CONNECTED_INDEPENDENTLY_RECURRENT:
            out.append((i, slice(w, w + layers[i]["units"])))
            w += layers[i]["units"]
    return out


def set_recurrent_uniform(m, cfg, low=0.0, high=1.0):
    """Overwrites every IndRNN layer's recurrent weights with seeded draws of
    U(low, high)."""
    rs = recurrent_slices(cfg)
    if not rs:
        return
    rng = np.random.default_rng(cfg.get("recurrent_seed", 3))
    p = m.get_array("parameters")
    for _, s in rs:
        p[s] = rng.uniform(low, high, s.stop - s.start).astype(np.float32)
    m.set_array("parameters", p)


def shakedrop_layers(cfg):
    """[(layer index, probability)] of the residual layers that use ShakeDrop."""
    return [(i, l["dropout"][1]) for i, l in enumerate(cfg["layers"])
            if l["type"] == LAYER.RESIDUAL and l.get("dropout") and l["dropout"][0] == LAYER_DROPOUT.SHAKEDROP]


def n_inputs(cfg):
    return cfg["layers"][0]["units"]


def n_outputs(cfg):
    return cfg["layers"][-1]["units"]


def build_model(m, cfg, batch=None):
    """Calls the reference's construction sequence on ``m``
    (run/deep-learning/mnist.cpp L:43-80 is the model for the order)."""
    layers = cfg["layers"]
    extra = {}
    if any(l.get("cells") for l in layers):
        # LSTM layers: `units` memory blocks of `cells` cells (Layer_Parameters::unit_parameters[0], [1]).
        extra["layer_units2"] = [l.get("cells", 0) for l in layers]
    m.compile([l["type"] for l in layers], [l["units"] for l in layers],
              seq_w=cfg.get("seq_w", 1), model_type=cfg["model_type"], **extra)
    for i, l in enumerate(layers):
        if l.get("af") is not None:
            m.set_layer_activation_function(i, l["af"])
    for i, l in enumerate(layers):
        if l.get("norm"):
            m.Set__Layer_Normalization(i, l["norm"])
    for i, l in enumerate(layers):
        if l.get("dropout"):
            # scale_weights=False: with True the reference multiplies a fresh
            # layer's weights by 0/keep (v1/learner/dropout.cpp L:250-256).
            m.set_dropout(i, l["dropout"][0], l["dropout"][1], False)
    brn = cfg.get("brn")
    if brn:
        m.Set__Normalization_Momentum_Average(brn["momentum"])
        m.Set__Normalization_Epsilon(brn["eps"])
        m.Set__Batch_Renormalization_r_Correction_Maximum(brn["r_max"])
        m.Set__Batch_Renormalization_d_Correction_Maximum(brn["d_max"])
    m.set_loss_fn(cfg["loss"])
    m.set_optimizer(cfg["optimizer"])
    for k, v in cfg.get("hparams", {}).items():
        m.set_hparam(k, v)
    if cfg.get("time_delays"):
        m.set_seq_w(cfg["time_delays"])
    m.set_max_batch_size(batch or cfg["batch"])
    m.set_mp(cfg.get("mp", True))
    return m


def synthetic_batch(cfg, batch=None, step=0):
    """Seeded inputs and targets, shapes [B, T*n_in] and [B, T*n_out]."""
    B = batch or cfg["batch"]
    T = cfg.get("seq_w", 1)
    rng = np.random.default_rng([cfg.get("data_seed", 0), step])
    ni, no = n_inputs(cfg), n_outputs(cfg)
    if cfg["inputs"] == "uniform":
        X = rng.random((B, T * ni), dtype=np.float32)
    else:
        X = rng.standard_normal((B, T * ni), dtype=np.float32)
    if cfg["targets"] == "onehot":
        labels = rng.integers(0, no, size=(B, T))
        Y = np.zeros((B, T, no), dtype=np.float32)
        np.put_along_axis(Y, labels[..., None], 1.0, axis=2)
        Y = Y.reshape(B, T * no)
    else:
        Y = rng.standard_normal((B, T * no), dtype=np.float32)
    return X, Y


def dropout_masks(cfg, step=0):
    """One Bernoulli(keep) mask per unit of every layer that uses Bernoulli
    dropout, shared by the whole batch (v1/learner/bernoulli_mp.cpp L:58-95).
    Returns {layer_index: uint8[T*units]}."""
    rng = np.random.default_rng([cfg.get("mask_seed", 1), step])
    T = cfg.get("seq_w", 1)
    out = {}
    for i, l in enumerate(cfg["layers"]):
        d = l.get("dropout")
        if d and d[0] in (LAYER_DROPOUT.BERNOULLI, LAYER_DROPOUT.BERNOULLI_INVERTED):
            out[i] = (rng.random(T * l["units"]) < d[1]).astype(np.uint8)
    return out
