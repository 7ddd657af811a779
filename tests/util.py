"""Shared helpers of the parity tests: error measures and a step tracer that
drives any backend exposing the reference's Model method names."""
from __future__ import annotations

import numpy as np

import configs


def rel_l2(a, b):
    """||a - b||_2 / ||b||_2 in float64."""
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / (den if den > 0 else 1.0))


def rel_max(a, b):
    """max|a - b| / max|b| in float64."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    den = np.abs(b).max()
    return float(np.abs(a - b).max() / (den if den > 0 else 1.0))


def rowwise_rel_l2(a, b):
    """Largest ||a[r] - b[r]||_2 / ||b[r]||_2 over the rows r of two [rows, n]
    tensors, in float64: a tensor-wide norm hides a row whose values are far
    below the rest, this does not.  Rows of b that are all zero are skipped."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    a = a.reshape(b.shape[0], -1)
    b = b.reshape(b.shape[0], -1)
    den = np.linalg.norm(b, axis=1)
    num = np.linalg.norm(a - b, axis=1)
    live = den > 0
    return float((num[live] / den[live]).max()) if live.any() else 0.0


def build(model, cfg, params=None, seed=None):
    configs.build_model(model, cfg)
    if params is not None:
        model.set_array("parameters", params)
    elif seed is not None:
        model.seed_weights(seed)
        model.initialize_weights_with_glorot_uniform()
    return model


def trace(model, cfg, steps=1, X=None, Y=None, masks=None):
    """Runs `steps` training steps on fixed inputs; returns the tensors the
    parity bar names: activations, errors and gradients of step 1, parameters
    after step 1 and after the last step, and the loss of every step."""
    B = cfg["batch"]
    if X is None:
        X, Y = configs.synthetic_batch(cfg)
    if masks is None:
        masks = configs.dropout_masks(cfg)
    model.train_begin(B)
    for li, mk in masks.items():
        model.set_dropout_mask(li, mk)
    nl = len(cfg["layers"])
    out = {}
    if hasattr(model, "reset_loss"):
        model.reset_loss()
    model.forward_pass(B, X)
    for li in range(1, nl):
        out[f"act{li}"] = model.get_layer_outputs(li, B).reshape(B, -1)
    model.compute_error(B, Y)
    model.backward_pass(B)
    for li in range(1, nl):
        out[f"delta{li}"] = model.get_layer_errors(li, B).reshape(B, -1)
    model.update_derivatives(B)
    model.merge_derivatives()
    losses = [model.get_loss()]
    out["grads"] = model.get_array("derivatives")
    model.update_weights(B, B)
    out["params1"] = model.get_array("parameters")
    for _ in range(1, steps):
        losses.append(model.train_step(B, X, Y))
    out["params_last"] = model.get_array("parameters")
    out["losses"] = np.asarray(losses, np.float64)
    for li, l in enumerate(cfg["layers"]):
        if l.get("norm"):
            n = l["units"] * cfg.get("seq_w", 1)
            out[f"mean_average{li}"] = model.get_layer_norm(li, "mean_average", n)
            out[f"variance_average{li}"] = model.get_layer_norm(li, "variance_average", n)
    return out


def copy_trained_state(src, dst, cfg):
    """Parameters and running averages of `src` into `dst`, so that a pass of
    both starts from the same bits."""
    dst.set_array("parameters", src.get_array("parameters"))
    for li, l in enumerate(cfg["layers"]):
        if l.get("norm"):
            n = l["units"] * cfg.get("seq_w", 1)
            for name in ("mean_average", "variance_average"):
                dst.set_layer_norm(li, name, src.get_layer_norm(li, name, n))


def compare(got, want, keys=None):
    """{key: (rel_l2, rel_max)} over the common keys."""
    keys = keys or [k for k in want if k in got]
    return {k: (rel_l2(got[k], want[k]), rel_max(got[k], want[k])) for k in keys}


KINKED = (3, 14, 16, 17)  # ELU, LEAKY_RELU, RELU, SELU: f' jumps at 0 (in the reference's formulas)


def near_kink(oracle_model, cfg, X, masks, band=1e-5):
    """Number of hidden pre-activations within `band` of 0 for activations whose
    derivative jumps there.  Such an element's derivative branch (x < 0) is
    decided by the last bits of a long sum, so two correct implementations (or
    the reference with two thread counts) may take different branches; the
    strict one-step comparisons use seeds where there is none."""
    B = cfg["batch"]
    for li, mk in masks.items():
        oracle_model.set_dropout_mask(li, mk)
    oracle_model.forward_pass(B, X)
    n = 0
    for li, l in enumerate(cfg["layers"][1:-1], start=1):
        if l.get("af") in KINKED and "Y" in oracle_model.layers[li]:
            lay = oracle_model.layers[li]
            n += int((np.abs(lay["PRE"] if "PRE" in lay else lay["Y"]) < band).sum())
    return n


def kink_free_parameters(cfg, make_oracle, X, masks, scale, tries=64, band=1e-5, prepare=None):
    """Seeded random weights (first seed for which no pre-activation lies on a
    derivative jump).  Returns (params, seed).  `prepare(model)` runs before the
    probing forward pass (e.g. to hand over ShakeDrop noise)."""
    for seed in range(tries):
        ora = build(make_oracle(), cfg)
        if prepare:
            prepare(ora)
        rng = np.random.default_rng(seed)
        p0 = ora.get_array("parameters")
        nw = ora.size("total_weights")
        p0[:nw] = (rng.standard_normal(nw) * scale).astype(np.float32)
        ora.set_array("parameters", p0)
        if near_kink(ora, cfg, X, masks, band) == 0:
            return p0, seed
    raise AssertionError("no kink-free seed found")


def shakedrop_step_draws(cfg, step, rows=None):
    """Draws of training step `step` for every ShakeDrop layer, taken from the
    reference's own generator classes (oracle/_ref).  Seed of a step =
    cfg['shakedrop_seed'] + 1000 * step."""
    import ref_binding

    layers = configs.shakedrop_layers(cfg)
    # One factor per element of a block's output: the width of the block's last
    # layer (the replay takes one width for all blocks).
    widths = {cfg["layers"][li + cfg["layers"][li]["units"]]["units"] for li, _ in layers}
    assert len(widths) == 1, "blocks of different widths need draws of their own"
    width = widths.pop()
    seed = cfg.get("shakedrop_seed", 2) + 1000 * step
    masks, fwd, bwd = ref_binding.shakedrop_draws(seed, [p for _, p in layers], rows or cfg["batch"], width)
    return seed, {li: (masks[k], fwd[k], bwd[k]) for k, (li, _) in enumerate(layers)}


def set_step_noise(model, cfg, step, draws=None):
    """Gives one training step its ShakeDrop noise: the reference is reseeded,
    every other backend receives the arrays the reference will draw."""
    if not configs.shakedrop_layers(cfg):
        return
    if draws is None:
        seed, arrays = shakedrop_step_draws(cfg, step)
    else:
        seed, arrays = draws
    if hasattr(model, "seed_shakedrop"):
        model.seed_shakedrop(seed)
    else:
        for li, (mk, fw, bw) in arrays.items():
            model.set_shakedrop_noise(li, mk, fw, bw)


def trace_noisy(model, cfg, steps=1, X=None, Y=None, draws=None):
    """`trace` for workloads whose steps consume ShakeDrop noise; `draws` maps a
    step index to (seed, {layer: (mask, forward, backward)})."""
    B = cfg["batch"]
    if X is None:
        X, Y = configs.synthetic_batch(cfg)
    model.train_begin(B)
    nl = len(cfg["layers"])
    out = {}
    losses = []
    for step in range(steps):
        set_step_noise(model, cfg, step, draws[step] if draws else None)
        if hasattr(model, "reset_loss"):
            model.reset_loss()
        model.forward_pass(B, X)
        if step == 0:
            for li in range(1, nl):
                out[f"act{li}"] = model.get_layer_outputs(li, B).reshape(B, -1)
        model.compute_error(B, Y)
        model.backward_pass(B)
        if step == 0:
            for li in range(1, nl):
                if cfg["layers"][li]["type"] == 3:
                    out[f"delta{li}"] = model.get_layer_errors(li, B).reshape(B, -1)
        model.update_derivatives(B)
        model.merge_derivatives()
        losses.append(model.get_loss())
        if step == 0:
            out["grads"] = model.get_array("derivatives")
        model.update_weights(B, B)
        if step == 0:
            out["params1"] = model.get_array("parameters")
    out["params_last"] = model.get_array("parameters")
    out["losses"] = np.asarray(losses, np.float64)
    return out
