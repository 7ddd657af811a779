"""Test infrastructure, not product code.

ctypes view of ``oracle/_ref/libdlref.so`` (the reference library's own
OpenMP training step, compiled from its sources by ``oracle/Makefile``).  The
class mirrors the method names of the reference's ``DL::v1::Model``
(lib/deep-learning/v1/learner/model.hpp L:752-3384) so that a parity test can
drive this checker and the CUDA library through the same builder function.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libdlref.so")

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
_szp = np.ctypeslib.ndpointer(dtype=np.uint64, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")

DROPIN_LIB_PATH = os.path.join(_HERE, "_ref", "libdlref_dropin.so")

_libs = {}


def available() -> bool:
    return os.path.exists(LIB_PATH)


def dropin_available() -> bool:
    """The reference built with its step routed to libdlb200 (`make -C oracle dropin`)."""
    return os.path.exists(DROPIN_LIB_PATH)


def lib(path=None):
    path = path or LIB_PATH
    if path in _libs:
        return _libs[path]
    L = C.CDLL(path)
    vp, sz, i, f, d, cp = C.c_void_p, C.c_size_t, C.c_int, C.c_float, C.c_double, C.c_char_p
    sig = {
        "ref_model_create": (vp, []),
        "ref_model_destroy": (None, [vp]),
        "ref_compile": (i, [vp, sz, sz, i, _i32p, _szp, sz]),
        "ref_compile2": (i, [vp, sz, sz, i, _i32p, _szp, _szp, sz]),
        "ref_set_layer_activation_function": (i, [vp, sz, i]),
        "ref_set_layer_normalization": (i, [vp, sz, i]),
        "ref_set_dropout": (i, [vp, sz, i, f, i]),
        "ref_set_normalization_momentum_average": (i, [vp, f]),
        "ref_set_normalization_epsilon": (i, [vp, f]),
        "ref_set_brn_r_correction_maximum": (i, [vp, f]),
        "ref_set_brn_d_correction_maximum": (i, [vp, f]),
        "ref_set_loss_fn": (i, [vp, i]),
        "ref_set_optimizer": (i, [vp, i]),
        "ref_set_hparam": (i, [vp, cp, d]),
        "ref_get_hparam": (d, [vp, cp]),
        "ref_set_max_batch_size": (i, [vp, sz]),
        "ref_set_mp": (i, [vp, i]),
        "ref_set_weight_decay": (i, [vp, C.c_double]),
        "ref_set_clip_gradient": (i, [vp, i, C.c_double]),
        "ref_set_constraint_recurrent_weight": (i, [vp, sz, C.c_double, C.c_double]),
        "ref_set_l2": (i, [vp, C.c_double]),
        "ref_save": (i, [vp, cp, cp]),
        "ref_load": (i, [vp, cp, cp]),
        "ref_set_propagation": (i, [vp, i]),
        "ref_set_accu_fn": (i, [vp, i]),
        "ref_set_accu_var": (i, [vp, C.c_double]),
        "ref_compute_loss": (i, [vp, sz, _f32p]),
        "ref_get_accu": (C.c_double, [vp, sz]),
        "ref_seed_uout": (i, [vp, C.c_uint]),
        "ref_uout_draws": (i, [C.c_uint, sz, sz, _szp, _f32p, _f32p]),
        "ref_set_seq_w": (i, [vp, sz]),
        "ref_seed_weights": (i, [vp, C.c_uint]),
        "ref_initialize_weights_with_glorot_uniform": (i, [vp]),
        "ref_get_size": (sz, [vp, cp]),
        "ref_layer_info": (i, [vp, sz, _szp]),
        "ref_get_array": (i, [vp, cp, _f32p, sz]),
        "ref_set_array": (i, [vp, cp, _f32p, sz]),
        "ref_get_layer_norm": (i, [vp, sz, cp, _f32p, sz]),
        "ref_set_layer_norm": (i, [vp, sz, cp, _f32p, sz]),
        "ref_set_dropout_mask": (i, [vp, sz, _u8p, sz]),
        "ref_seed_shakedrop": (i, [vp, C.c_uint]),
        "ref_shakedrop_draws": (i, [C.c_uint, sz, sz, sz, _f32p, _u8p, _f32p, _f32p]),
        "ref_train_begin": (i, [vp, sz]),
        "ref_forward_pass": (i, [vp, sz, _f32p]),
        "ref_compute_error": (i, [vp, sz, _f32p]),
        "ref_backward_pass": (i, [vp, sz]),
        "ref_update_derivatives": (i, [vp, sz]),
        "ref_merge_derivatives": (i, [vp]),
        "ref_get_loss": (d, [vp]),
        "ref_reset_loss": (i, [vp]),
        "ref_update_weights": (i, [vp, sz, sz]),
        "ref_train_step": (i, [vp, sz, _f32p, _f32p, C.POINTER(d)]),
        "ref_get_layer_outputs": (i, [vp, sz, sz, _f32p]),
        "ref_get_layer_errors": (i, [vp, sz, sz, i, _f32p]),
        "ref_optimizer_sweep": (d, [i, sz, i, i, _f32p, _f32p, _f32p, _f32p, _f32p, _f64p]),
    }
    if path == DROPIN_LIB_PATH:
        sig["ref_set_b200"] = (i, [vp, i, i])
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _libs[path] = L
    return L


def _ck(rc, what):
    if rc != 0:
        raise RuntimeError(f"reference call failed: {what}")


class RefModel:
    """Same method names as the CUDA library's Python ``Model``."""

    backend = "reference-openmp"
    lib_path = None

    def __init__(self):
        self.L = lib(self.lib_path)
        self.h = self.L.ref_model_create()

    def close(self):
        if self.h:
            self.L.ref_model_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # --- construction ---------------------------------------------------
    def compile(self, layer_types, layer_units, seq_w=1, model_type=3, allowable_memory=48 << 30, layer_units2=None):
        lt = np.ascontiguousarray(layer_types, dtype=np.int32)
        lu = np.ascontiguousarray(layer_units, dtype=np.uint64)
        if layer_units2 is not None:
            lu2 = np.ascontiguousarray(layer_units2, dtype=np.uint64)
            _ck(self.L.ref_compile2(self.h, len(lt), seq_w, model_type, lt, lu, lu2, allowable_memory), "compile")
            return
        _ck(self.L.ref_compile(self.h, len(lt), seq_w, model_type, lt, lu, allowable_memory), "compile")

    def set_layer_activation_function(self, layer, af):
        _ck(self.L.ref_set_layer_activation_function(self.h, layer, af), "set_layer_activation_function")

    def Set__Layer_Normalization(self, layer, norm):
        _ck(self.L.ref_set_layer_normalization(self.h, layer, norm), "Set__Layer_Normalization")

    def set_dropout(self, layer, kind, value, scale_weights=False):
        _ck(self.L.ref_set_dropout(self.h, layer, kind, value, int(scale_weights)), "set_dropout")

    def Set__Normalization_Momentum_Average(self, v):
        _ck(self.L.ref_set_normalization_momentum_average(self.h, v), "momentum")

    def Set__Normalization_Epsilon(self, v):
        _ck(self.L.ref_set_normalization_epsilon(self.h, v), "epsilon")

    def Set__Batch_Renormalization_r_Correction_Maximum(self, v):
        _ck(self.L.ref_set_brn_r_correction_maximum(self.h, v), "r_max")

    def Set__Batch_Renormalization_d_Correction_Maximum(self, v):
        _ck(self.L.ref_set_brn_d_correction_maximum(self.h, v), "d_max")

    def set_loss_fn(self, loss):
        _ck(self.L.ref_set_loss_fn(self.h, loss), "set_loss_fn")

    def set_optimizer(self, opt):
        _ck(self.L.ref_set_optimizer(self.h, opt), "set_optimizer")

    def set_hparam(self, name, value):
        _ck(self.L.ref_set_hparam(self.h, name.encode(), float(value)), f"set_hparam {name}")

    def get_hparam(self, name):
        return self.L.ref_get_hparam(self.h, name.encode())

    def set_max_batch_size(self, b):
        _ck(self.L.ref_set_max_batch_size(self.h, b), "set_max_batch_size")

    def set_mp(self, on):
        _ck(self.L.ref_set_mp(self.h, int(on)), "set_mp")

    def set_seq_w(self, delays):
        _ck(self.L.ref_set_seq_w(self.h, delays), "set_seq_w")

    def set_propagation(self, state):
        """0: inference, 1: training (PROPAGATION, v1/data/enum/propagation.hpp)."""
        _ck(self.L.ref_set_propagation(self.h, int(state)), "set_propagation")

    def set_accu_fn(self, fn):
        _ck(self.L.ref_set_accu_fn(self.h, int(fn)), "set_accu_fn")

    def set_accu_var(self, v):
        _ck(self.L.ref_set_accu_var(self.h, float(v)), "set_accu_var")

    def compute_loss(self, batch, Y):
        Y = np.ascontiguousarray(Y, dtype=np.float32)
        _ck(self.L.ref_compute_loss(self.h, batch, Y), "compute_loss")

    def get_accu(self, rows_total):
        return float(self.L.ref_get_accu(self.h, rows_total))

    def seed_uout(self, seed):
        _ck(self.L.ref_seed_uout(self.h, seed), "seed_uout")

    def set_weight_decay(self, value):
        _ck(self.L.ref_set_weight_decay(self.h, float(value)), "set_weight_decay")

    def save(self, path_params, path_spec):
        _ck(self.L.ref_save(self.h, path_params.encode(), path_spec.encode()), "save")

    def load(self, path_params, path_spec):
        _ck(self.L.ref_load(self.h, path_params.encode(), path_spec.encode()), "load")

    def set_l2(self, value):
        _ck(self.L.ref_set_l2(self.h, float(value)), "set_l2")

    def set_clip_gradient(self, use, value):
        _ck(self.L.ref_set_clip_gradient(self.h, int(bool(use)), float(value)), "set_clip_gradient")

    def set_constraint_recurrent_weight(self, layer, lower, upper):
        _ck(self.L.ref_set_constraint_recurrent_weight(self.h, layer, float(lower), float(upper)),
            "set_constraint_recurrent_weight")

    def seed_weights(self, seed):
        _ck(self.L.ref_seed_weights(self.h, seed), "seed")

    def initialize_weights_with_glorot_uniform(self):
        _ck(self.L.ref_initialize_weights_with_glorot_uniform(self.h), "glorot")

    # --- state ----------------------------------------------------------
    def size(self, name):
        v = self.L.ref_get_size(self.h, name.encode())
        if v == 2**64 - 1:
            raise KeyError(name)
        return int(v)

    def layer_info(self, layer):
        out = np.zeros(10, dtype=np.uint64)
        _ck(self.L.ref_layer_info(self.h, layer, out), "layer_info")
        keys = ("type", "n_out", "first_connection", "last_connection", "first_bias", "last_bias",
                "norm", "dropout", "group", "first_norm_unit")
        return {k: int(v) for k, v in zip(keys, out)}

    def get_array(self, name, n=None):
        n = self.size("total_parameters") if n is None else n
        out = np.empty(n, dtype=np.float32)
        _ck(self.L.ref_get_array(self.h, name.encode(), out, n), f"get_array {name}")
        return out

    def set_array(self, name, arr):
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        _ck(self.L.ref_set_array(self.h, name.encode(), arr, arr.size), f"set_array {name}")

    def get_layer_norm(self, layer, name, n):
        out = np.empty(n, dtype=np.float32)
        _ck(self.L.ref_get_layer_norm(self.h, layer, name.encode(), out, n), f"get_layer_norm {name}")
        return out

    def set_layer_norm(self, layer, name, arr):
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        _ck(self.L.ref_set_layer_norm(self.h, layer, name.encode(), arr, arr.size), f"set_layer_norm {name}")

    def set_dropout_mask(self, layer, mask):
        mask = np.ascontiguousarray(mask, dtype=np.uint8)
        _ck(self.L.ref_set_dropout_mask(self.h, layer, mask, mask.size), "set_dropout_mask")

    def seed_shakedrop(self, seed):
        _ck(self.L.ref_seed_shakedrop(self.h, seed), "seed_shakedrop")

    # --- step -----------------------------------------------------------
    def train_begin(self, batch):
        _ck(self.L.ref_train_begin(self.h, batch), "train_begin")

    def forward_pass(self, batch, X):
        X = np.ascontiguousarray(X, dtype=np.float32)
        self._x = X
        _ck(self.L.ref_forward_pass(self.h, batch, X), "forward_pass")

    def compute_error(self, batch, Y):
        Y = np.ascontiguousarray(Y, dtype=np.float32)
        self._y = Y
        _ck(self.L.ref_compute_error(self.h, batch, Y), "compute_error")

    def backward_pass(self, batch):
        _ck(self.L.ref_backward_pass(self.h, batch), "backward_pass")

    def update_derivatives(self, batch):
        _ck(self.L.ref_update_derivatives(self.h, batch), "update_derivatives")

    def merge_derivatives(self):
        _ck(self.L.ref_merge_derivatives(self.h), "merge")

    def get_loss(self):
        return self.L.ref_get_loss(self.h)

    def reset_loss(self):
        _ck(self.L.ref_reset_loss(self.h), "reset_loss")

    def update_weights(self, batch, training_size):
        _ck(self.L.ref_update_weights(self.h, batch, training_size), "update_weights")

    def train_step(self, batch, X, Y):
        X = np.ascontiguousarray(X, dtype=np.float32)
        Y = np.ascontiguousarray(Y, dtype=np.float32)
        loss = C.c_double(0.0)
        _ck(self.L.ref_train_step(self.h, batch, X, Y, C.byref(loss)), "train_step")
        return loss.value

    def get_layer_outputs(self, layer, batch):
        n_out = self.layer_info(layer)["n_out"]
        T = self.size("seq_w")
        out = np.empty((T, batch, n_out), dtype=np.float32)
        _ck(self.L.ref_get_layer_outputs(self.h, layer, batch, out), "get_layer_outputs")
        return out

    def get_layer_errors(self, layer, batch, which=0):
        n_out = self.layer_info(layer)["n_out"]
        T = self.size("seq_w")
        out = np.empty((T, batch, n_out), dtype=np.float32)
        _ck(self.L.ref_get_layer_errors(self.h, layer, batch, which, out), "get_layer_errors")
        return out


class DropinModel(RefModel):
    """The reference's own Model class, built with its step entry points routed to
    libdlb200 (oracle/dropin_patch.py, oracle/dropin_glue.cpp): construction and
    the step go through the reference's methods; after `set_b200(True)` the
    numerical work of the step runs in the CUDA library."""

    backend = "reference-with-dlb200"
    lib_path = DROPIN_LIB_PATH

    def set_b200(self, on, device=0):
        _ck(self.L.ref_set_b200(self.h, int(bool(on)), device), "set_b200")


def uout_draws(seed, betas, rows, widths):
    """[noise [rows, width] per layer] that a serial reference forward pass
    draws after RefModel.seed_uout(seed)."""
    w = np.ascontiguousarray(widths, dtype=np.uint64)
    b = np.ascontiguousarray(betas, dtype=np.float32)
    out = np.empty(int(rows * w.sum()), dtype=np.float32)
    _ck(lib().ref_uout_draws(seed, len(w), rows, w, b, out), "uout_draws")
    res, o = [], 0
    for n in w:
        res.append(out[o:o + rows * int(n)].reshape(rows, int(n)).copy())
        o += rows * int(n)
    return res


def shakedrop_draws(seed, probabilities, rows, width):
    """(masks [n, rows], forward [n, rows, width], backward [n, rows, width]) that
    a serial reference step draws after RefModel.seed_shakedrop(seed)."""
    p = np.ascontiguousarray(probabilities, dtype=np.float32)
    n = p.size
    masks = np.zeros((n, rows), np.uint8)
    fwd = np.ones((n, rows, width), np.float32)
    bwd = np.ones((n, rows, width), np.float32)
    _ck(lib().ref_shakedrop_draws(seed, n, rows, width, p, masks, fwd, bwd), "shakedrop_draws")
    return masks, fwd, bwd


def optimizer_sweep(optimizer, p, grad_fill, m, v, vhat, steps, hparams, use_mp=True):
    """Runs the reference's flat update loop in place; returns seconds."""
    hp = np.ascontiguousarray(hparams, dtype=np.float64)
    return lib().ref_optimizer_sweep(optimizer, p.size, steps, int(use_mp), p, grad_fill, m, v, vhat, hp)
