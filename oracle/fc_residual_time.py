"""Test infrastructure, not product code.

CPU restatement (numpy fp32) of residual blocks of fully connected layers inside
a time-stepped model (seq_w > 1), on top of oracle/fc_residual.py.  Pinned
against the compiled reference in tests/test_oracle_residual.py.

The reference runs such a model layer by layer and, inside a layer, time step
by time step (Recurrent__Forward_Pass__Residual__OpenMP and
Recurrent__Forward_Pass__Residual__Layer__OpenMP,
lib/deep-learning/v1/learner/fwp_rec_mp.cpp L:510-700; backward
v1/learner/bwp_rec_mp.cpp): without recurrent connections the time steps only
share the weights, so a step over T time steps is T feed-forward steps whose
gradients add up, with

  * batch-renormalization statistics and running averages of their own per time
    step (allocate.cpp L:1348-1356: [T, units] arrays),
  * Bernoulli masks mask[t * width + u] per time step,
  * ShakeDrop row flags flag[t * batch + b] and draws [T * batch, width]
    (fwp_mp.cpp L:4935-4955),
  * the error on the time steps t >= n_time_delay, each with the divisor of one
    batch (compute_error_rec_mp, v1/learner/compute_error_mp.cpp L:143-265); with
    a softmax output the error of every time step is taken against the target of
    time step 0 (L:237-247), which is what the reference computes.

Layers are fully connected (no recurrent layer types).  Inputs are rows of
T * n_in values, outputs [T, rows, units] as in the reference.
"""
from __future__ import annotations

import numpy as np

from fc_residual import LAYER_RESIDUAL, ResidualOracleModel
from fc_step import AF_SOFTMAX, LOSS_CROSS_ENTROPY, NORM_NONE, OracleModel, f32, loss_and_delta

# What one feed-forward pass leaves in a layer's dict and a later pass reads.
_PER_STEP = ("A", "IN", "Y", "Z", "norm_in", "x_hat", "delta")


class ResidualTimeOracleModel(ResidualOracleModel):
    backend = "numpy-restatement-residual-time"

    def compile(self, layer_types, layer_units, seq_w=1, model_type=4, allowable_memory=None):
        self.T = int(seq_w)
        self.time_delay = 0
        ResidualOracleModel.compile(self, layer_types, layer_units, 1, model_type, allowable_memory)

    def set_seq_w(self, delays):
        self.time_delay = int(delays)

    def size(self, name):
        if name == "seq_w":
            return self.T
        return super().size(name)

    # --- per-time-step views ----------------------------------------------
    def _layout(self):
        super()._layout()
        for l in self.layers:
            if l["norm"] != NORM_NONE and "states" not in l:
                n = l["norm_units"]
                l["states"] = [dict(mean_average=np.zeros(n, f32), variance_average=np.ones(n, f32))
                               for _ in range(self.T)]

    def _enter(self, t, batch):
        """Makes the layer dicts those of time step t."""
        for l in self.layers:
            saved = l.setdefault("steps", [dict() for _ in range(self.T)])[t]
            for k in _PER_STEP:
                if k in saved:
                    l[k] = saved[k]
                else:
                    l.pop(k, None)
            if "states" in l:
                l["state"] = l["states"][t]
            if l.get("mask_all") is not None:
                w = l["mask_all"].size // self.T
                l["mask"] = l["mask_all"][t * w:(t + 1) * w]
            if l.get("sd_all") is not None:
                m, fw, bw = l["sd_all"]
                rows = m.size // self.T
                l["sd_mask"] = m[t * rows:(t + 1) * rows]
                l["sd_fwd"] = fw[t * rows:(t + 1) * rows]
                l["sd_bwd"] = bw[t * rows:(t + 1) * rows]

    def _leave(self, t):
        for l in self.layers:
            l["steps"][t] = {k: l[k] for k in _PER_STEP if k in l}

    def set_dropout_mask(self, layer, mask):
        """Flags of all time steps, [T * width]."""
        self.layers[layer]["mask_all"] = np.asarray(mask, np.uint8).astype(bool)

    def set_shakedrop_noise(self, layer, mask, forward, backward):
        """Row flags [T * rows] and draws [T * rows, width] of one residual layer."""
        self.layers[layer]["sd_all"] = (np.asarray(mask, np.uint8).astype(bool), np.asarray(forward, f32),
                                        np.asarray(backward, f32))

    def get_layer_norm(self, layer, name, n):
        l = self.layers[layer]
        if name in ("scale", "shift"):
            return super().get_layer_norm(layer, name, n)
        key = {"r_correction": "r", "d_correction": "d"}.get(name, name)
        return np.concatenate([st[key] for st in l["states"]])

    def get_accu(self, rows_total):
        return OracleModel.get_accu(self, rows_total * (self.T - self.time_delay))

    def set_layer_norm(self, layer, name, arr):
        l = self.layers[layer]
        if name in ("scale", "shift"):
            sl = self._gamma_slice(l) if name == "scale" else self._beta_slice(l)
            self.params[sl] = np.asarray(arr, f32)
            return
        key = {"r_correction": "r", "d_correction": "d"}.get(name, name)
        for st, part in zip(l["states"], np.asarray(arr, f32).reshape(self.T, -1)):
            st[key] = part.copy()

    # --- step ---------------------------------------------------------------
    def forward_pass(self, batch, X):
        n_in = self.layers[0]["units"]
        x = np.asarray(X[:batch], f32).reshape(batch, self.T, n_in)
        for t in range(self.T):
            self._enter(t, batch)
            ResidualOracleModel.forward_pass(self, batch, np.ascontiguousarray(x[:, t]))
            self._leave(t)

    def compute_error(self, batch, Y):
        o = self.layers[-1]
        W = o["units"]
        y = np.asarray(Y[:batch], f32).reshape(batch, self.T, W)
        for t in range(self.T):
            self._enter(t, batch)
            if t >= self.time_delay:
                OracleModel.compute_error(self, batch, np.ascontiguousarray(y[:, t]))
                if o["af"] == AF_SOFTMAX:
                    # The softmax branch of compute_error_rec_mp reads the target of
                    # time step 0 for every time step (`Ym[i][k]`,
                    # compute_error_mp.cpp L:237-247); the loss reads the right one.
                    _, o["delta"] = loss_and_delta(self.loss, o["af"], o["Y"], o["A"],
                                                   np.ascontiguousarray(y[:, 0]), self.global_rows)
            else:
                o["delta"] = np.zeros((batch, W), f32)
            self._leave(t)

    def backward_pass(self, batch):
        for t in range(self.T - 1, -1, -1):
            self._enter(t, batch)
            ResidualOracleModel.backward_pass(self, batch)
            self._leave(t)

    def update_derivatives(self, batch):
        for t in range(self.T):
            self._enter(t, batch)
            ResidualOracleModel.update_derivatives(self, batch)
            self._leave(t)

    def compute_loss(self, batch, Y):
        o = self.layers[-1]
        W = o["units"]
        y = np.asarray(Y[:batch], f32).reshape(batch, self.T, W)
        for t in range(self.time_delay, self.T):
            self._enter(t, batch)
            OracleModel.compute_loss(self, batch, np.ascontiguousarray(y[:, t]))
            self._leave(t)

    def get_loss(self):
        if self.loss_rows == 0:
            return 1.0
        total = float(self.allreduce(np.array([self.loss_sum], np.float64))[0])
        rows = self.loss_rows * self.world
        if self.loss == LOSS_CROSS_ENTROPY:
            return total / rows
        return total / (rows * self.layers[-1]["units"])

    def _stack(self, layer, key, batch):
        return np.stack([self.layers[layer]["steps"][t][key][:batch] for t in range(self.T)])

    def get_layer_outputs(self, layer, batch):
        return self._stack(layer, "A", batch)

    def get_layer_errors(self, layer, batch, which=0):
        return self._stack(layer, "delta", batch)
