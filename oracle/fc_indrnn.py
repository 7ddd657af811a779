"""Test infrastructure, not product code.

CPU restatement (numpy fp32) of the reference's recurrent path for stacks of
independently recurrent (IndRNN) and fully connected layers, on top of
oracle/fc_step.py.  Pinned against the compiled reference in
tests/test_oracle_indrnn.py and against tests/golden/indrnn_*.npz.

Layer-major, time-minor as the reference (v1/learner/fwp_rec_mp.cpp L:29-110,
L:335-348): for a layer, every time step t runs FC product, bias or batch
renormalization with statistics of its own per t, then for an IndRNN layer
(L:762-800)
    pre_t = y_t + u * h_{t-1}   (t = 0: pre_0 = y_0),   h_t = f(pre_t).
Tensors are [T, rows, units]; a row of the caller's input holds T * n values.

Backward (v1/learner/bwp_rec_mp.cpp L:29-110, L:386-394; bwp_mp.cpp
L:1188-1263), t from T-1 down to 0:
    f'_t = f'(pre_t, h_t);  delta_t = dA_t f'_t;
    dAF_t = delta_t + u f'_t dAF_{t+1}     (t = T-1: dAF = delta)
and what follows (normalization backward, weight gradients, the error passed
down) uses dAF.  du[h] += sum over rows and t >= 1 of h_{t-1} dAF_t
(v1/learner/update_derivative_rec_mp.cpp L:460-487).  The output error exists
only for t >= n_time_delay (v1/learner/compute_error_mp.cpp L:143-265).  After
the update the recurrent weights are clamped to +-mag^(1/T), mag = 2 with the
reference's default clip_gradient (v1/ops/constraints/constraint.cpp L:64-95,
L:271-289).  Parameter order: an IndRNN layer's u follows its W
(v1/learner/connections_prepare.cpp L:46-81); its gamma starts at 0.1
(v1/learner/allocate.cpp L:1485-1507).
"""
from __future__ import annotations

import numpy as np

import fc_step
from fc_step import (AF_SOFTMAX, LOSS_CROSS_ENTROPY, NORM_NONE, OracleModel, af_derive, af_fire, brn_backward, brn_forward,
                     f32, loss_and_delta, optimizer_scalars, optimizer_update, softmax)

LAYER_FC, LAYER_INDRNN = 3, 4


class IndRnnOracleModel(OracleModel):
    backend = "numpy-restatement-indrnn"

    def compile(self, layer_types, layer_units, seq_w=1, model_type=4, allowable_memory=None):
        self.T = int(seq_w)
        self.time_delay = 0
        self.layers = [dict(type=int(t), units=int(u), af=None, norm=NORM_NONE, dropout=(0, 0.0), mask=None)
                       for t, u in zip(layer_types, layer_units)]
        self._layout()

    def set_seq_w(self, delays):
        self.time_delay = int(delays)

    def _layout(self):
        w = 0
        for i in range(1, len(self.layers)):
            l = self.layers[i]
            l["fan_in"] = self.layers[i - 1]["units"]
            l["first_connection"] = w
            w += l["units"] * l["fan_in"]
            if l["type"] == LAYER_INDRNN:
                l["first_recurrent"] = w
                w += l["units"]
            l["last_connection"] = w
        self.total_weights = w
        b = w
        for l in self.layers[1:]:
            l["first_bias"], b = b, b + l["units"]
            l["last_bias"] = b
        self.total_bias = b - w
        any_norm = any(l["norm"] != NORM_NONE for l in self.layers)
        u = 0
        for l in self.layers:
            l["first_norm_unit"], u = u, u + l["units"]
        self.total_norm = u if any_norm else 0
        P = self.total_weights + self.total_bias + 2 * self.total_norm
        old = self.params
        self.params = np.zeros(P, f32)
        if old is not None:
            k = self.total_weights + self.total_bias
            self.params[:k] = old[:k]
        gs = self.total_weights + self.total_bias
        if self.total_norm:
            for l in self.layers:
                g0 = gs + l["first_norm_unit"]
                self.params[g0:g0 + l["units"]] = 0.1 if l["type"] == LAYER_INDRNN else 1.0
        self.grads = np.zeros(P, f32)
        self.m1, self.m2, self.m2hat = np.zeros(P, f32), np.zeros(P, f32), np.zeros(P, f32)
        for l in self.layers:
            if l["norm"] != NORM_NONE and "states" not in l:
                n = l["units"]
                l["states"] = [dict(mean_average=np.zeros(n, f32), variance_average=np.ones(n, f32))
                               for _ in range(self.T)]

    def size(self, name):
        if name == "seq_w":
            return self.T
        return super().size(name)

    def get_layer_norm(self, layer, name, n):
        l = self.layers[layer]
        if name in ("scale", "shift"):
            return super().get_layer_norm(layer, name, n)
        key = {"r_correction": "r", "d_correction": "d"}.get(name, name)
        return np.concatenate([st[key] for st in l["states"]])

    def set_layer_norm(self, layer, name, arr):
        l = self.layers[layer]
        key = {"r_correction": "r", "d_correction": "d"}.get(name, name)
        for st, part in zip(l["states"], np.asarray(arr, f32).reshape(self.T, -1)):
            st[key] = part.copy()

    def _W(self, l):
        n = l["units"] * l["fan_in"]
        return self.params[l["first_connection"]:l["first_connection"] + n].reshape(l["units"], l["fan_in"])

    def _u(self, l):
        return self.params[l["first_recurrent"]:l["first_recurrent"] + l["units"]]

    # --- step -----------------------------------------------------------
    def forward_pass(self, batch, X):
        T = self.T
        n_in = self.layers[0]["units"]
        a = np.ascontiguousarray(np.asarray(X[:batch], f32).reshape(batch, T, n_in).transpose(1, 0, 2))
        # Dropout on the inputs, on the model's copy of the batch and per time step
        # (Model::assign_inputs_rec_mp, v1/learner/assign_inputs.cpp L:219-266):
        # the Bernoulli kinds by the input layer's mask in training, the plain
        # kind by its keep probability at inference.
        kind0, value0 = self.layers[0]["dropout"]
        if kind0 in (fc_step.DROPOUT_BERNOULLI, fc_step.DROPOUT_BERNOULLI_INVERTED):
            for t in range(T):
                if self.training:
                    a[t] = fc_step.apply_dropout(a[t], kind0, value0, self.layers[0]["mask"][t * n_in:(t + 1) * n_in])
                elif kind0 == fc_step.DROPOUT_BERNOULLI:
                    a[t] = (a[t] * f32(value0)).astype(f32)
        self.layers[0]["A"] = a
        for i in range(1, len(self.layers)):
            l = self.layers[i]
            H = l["units"]
            W = self._W(l)
            Z = np.empty((T, batch, H), f32)
            Y = np.empty((T, batch, H), f32)
            XH = np.empty((T, batch, H), f32)
            A = np.empty((T, batch, H), f32)
            PRE = np.empty((T, batch, H), f32)
            for t in range(T):
                z = (a[t] @ W.T).astype(f32)
                if l["norm"] == NORM_NONE:
                    z = (z + self.params[l["first_bias"]:l["last_bias"]]).astype(f32)
                    y = z
                elif not self.training:
                    # The running averages of this time step (fwp_mp.cpp L:4461-4491).
                    st = l["states"][t]
                    y = (self.params[self._gamma_slice(l)] * ((z - st["mean_average"]) / st["variance_average"])
                         + self.params[self._beta_slice(l)]).astype(f32)
                else:
                    st = l["states"][t]
                    st["gamma"] = self.params[self._gamma_slice(l)]
                    st["beta"] = self.params[self._beta_slice(l)]
                    XH[t], y = brn_forward(z, st, self._brn_of(l), self.global_rows, self.allreduce)
                Z[t], Y[t] = z, y
                if l["type"] == LAYER_INDRNN:
                    PRE[t] = y if t == 0 else (y + self._u(l) * A[t - 1]).astype(f32)
                    A[t] = af_fire(l["af"], PRE[t])
                else:
                    PRE[t] = y
                    A[t] = softmax(y) if l["af"] == AF_SOFTMAX else af_fire(l["af"], y)
                # Bernoulli dropout of time step t: flags mask[t * units + u], applied
                # in place, so that the recurrence of step t + 1 reads the masked
                # output (fwp_mp.cpp L:1228-1262, L:4842-4868); at inference the
                # keep probability scales instead (fwp_rec_mp.cpp L:299-312).
                kind, value = l["dropout"]
                if kind == fc_step.DROPOUT_UOUT and i + 1 < len(self.layers) and self.training:
                    # UOut of time step t, in place like the masks: draws [T * batch, units],
                    # rows t * batch .. of them (fwp_mp.cpp L:1252-1257, L:4959-4985).
                    nz = l["noise"].reshape(T, -1, H)[t, :batch]
                    A[t] = fc_step.apply_dropout(A[t], kind, value, None, nz)
                if kind in (fc_step.DROPOUT_BERNOULLI, fc_step.DROPOUT_BERNOULLI_INVERTED) and i + 1 < len(self.layers):
                    if not self.training:
                        if kind == fc_step.DROPOUT_BERNOULLI:
                            A[t] = (A[t] * f32(value)).astype(f32)
                    else:
                        A[t] = fc_step.apply_dropout(A[t], kind, value, l["mask"][t * H:(t + 1) * H])
            l.update(Z=Z, Y=Y, XH=XH, A=A, PRE=PRE)
            a = A

    def compute_error(self, batch, Y):
        o = self.layers[-1]
        T, n_out = self.T, o["units"]
        y = np.asarray(Y[:batch], f32).reshape(batch, T, n_out).transpose(1, 0, 2)
        delta = np.zeros((T, batch, n_out), f32)
        for t in range(self.time_delay, T):
            total, delta[t] = loss_and_delta(self.loss, o["af"], o["Y"][t], o["A"][t], y[t], self.global_rows)
            self.loss_sum += total
            if o["af"] == AF_SOFTMAX:
                # The softmax branch reads the target of time step 0 for every time
                # step (`Ym[i][k]`, compute_error_mp.cpp L:237-247); the loss above
                # reads the right one.
                _, delta[t] = loss_and_delta(self.loss, o["af"], o["Y"][t], o["A"][t], y[0], self.global_rows)
        o["delta"] = delta
        self.loss_rows += batch * (T - self.time_delay)

    def backward_pass(self, batch):
        T = self.T
        for gi in range(len(self.layers) - 1, 1, -1):
            nxt, l = self.layers[gi], self.layers[gi - 1]
            Wn = self._W(nxt)
            dA = np.stack([(nxt["delta"][t] @ Wn).astype(f32) for t in range(T)])
            delta = np.empty_like(dA)
            if l["type"] == LAYER_INDRNN:
                u = self._u(l)
                dAF = np.empty_like(dA)
                for t in range(T - 1, -1, -1):
                    fp = af_derive(l["af"], l["PRE"][t], l["A"][t])
                    d = (dA[t] * fp).astype(f32)
                    dAF[t] = d if t == T - 1 else (d + u * fp * dAF[t + 1]).astype(f32)
                du = np.zeros(l["units"], np.float64)
                for t in range(1, T):
                    du += (l["A"][t - 1].astype(np.float64) * dAF[t]).sum(axis=0)
                self.grads[l["first_recurrent"]:l["first_recurrent"] + l["units"]] += du.astype(f32)
                e = dAF
            else:
                e = np.stack([(dA[t] * af_derive(l["af"], l["Y"][t], l["A"][t])).astype(f32) for t in range(T)])
            for t in range(T - 1, -1, -1):
                if l["norm"] != NORM_NONE:
                    delta[t], dg, db = brn_backward(e[t], l["Z"][t], l["XH"][t], l["states"][t], self.global_rows,
                                                    self.allreduce)
                    self.grads[self._gamma_slice(l)] += dg
                    self.grads[self._beta_slice(l)] += db
                else:
                    delta[t] = e[t]
            l["delta"] = delta

    def update_derivatives(self, batch):
        T = self.T
        for i in range(1, len(self.layers)):
            l = self.layers[i]
            x = self.layers[i - 1]["A"]
            n = l["units"] * l["fan_in"]
            dW = np.zeros((l["units"], l["fan_in"]), np.float64)
            for t in range(T):
                dW += l["delta"][t].T.astype(np.float64) @ x[t]
            self.grads[l["first_connection"]:l["first_connection"] + n] += dW.astype(f32).ravel()
            if l["norm"] == NORM_NONE:
                self.grads[l["first_bias"]:l["last_bias"]] += l["delta"].sum(axis=(0, 1), dtype=np.float64).astype(f32)

    def get_loss(self):
        if self.loss_rows == 0:
            return 1.0
        total = float(self.allreduce(np.array([self.loss_sum], np.float64))[0])
        rows = self.loss_rows * self.world
        if self.loss == LOSS_CROSS_ENTROPY:
            return total / rows
        return total / (rows * self.layers[-1]["units"])

    def compute_loss(self, batch, Y):
        """compute_loss_rec_mp (v1/learner/compute_loss_mp.cpp L:115-205): every
        row's time steps t >= n_time_delay as rows of the feed-forward form."""
        T, d, W = self.T, self.time_delay, self.layers[-1]["units"]
        y = np.asarray(Y[:batch], f32).reshape(batch, T, W).transpose(1, 0, 2)[d:].reshape(-1, W)
        full = self.layers[-1]["A"]
        try:
            self.layers[-1]["A"] = full[d:, :batch].reshape(-1, W)
            OracleModel.compute_loss(self, (T - d) * batch, y)
        finally:
            self.layers[-1]["A"] = full

    def get_accu(self, rows_total):
        return OracleModel.get_accu(self, rows_total * (self.T - self.time_delay))

    def update_weights(self, batch, training_size):
        self._clip_gradient()
        k = optimizer_scalars(self.optimizer, self.hp, self.opt_state)
        optimizer_update(self.optimizer, k, self.params, self.grads, self.m1, self.m2, self.m2hat,
                         *self._decay(batch, training_size))
        # mag = clip(clip_gradient, 2, 10): Compute__Regularization__Constraint_
        # Recurrent_Weight__Default, v1/ops/constraints/constraint.cpp L:64-95.
        for l in self.layers[1:]:
            if l["type"] == LAYER_INDRNN:
                lo, hi = self._recurrent_bounds(l)
                if lo != 0 or hi != 0:  # Layer::Use__Regularization__Constraint_Recurrent_Weight, L:28-31
                    s = slice(l["first_recurrent"], l["first_recurrent"] + l["units"])
                    self.params[s] = np.clip(self.params[s], lo, hi)

    def _recurrent_bounds(self, l):
        """The layer's own bounds when set by hand, else the default."""
        if l.get("rec_bounds") is not None:
            return l["rec_bounds"]
        mag = f32(min(max(self.hp.get("clip_gradient", 1.0), 2.0), 10.0))
        bound = f32(np.power(mag, f32(1) / f32(self.T), dtype=f32))
        return -bound, bound

    def set_constraint_recurrent_weight(self, layer, lower, upper):
        """Model::Set__Regularization__Constraint_Recurrent_Weight(index, lower, upper)
        (v1/ops/constraints/constraint.cpp L:143-243).  Bounds equal to the default
        keep following clip_gradient (Check__Use__..__Default, L:41-57)."""
        l = self.layers[layer]
        assert l["type"] == LAYER_INDRNN and lower <= upper
        l["rec_bounds"] = None
        dlo, dhi = self._recurrent_bounds(l)
        if abs(f32(lower) - dlo) > 1e-8 or abs(f32(upper) - dhi) > 1e-8:
            l["rec_bounds"] = (f32(lower), f32(upper))

    def get_layer_outputs(self, layer, batch):
        return self.layers[layer]["A"][:, :batch].copy()

    def get_layer_errors(self, layer, batch, which=0):
        return self.layers[layer]["delta"][:, :batch].copy()
