"""Test infrastructure, not product code.

CPU restatement (numpy fp32) of the reference's residual blocks of fully
connected layers with ShakeDrop, on top of oracle/fc_step.py.  Pinned against
the compiled reference in tests/test_oracle_residual.py and against the
committed fixture tests/golden/residual_*.npz.

A RESIDUAL layer of depth d is followed by its d block layers (the reference's
layer list, lib/deep-learning/v1/learner/compile.cpp).  Block layers are
pre-activation layers (v1/learner/fwp_mp.cpp L:3951-4192):

    first block layer:  s_1 = x W_1^T (+ b_1)            (no activation)
    later block layers: n_j = [batch renorm over the layer's INPUT units](s_{j-1})
                        a_j = dropout(f_j(n_j));  s_j = a_j W_j^T (+ b_j)

then (L:3777-3911) the residual layer's own normalization (if set), ShakeDrop
(L:4922-4957: rows drawn with probability p get every element multiplied by a
fresh U(-1,1)), and out = x + block (widths equal here; the reference's
zero-padded shortcut for unequal widths is outside this restatement).

Backward (v1/learner/bwp_mp.cpp L:310-406, L:658-874, L:933-966): the error of
the block output is the error of the residual output; rows that were perturbed
forward get every element multiplied by a fresh U(0,1); then the block layers
from last to first; the layer below the block receives the shortcut error plus
delta_1 W_1.  The batch-renormalization units of a block layer number its
fan-in, not its width.
"""
from __future__ import annotations

import numpy as np

import fc_step
from fc_step import (AF_SOFTMAX, NORM_NONE, OracleModel, af_derive, af_fire, apply_dropout, brn_backward,
                     brn_forward, f32, softmax)

LAYER_FC, LAYER_RESIDUAL = 3, 9
DROPOUT_SHAKEDROP = 5


class ResidualOracleModel(OracleModel):
    backend = "numpy-restatement-residual"

    # --- construction ---------------------------------------------------
    def compile(self, layer_types, layer_units, seq_w=1, model_type=3, allowable_memory=None):
        assert seq_w == 1
        self.layers = []
        width = None
        i = 0
        types, units = list(layer_types), [int(u) for u in layer_units]
        while i < len(types):
            if types[i] == LAYER_RESIDUAL:
                depth = units[i]
                res = dict(type=LAYER_RESIDUAL, units=width, depth=depth, af=None, norm=NORM_NONE,
                           dropout=(0, 0.0), mask=None, group=0, norm_units=width)
                self.layers.append(res)
                fan = width
                for j in range(depth):
                    i += 1
                    assert types[i] == LAYER_FC
                    self.layers.append(dict(type=LAYER_FC, units=units[i], fan_in=fan, af=None, norm=NORM_NONE,
                                            dropout=(0, 0.0), mask=None, group=1, block_input=(j == 0),
                                            norm_units=fan))
                    fan = units[i]
                # The residual output is as wide as the wider of shortcut and block;
                # the narrower one is added from column `pad` on
                # (v1/learner/compile.cpp L:337-352, Forward_Pass__Zero_Padded_Identity__OpenMP,
                # fwp_mp.cpp L:5058-5123).
                res["units"] = max(width, fan)
                res["norm_units"] = fan   # the layer's own normalization acts on the block output
                res["pad"] = (abs(width - fan) + 1) // 2
                res["shortcut_width"], res["block_width"] = width, fan
                width = res["units"]
            else:
                self.layers.append(dict(type=LAYER_FC, units=units[i], fan_in=width, af=None, norm=NORM_NONE,
                                        dropout=(0, 0.0), mask=None, group=0, block_input=False,
                                        norm_units=units[i]))
                width = units[i]
            i += 1
        self._layout()

    def _layout(self):
        w = 0
        fcs = [l for l in self.layers[1:] if l["type"] == LAYER_FC]
        for l in fcs:
            l["first_connection"], w = w, w + l["units"] * l["fan_in"]
            l["last_connection"] = w
        self.total_weights = w
        b = w
        for l in fcs:
            l["first_bias"], b = b, b + l["units"]
            l["last_bias"] = b
        self.total_bias = b - w
        any_norm = any(l["norm"] != NORM_NONE for l in self.layers)
        u = 0
        for l in self.layers:
            l["first_norm_unit"], u = u, u + l["norm_units"]
        self.total_norm = u if any_norm else 0
        P = self.total_weights + self.total_bias + 2 * self.total_norm
        old = self.params
        self.params = np.zeros(P, f32)
        if old is not None:
            k = self.total_weights + self.total_bias
            self.params[:k] = old[:k]
        gs = self.total_weights + self.total_bias
        self.params[gs:gs + self.total_norm] = 1.0
        self.grads = np.zeros(P, f32)
        self.m1, self.m2, self.m2hat = np.zeros(P, f32), np.zeros(P, f32), np.zeros(P, f32)
        for l in self.layers:
            if l["norm"] != NORM_NONE and "state" not in l:
                n = l["norm_units"]
                l["state"] = dict(mean_average=np.zeros(n, f32), variance_average=np.ones(n, f32))

    def _gamma_slice(self, l):
        s = self.total_weights + self.total_bias + l["first_norm_unit"]
        return slice(s, s + l["norm_units"])

    def _beta_slice(self, l):
        s = self.total_weights + self.total_bias + self.total_norm + l["first_norm_unit"]
        return slice(s, s + l["norm_units"])

    def set_dropout(self, layer, kind, value, scale_weights=False):
        assert not scale_weights
        self.layers[layer]["dropout"] = (kind, value)

    def set_shakedrop_noise(self, layer, mask, forward, backward):
        """Row flags and the forward U(-1,1) / backward U(0,1) draws of one
        residual layer (rows x width; only flagged rows are used)."""
        l = self.layers[layer]
        l["sd_mask"] = np.asarray(mask, np.uint8).astype(bool)
        l["sd_fwd"] = np.asarray(forward, f32)
        l["sd_bwd"] = np.asarray(backward, f32)

    def size(self, name):
        if name == "n_out":
            return self.layers[-1]["units"]
        return super().size(name)

    def layer_info(self, layer):
        l = self.layers[layer]
        return dict(type=l["type"], n_out=l["units"], first_connection=l.get("first_connection", 0),
                    last_connection=l.get("last_connection", 0), first_bias=l.get("first_bias", 0),
                    last_bias=l.get("last_bias", 0), norm=l["norm"], dropout=l["dropout"][0], group=l["group"],
                    first_norm_unit=l["first_norm_unit"] if self.total_norm else 0)

    # --- helpers --------------------------------------------------------
    def _W(self, l):
        return self.params[l["first_connection"]:l["last_connection"]].reshape(l["units"], l["fan_in"])

    def _norm_in(self, l, x):
        """Batch renorm of a layer over `x`; remembers what backward needs.  At
        inference the running averages (fwp_mp.cpp L:4461-4491)."""
        st = l["state"]
        if not self.training:
            return (self.params[self._gamma_slice(l)] * ((x - st["mean_average"]) / st["variance_average"])
                    + self.params[self._beta_slice(l)]).astype(f32)
        st["gamma"] = self.params[self._gamma_slice(l)]
        st["beta"] = self.params[self._beta_slice(l)]
        l["norm_in"] = x
        l["x_hat"], y = brn_forward(x, st, self._brn_of(l), self.global_rows, self.allreduce)
        return y

    def _norm_back(self, l, dy):
        dx, dg, db = brn_backward(dy, l["norm_in"], l["x_hat"], l["state"], self.global_rows, self.allreduce)
        self.grads[self._gamma_slice(l)] += dg
        self.grads[self._beta_slice(l)] += db
        return dx

    # --- step -----------------------------------------------------------
    def forward_pass(self, batch, X):
        a = np.ascontiguousarray(X[:batch], f32)
        self.layers[0]["A"] = a
        i = 1
        while i < len(self.layers):
            l = self.layers[i]
            if l["type"] == LAYER_RESIDUAL:
                x = a
                h = x
                for j in range(l["depth"]):
                    b = self.layers[i + 1 + j]
                    if b["block_input"]:
                        assert b["norm"] == NORM_NONE, "normalised block-input layers are outside this restatement"
                        b["IN"] = h
                    else:
                        n = self._norm_in(b, h) if b["norm"] != NORM_NONE else h
                        b["Y"] = n
                        if self.training:
                            b["IN"] = apply_dropout(af_fire(b["af"], n), b["dropout"][0], b["dropout"][1], b["mask"])
                        else:  # plain Bernoulli dropout scales by the keep probability, L:4870-4892
                            b["IN"] = af_fire(b["af"], n)
                            if b["dropout"][0] == fc_step.DROPOUT_BERNOULLI:
                                b["IN"] = (b["IN"] * f32(b["dropout"][1])).astype(f32)
                    s = (b["IN"] @ self._W(b).T).astype(f32)
                    if b["norm"] == NORM_NONE:
                        s = (s + self.params[b["first_bias"]:b["last_bias"]]).astype(f32)
                    b["A"] = s
                    h = s
                o = self._norm_in(l, h) if l["norm"] != NORM_NONE else h
                if l["dropout"][0] == DROPOUT_SHAKEDROP and not self.training:
                    # Inference: the block output times 1 - p (fwp_mp.cpp L:3876-3897).
                    o = (o * (f32(1) - f32(l["dropout"][1]))).astype(f32)
                elif l["dropout"][0] == DROPOUT_SHAKEDROP:
                    o = np.where(l["sd_mask"][:batch, None], o * l["sd_fwd"][:batch], o).astype(f32)
                # The reference normalises / perturbs in place in the last block
                # layer's output buffer, which is what a reader of that layer sees.
                self.layers[i + l["depth"]]["A"] = o
                a = np.zeros((x.shape[0], l["units"]), f32)
                sa = l["pad"] if x.shape[1] < l["units"] else 0
                sb = l["pad"] if o.shape[1] < l["units"] else 0
                if o.shape[1] >= x.shape[1]:   # the wider one is copied, the narrower one added
                    a[:, sb:sb + o.shape[1]] = o
                    a[:, sa:sa + x.shape[1]] += x
                else:
                    a[:, sa:sa + x.shape[1]] = x
                    a[:, sb:sb + o.shape[1]] += o
                l["A"] = a
                i += l["depth"] + 1
                continue
            W = self._W(l)
            z = (a @ W.T).astype(f32)
            if l["norm"] == NORM_NONE:
                z = (z + self.params[l["first_bias"]:l["last_bias"]]).astype(f32)
                y = z
            else:
                y = self._norm_in(l, z)
            l["Z"], l["Y"] = z, y
            if l["af"] == AF_SOFTMAX:
                a = softmax(y)
            elif not self.training:
                a = af_fire(l["af"], y)
                if l["dropout"][0] == fc_step.DROPOUT_BERNOULLI:
                    a = (a * f32(l["dropout"][1])).astype(f32)
            else:
                a = apply_dropout(af_fire(l["af"], y), l["dropout"][0], l["dropout"][1], l["mask"])
            l["A"] = a
            l["IN"] = self._below(i)["A"]
            i += 1

    def _below(self, i):
        """Top-level layer whose output feeds top-level layer i."""
        j = i - 1
        while self.layers[j].get("group") == 1:
            j -= 1
        return self.layers[j]

    def _top_level(self):
        return [i for i, l in enumerate(self.layers) if l.get("group", 0) == 0]

    def backward_pass(self, batch):
        tops = self._top_level()
        # dOut of every top-level layer above the input, from the output down.
        dout = {tops[-1]: None}
        for pos in range(len(tops) - 1, 0, -1):
            i = tops[pos]
            l = self.layers[i]
            if l["type"] == LAYER_RESIDUAL:
                d = dout[i]
                # Backward_Pass__Residual__OpenMP (bwp_mp.cpp L:1078-1140): the
                # narrower of shortcut and block reads its window of the error.
                wa, wb = l["shortcut_width"], l["block_width"]
                sa = l["pad"] if wa < l["units"] else 0
                sb = l["pad"] if wb < l["units"] else 0
                do = np.ascontiguousarray(d[:, sb:sb + wb])
                if l["dropout"][0] == DROPOUT_SHAKEDROP:
                    do = np.where(l["sd_mask"][:batch, None], do * l["sd_bwd"][:batch], do).astype(f32)
                if l["norm"] != NORM_NONE:
                    do = self._norm_back(l, do)
                delta = do
                for j in range(l["depth"], 0, -1):
                    b = self.layers[i + j]
                    b["delta"] = delta
                    if b["block_input"]:
                        break
                    da = (delta @ self._W(b)).astype(f32)
                    e = (da * af_derive(b["af"], b["Y"], b["IN"])).astype(f32)
                    if b["norm"] != NORM_NONE:
                        e = self._norm_back(b, e)
                    delta = e
                first = self.layers[i + 1]
                l["delta"] = d
                if pos > 1:   # no error into the input layer
                    dout[tops[pos - 1]] = (d[:, sa:sa + wa] + (first["delta"] @ self._W(first)).astype(f32)).astype(f32)
            else:
                if dout[i] is not None:   # hidden standalone layer
                    e = (dout[i] * af_derive(l["af"], l["Y"], l["A"])).astype(f32)
                    if l["norm"] != NORM_NONE:
                        e = self._norm_back(l, e)
                    l["delta"] = e
                if pos > 1:
                    dout[tops[pos - 1]] = (l["delta"] @ self._W(l)).astype(f32)

    def update_derivatives(self, batch):
        for l in self.layers[1:]:
            if l["type"] != LAYER_FC:
                continue
            dW = (l["delta"].T @ l["IN"]).astype(f32)
            self.grads[l["first_connection"]:l["last_connection"]] += dW.ravel()
            if l["norm"] == NORM_NONE:
                self.grads[l["first_bias"]:l["last_bias"]] += l["delta"].sum(axis=0, dtype=np.float64).astype(f32)

    def get_layer_outputs(self, layer, batch):
        return self.layers[layer]["A"][None, :batch].copy()

    def get_layer_errors(self, layer, batch, which=0):
        return self.layers[layer]["delta"][None, :batch].copy()
