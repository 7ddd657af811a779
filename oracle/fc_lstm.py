"""Test infrastructure, not product code.

CPU restatement (numpy fp32) of the reference's LSTM layer inside a time-stepped
stack of fully connected layers, on top of oracle/fc_step.py.  Pinned against
the compiled reference in tests/test_oracle_lstm.py.

An LSTM layer has `blocks` memory blocks of `cells` cells each (C = blocks *
cells outputs); a block's input, forget and output gate are shared by its
cells, with peephole connections from the block's own cell states (reference:
lib/deep-learning/v1/learner/fwp_rec_mp.cpp L:802-1526, forward;
v1/learner/bwp_rec_mp.cpp L:1006-1582, backward;
v1/learner/update_derivative_rec_mp.cpp L:489-774, weight gradients).  With x_t
the layer's input, h_t its output, c_t the cell states and k the cells of block b:

    z_t = tanh(W_z x_t + R_z h_{t-1} + b_z)                       (per cell)
    i_t = sigm(W_i x_t + R_i h_{t-1} + b_i + sum_k p_i[k] c_{t-1}[k])   (per block)
    f_t = sigm(W_f x_t + R_f h_{t-1} + b_f + sum_k p_f[k] c_{t-1}[k])
    c_t = z_t i_t + c_{t-1} f_t
    o_t = sigm(W_o x_t + R_o h_{t-1} + b_o + sum_k p_o[k] c_t[k])
    h_t = tanh(c_t) o_t

At t = 0 there is no recurrent term, no peephole into i, no forget gate.  tanh is
the reference's 2 / (1 + exp(-2x)) - 1 (v1/ops/activations/functions.hpp L:44).

Parameter layout (v1/learner/connections_prepare.cpp L:83-225), block after
block: per cell [W_z (I) | R_z (C)], then W_i, W_f, W_o (I each), R_i, R_f, R_o
(C each), p_i, p_f, p_o (cells each).  Biases: Prepare__Bias__LSTM (L:240-262)
reserves C + 3 * blocks entries for the layer but leaves first_bias_connection_index
at the block part, and the kernels index b_z from there: b_z[c] = bias[C + c],
b_i[b] = bias[2C + b], b_f[b] = bias[2C + blocks + b], b_o[b] = bias[2C + 2 blocks + b]
relative to the layer's reserved range, the last C of which lie in the next
layer's biases.  The restatement uses the same indices, so the aliasing is the
reference's.  Layers other than LSTM are fully connected without normalization
and without dropout.
"""
from __future__ import annotations

import numpy as np

from fc_step import (AF_SOFTMAX, LOSS_CROSS_ENTROPY, NORM_NONE, OracleModel, af_derive, af_fire, f32, loss_and_delta,
                     softmax)

LAYER_FC, LAYER_LSTM = 3, 7


def sigm(x):
    return (f32(1) / (f32(1) + np.exp(-x, dtype=f32))).astype(f32)


def tanh_ref(x):
    return (f32(2) / (f32(1) + np.exp(f32(-2) * x, dtype=f32)) - f32(1)).astype(f32)


class LstmOracleModel(OracleModel):
    backend = "numpy-restatement-lstm"

    def compile(self, layer_types, layer_units, seq_w=1, model_type=4, allowable_memory=None, layer_units2=None):
        self.T = int(seq_w)
        self.time_delay = 0
        u2 = layer_units2 or [0] * len(layer_types)
        self.layers = []
        for t, u, k in zip(layer_types, layer_units, u2):
            if int(t) == LAYER_LSTM:
                self.layers.append(dict(type=LAYER_LSTM, blocks=int(u), cells=int(k), units=int(u) * int(k), af=None,
                                        norm=NORM_NONE, dropout=(0, 0.0), mask=None))
            else:
                self.layers.append(dict(type=int(t), units=int(u), af=None, norm=NORM_NONE, dropout=(0, 0.0), mask=None))
        self._layout()

    def set_seq_w(self, delays):
        self.time_delay = int(delays)

    def size(self, name):
        if name == "seq_w":
            return self.T
        return super().size(name)

    def _layout(self):
        w = 0
        for i in range(1, len(self.layers)):
            l = self.layers[i]
            I = l["fan_in"] = self.layers[i - 1]["units"]
            l["first_connection"] = w
            if l["type"] == LAYER_LSTM:
                B, K, C = l["blocks"], l["cells"], l["units"]
                idx = dict(Wz=[], Rz=[], Wi=[], Wf=[], Wo=[], Ri=[], Rf=[], Ro=[], pi=[], pf=[], po=[])
                for b in range(B):
                    for k in range(K):
                        idx["Wz"].append(w); w += I
                        idx["Rz"].append(w); w += C
                    for name in ("Wi", "Wf", "Wo"):
                        idx[name].append(w); w += I
                    for name in ("Ri", "Rf", "Ro"):
                        idx[name].append(w); w += C
                    for name in ("pi", "pf", "po"):
                        idx[name].append(w); w += K
                l["idx"] = idx
            else:
                w += l["units"] * I
            l["last_connection"] = w
        self.total_weights = w
        b = w
        for l in self.layers[1:]:
            n = l["units"] + 3 * l["blocks"] if l["type"] == LAYER_LSTM else l["units"]
            l["first_bias"], b = b, b + n
            l["last_bias"] = b
        self.total_bias = b - w
        self.total_norm = 0
        P = self.total_weights + self.total_bias
        old = self.params
        self.params = np.zeros(P, f32)
        if old is not None and old.size == P:
            self.params[:] = old
        self.grads = np.zeros(P, f32)
        self.m1, self.m2, self.m2hat = np.zeros(P, f32), np.zeros(P, f32), np.zeros(P, f32)

    # --- views into the flat vectors -------------------------------------
    def _rows(self, vec, starts, n):
        return np.stack([vec[s:s + n] for s in starts])

    def _lstm_weights(self, l, vec):
        I, C, K = l["fan_in"], l["units"], l["cells"]
        ix = l["idx"]
        g = lambda name, n: self._rows(vec, ix[name], n)
        return dict(Wz=g("Wz", I), Rz=g("Rz", C), Wi=g("Wi", I), Wf=g("Wf", I), Wo=g("Wo", I), Ri=g("Ri", C),
                    Rf=g("Rf", C), Ro=g("Ro", C), pi=g("pi", K), pf=g("pf", K), po=g("po", K))

    def _lstm_bias_index(self, l):
        """Indices into the flat vector as the reference's kernels form them."""
        C, B = l["units"], l["blocks"]
        base = l["first_bias"] + C   # first_bias_connection_index after Prepare__Bias__LSTM
        return dict(z=base + np.arange(C), i=base + C + np.arange(B), f=base + C + B + np.arange(B),
                    o=base + C + 2 * B + np.arange(B))

    def _W(self, l):
        return self.params[l["first_connection"]:l["last_connection"]].reshape(l["units"], l["fan_in"])

    # --- step ---------------------------------------------------------------
    def forward_pass(self, batch, X):
        T = self.T
        n_in = self.layers[0]["units"]
        a = np.ascontiguousarray(np.asarray(X[:batch], f32).reshape(batch, T, n_in).transpose(1, 0, 2))
        self.layers[0]["A"] = a
        for i in range(1, len(self.layers)):
            l = self.layers[i]
            if l["type"] == LAYER_LSTM:
                a = self._lstm_forward(l, a, batch)
                continue
            W = self._W(l)
            bias = self.params[l["first_bias"]:l["last_bias"]]
            Z = np.stack([((a[t] @ W.T).astype(f32) + bias).astype(f32) for t in range(T)])
            A = np.stack([softmax(Z[t]) if l["af"] == AF_SOFTMAX else af_fire(l["af"], Z[t]) for t in range(T)])
            l.update(Z=Z, Y=Z, A=A, IN=a)
            a = A

    def _lstm_forward(self, l, x, batch):
        T, C, B, K = self.T, l["units"], l["blocks"], l["cells"]
        w = self._lstm_weights(l, self.params)
        bi = self._lstm_bias_index(l)
        P = self.params
        blk = np.repeat(np.arange(B), K)          # block of every cell
        z = np.zeros((T, batch, C), f32); c = np.zeros_like(z); ca = np.zeros_like(z); h = np.zeros_like(z)
        gi = np.zeros((T, batch, B), f32); gf = np.zeros_like(gi); go = np.zeros_like(gi)
        for t in range(T):
            sz = (x[t] @ w["Wz"].T).astype(f32)
            si = (x[t] @ w["Wi"].T).astype(f32)
            sf = (x[t] @ w["Wf"].T).astype(f32)
            so = (x[t] @ w["Wo"].T).astype(f32)
            if t > 0:
                sz = (sz + (h[t - 1] @ w["Rz"].T).astype(f32)).astype(f32)
                si = (si + (h[t - 1] @ w["Ri"].T).astype(f32)).astype(f32)
                sf = (sf + (h[t - 1] @ w["Rf"].T).astype(f32)).astype(f32)
                so = (so + (h[t - 1] @ w["Ro"].T).astype(f32)).astype(f32)
            sz = (sz + P[bi["z"]]).astype(f32)
            si = (si + P[bi["i"]]).astype(f32)
            sf = (sf + P[bi["f"]]).astype(f32)
            so = (so + P[bi["o"]]).astype(f32)
            if t > 0:
                cp = c[t - 1].reshape(batch, B, K)
                si = (si + (cp * w["pi"]).sum(axis=2, dtype=f32)).astype(f32)
                sf = (sf + (cp * w["pf"]).sum(axis=2, dtype=f32)).astype(f32)
            gi[t] = sigm(si)
            z[t] = tanh_ref(sz)
            c[t] = (z[t] * gi[t][:, blk]).astype(f32)
            if t > 0:
                gf[t] = sigm(sf)
                c[t] = (c[t] + c[t - 1] * gf[t][:, blk]).astype(f32)
            ca[t] = tanh_ref(c[t])
            so = (so + (c[t].reshape(batch, B, K) * w["po"]).sum(axis=2, dtype=f32)).astype(f32)
            go[t] = sigm(so)
            h[t] = (ca[t] * go[t][:, blk]).astype(f32)
        l.update(IN=x, z=z, c=c, ca=ca, A=h, gi=gi, gf=gf, go=go, blk=blk)
        return h

    def compute_error(self, batch, Y):
        o = self.layers[-1]
        T, n_out = self.T, o["units"]
        y = np.asarray(Y[:batch], f32).reshape(batch, T, n_out).transpose(1, 0, 2)
        delta = np.zeros((T, batch, n_out), f32)
        for t in range(self.time_delay, T):
            total, delta[t] = loss_and_delta(self.loss, o["af"], o["Y"][t], o["A"][t], y[t], self.global_rows)
            self.loss_sum += total
            if o["af"] == AF_SOFTMAX:   # the target of time step 0, compute_error_mp.cpp L:237-247
                _, delta[t] = loss_and_delta(self.loss, o["af"], o["Y"][t], o["A"][t], y[0], self.global_rows)
        o["delta"] = delta
        self.loss_rows += batch * (T - self.time_delay)

    def backward_pass(self, batch):
        T = self.T
        for gi in range(len(self.layers) - 1, 0, -1):
            l = self.layers[gi]
            if l["type"] == LAYER_LSTM:
                dx = self._lstm_backward(l, batch)
            else:
                W = self._W(l)
                dx = np.stack([(l["delta"][t] @ W).astype(f32) for t in range(T)])
            if gi == 1:
                break
            below = self.layers[gi - 1]
            if below["type"] == LAYER_LSTM:
                below["dH"] = dx
            else:
                below["delta"] = np.stack([(dx[t] * af_derive(below["af"], below["Y"][t], below["A"][t])).astype(f32)
                                           for t in range(T)])

    def _lstm_backward(self, l, batch):
        """From dH (the error of the layer's outputs) to the gate errors and the
        error of the layer's inputs."""
        T, C, B, K = self.T, l["units"], l["blocks"], l["cells"]
        w = self._lstm_weights(l, self.params)
        blk = l["blk"]
        dH = l["dH"].copy()
        dz = np.zeros((T, batch, C), f32); dc = np.zeros_like(dz)
        di = np.zeros((T, batch, B), f32); df = np.zeros_like(di); do = np.zeros_like(di)
        blocksum = lambda v: v.reshape(batch, B, K).sum(axis=2, dtype=f32)
        for t in range(T - 1, -1, -1):
            if t < T - 1:
                dH[t] = (dH[t] + (dz[t + 1] @ w["Rz"]).astype(f32) + (di[t + 1] @ w["Ri"]).astype(f32)
                         + (df[t + 1] @ w["Rf"]).astype(f32) + (do[t + 1] @ w["Ro"]).astype(f32)).astype(f32)
            go = l["go"][t]
            do[t] = (go * (f32(1) - go) * blocksum(dH[t] * l["ca"][t])).astype(f32)
            e = (dH[t] * go[:, blk] * (f32(1) - l["ca"][t] * l["ca"][t])).astype(f32)
            e = (e + w["po"].reshape(-1) * do[t][:, blk]).astype(f32)
            if t < T - 1:
                e = (e + w["pi"].reshape(-1) * di[t + 1][:, blk] + w["pf"].reshape(-1) * df[t + 1][:, blk]
                     + dc[t + 1] * l["gf"][t + 1][:, blk]).astype(f32)
            dc[t] = e
            gi_ = l["gi"][t]
            dz[t] = (e * gi_[:, blk] * (f32(1) - l["z"][t] * l["z"][t])).astype(f32)
            di[t] = (gi_ * (f32(1) - gi_) * blocksum(e * l["z"][t])).astype(f32)
            if t > 0:
                gf_ = l["gf"][t]
                df[t] = (gf_ * (f32(1) - gf_) * blocksum(e * l["c"][t - 1])).astype(f32)
        l.update(dz=dz, di=di, df=df, do=do, delta=dH)
        return np.stack([((dz[t] @ w["Wz"]) + (di[t] @ w["Wi"]) + (df[t] @ w["Wf"]) + (do[t] @ w["Wo"])).astype(f32)
                         for t in range(T)])

    def update_derivatives(self, batch):
        T = self.T
        for i in range(1, len(self.layers)):
            l = self.layers[i]
            x = l["IN"]
            if l["type"] != LAYER_LSTM:
                dW = sum(l["delta"][t].T.astype(np.float64) @ x[t] for t in range(T))
                self.grads[l["first_connection"]:l["last_connection"]] += dW.astype(f32).ravel()
                self.grads[l["first_bias"]:l["last_bias"]] += l["delta"].sum(axis=(0, 1), dtype=np.float64).astype(f32)
                continue
            I, C, B, K = l["fan_in"], l["units"], l["blocks"], l["cells"]
            h, c = l["A"], l["c"]
            acc = lambda d, v, rng: sum(d[t + s].T.astype(np.float64) @ v[t] for t, s in rng).astype(f32)
            now = [(t, 0) for t in range(T)]
            nxt = [(t, 1) for t in range(T - 1)]
            g = dict(Wz=acc(l["dz"], x, now), Wi=acc(l["di"], x, now), Wf=acc(l["df"], x, now), Wo=acc(l["do"], x, now))
            if T > 1:
                g.update(Rz=acc(l["dz"], h, nxt), Ri=acc(l["di"], h, nxt), Rf=acc(l["df"], h, nxt), Ro=acc(l["do"], h, nxt))
            cb = c.reshape(T, batch, B, K).astype(np.float64)
            g["po"] = np.einsum("tnb,tnbk->bk", l["do"].astype(np.float64), cb).astype(f32)
            if T > 1:
                g["pi"] = np.einsum("tnb,tnbk->bk", l["di"][1:].astype(np.float64), cb[:-1]).astype(f32)
                g["pf"] = np.einsum("tnb,tnbk->bk", l["df"][1:].astype(np.float64), cb[:-1]).astype(f32)
            widths = dict(Wz=I, Wi=I, Wf=I, Wo=I, Rz=C, Ri=C, Rf=C, Ro=C, pi=K, pf=K, po=K)
            for name, mat in g.items():
                for row, start in enumerate(l["idx"][name]):
                    self.grads[start:start + widths[name]] += mat[row]
            bi = self._lstm_bias_index(l)
            for name, d in (("z", l["dz"]), ("i", l["di"]), ("f", l["df"]), ("o", l["do"])):
                np.add.at(self.grads, bi[name], d.sum(axis=(0, 1), dtype=np.float64).astype(f32))

    def get_loss(self):
        if self.loss_rows == 0:
            return 1.0
        total = float(self.allreduce(np.array([self.loss_sum], np.float64))[0])
        rows = self.loss_rows * self.world
        if self.loss == LOSS_CROSS_ENTROPY:
            return total / rows
        return total / (rows * self.layers[-1]["units"])

    def get_layer_outputs(self, layer, batch):
        return self.layers[layer]["A"][:, :batch].copy()

    def get_layer_errors(self, layer, batch, which=0):
        return self.layers[layer]["delta"][:, :batch].copy()
