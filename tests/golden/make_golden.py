"""Generates the committed golden fixtures of the fully-connected training step
from the reference library's own code (oracle/_ref/libdlref.so, built by
`make -C oracle` where the reference sources are present).

    python tests/golden/make_golden.py [fixture names]

Each fixture is a small .npz holding the seeded inputs, targets, dropout masks
and initial parameters of one workload and what the reference produced from
them: activations, errors and gradients of the first step, parameters after
step 1 and after the last step, every step's loss and the running batch
renormalization statistics.  The workloads are reduced shapes of the benchmark
configurations so that the files stay a few hundred KB in total.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for sub in ("deep-learning_b200", "oracle", "tests"):
    sys.path.insert(0, os.path.join(ROOT, sub))

import configs  # noqa: E402
import ref_binding  # noqa: E402
import util  # noqa: E402
from enums import ACTIVATION, LAYER_DROPOUT, OPTIMIZER  # noqa: E402


def cases():
    """name -> (config, steps).  Also imported by the tests."""
    brn = configs.deep_brn_mlp
    return {
        "mlp_softmax_adam": (configs.mlp_softmax(n_in=36, hidden=24, n_out=10, batch=16), 12),
        "brn_selu_bernoulli_amsbound": (brn(20, 32, 2, 12, 24), 12),
        "brn_elu_inverted_adabound": (brn(20, 32, 2, 12, 24, af=ACTIVATION.ELU, optimizer=OPTIMIZER.ADABOUND,
                                          dropout=LAYER_DROPOUT.BERNOULLI_INVERTED), 12),
        "brn_isrlu_nosadam": (brn(20, 32, 2, 12, 24, af=ACTIVATION.ISRLU, optimizer=OPTIMIZER.NOSADAM), 12),
        "brn_relu_amsgrad_nodrop": (brn(20, 32, 2, 12, 24, af=ACTIVATION.RELU, optimizer=OPTIMIZER.AMSGRAD,
                                        dropout=None), 12),
        "brn_lrelu_adam_ragged": (brn(19, 30, 2, 7, 13, af=ACTIVATION.LEAKY_RELU, optimizer=OPTIMIZER.ADAM), 12),
    }


def noisy_cases():
    """Workloads whose steps consume ShakeDrop noise: name -> (config, steps)."""
    return {
        "residual_elu_shakedrop_adam": (configs.residual_mlp(width=24, blocks=3, n_out=7, batch=16), 6),
    }


def recurrent_cases():
    """Time-stepped (IndRNN) workloads: name -> (config, steps)."""
    rnn = configs.indrnn_stack
    all_steps = rnn(n_in=9, hidden=14, depth=2, n_out=5, seq_w=6, batch=7, af=ACTIVATION.LEAKY_RELU,
                    optimizer=OPTIMIZER.ADAM, norm=False)
    all_steps["time_delays"] = 0  # an error on every time step
    all_steps["name"] += "_alltimes"
    return {
        "indrnn_relu_brn_adabound": (rnn(n_in=10, hidden=16, depth=2, n_out=6, seq_w=12, batch=8), 12),
        "indrnn_lrelu_nonorm_adam_alltimes": (all_steps, 12),
    }


def lstm_cases():
    """LSTM workloads: name -> (config, steps).  The layer after an LSTM layer is at
    least as wide as the LSTM layer has cells: the reference reads that many bias
    entries past the LSTM layer's own, out of its parameter vector otherwise."""
    c = configs.lstm_stack
    last = c(n_in=5, blocks=4, cells=1, depth=1, n_out=6, seq_w=6, batch=7)
    last["time_delays"] = 5   # an error on the last time step only
    last["name"] += "_laststep"
    return {
        "lstm_3x2_peephole_adam": (c(n_in=4, blocks=3, cells=2, depth=1, n_out=8, seq_w=3, batch=5), 6),
        "lstm_two_layers": (c(n_in=4, blocks=3, cells=2, depth=2, n_out=8, seq_w=5, batch=6), 6),
        "lstm_under_fc": (c(n_in=6, blocks=2, cells=3, depth=2, n_out=7, seq_w=4, batch=5, hidden_fc=6), 6),
        "lstm_last_step_only": (last, 6),
    }


def make_lstm(name, cfg, steps):
    """The biases are drawn at random first, so that the reference's bias indices
    are told apart from any other.  Serial mode: the reference's LSTM code leaves
    its heap damaged (glibc reports it when the process frees), so every fixture
    comes from a process of its own that leaves without cleaning up."""
    ref = util.build(ref_binding.RefModel(), dict(cfg, mp=False), seed=0)
    p0 = ref.get_array("parameters")
    nw = ref.size("total_weights")
    p0[nw:] = (np.random.default_rng(1).standard_normal(p0.size - nw) * 0.1).astype(np.float32)
    ref.set_array("parameters", p0)
    X, Y = configs.synthetic_batch(cfg)
    out = util.trace(ref, cfg, steps=steps, X=X, Y=Y)
    blob = {"in_X": X, "in_Y": Y, "in_params": p0, "steps": np.int64(steps)}
    blob.update({f"out_{k}": v for k, v in out.items()})
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **blob)
    print(f"{name}: {os.path.getsize(path)} bytes, loss {out['losses'][0]:.6f} -> {out['losses'][-1]:.6f}", flush=True)


def make_plain(name, cfg, steps):
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    configs.set_recurrent_uniform(ref, cfg)
    p0 = ref.get_array("parameters")
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    out = util.trace(ref, cfg, steps=steps, X=X, Y=Y, masks=masks)
    blob = {"in_X": X, "in_Y": Y, "in_params": p0, "steps": np.int64(steps)}
    for li, mk in masks.items():
        blob[f"in_mask{li}"] = mk
    blob.update({f"out_{k}": v for k, v in out.items()})
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **blob)
    print(f"{name}: {os.path.getsize(path)} bytes, loss {out['losses'][0]:.6f} -> {out['losses'][-1]:.6f}")


def make_noisy(name, cfg, steps):
    ref = util.build(ref_binding.RefModel(), cfg, seed=0)
    p0 = ref.get_array("parameters")
    X, Y = configs.synthetic_batch(cfg)
    draws = [util.shakedrop_step_draws(cfg, s) for s in range(steps)]
    out = util.trace_noisy(ref, cfg, steps=steps, X=X, Y=Y, draws=draws)
    blob = {"in_X": X, "in_Y": Y, "in_params": p0, "steps": np.int64(steps)}
    for s, (seed, arrays) in enumerate(draws):
        blob[f"in_sdseed{s}"] = np.int64(seed)
        for li, (mk, fw, bw) in arrays.items():
            blob[f"in_sd{s}_{li}_mask"], blob[f"in_sd{s}_{li}_fwd"], blob[f"in_sd{s}_{li}_bwd"] = mk, fw, bw
    blob.update({f"out_{k}": v for k, v in out.items()})
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **blob)
    print(f"{name}: {os.path.getsize(path)} bytes, loss {out['losses'][0]:.6f} -> {out['losses'][-1]:.6f}")


def main():
    """With arguments, regenerates only the named fixtures."""
    if not ref_binding.available():
        sys.exit("oracle/_ref/libdlref.so is missing: run `make -C oracle` where the reference sources are")
    if len(sys.argv) == 3 and sys.argv[1] == "--one-lstm":
        make_lstm(sys.argv[2], *lstm_cases()[sys.argv[2]])
        os._exit(0)
    only = set(sys.argv[1:])
    for name, (cfg, steps) in {**cases(), **recurrent_cases()}.items():
        if not only or name in only:
            make_plain(name, cfg, steps)
    for name, (cfg, steps) in noisy_cases().items():
        if not only or name in only:
            make_noisy(name, cfg, steps)
    import subprocess
    for name in lstm_cases():
        if not only or name in only:
            subprocess.run([sys.executable, os.path.abspath(__file__), "--one-lstm", name], check=True)


if __name__ == "__main__":
    main()
