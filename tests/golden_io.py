"""Loads the committed golden fixtures (tests/golden/*.npz) and replays them on
a backend."""
import importlib.util
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden")

_spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)

CASES = make_golden.cases()
RECURRENT_CASES = make_golden.recurrent_cases()
LSTM_CASES = make_golden.lstm_cases()


def load(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    cfg, steps = {**CASES, **RECURRENT_CASES, **LSTM_CASES}[name]
    masks = {int(k[len("in_mask"):]): z[k] for k in z.files if k.startswith("in_mask")}
    want = {k[len("out_"):]: z[k] for k in z.files if k.startswith("out_")}
    return cfg, int(z["steps"]), z["in_X"], z["in_Y"], masks, z["in_params"], want


NOISY_CASES = make_golden.noisy_cases()


def load_noisy(name):
    """(cfg, steps, X, Y, draws, initial parameters, expected) of a fixture whose
    steps consume ShakeDrop noise; draws[step] = (seed, {layer: (mask, fwd, bwd)})."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    cfg, _ = NOISY_CASES[name]
    steps = int(z["steps"])
    draws = []
    for s in range(steps):
        arrays = {}
        for k in z.files:
            if k.startswith(f"in_sd{s}_") and k.endswith("_mask"):
                li = int(k.split("_")[2])
                arrays[li] = (z[k], z[f"in_sd{s}_{li}_fwd"], z[f"in_sd{s}_{li}_bwd"])
        draws.append((int(z[f"in_sdseed{s}"]), arrays))
    want = {k[len("out_"):]: z[k] for k in z.files if k.startswith("out_")}
    return cfg, steps, z["in_X"], z["in_Y"], draws, z["in_params"], want
