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


def load(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    cfg, steps = CASES[name]
    masks = {int(k[len("in_mask"):]): z[k] for k in z.files if k.startswith("in_mask")}
    want = {k[len("out_"):]: z[k] for k in z.files if k.startswith("out_")}
    return cfg, int(z["steps"]), z["in_X"], z["in_Y"], masks, z["in_params"], want
