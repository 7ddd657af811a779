"""The reference library built with its training step routed to libdlb200
(oracle/dropin_patch.py inserts one hook per entry point, oracle/dropin_glue.cpp
is the binding INTEGRATION.md describes: Model::set_b200 replays the model's
construction on a dlb_model and forward_pass / compute_error / backward_pass /
update_derivatives / merge_mp_derivatives / update_weights / get_loss call the
library).  The reference's own Model object is built, initialised and driven by
the same calls as always; with the switch on, the loss curve and the weights must
follow the unpatched reference's.

The reference's Driver::train needs its Datasets classes, which are not part of
this build (Boost / Eigen dependencies); the harness repeats the body of
Driver::train_mp (drivers/driver.cpp L:227-266) around the same Model methods.
The two builds of the reference run in processes of their own.
"""
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for sub in ("deep-learning_b200", "oracle", "tests"):
    sys.path.insert(0, os.path.join(ROOT, sub))

import configs  # noqa: E402
import ref_binding  # noqa: E402

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (ref_binding.available() and ref_binding.dropin_available()),
                                 reason="oracle/_ref (reference and drop-in builds) not present on this machine")]

STEPS = 30
CASES = {
    "mlp_softmax": lambda: configs.mlp_softmax(),                       # BASELINE configuration 1
    "deep_brn_mlp": lambda: configs.deep_brn_mlp(256, 512, 2, 256, 256),  # configuration 2, reduced
}


def run(case, dropin, out):
    """Builds the reference's Model for `case`, trains STEPS steps on one batch and
    saves losses and weights; `dropin`: the patched build with the switch on."""
    import util

    cfg = CASES[case]()
    model = util.build(ref_binding.DropinModel() if dropin else ref_binding.RefModel(), cfg, seed=0)
    B = cfg["batch"]
    X, Y = configs.synthetic_batch(cfg)
    model.train_begin(B)
    for li, mk in configs.dropout_masks(cfg).items():
        model.set_dropout_mask(li, mk)
    if dropin:
        model.set_b200(True)
    losses = [model.train_step(B, X, Y) for _ in range(STEPS)]
    np.savez(out, losses=np.asarray(losses), params=model.get_array("parameters"))


@pytest.mark.parametrize("case", sorted(CASES))
def test_reference_model_over_the_library_follows_the_reference(case):
    import util

    with tempfile.TemporaryDirectory() as tmp:
        outs = []
        for dropin in (0, 1):
            out = os.path.join(tmp, f"{dropin}.npz")
            p = subprocess.run([sys.executable, os.path.abspath(__file__), "--run", case, str(dropin), out],
                               capture_output=True, text=True, timeout=900)
            assert p.returncode == 0, p.stderr[-3000:]
            assert "dlb drop-in:" not in p.stderr, p.stderr[-3000:]
            outs.append(np.load(out))
    ref, got = outs
    print("losses", ref["losses"][[0, 1, STEPS - 1]], got["losses"][[0, 1, STEPS - 1]])
    assert ref["losses"][-1] < ref["losses"][0]                   # it trains
    assert util.rel_l2(got["losses"][:1], ref["losses"][:1]) <= 1e-5
    assert util.rel_l2(got["losses"], ref["losses"]) <= 1e-4
    assert util.rel_l2(got["params"], ref["params"]) <= 1e-4
    assert not np.array_equal(got["params"], ref["params"])        # two implementations, not one twice


if __name__ == "__main__" and len(sys.argv) > 1 and sys.argv[1] == "--run":
    run(sys.argv[2], bool(int(sys.argv[3])), sys.argv[4])
