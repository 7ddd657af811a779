"""The C ABI boundary without a GPU: the shared library loads, exports every
function include/dlb200.h declares, the Python binding covers the same set, and
asking for a device fails loudly instead of falling back to a CPU path."""
import ctypes
import os
import re

import pytest

import dlb200

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "dlb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dlb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_functions():
    names = declared_functions()
    assert len(names) > 60
    for must in ("dlb_fc_forward", "dlb_fc_backward_input", "dlb_fc_weight_gradient", "dlb_brn_forward_sums",
                 "dlb_activation_forward", "dlb_optimizer_step", "dlb_model_forward_pass"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(dlb200.LIB_PATH)
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in include/dlb200.h but not exported: {missing}"


def test_binding_covers_header():
    declared = set(declared_functions())
    bound = set(dlb200.SIGNATURES)
    assert declared == bound, f"only in header: {declared - bound}; only in binding: {bound - declared}"


def test_status_strings_and_version():
    L = dlb200.lib()
    assert L.dlb_version() >= 100
    assert L.dlb_status_string(0) == b"ok"
    assert b"CPU" in L.dlb_status_string(6)


def test_optimizer_prepare_is_host_only():
    """dlb_optimizer_prepare derives the step scalars on the host exactly as the
    reference does from its float time step; it needs no device."""
    import fc_step
    import numpy as np

    L = dlb200.lib()
    hyper = (ctypes.c_float * 8)(1e-3, 0.9, 0.999, 1e-8, 0.1, 0.1, 1e-3, 1.0)
    hp = dict(adam_learning_rate=1e-3, adam_beta1=0.9, adam_beta2=0.999, adam_epsilon=1e-8, adam_gamma=0.1,
              learning_rate_final=0.1, learning_gamma=1e-3)
    for rule in (1, 2, 3, 4, 5, 9):
        t, prev, state = ctypes.c_float(0), ctypes.c_float(0), {}
        for _ in range(5):
            k = dlb200.OptimizerScalars()
            assert L.dlb_optimizer_prepare(rule, hyper, ctypes.byref(t), ctypes.byref(prev), ctypes.byref(k)) == 0
            want = fc_step.optimizer_scalars(rule, hp, state)
            np.testing.assert_allclose(k.lr_t, want["lr_t"], rtol=2e-6)
            np.testing.assert_allclose(k.beta2, want["beta2"], rtol=2e-6)
            np.testing.assert_allclose([k.lower_bound, k.upper_bound], [want["lo"], want["hi"]], rtol=2e-6)
    assert L.dlb_optimizer_prepare(7, hyper, ctypes.byref(t), ctypes.byref(prev), ctypes.byref(k)) == 3   # iRPROP-


def test_no_cpu_fallback():
    import subprocess
    import sys

    code = ("import sys; sys.path.insert(0, %r); import dlb200\n"
            "try:\n    dlb200.Context(0)\nexcept dlb200.DlbError as e:\n    print('REFUSED', e)\n"
            "else:\n    print('CREATED')\n") % os.path.join(ROOT, "deep-learning_b200")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120).stdout
    assert "REFUSED" in out and "no CPU path" in out
