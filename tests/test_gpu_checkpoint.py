"""The reference's text checkpoint format: files written by the library are the
bytes the compiled reference writes for the same state, the reference's loader
reads them, and the library reads the reference's."""
import os

import numpy as np
import pytest

import configs
import dlb200
import ref_binding
import util
from enums import LOSS_FN

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_binding.available(), reason="oracle/_ref not built on this machine")]

CASES = {
    "brn_mlp": lambda: configs.deep_brn_mlp(6, 8, 2, 4, 8),
    "softmax_mlp": lambda: configs.mlp_softmax(7, 5, 3, 8),
    "residual": lambda: configs.residual_mlp(6, 2, 4, 8),
    "residual_wider_blocks": lambda: configs.residual_mlp(5, 2, 4, 8, block_width=8),
    "indrnn": lambda: configs.indrnn_stack(n_in=3, hidden=5, depth=2, n_out=2, seq_w=3, batch=6),
}


def _trained(gpu_ctx, cfg):
    mod = util.build(dlb200.Model(gpu_ctx), cfg, seed=3)
    if configs.shakedrop_layers(cfg):
        util.trace_noisy(mod, cfg, steps=2)
    else:
        util.trace(mod, cfg, steps=2)
    return mod


@pytest.mark.parametrize("case", sorted(CASES))
def test_files_are_the_reference_s_bytes_and_load_both_ways(gpu_ctx, case, tmp_path):
    cfg = CASES[case]()
    B, last = cfg["batch"], len(cfg["layers"]) - 1
    mod = _trained(gpu_ctx, cfg)
    # use_mp is the reference's threading switch; the library always writes 1.
    ref = util.build(ref_binding.RefModel(), dict(cfg, mp=True), seed=0)
    util.copy_trained_state(mod, ref, cfg)
    for model in (mod, ref):
        model.set_accu_fn(1 if cfg["loss"] == LOSS_FN.CROSS_ENTROPY else 3)
    ours = (str(tmp_path / "ours.net"), str(tmp_path / "ours.nn"))
    theirs = (str(tmp_path / "theirs.net"), str(tmp_path / "theirs.nn"))
    mod.save(*ours)
    ref.save(*theirs)
    for a, b in zip(ours, theirs):
        got, want = open(a, "rb").read(), open(b, "rb").read()
        if got != want:
            ga, wa = got.split(b"\r\n"), want.split(b"\r\n")
            first = next((i for i, (x, y) in enumerate(zip(ga, wa)) if x != y), min(len(ga), len(wa)))
            raise AssertionError(f"{os.path.basename(a)} line {first + 1}: {ga[first:first + 1]} != {wa[first:first + 1]}")

    # The reference reads our files.
    X, _ = configs.synthetic_batch(dict(cfg, data_seed=5))
    back = ref_binding.RefModel()
    back.load(*ours)
    back.set_max_batch_size(B)
    back.set_mp(True)
    back.train_begin(B)
    back.set_propagation(0)
    back.forward_pass(B, X)
    mod.set_propagation(0)
    mod.forward_pass(B, X)
    assert util.rel_l2(mod.get_layer_outputs(last, B).reshape(-1), back.get_layer_outputs(last, B).reshape(-1)) <= 1e-5
    # Weights and biases come back bit for bit (16 significant digits carry a
    # float); the scale / shift slots of layers without normalization are not in the file.
    nw = mod.size("total_weights") + mod.size("total_bias")
    assert np.array_equal(back.get_array("parameters")[:nw], mod.get_array("parameters")[:nw])

    # We read the reference's files.
    again = dlb200.Model(gpu_ctx)
    again.load(*theirs)
    assert np.array_equal(again.get_array("parameters"), mod.get_array("parameters"))
    again.train_begin(B)
    again.set_propagation(0)
    again.forward_pass(B, X)
    assert np.array_equal(again.get_layer_outputs(last, B), mod.get_layer_outputs(last, B))
    rewritten = (str(tmp_path / "again.net"), str(tmp_path / "again.nn"))
    again.save(*rewritten)
    for a, b in zip(rewritten, theirs):
        assert open(a, "rb").read() == open(b, "rb").read()
    assert gpu_ctx.sync() == 0


def test_a_file_outside_the_supported_path_is_refused(gpu_ctx, tmp_path):
    cfg = CASES["brn_mlp"]()
    mod = _trained(gpu_ctx, cfg)
    files = (str(tmp_path / "a.net"), str(tmp_path / "a.nn"))
    mod.save(*files)
    text = open(files[0], "rb").read().replace(b"  Hidden layer 1:\r\n    type_layer 3", b"  Hidden layer 1:\r\n    type_layer 6")
    open(files[0], "wb").write(text)
    with pytest.raises(dlb200.DlbError, match="outside the supported path"):
        dlb200.Model(gpu_ctx).load(*files)
    with pytest.raises(dlb200.DlbError):
        dlb200.Model(gpu_ctx).load(str(tmp_path / "missing.net"), files[1])


def test_checkpointer_rotation_moments_and_resume(gpu_ctx, tmp_path):
    """Checkpoint directories as DL::Checkpointer writes them (nn/checkpointer.cpp
    L:94-160): ckpt-<step>/model.net + model.nn, a `checkpoint` file naming the
    newest, the newest max_to_keep kept; the interval policy of
    CheckpointerInterval (L:230-250); and the side file with the optimizer's
    moments, with which a run resumed from the directory continues bit for bit."""
    import os
    import time

    cfg = configs.deep_brn_mlp(64, 128, 2, 32, 96)
    B = cfg["batch"]
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)

    def with_masks(m):
        for li, mk in masks.items():
            m.set_dropout_mask(li, mk)
        return m

    model = with_masks(util.build(dlb200.Model(gpu_ctx), cfg, seed=7))
    ck = dlb200.Checkpointer(model, str(tmp_path), max_to_keep=2, interval=3)
    saved_at = []
    for g in range(8):
        model.train_step(B, X, Y)
        if ck(g):
            saved_at.append(g)
            time.sleep(0.02)   # rotation orders the directories by time of last write
    assert saved_at == [0, 3, 6]                                   # due steps 0, 3, 6
    assert sorted(os.listdir(tmp_path)) == ["checkpoint", "ckpt-3", "ckpt-6"]   # ckpt-0 rotated out
    assert open(tmp_path / "checkpoint", "rb").read() == b"model_checkpoint_path: ckpt-6"
    assert sorted(os.listdir(tmp_path / "ckpt-6")) == ["model.net", "model.nn", "model.opt"]
    assert not ck(7) and ck(7, force=True)                         # not due, then forced
    assert sorted(os.listdir(tmp_path)) == ["checkpoint", "ckpt-6", "ckpt-7"]
    # Resume: a fresh model loads the newest checkpoint and continues exactly.
    resumed = dlb200.Model(gpu_ctx)
    assert dlb200.Checkpointer(resumed, str(tmp_path)).load()
    with_masks(resumed)
    util.copy_trained_state(model, resumed, cfg)                   # running averages travel in model.net already
    for key in ("parameters", "first_moment", "second_moment", "second_moment_hat"):
        assert np.array_equal(resumed.get_array(key), model.get_array(key)), key
    assert resumed.get_hparam("optimizer_time_step") == model.get_hparam("optimizer_time_step") == 8.0
    a = [model.train_step(B, X, Y) for _ in range(3)]
    b = [resumed.train_step(B, X, Y) for _ in range(3)]
    np.testing.assert_allclose(b, a, rtol=1e-12)
    assert np.array_equal(resumed.get_array("parameters"), model.get_array("parameters"))
    # Without the side file (a checkpoint the reference wrote) the moments start at zero.
    os.remove(tmp_path / "ckpt-7" / "model.opt")
    plain = dlb200.Model(gpu_ctx)
    assert dlb200.Checkpointer(plain, str(tmp_path)).load()
    assert not plain.get_array("first_moment").any()
    empty = dlb200.Model(gpu_ctx)
    assert not dlb200.Checkpointer(empty, str(tmp_path / "nothing_here")).load()
    assert gpu_ctx.sync() == 0


def test_l2_is_kept_and_saved_but_does_not_touch_the_step(gpu_ctx, tmp_path):
    """Model::set_l2: the reference's update calls its L2 routine over an empty
    range (tests/test_oracle.py pins that), so the value only travels through the
    hyperparameter file."""
    cfg = configs.deep_brn_mlp(64, 128, 2, 32, 96)
    B = cfg["batch"]
    X, Y = configs.synthetic_batch(cfg)
    a = util.build(dlb200.Model(gpu_ctx), cfg, seed=7)
    b = util.build(dlb200.Model(gpu_ctx), cfg, seed=7)
    b.set_l2(0.1)
    for m in (a, b):
        m.train_step(B, X, Y)
    assert np.array_equal(a.get_array("parameters"), b.get_array("parameters"))
    b.save(str(tmp_path / "m.net"), str(tmp_path / "m.nn"))
    assert "regularization__l2 0.1" in open(tmp_path / "m.nn", "rb").read().decode().replace("0.1000000014901161", "0.1")
    c = dlb200.Model(gpu_ctx)
    c.load(str(tmp_path / "m.net"), str(tmp_path / "m.nn"))
    with pytest.raises(dlb200.DlbError):
        b.set_l2(1.5)
    assert gpu_ctx.sync() == 0
