"""Two GPUs, one process each: the rows are sharded, batch-renormalization sums
and gradients cross NVLink through the library's NCCL communicator, and every
rank must end with the parameters of the single-GPU full-batch run."""
import os
import subprocess
import sys
import tempfile
import time

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

pytestmark = pytest.mark.gpu


def _gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=60).stdout
        return sum(1 for l in out.splitlines() if l.startswith("GPU "))
    except (OSError, subprocess.TimeoutExpired):
        return 0


def _cfg(kind="brn_mlp"):
    import configs

    if kind == "indrnn":
        return configs.indrnn_stack(n_in=64, hidden=128, depth=2, n_out=32, seq_w=6, batch=64)
    if kind == "residual":
        return configs.residual_mlp(width=256, blocks=2, n_out=10, batch=128)
    return configs.deep_brn_mlp(256, 512, 2, 128, 256)


def _run(model, cfg, X, Y, masks, steps, first_row=0):
    """`steps` training steps; ShakeDrop noise, where the model has any, is drawn
    on the device by global row index, so that shards draw their rows of the
    full batch's arrays."""
    import configs
    import util

    if not configs.shakedrop_layers(cfg):
        return util.trace(model, cfg, steps=steps, X=X, Y=Y, masks=masks)
    B = cfg["batch"]
    model.train_begin(B)
    out, losses = {}, []
    for step in range(steps):
        model.draw_noise(B, 99, step, first_row)
        model.reset_loss()
        model.forward_pass(B, X)
        model.compute_error(B, Y)
        model.backward_pass(B)
        model.update_derivatives(B)
        model.merge_derivatives()
        losses.append(model.get_loss())
        if step == 0:
            out["grads"] = model.get_array("derivatives")
        model.update_weights(B, B)
        if step == 0:
            out["params1"] = model.get_array("parameters")
    out["params_last"] = model.get_array("parameters")
    out["losses"] = np.asarray(losses, np.float64)
    return out


def worker(rank, world, tmp, kind="brn_mlp"):
    for sub in ("deep-learning_b200", "oracle", "tests"):
        sys.path.insert(0, os.path.join(ROOT, sub))
    import configs
    import dlb200
    import util

    ctx = dlb200.Context(rank)
    id_path = os.path.join(tmp, "nccl_id")
    if rank == 0:
        with open(id_path + ".tmp", "wb") as f:
            f.write(ctx.unique_id())
        os.replace(id_path + ".tmp", id_path)
    deadline = time.time() + 120
    while not os.path.exists(id_path):
        if time.time() > deadline:
            raise SystemExit("rank 0 never published the communicator id")
        time.sleep(0.05)
    ctx.comm_init(open(id_path, "rb").read(), rank, world)
    # Two processes on two GPUs of one host: the statistics cross NVLink through
    # the peer-memory exchange unless the environment turned it off.
    assert ctx.peer_exchange() == (os.environ.get("DLB_PEER_EXCHANGE", "1") != "0")
    one_call = kind.startswith("one_call")
    cfg = _cfg(("residual" if kind.endswith("residual") else "brn_mlp") if one_call else kind)
    B = cfg["batch"]
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    shard = B // world
    lo, hi = rank * shard, (rank + 1) * shard
    p0 = np.load(os.path.join(tmp, "p0.npy"))
    if one_call:
        # One-call steps: the owner-computes update of the weight matrices (default)
        # beside all-reduce + replicated update, then one step through the
        # separate entry points, whose replicated update needs the moments back.
        out = {}
        for name, on in (("owners", 1), ("replicated", 0)):
            m = util.build(dlb200.Model(ctx), dict(cfg, batch=shard), params=p0)
            m.set_global_batch(B)
            m.set_sharded_update(on)
            m.train_begin(shard)
            for li, mk in masks.items():
                m.set_dropout_mask(li, mk)
            noisy = bool(configs.shakedrop_layers(cfg))

            def step(k):
                if noisy:
                    m.draw_noise(shard, 99, k, lo)
                return m.train_step(shard, X[lo:hi], Y[lo:hi])

            losses = [step(k) for k in range(3)]
            out[name + "_params3"] = m.get_array("parameters")
            out[name + "_grads3"] = m.get_array("derivatives")
            losses.append(step(3))
            for mom in ("first_moment", "second_moment") + (() if noisy else ("second_moment_hat",)):
                out[name + "_" + mom] = m.get_array(mom)
            if noisy:
                m.draw_noise(shard, 99, 4, lo)
            m.reset_loss()
            m.forward_pass(shard, X[lo:hi])
            m.compute_error(shard, Y[lo:hi])
            m.backward_pass(shard)
            m.update_derivatives(shard)
            m.merge_derivatives()
            m.update_weights(B, B)
            out[name + "_params5"] = m.get_array("parameters")
            out[name + "_losses"] = np.asarray(losses, np.float64)
        assert ctx.sync() == 0
        np.savez(os.path.join(tmp, f"rank{rank}.npz"), **out)
        return
    m = util.build(dlb200.Model(ctx), dict(cfg, batch=shard), params=p0)
    m.set_global_batch(B)
    out = _run(m, dict(cfg, batch=shard), X[lo:hi], Y[lo:hi], masks, 4, first_row=lo)
    assert ctx.sync() == 0
    np.savez(os.path.join(tmp, f"rank{rank}.npz"), grads=out["grads"], params1=out["params1"],
             params_last=out["params_last"], losses=out["losses"])


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_two_gpu_shards_equal_single_gpu_full_batch(gpu_ctx):
    import configs
    import dlb200
    import fc_step
    import util

    cfg = _cfg()
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    p0, _ = util.kink_free_parameters(cfg, fc_step.OracleModel, X, masks, scale=1.0 / np.sqrt(512))
    want = util.trace(util.build(dlb200.Model(gpu_ctx), cfg, params=p0), cfg, 4, X, Y, masks)
    with tempfile.TemporaryDirectory() as tmp:
        np.save(os.path.join(tmp, "p0.npy"), p0)
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        procs = [subprocess.Popen([sys.executable, os.path.abspath(__file__), "--worker", str(r), "2", tmp], env=env)
                 for r in range(2)]
        for p in procs:
            assert p.wait(timeout=600) == 0
        for r in range(2):
            got = np.load(os.path.join(tmp, f"rank{r}.npz"))
            # Same arithmetic, sums split in two and added in double: the shards
            # reproduce the full batch to rounding of the statistics.
            for key in ("grads", "params1", "losses"):
                assert util.rel_l2(got[key], want[key]) <= 1e-5, (r, key)
            assert util.rel_l2(got["params_last"], want["params_last"]) <= 1e-4, r
        a, b = np.load(os.path.join(tmp, "rank0.npz")), np.load(os.path.join(tmp, "rank1.npz"))
        assert np.array_equal(a["params_last"], b["params_last"])   # replicas stay bit-identical


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_two_gpu_owner_computes_update_of_residual_blocks(gpu_ctx):
    """The same for residual blocks, where the matrices are updated by their
    owners behind the weight-gradient products, after the backward pass."""
    import dlb200
    import util

    cfg = _cfg("residual")
    p0 = util.build(dlb200.Model(gpu_ctx), cfg, seed=5).get_array("parameters")
    with tempfile.TemporaryDirectory() as tmp:
        np.save(os.path.join(tmp, "p0.npy"), p0)
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        procs = [subprocess.Popen([sys.executable, os.path.abspath(__file__), "--worker", str(r), "2", tmp,
                                   "one_call_residual"], env=env) for r in range(2)]
        for p in procs:
            assert p.wait(timeout=600) == 0
        ranks = [np.load(os.path.join(tmp, f"rank{r}.npz")) for r in range(2)]
        for r, got in enumerate(ranks):
            for key in ("params3", "grads3", "first_moment", "second_moment", "params5"):
                assert np.array_equal(got["owners_" + key], got["replicated_" + key]), (r, key)
            assert not got["owners_grads3"].any()
            assert got["owners_first_moment"].any()
            assert not np.array_equal(got["owners_params3"], p0)
        assert np.array_equal(ranks[0]["owners_params5"], ranks[1]["owners_params5"])


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_two_gpu_owner_computes_update_equals_replicated_update(gpu_ctx):
    """One-call steps on two ranks: reduce-scatter, update of the owned rows and
    gather of the weights give, bit for bit, what all-reduce and the same update
    on both ranks give (with two ranks both sums are a + b), the cleared
    gradients and the gathered moments included; a later step through the
    separate entry points carries on from the gathered moments; and both are the
    single-GPU full-batch run to rounding of the statistics."""
    import configs
    import dlb200
    import fc_step
    import util

    cfg = _cfg()
    B = cfg["batch"]
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    p0, _ = util.kink_free_parameters(cfg, fc_step.OracleModel, X, masks, scale=1.0 / np.sqrt(512))
    single = util.build(dlb200.Model(gpu_ctx), cfg, params=p0)
    single.train_begin(B)
    for li, mk in masks.items():
        single.set_dropout_mask(li, mk)
    want_losses = [single.train_step(B, X, Y) for _ in range(3)]
    want3 = single.get_array("parameters")
    with tempfile.TemporaryDirectory() as tmp:
        np.save(os.path.join(tmp, "p0.npy"), p0)
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        procs = [subprocess.Popen([sys.executable, os.path.abspath(__file__), "--worker", str(r), "2", tmp, "one_call"],
                                  env=env) for r in range(2)]
        for p in procs:
            assert p.wait(timeout=600) == 0
        ranks = [np.load(os.path.join(tmp, f"rank{r}.npz")) for r in range(2)]
        for r, got in enumerate(ranks):
            for key in ("params3", "grads3", "first_moment", "second_moment", "second_moment_hat", "params5"):
                assert np.array_equal(got["owners_" + key], got["replicated_" + key]), (r, key)
            # The loss is a sum of doubles added in whatever order the blocks finish.
            assert np.allclose(got["owners_losses"], got["replicated_losses"], rtol=1e-12, atol=0)
            assert not got["owners_grads3"].any()          # cleared, the slices of the other rank too
            assert got["owners_first_moment"].any()
            assert util.rel_l2(got["owners_params3"], want3) <= 1e-4, r
            assert np.allclose(got["owners_losses"][:3], want_losses, rtol=1e-5)
        for key in ("owners_params3", "owners_params5", "owners_second_moment_hat"):
            assert np.array_equal(ranks[0][key], ranks[1][key]), key


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("kind", ["indrnn", "residual"])
def test_two_gpu_shards_of_the_other_model_families(gpu_ctx, kind):
    """The same for a time-stepped IndRNN stack (per-time-step statistics, 2 T H
    doubles per exchange) and for residual blocks with ShakeDrop noise drawn on
    the device by global row index."""
    import dlb200
    import util

    cfg = _cfg(kind)
    X, Y = __import__("configs").synthetic_batch(cfg)
    seeded = util.build(dlb200.Model(gpu_ctx), cfg, seed=5)
    p0 = seeded.get_array("parameters")
    want = _run(util.build(dlb200.Model(gpu_ctx), cfg, params=p0), cfg, X, Y, {}, 4)
    with tempfile.TemporaryDirectory() as tmp:
        np.save(os.path.join(tmp, "p0.npy"), p0)
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        procs = [subprocess.Popen([sys.executable, os.path.abspath(__file__), "--worker", str(r), "2", tmp, kind],
                                  env=env) for r in range(2)]
        for p in procs:
            assert p.wait(timeout=600) == 0
        a, b = np.load(os.path.join(tmp, "rank0.npz")), np.load(os.path.join(tmp, "rank1.npz"))
        for key in ("grads", "params1", "losses"):
            assert util.rel_l2(a[key], want[key]) <= 2e-5, key
        # Later steps may meet a derivative jump; only the scale of the agreement is checked.
        assert util.rel_l2(a["params_last"], want["params_last"]) <= 1e-3
        assert np.array_equal(a["params_last"], b["params_last"])   # replicas stay bit-identical


if __name__ == "__main__" and len(sys.argv) > 1 and sys.argv[1] == "--worker":
    worker(int(sys.argv[2]), int(sys.argv[3]), sys.argv[4], sys.argv[5] if len(sys.argv) > 5 else "brn_mlp")
