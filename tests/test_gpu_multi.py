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


def _cfg():
    import configs

    return configs.deep_brn_mlp(256, 512, 2, 128, 256)


def worker(rank, world, tmp):
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
    cfg = _cfg()
    B = cfg["batch"]
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    shard = B // world
    lo, hi = rank * shard, (rank + 1) * shard
    p0 = np.load(os.path.join(tmp, "p0.npy"))
    m = util.build(dlb200.Model(ctx), dict(cfg, batch=shard), params=p0)
    m.set_global_batch(B)
    out = util.trace(m, dict(cfg, batch=shard), steps=4, X=X[lo:hi], Y=Y[lo:hi], masks=masks)
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


if __name__ == "__main__" and len(sys.argv) > 1 and sys.argv[1] == "--worker":
    worker(int(sys.argv[2]), int(sys.argv[3]), sys.argv[4])
