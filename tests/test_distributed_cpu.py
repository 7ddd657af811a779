"""Data-parallel sharding of the step on CPU: two gloo ranks each hold half of
the rows and exchange exactly what the GPU path exchanges over NCCL (the two
batch-renormalization forward sums, the two backward sums, the gradient vector
and the loss); the result must equal the single-process full-batch step."""
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _cfg():
    import configs
    from enums import OPTIMIZER

    return configs.deep_brn_mlp(24, 40, 2, 12, 32, optimizer=OPTIMIZER.AMSBOUND)


def worker(rank, world, port, out_path):
    for sub in ("deep-learning_b200", "oracle", "tests"):
        sys.path.insert(0, os.path.join(ROOT, sub))
    import torch
    import torch.distributed as dist

    import configs
    import fc_step
    import util

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = _cfg()
    B = cfg["batch"]
    X, Y = configs.synthetic_batch(cfg)
    masks = configs.dropout_masks(cfg)
    full = util.build(fc_step.OracleModel(), cfg)
    rng = np.random.default_rng(0)
    p0 = full.get_array("parameters")
    nw = full.size("total_weights")
    p0[:nw] = (rng.standard_normal(nw) / 6).astype(np.float32)

    def allreduce(a):
        t = torch.from_numpy(np.ascontiguousarray(a, np.float64).copy())
        dist.all_reduce(t)
        return t.numpy()

    shard = B // world
    lo, hi = rank * shard, (rank + 1) * shard
    m = util.build(fc_step.OracleModel(), dict(cfg, batch=shard), params=p0)
    m.allreduce, m.world = allreduce, world
    m.set_global_batch(B)
    out = util.trace(m, dict(cfg, batch=shard), steps=5, X=X[lo:hi], Y=Y[lo:hi], masks=masks)
    if rank == 0:
        np.savez(out_path, **{k: v for k, v in out.items() if k in ("grads", "params1", "params_last", "losses")},
                 p0=p0)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_shards_equal_full_batch():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import configs
    import fc_step
    import util

    port = 29500 + os.getpid() % 2000
    with tempfile.TemporaryDirectory() as tmp:
        out_path = os.path.join(tmp, "rank0.npz")
        procs = [subprocess.Popen([sys.executable, os.path.abspath(__file__), "--worker", str(r), "2", str(port),
                                   out_path]) for r in range(2)]
        for p in procs:
            assert p.wait(timeout=300) == 0
        got = np.load(out_path)
        cfg = _cfg()
        X, Y = configs.synthetic_batch(cfg)
        want = util.trace(util.build(fc_step.OracleModel(), cfg, params=got["p0"]), cfg, steps=5, X=X, Y=Y,
                          masks=configs.dropout_masks(cfg))
        for key in ("grads", "params1", "params_last", "losses"):
            assert util.rel_l2(got[key], want[key]) <= 2e-6, key


if __name__ == "__main__" and len(sys.argv) > 1 and sys.argv[1] == "--worker":
    worker(int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), sys.argv[5])
