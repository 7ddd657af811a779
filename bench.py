"""Throughput of the fully-connected training step (forward + backward + update).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1 runs in this process; for N > 1 the script is launched once per GPU by
torch.distributed.run and reads RANK / LOCAL_RANK / WORLD_SIZE / MASTER_*.
Rank 0 prints ONE JSON line.

Workload: the deep batch-renormalised MLP 1024 -> 4 x 4096 -> 1024 (FC + batch
renorm + SELU + Bernoulli dropout keep 0.9 per hidden layer, linear output, MSE,
AMSBound), fp32, 4096 rows per GPU, synthetic N(0,1) inputs and targets and
Glorot-uniform weights.  Across GPUs the rows are sharded (weak scaling: every
GPU keeps 4096 rows); batch-renormalization sums and the gradient vector are
all-reduced over NCCL so that every rank holds the full-batch result.

`value`   samples/s with inputs resident in HBM, timed with CUDA events on the
          library's stream, max over ranks.
`e2e`     the same step through Model.stage_batch + Model.train_step_staged with
          HOST (pinned) inputs: every step's host-to-device copy of inputs and
          targets (started one step ahead, so that it runs under the previous
          step's kernels) and the device-to-host read of its loss are inside
          the timed region.
`roofline` the tcgen05 GEMM kernel: algorithmic FLOPs (2*M*N*K per launch, not
          multiplied by the three tensor-core products per FLOP) over the summed
          event-timed launch durations inside the timed region.
`cpu_baseline` the reference's own OpenMP step (oracle/_ref, compiled from the
          reference's sources) on this host's cores, on a bounded sample.
--impl reference times only that CPU implementation.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "deep-learning_b200"))

import numpy as np  # noqa: E402

import configs  # noqa: E402

METRIC = "train samples/sec (fwd+bwd+update)"
UNIT = "samples/s"
ROWS_PER_GPU = 4096
# TF32 dense GEMM measured on this pool's B200 with cuBLAS (torch.matmul,
# allow_tf32, 8192^3): 745 TFLOP/s best of 10, 591 TFLOP/s over a 3 s loop.  A
# 3xTF32 product issues three TF32 MMAs per fp32-equivalent FLOP.
TF32_TFLOPS_BURST, TF32_TFLOPS_SUSTAINED = 745.3, 591.1
CPU_SAMPLE_ROWS = 512


def env_int(name, default):
    return int(os.environ.get(name, default))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def gemm_traffic_per_launch():
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the GEMM
    kernel at M = N = K = 4096 (9 of the 14 launches of a step have that shape),
    from the ncu capture summarised in
    profiles/gemm_x3_pair_kernel_4096x4096x4096.md: 337 MB + 55.8 MB."""
    return 393.0e6


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs.  The
    sampler is started before the warm-up steps (nvidia-smi takes a few hundred
    milliseconds to deliver its first line, longer than a short timed region);
    `mark()` notes where the timed region begins.  Samples from the mark on are
    reported; with fewer than three of them, the warm-up steps' samples (the same
    kernels under the same load) are included and `window` says so."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device = device
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        self.offset = 0

    def mark(self):
        try:
            self.offset = os.path.getsize(self.file.name)
        except OSError:
            self.offset = 0

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "25"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

        def parse(offset):
            self.file.seek(offset)
            sm, mx, reasons = [], [], set()
            for line in self.file:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 8:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[4:8]):
                    if val == "Active":
                        reasons.add(name)
            return sm, mx, reasons

        sm, mx, reasons = parse(self.offset)
        window = "timed region and end-to-end region"
        if len(sm) < 3:
            sm, mx, reasons = parse(0)
            window = "warm-up steps, timed region and end-to-end region"
        self.file.close()
        os.unlink(self.file.name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm),
                       window=window)
        return out


# name -> (rows per GPU, rows of the CPU sample or None, description).  The
# default is the workload the metric is quoted on; the others are the
# multi-GPU residual workload at its per-GPU shard and the IndRNN workload.
WORKLOADS = {
    "deep_brn_mlp": (ROWS_PER_GPU, CPU_SAMPLE_ROWS,
                     "deep batch-renorm MLP {units}, FC + batch renorm(r_max 3, d_max 5, momentum 0.99, eps 1e-5) "
                     "+ SELU + Bernoulli dropout keep 0.9, MSE, AMSBound(final_lr 0.1, gamma 1e-3)"),
    "deep_brn_mlp_small": (1024, 256, "reduced deep batch-renorm MLP {units} (same layer recipe)"),
    "residual_mlp": (8192, None,
                     "residual MLP, 16 blocks of width 8192 (FC - batch renorm - ELU - FC, ShakeDrop skip with "
                     "linear decay to 0.5, draws passed in and kept for the timed steps), softmax cross-entropy "
                     "over 1000 classes, Adam; 8192 rows per GPU = the 65536-row batch sharded over 8"),
    "indrnn": (1024, 16,
               "IndRNN stack 512 - 4 x 2048 - 512, ReLU recurrence, recurrent weights U(0,1), sequence length "
               "{seq_w}, batch renorm (statistics per time step) in every recurrent layer, MSE on the last step, "
               "AdaBound; a sample is one sequence"),
}


def workload(args):
    if args.workload not in WORKLOADS:
        raise SystemExit(f"unknown workload {args.workload}")
    rows = args.rows or WORKLOADS[args.workload][0]
    if args.workload == "deep_brn_mlp":
        return configs.deep_brn_mlp(batch=rows)
    if args.workload == "deep_brn_mlp_small":
        return configs.deep_brn_mlp(256, 1024, 4, 256, batch=rows)
    if args.workload == "residual_mlp":
        return configs.residual_mlp(batch=rows)
    return configs.indrnn_stack(seq_w=args.seq_w, batch=rows)


def workload_config(args, cfg, world, extra=None):
    layers = cfg["layers"]
    units = "-".join(str(l["units"]) for l in layers if l["type"] != configs.LAYER.RESIDUAL)
    out = {
        "workload": WORKLOADS[args.workload][2].format(units=units, seq_w=cfg.get("seq_w", 1)),
        "rows_per_gpu": cfg["batch"], "global_batch": cfg["batch"] * world, "parallelism": f"dp{world}",
        "l2": "per-step working set (weights, residual planes, gradients, three moment vectors, activations: "
              "1.4 GB and up) is larger than the 126 MB L2; no explicit flush",
    }
    if extra:
        out.update(extra)
    return out


def shakedrop_noise(model, cfg, rows, seed):
    """Row flags and draws for every ShakeDrop layer (the reference draws them
    on the host each step; here they are an input, like the dropout masks)."""
    rng = np.random.default_rng(seed)
    width = cfg["layers"][0]["units"]
    fwd = rng.uniform(-1, 1, (rows, width)).astype(np.float32)
    bwd = rng.uniform(0, 1, (rows, width)).astype(np.float32)
    for li, p in configs.shakedrop_layers(cfg):
        model.set_shakedrop_noise(li, (rng.random(rows) < p).astype(np.uint8), fwd, bwd)


# ----------------------------------------------------------------------------
def cpu_reference_rate(cfg_full, rows, steps, warmup):
    """samples/s of the reference's own OpenMP training step on this host."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_binding

    if not ref_binding.available():
        import fc_step  # the CPU restatement stands in where the reference was not compiled

        kind, model = "port", fc_step.OracleModel()
    else:
        kind, model = "reference", ref_binding.RefModel()
    cfg = dict(cfg_full, batch=rows)
    configs.build_model(model, cfg)
    if kind == "reference":
        model.seed_weights(0)
        model.initialize_weights_with_glorot_uniform()
        configs.set_recurrent_uniform(model, cfg)
    else:
        rng = np.random.default_rng(0)
        p = model.get_array("parameters")
        nw = model.size("total_weights")
        p[:nw] = (rng.standard_normal(nw) / 64).astype(np.float32)
        model.set_array("parameters", p)
    X, Y = configs.synthetic_batch(cfg)
    model.train_begin(rows)
    for li, mk in configs.dropout_masks(cfg).items():
        model.set_dropout_mask(li, mk)
    for _ in range(warmup):
        model.train_step(rows, X, Y)
    t0 = time.perf_counter()
    for _ in range(steps):
        model.train_step(rows, X, Y)
    dt = time.perf_counter() - t0
    cores = model.size("number_threads") if kind == "reference" else 1
    return {"value": rows * steps / dt, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": f"{steps} step(s) of {rows} rows at full layer widths after {warmup} warm-up step(s); "
                      f"host has {os.cpu_count()} logical cores"}, dt / steps


def run_reference(args, rank, world):
    if rank != 0:
        return
    cfg = workload(args)
    sample_rows = WORKLOADS[args.workload][1]
    if sample_rows is None:
        print(json.dumps({"impl": "reference", "unavailable": "the reference's OpenMP step keeps one gradient copy "
                          "per thread; at this workload's 8.6e9 parameters that does not fit this host"}), flush=True)
        return
    base, step_s = cpu_reference_rate(cfg, sample_rows, max(1, args.steps), max(0, args.warmup))
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, cfg, 1, {"rows_per_gpu": sample_rows, "global_batch": sample_rows,
                                                 "parallelism": f"openmp x{base['cores']}"}),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------
def run_ours(args, rank, local_rank, world):
    import dlb200

    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        # CPU control plane (rendezvous, barriers, max over ranks); the data
        # path uses the library's own NCCL communicator.
        dist.init_process_group("gloo", rank=rank, world_size=world)
    ctx = dlb200.Context(local_rank)
    sampler = ClockSampler(local_rank)   # started here: the model set-up below covers nvidia-smi's start-up
    if rank == 0:
        sampler.start()
    if world > 1:
        box = [ctx.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        ctx.comm_init(box[0], rank, world)

    cfg = workload(args)
    rows = cfg["batch"]
    model = configs.build_model(dlb200.Model(ctx), cfg)
    model.seed_weights(0)
    model.initialize_weights_with_glorot_uniform()
    configs.set_recurrent_uniform(model, cfg)
    model.set_global_batch(rows * world)
    for li, mk in configs.dropout_masks(cfg).items():
        model.set_dropout_mask(li, mk)
    shakedrop_noise(model, cfg, rows, 2 + rank)
    Xh, Yh = configs.synthetic_batch(dict(cfg, data_seed=1000 + rank))
    Xp = dlb200.pinned_empty(Xh.shape)
    Yp = dlb200.pinned_empty(Yh.shape)
    Xp[...] = Xh
    Yp[...] = Yh
    Xd, Yd = ctx.array(Xh), ctx.array(Yh)

    def barrier():
        ctx.sync()
        if dist:
            dist.barrier()

    def max_over_ranks(v):
        if not dist:
            return v
        import torch

        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    # ---- device-resident throughput ------------------------------------
    for _ in range(max(args.warmup, 3)):
        model.train_step_device(rows, Xd, Yd)
    barrier()
    if rank == 0:
        sampler.mark()
    ctx.gemm_profile(True)
    ctx.gemm_profile_read()
    launches0 = ctx.launch_count()
    barrier()
    ctx.timer_start()
    for _ in range(args.steps):
        model.train_step_device(rows, Xd, Yd)
    ms = ctx.timer_stop()
    barrier()
    ms = max_over_ranks(ms)
    launches = ctx.launch_count() - launches0
    g_n, g_ms, g_flops = ctx.gemm_profile_read()
    ctx.gemm_profile(False)
    status = ctx.sync()
    if status != 0:
        raise SystemExit(f"device status {status} after the timed region")

    # ---- end to end: host inputs in, loss out ----------------------------
    # Every step's batch crosses PCIe inside the timed region; the copy of batch
    # i+1 is started before the step on batch i so that it runs under its kernels.
    for _ in range(2):  # warm-up: both staging slots get their device buffers
        model.stage_batch(rows, Xp, Yp)
    for _ in range(2):
        model.train_step_staged()
    ctx.sync()
    barrier()
    t0 = time.perf_counter()
    loss = 0.0
    model.stage_batch(rows, Xp, Yp)
    for i in range(args.steps):
        if i + 1 < args.steps:
            model.stage_batch(rows, Xp, Yp)
        loss = model.train_step_staged()
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    clocks = sampler.stop() if rank == 0 else None
    if rank != 0:
        return

    peaks, peak_kind = measured_peaks()
    ms_per_step = ms / args.steps
    value = rows * world * args.steps / (ms / 1e3)
    achieved = g_flops / (g_ms / 1e3) / 1e12 if g_ms > 0 else 0.0
    peak = float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops")))
    f16 = ctx.gemm_kind() == 1
    x3_sustained = peak / 3 if f16 else TF32_TFLOPS_SUSTAINED / 3
    x3_burst = float(peaks.get("bf16_tflops", peak)) / 3 if f16 else TF32_TFLOPS_BURST / 3
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(args, cfg, world),
        "e2e": {"value": rows * world * args.steps / e2e_s, "unit": UNIT,
                "h2d_bytes_per_step": int(Xp.nbytes + Yp.nbytes), "d2h_bytes_per_step": 8,
                "ms_per_step": e2e_s / args.steps * 1e3, "last_loss": loss},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {
            "kernel": ("gemm_x3_pair_kernel (tcgen05 cta_group::2, all FC products; 3xFP16 planes, kind::f16)"
                       if f16 else "gemm_x3_kernel (tcgen05, all FC products; 3xTF32, kind::tf32)"),
            "bound": "tensor",
            "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
            "peak_source": f"MEASURED_PEAKS.json bf16 dense, sustained ({peak_kind})",
            "traffic": gemm_traffic_per_launch(),
            "launches_timed": g_n, "avg_launch_ms": g_ms / g_n if g_n else None,
            "share_of_step": g_ms / ms if ms else None,
            # `achieved` counts 2*M*N*K per launch; the kernel issues three
            # tensor-core products per such FLOP, so its ceiling is a third of
            # the dense peak of its input type and `issued` is what the pipe ran.
            "split3": {"issued_tflops": 3 * achieved, "ceiling": x3_sustained, "frac": achieved / x3_sustained,
                       "ceiling_burst": x3_burst,
                       "note": "fp32-equivalent ceiling of a three-product split: dense peak of the input type / 3 ("
                               + ("bf16/fp16 from MEASURED_PEAKS.json" if f16 else
                                  "TF32 measured on this pool with cuBLAS: 745 burst, 591 sustained") + ")"},
        },
    }
    sample_rows = WORKLOADS[args.workload][1]
    if world == 1 and not args.no_cpu_baseline and sample_rows is not None:
        base, _ = cpu_reference_rate(cfg, sample_rows, 2, 1)
        line["cpu_baseline"] = base
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="deep_brn_mlp")
    ap.add_argument("--rows", type=int, default=0, help="rows per GPU (default: the workload's own)")
    ap.add_argument("--seq-w", type=int, default=256, help="sequence length of the indrnn workload")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank, local_rank, world = env_int("RANK", 0), env_int("LOCAL_RANK", 0), env_int("WORLD_SIZE", 1)
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
