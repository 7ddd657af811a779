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
summed over NCCL so that every rank holds the full-batch result (the gradient
of a weight matrix is reduce-scattered by rows, each rank updates the rows it
owns and the updated rows are gathered: `comm`, `strong` at N > 1).

`value`   samples/s with inputs resident in HBM, timed with CUDA events on the
          library's stream, max over ranks.
`e2e`     the same step through Model.stage_batch + Model.train_step_staged with
          HOST (pinned) inputs: every step's host-to-device copy of inputs and
          targets (started one step ahead, so that it runs under the previous
          step's kernels) and the device-to-host read of its loss are inside
          the timed region.
`e2e_dropin` the same step as the reference's own loop calls it: arrays of host
          row pointers (pageable memory) through the step entry points
          forward_pass / compute_error / backward_pass / update_derivatives /
          merge_derivatives / update_weights and a blocking loss read per step.
`roofline` the tcgen05 GEMM kernel: algorithmic FLOPs (2*M*N*K per launch, not
          multiplied by the three tensor-core products per FLOP) over the summed
          event-timed launch durations inside the timed region.
`range_guard` counters of the fp16 operand form's range guard over the whole
          run: operand tensors flagged, products that ran on the fp32 kernel,
          tensors whose planes were written a second time (all 0 here).
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


def gemm_traffic(f16):
    """(bytes, where from): DRAM bytes one launch of the product kernel moved
    under ncu (read + written), from the record kept beside the profile
    summaries for the operand form that ran; the capture is of the 4096^3
    product, 9 of the 14 launches of a step."""
    path = os.path.join(ROOT, "profiles", "gemm_traffic.json")
    try:
        with open(path) as f:
            e = json.load(f)["f16x3" if f16 else "tf32x3"]
        shape = "x".join(str(v) for v in e["shape"])
        return e["dram_bytes_read"] + e["dram_bytes_write"], f"ncu capture of {e['kernel']} at {shape} (profiles/{e['summary']})"
    except (OSError, KeyError, ValueError):
        return None, "no capture on record"


def gemm_algorithmic_bytes(cfg, rows, f16=True):
    """Operand and result bytes of the FC products of one step, each counted
    once: per product (M, N, K) two operand planes of 2 bytes (or the fp32
    tensor and its residual plane) per element read, M x N floats written.
    Returns (total bytes, number of products)."""
    per_elem = 4 if f16 else 8
    widths = [l["units"] for l in cfg["layers"] if l["type"] != configs.LAYER.RESIDUAL]
    T = cfg.get("seq_w", 1)
    total, count = 0, 0
    for i in range(1, len(widths)):
        fan_in, fan_out, m = widths[i - 1], widths[i], rows * T
        shapes = [(m, fan_out, fan_in), (fan_out, fan_in, m)]        # forward, weight gradient
        if i > 1:
            shapes.append((m, fan_in, fan_out))                         # input gradient
        for (M, N, K) in shapes:
            total += per_elem * (M * K + N * K) + 4 * M * N
            count += 1
    return total, count


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
    if args.workload == "optimizer_sweep":
        raise SystemExit("optimizer_sweep has no model")
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
        "noise": "Bernoulli masks (and ShakeDrop draws) are inputs set once before the steps: the reference draws "
                 "its masks once per Driver::train call, not per step",
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
    if args.workload == "optimizer_sweep":
        return reference_optimizer_sweep(args)
    cfg = workload(args)
    # --rows asks for that many rows per step (4096 = the library arm's batch, at
    # about half a minute per step on 16 cores); the default is a bounded sample.
    sample_rows = args.rows or WORKLOADS[args.workload][1]
    if WORKLOADS[args.workload][1] is None:
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

    j_n, j_ms, x_n, x_ms = ctx.comm_profile_read()
    comm = {"allreduce_exposed_ms": max_over_ranks(j_ms / args.steps), "stats_exchange_ms": max_over_ranks(x_ms / args.steps),
            "stats_exchanges_per_step": x_n / args.steps, "gemm_avg_launch_ms": max_over_ranks(g_ms / g_n if g_n else 0.0),
            "what": "per step, largest over the ranks, from CUDA events on the compute stream: time it stood still "
                    "waiting for the overlapped gradient all-reduces; summed duration of the exchanges of "
                    "batch-renormalization sums; average duration of an FC product (against the 1-GPU figure: "
                    "the slowdown from sharing SMs and HBM with the transfers)"} if world > 1 else None

    # ---- end to end: host inputs in, loss out ----------------------------
    # Every step's batch crosses PCIe inside the timed region; the copy of batch
    # i+1 is started before the step on batch i so that it runs under its kernels.
    # Every step reads a loss back (8 bytes): with a lag of one step it is the loss
    # of the step before, so that the host never waits for the step it has just
    # enqueued; the last step's loss is read before the clock stops.
    def end_to_end(lag, steps):
        model.set_loss_lag(lag)
        for _ in range(2):  # warm-up: both staging slots get their device buffers
            model.stage_batch(rows, Xp, Yp)
        for _ in range(2):
            model.train_step_staged()
        ctx.sync()
        barrier()
        t0 = time.perf_counter()
        model.stage_batch(rows, Xp, Yp)
        for i in range(steps):
            if i + 1 < steps:
                model.stage_batch(rows, Xp, Yp)
            last = model.train_step_staged()
        if lag:
            last = model.get_loss()
        barrier()
        return max_over_ranks(time.perf_counter() - t0), last

    in_order_s, _ = end_to_end(0, args.steps)
    e2e_s, loss = end_to_end(1, args.steps)
    model.set_loss_lag(0)

    # ---- the reference's own loop over the step entry points --------------
    # What Driver::train_mp does with the library behind Model: arrays of host
    # row pointers into pageable memory go into forward_pass / compute_error,
    # then backward_pass, update_derivatives, merge, update_weights, and the loss
    # is read after the update.  No staging ahead, no lag: the boundary as the
    # reference calls it.
    def dropin_loop(steps):
        import ctypes as C

        L, h = model.L, model.h
        Xr = (C.c_void_p * rows)(*[Xh.ctypes.data + i * Xh.strides[0] for i in range(rows)])
        Yr = (C.c_void_p * rows)(*[Yh.ctypes.data + i * Yh.strides[0] for i in range(rows)])
        g = rows * world

        def one():
            dlb200.check(L.dlb_model_reset_loss(h), "reset_loss")
            dlb200.check(L.dlb_model_forward_pass(h, rows, Xr), "forward_pass")
            dlb200.check(L.dlb_model_compute_error(h, rows, Yr), "compute_error")
            dlb200.check(L.dlb_model_backward_pass(h, rows), "backward_pass")
            dlb200.check(L.dlb_model_update_derivatives(h, rows), "update_derivatives")
            dlb200.check(L.dlb_model_merge_derivatives(h), "merge_derivatives")
            dlb200.check(L.dlb_model_update_weights(h, g, g), "update_weights")
            return model.get_loss()

        for _ in range(2):
            one()
        ctx.sync()
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            last = one()
        ctx.sync()
        barrier()
        return max_over_ranks(time.perf_counter() - t0), last

    dropin_s, dropin_loss = dropin_loop(args.steps)

    # ---- strong scaling: the 4096-row batch itself sharded over the GPUs -----
    strong = None
    if world > 1 and args.workload == "deep_brn_mlp":
        rows_s = rows // world
        Xs, Ys = ctx.array(Xh[:rows_s]), ctx.array(Yh[:rows_s])
        model.set_global_batch(rows_s * world)
        for _ in range(3):
            model.train_step_device(rows_s, Xs, Ys)
        barrier()
        ctx.timer_start()
        for _ in range(args.steps):
            model.train_step_device(rows_s, Xs, Ys)
        ms_s = max_over_ranks(ctx.timer_stop())
        barrier()
        model.set_global_batch(rows * world)
        strong = {"global_batch": rows_s * world, "rows_per_gpu": rows_s, "ms_per_step": ms_s / args.steps,
                  "value": rows_s * world * args.steps / (ms_s / 1e3), "unit": UNIT,
                  "what": "the same model with the 4096-row batch sharded over the GPUs (fixed total work), "
                          "device-resident inputs, timed like `value`"}
    clocks = sampler.stop() if rank == 0 else None
    guard = ctx.guard_counters()
    if rank != 0:
        return

    peaks, peak_kind = measured_peaks()
    ms_per_step = ms / args.steps
    value = rows * world * args.steps / (ms / 1e3)
    achieved = g_flops / (g_ms / 1e3) / 1e12 if g_ms > 0 else 0.0
    peak = float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops")))
    f16 = ctx.gemm_kind() == 1
    traffic, traffic_source = gemm_traffic(f16)
    plain_stack = args.workload in ("deep_brn_mlp", "deep_brn_mlp_small")
    algo_bytes, algo_count = gemm_algorithmic_bytes(cfg, rows, f16) if plain_stack else (0, 1)
    x3_sustained = peak / 3 if f16 else TF32_TFLOPS_SUSTAINED / 3
    x3_burst = float(peaks.get("bf16_tflops", peak)) / 3 if f16 else TF32_TFLOPS_BURST / 3
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(args, cfg, world),
        "e2e": {"value": rows * world * args.steps / e2e_s, "unit": UNIT,
                "h2d_bytes_per_step": int(Xp.nbytes + Yp.nbytes), "d2h_bytes_per_step": 8,
                "ms_per_step": e2e_s / args.steps * 1e3, "last_loss": loss,
                "loss_read": "every step reads the loss of the step before from page-locked memory (lag of one step), "
                             "the last step's before the clock stops",
                "in_order": {"value": rows * world * args.steps / in_order_s, "ms_per_step": in_order_s / args.steps * 1e3,
                             "what": "each step waits for its own loss after enqueuing its update"}},
        "e2e_dropin": {"value": rows * world * args.steps / dropin_s, "unit": UNIT, "ms_per_step": dropin_s / args.steps * 1e3,
                       "h2d_bytes_per_step": int(Xh.nbytes + Yh.nbytes), "d2h_bytes_per_step": 8, "last_loss": dropin_loss,
                       "what": "the reference's own loop (Driver::train_mp) over the step entry points it would bind: "
                               "host row-pointer arrays into pageable memory through dlb_model_forward_pass / "
                               "compute_error, then backward_pass, update_derivatives, merge_derivatives, "
                               "update_weights and a blocking get_loss every step; nothing staged ahead"},
        "gpu_launches": launches,
        "range_guard": {"operand_tensors_flagged": guard[0], "products_on_fp32_fallback": guard[1],
                        "tensors_split_again": ctx.guard_resplits(),
                        "note": "3xFP16 form, whole run: operand tensors with lines too small for the tensor's scale, "
                                "products that therefore ran on the fp32 kernel, tensors split a second time after "
                                "outgrowing their predicted scale (expected 0 0 0 on this workload)"},
        "clocks": clocks,
        "comm": comm, "strong": strong,
        "roofline": {
            "kernel": ("gemm_x3_pair_kernel (tcgen05 cta_group::2, all FC products; 3xFP16 planes, kind::f16)"
                       if f16 else "gemm_x3_kernel (tcgen05, all FC products; 3xTF32, kind::tf32)"),
            "bound": "tensor",
            "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
            "peak_source": f"MEASURED_PEAKS.json bf16 dense, sustained ({peak_kind})",
            "traffic": traffic, "traffic_source": traffic_source,
            "algorithmic_bytes_avg_launch": algo_bytes / algo_count if plain_stack else None,
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


# ----------------------------------------------------------------------------
# Optimizer-only workload: a flat fp32 vector sharded by index range, no exchange.
SWEEP_SIZES = (1_000_000, 100_000_000, 1_000_000_000)
# name -> (rule code of the C ABI, algorithmic bytes per element: read p, g, m, v
# and write p, m, v, g <- 0; + 8 for the running maximum of AMSGrad / AMSBound)
SWEEP_RULES = {"adam": (2, 32), "amsgrad": (5, 40), "adamax": (3, 32), "nosadam": (9, 32), "amsbound": (4, 40)}
SWEEP_HYPER = (1e-3, 0.9, 0.999, 1e-8, 0.1, 0.1, 1e-3)


def sweep_config(world, extra=None):
    out = {"workload": "optimizer-only sweep over a flat fp32 vector of 1e6 / 1e8 / 1e9 elements, p ~ N(0, 0.02), "
                       "g ~ N(0, 1e-3) refilled before every step (outside the timed kernel), zero moments, 10 steps "
                       "each of Adam, AMSGrad, AdaMax, NosAdam (gamma 0.1), AMSBound (final_lr 0.1, gamma 1e-3)",
           "parallelism": f"index ranges over {world} GPU(s), no exchange",
           "l2": "1e8 and 1e9 elements: arrays of 0.4 to 4 GB each, larger than the 126 MB L2; 1e6 elements: a 256 MB "
                 "buffer is written between timed steps to flush L2"}
    if extra:
        out.update(extra)
    return out


def run_optimizer_sweep(args, rank, local_rank, world):
    import ctypes as C

    import dlb200

    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("gloo", rank=rank, world_size=world)
    ctx = dlb200.Context(local_rank)
    L = ctx.L
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    def max_over_ranks(v):
        if not dist:
            return v
        import torch

        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    rng = np.random.default_rng(100 + rank)
    block = rng.standard_normal(1 << 22, dtype=np.float32)
    flush = ctx.empty(64 << 20)   # 256 MB
    steps, warmup = args.steps, max(args.warmup, 3)
    table, launches = {}, 0
    sizes = [int(s) for s in args.sizes.split(",")] if args.sizes else SWEEP_SIZES
    for size in sizes:
        n = size // world // 4 * 4
        bufs = {k: ctx.empty(n) for k in ("p0", "g0", "p", "g", "m", "v", "vh")}

        def fill(dst, scale):
            # One seeded block of normal draws repeated over the vector.
            head = min(n, block.size)
            dlb200.check(L.dlb_memcpy_h2d(ctx.h, dst.ptr, dlb200._ptr(np.ascontiguousarray(block[:head] * np.float32(scale))),
                                          head * 4))
            ctx.sync()
            have = head
            while have < n:
                step_n = min(have, n - have)
                dlb200.check(L.dlb_memcpy_d2d(ctx.h, dst.offset(have), dst.ptr, step_n * 4))
                have += step_n
            ctx.sync()

        fill(bufs["p0"], 0.02)
        fill(bufs["g0"], 1e-3)
        table[str(size)] = {}
        for name, (rule, bytes_per) in SWEEP_RULES.items():
            dlb200.check(L.dlb_memcpy_d2d(ctx.h, bufs["p"].ptr, bufs["p0"].ptr, n * 4))
            for k in ("m", "v", "vh"):
                dlb200.check(L.dlb_memset(ctx.h, bufs[k].ptr, 0, n * 4))
            hyper = (C.c_float * 8)(*SWEEP_HYPER, 1.0)
            t, prev = C.c_float(0), C.c_float(0)
            total_ms = 0.0
            for it in range(warmup + steps):
                k = dlb200.OptimizerScalars()
                dlb200.check(L.dlb_optimizer_prepare(rule, hyper, C.byref(t), C.byref(prev), C.byref(k)))
                dlb200.check(L.dlb_memcpy_d2d(ctx.h, bufs["g"].ptr, bufs["g0"].ptr, n * 4))
                if size < 50_000_000:
                    dlb200.check(L.dlb_memset(ctx.h, flush.ptr, it & 0xff, flush.nbytes))
                if it == warmup:
                    ctx.sync()
                    if dist:
                        dist.barrier()
                    if rank == 0 and size == sizes[-1] and name == "adam":
                        sampler.mark()
                ctx.timer_start()
                dlb200.check(L.dlb_optimizer_step(ctx.h, rule, C.byref(k), bufs["p"].ptr, bufs["g"].ptr, bufs["m"].ptr,
                                                  bufs["v"].ptr, bufs["vh"].ptr, None, n))
                ms = ctx.timer_stop()
                if it >= warmup:
                    total_ms += ms
                    launches += 1
            total_ms = max_over_ranks(total_ms)
            gbs = bytes_per * n * world * steps / (total_ms / 1e3) / 1e9
            table[str(size)][name] = {"gb_per_s": gbs, "gb_per_s_per_gpu": gbs / world, "ms_per_step": total_ms / steps,
                                      "bytes_per_element": bytes_per}
        if ctx.sync() != 0:
            raise SystemExit("device status after the sweep")
        for b in bufs.values():
            b.free()

    # End to end at the middle size: the gradient arrives from pinned host memory
    # every step and the first parameters are read back.
    e2e = None
    size = sizes[min(1, len(sizes) - 1)]
    n = size // world // 4 * 4
    gh = dlb200.pinned_empty(n)
    gh[...] = np.resize(block * np.float32(1e-3), n)
    bufs = {k: ctx.zeros(n) for k in ("p", "g", "m", "v", "vh")}
    rule, bytes_per = SWEEP_RULES["amsbound"]
    hyper = (C.c_float * 8)(*SWEEP_HYPER, 1.0)
    t, prev = C.c_float(0), C.c_float(0)
    back = np.zeros(2, np.float32)
    for it in range(2 + steps):
        if it == 2:
            ctx.sync()
            if dist:
                dist.barrier()
            t0 = time.perf_counter()
        k = dlb200.OptimizerScalars()
        dlb200.check(L.dlb_optimizer_prepare(rule, hyper, C.byref(t), C.byref(prev), C.byref(k)))
        dlb200.check(L.dlb_memcpy_h2d(ctx.h, bufs["g"].ptr, dlb200._ptr(gh), n * 4))
        dlb200.check(L.dlb_optimizer_step(ctx.h, rule, C.byref(k), bufs["p"].ptr, bufs["g"].ptr, bufs["m"].ptr,
                                          bufs["v"].ptr, bufs["vh"].ptr, None, n))
        dlb200.check(L.dlb_memcpy_d2h(ctx.h, dlb200._ptr(back), bufs["p"].ptr, 8))
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    e2e = {"value": bytes_per * n * world * steps / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": int(n * 4),
           "d2h_bytes_per_step": 8, "ms_per_step": e2e_s / steps * 1e3,
           "what": f"AMSBound over {size:.0e} elements with the gradient copied from pinned host memory each step"}
    clocks = sampler.stop() if rank == 0 else None
    if rank != 0:
        return
    peaks, peak_kind = measured_peaks()
    peak = float(peaks["hbm_gbs"])
    big = table[str(sizes[-1])]
    total_bytes = sum(v["bytes_per_element"] for v in big.values())
    total_ms = sum(v["ms_per_step"] for v in big.values())
    n_big = sizes[-1] // world // 4 * 4
    value = total_bytes * n_big * world / (total_ms / 1e3) / 1e9
    for rules in table.values():
        for v in rules.values():
            v["frac_of_hbm_peak"] = v["gb_per_s_per_gpu"] / peak
    line = {
        "metric": "optimizer update HBM GB/s (flat fp32 vector)", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": total_ms / len(big), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": sweep_config(world, {"value_is": f"all GPUs together at {sizes[-1]:.0e} elements, the five rules "
                                                   "weighted by their time"}),
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
        "roofline": {"kernel": "optimizer_kernel<rule> (one streaming pass over p, g, m, v[, v_hat])", "bound": "hbm",
                     "achieved": value / world, "peak": peak, "unit": "GB/s", "frac": value / world / peak,
                     "peak_source": f"MEASURED_PEAKS.json copy bandwidth ({peak_kind})", "traffic": None,
                     "traffic_source": "no capture at this size; the in-step pass is in profiles/elementwise_kernels_deep_brn_mlp.md"},
        "sweep": table,
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_optimizer_sweep(min(100_000_000, sizes[-1]), 3)
    print(json.dumps(line), flush=True)


def cpu_optimizer_sweep(n, steps):
    """GB/s of the reference's own update loops (Update_Parameters__*__OpenMP) on
    this host: `steps` steps of each rule the reference implements (AdaMax has no
    loop there) over n elements."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_binding

    if not ref_binding.available():
        return {"value": None, "unit": "GB/s", "cores": 0, "kind": "port", "sample": "oracle/_ref is not built"}
    rng = np.random.default_rng(0)
    block = rng.standard_normal(1 << 22, dtype=np.float32)
    p = np.resize(block * np.float32(0.02), n)
    g = np.resize(block * np.float32(1e-3), n)
    total_bytes, total_s, per_rule = 0.0, 0.0, {}
    for name, (rule, bytes_per) in SWEEP_RULES.items():
        if name == "adamax":
            continue
        m, v, vh = (np.full(n, 0, np.float32) for _ in range(3))   # touched, not lazily mapped
        secs = ref_binding.optimizer_sweep(rule, p.copy(), g, m, v, vh, steps, list(SWEEP_HYPER))
        per_rule[name] = bytes_per * n * steps / secs / 1e9
        total_bytes += bytes_per * n * steps
        total_s += secs
    return {"value": total_bytes / total_s / 1e9, "unit": "GB/s", "cores": os.cpu_count(), "kind": "reference",
            "per_rule_gb_per_s": per_rule,
            "sample": f"{steps} steps of Adam, AMSGrad, NosAdam, AMSBound over {n:.0e} elements (the reference has no "
                      f"AdaMax loop); host has {os.cpu_count()} logical cores"}


def reference_optimizer_sweep(args):
    base = cpu_optimizer_sweep(100_000_000, max(1, args.steps))
    line = {"impl": "reference", "metric": "optimizer update HBM GB/s (flat fp32 vector)", "value": base["value"],
            "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": None,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": sweep_config(1, {"parallelism": f"openmp x{base['cores']}"}), "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
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
    ap.add_argument("--sizes", default="", help="optimizer_sweep: comma-separated vector lengths (default 1e6,1e8,1e9)")
    args = ap.parse_args()
    rank, local_rank, world = env_int("RANK", 0), env_int("LOCAL_RANK", 0), env_int("WORLD_SIZE", 1)
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif args.workload == "optimizer_sweep":
        run_optimizer_sweep(args, rank, local_rank, world)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
