#!/usr/bin/env python
"""Benchmark of the BLSTM training step (frames/s) on 1..8 B200.

    python bench.py --gpus N --steps K --warmup W [--workload cfg1] [--impl reference]

A step is one pass of the hot path over one fraction of synthetic input: load -> forward through
all layers -> SSE -> BPTT backward -> weight gradients -> [all-reduce] -> steepest-descent update.
The default workload is configuration 4 (382 -> 3x blstm 512/direction -> 187 -> sse, ONE fraction of
256 parallel sequences of 600..1000 frames).  With N > 1 (launched by torch.distributed.run, one
process per GPU) the same 256 sequences are dealt to the ranks in snake order, every rank processes
its 256/N sequences and the weight gradients are summed with NCCL before the update (strong
scaling: the job is the same at every N).  After the timed steps such a run checks itself: the
weights must be bit-identical on all ranks, and the summed error and all-reduced gradients of the
sharded first step must equal what rank 0 computes on the unsharded fraction.  The other
configurations (--workload cfg0..cfg3) give every rank a fraction of its own (weak scaling).

`value`  : real (unpadded) frames of all ranks per second, inputs already resident in HBM,
           timed with CUDA events on the library's stream, max over ranks.
`e2e`    : the same metric through b2_net_train_step with pinned HOST buffers: the host->device
           copy of the fraction and the device->host read of the error are inside the timed region.
`--impl reference` times the reference toolkit's own Cpu-device code (oracle/_ref, OpenMP Thrust
host backend, all host threads; the C restatement if that library did not travel) on a bounded
sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "project-currennt-public_b200"))

# (workload, phase, recurrence path) -> DRAM bytes per cell-step (one unit, one frame slot) measured with ncu
TRAFFIC_BYTES_PER_CELL_STEP = {
    ("cfg1", "lstm_fwd_recurrence", "persistent_ffma"): 26.1,
    ("cfg1", "lstm_bwd_recurrence", "persistent_ffma"): 32.2,
    ("cfg4", "lstm_fwd_recurrence", "persistent_tensor_core"): 32.3,
    ("cfg4", "lstm_bwd_recurrence", "persistent_tensor_core"): 36.0,
}

METRIC = "blstm_train_step_frames_per_sec"
UNIT = "frames/s"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=float(d["hbm_gbs"]), bf16=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), src="measured")
    return dict(hbm=6650.0, bf16=1400.0, src="fallback")


class ClockSampler(threading.Thread):
    """samples nvidia-smi clocks and throttle reasons while the timed region runs"""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.stop_flag, self.rows = index, False, []

    def run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q, "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            time.sleep(0.05)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(int(r[0]) for r in self.rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower() == "active" for r in self.rows if len(r) > 2 + i)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None,
                "sm_max_mhz": int(self.rows[0][1]) if self.rows[0][1].isdigit() else None, "reasons": reasons,
                "samples": len(self.rows)}


def workload_for(name, rank):
    from b2lstm import workloads
    cfg = int(name.replace("cfg", ""))
    return cfg, workloads.build(cfg, rank=rank)


# ---- algorithmic work per phase (per step, this rank) -----------------------------------------------
def phase_work(layers, T, P, real_frames, count_padding=True):
    """{phase: (kind, amount)}: flops for GEMM phases, bytes for HBM phases (40 B forward / 44 B
    backward per cell-step).  count_padding: over all T*P frame slots (what the kernels process) or
    over the real frames only (the algorithmic work the roofline is quoted on)."""
    N = T * P if count_padding else real_frames
    w = {}

    def add(k, kind, v):
        w[k] = (kind, w.get(k, (kind, 0))[1] + v)
    for i in range(1, len(layers)):
        ty, ls, pls = layers[i]["type"], layers[i]["size"], layers[i - 1]["size"]
        if ty.startswith("feedforward"):
            add("ff_forward_gemm", "flops", 2.0 * ls * pls * N)
            add("ff_backward_gemm", "flops", 2.0 * ls * pls * N * (2 if i > 1 else 1))
            add("ff_bias_act", "bytes", 8.0 * ls * N)
            add("ff_delta", "bytes", 12.0 * ls * N)
            add("ff_bias_grad", "bytes", 4.0 * ls * N)
        elif ty in ("lstm", "blstm"):
            els = ls // 2 if ty == "blstm" else ls
            add("lstm_proj_gemm", "flops", 8.0 * ls * pls * N)
            add("lstm_dx_gemm", "flops", 8.0 * ls * pls * N if i > 1 else 0.0)
            add("lstm_dw_in_gemm", "flops", 8.0 * ls * pls * N)
            add("lstm_dw_rec_gemm", "flops", 8.0 * ls * els * (N - P))
            add("lstm_fwd_recurrence", "bytes", 40.0 * ls * N)
            add("lstm_bwd_recurrence", "bytes", 44.0 * ls * N)
            add("lstm_fwd_recurrence_flops", "flops", 8.0 * ls * els * (N - P))
            add("lstm_bwd_recurrence_flops", "flops", 8.0 * ls * els * (N - P))
            add("lstm_vector_grads", "bytes", 28.0 * ls * N)
        elif ty == "sse":
            add("sse_loss", "bytes", 8.0 * ls * N)
            add("sse_grad", "bytes", 12.0 * ls * N)
    return w


def scaling_of(args, world):
    """cfg4 is ONE fraction of 256 sequences dealt to the ranks (strong scaling) unless --weak is given"""
    return "strong" if (args.workload == "cfg4" and not args.weak) else "weak"


def run_reference(args, rank, world):
    """Reference arm: the reference's own Cpu code on the host cores, bounded sample of the workload."""
    if rank != 0:
        return
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the reference arm uses every host core
    # whatever the launcher set (the OpenMP runtime reads the variable when the library is loaded, below)
    ncores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    os.environ["OMP_NUM_THREADS"] = str(ncores)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from oracle import OracleNet, ref_available
    from b2lstm import workloads
    cfg = int(args.workload.replace("cfg", ""))
    kind = "ref_omp" if ref_available(omp=True) else "port"
    cores = ncores if kind == "ref_omp" else 1
    # bounded sample: the configuration's layer sizes on P_s sequences of reduced length
    c = workloads.CONFIGS[cfg]
    P_s = min(c["P"], 8)
    # frames of the sample as a share of the workload's sequence lengths: about one to two seconds of work per
    # step for the OpenMP build of the reference on a few dozen cores
    scale = args.cpu_scale if args.cpu_scale > 0 else {0: 1.0, 1: 0.05, 2: 0.01, 3: 0.02, 4: 0.06}[cfg]

    def one(scale):
        wl = workloads.build(cfg, scale_frames=scale, P=P_s)
        net = OracleNet(wl["layers"], P_s, int(wl["lens"].max()), kind)
        for i, w in wl["weights"].items():
            net.set_weights(i, w)
        t0 = time.perf_counter()
        net.load(wl["lens"], wl["x"], wl["tg"])
        net.forward()
        net.backward()
        net.sgd_update(1e-5, 0.9)
        dt = time.perf_counter() - t0
        net.close()
        return int(wl["lens"].sum()), dt
    # The sample is FIXED per workload (no calibration against the clock): the same frames at every N and in
    # every run, so that the figure is comparable between runs.  One untimed pass warms the caches up.
    scale2 = scale
    for _ in range(max(1, args.warmup)):
        one(scale2)
    tot_f, tot_t = 0, 0.0
    for _ in range(args.steps):
        f, t = one(scale2)
        tot_f += f
        tot_t += t
    v = tot_f / tot_t
    sample = "%s layer sizes, %d sequences x ~%d frames per step (%d real frames/step), %d steps" % (
        args.workload, P_s, int(c["len_hi"] * scale2), tot_f // max(1, args.steps), args.steps)
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * tot_t / max(1, args.steps), "higher_is_better": True,
            "scaling": scaling_of(args, world), "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workloads.CONFIGS[cfg]["name"], "sample": sample, "omp_threads": cores},
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "reference" if kind == "ref_omp" else "port",
                             "sample": sample},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def dp_correctness_record(net, wl, full, rank, world, dist, torch, args):
    """What the data-parallel job computed, checked after the timed steps (N > 1).
    (1) The weights of every layer are bit-identical on all ranks (byte-wise maximum == minimum over ranks).
    (2) Strong scaling only: from fresh, identical weights every rank runs forward + backward on its shard (the
        backward pass all-reduces the gradients); rank 0 then runs the UNSHARDED fraction on one GPU.  Summed
        error: relative 1e-5.  Every gradient block: relative L2 and max-abs ratio 1e-4."""
    import numpy as np
    import b2lstm
    rec = {"weights_identical_on_all_ranks": True}
    for i in wl["weights"]:
        w = torch.from_numpy(net.get_weights(i).view(np.int32).copy()).cuda()
        hi, lo = w.clone(), w.clone()
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        if not bool(torch.equal(hi, lo)):
            rec["weights_identical_on_all_ranks"] = False
    if full is None:
        return rec
    for i, w in wl["weights"].items():
        net.set_weights(i, w)
    net.load_fraction(wl["lens"], wl["x"], wl["tg"])
    err = net.dp_allreduce_scalar(net.forward())
    net.backward()
    net.synchronize()
    grads = {i: net.weight_updates(i) for i in wl["weights"]}
    dist.barrier()
    if rank == 0:
        layers = full["layers"]
        one = b2lstm.Net(layers, full["P"], int(full["lens"].max()))
        one.set_recurrence_mode(args.recurrence)
        one.set_force_ffma(args.ffma)
        for i, w in full["weights"].items():
            one.set_weights(i, w)
        one.load_fraction(full["lens"], full["x"], full["tg"])
        err1 = one.forward()
        one.backward()
        one.synchronize()
        worst_l2, worst_max = 0.0, 0.0
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import parity
        for i in full["weights"]:
            g1 = one.weight_updates(i).astype(np.float64)
            g = grads[i].astype(np.float64)
            for name, sl in parity.weight_blocks(layers, i).items():
                a, b = g[sl], g1[sl]
                nb = np.linalg.norm(b)
                if nb > 0:
                    worst_l2 = max(worst_l2, float(np.linalg.norm(a - b) / nb))
                    worst_max = max(worst_max, float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)))
        one.close()
        rec.update({"error_sharded": err, "error_one_gpu": err1, "error_rel_diff": abs(err - err1) / max(abs(err1), 1e-30),
                    "gradient_rel_l2_worst_block": worst_l2, "gradient_max_abs_ratio_worst_block": worst_max,
                    "ok": bool(rec["weights_identical_on_all_ranks"] and abs(err - err1) <= 1e-5 * abs(err1)
                               and worst_l2 <= 1e-4 and worst_max <= 1e-4)})
    dist.barrier()
    return rec


def run_gemm_microbench(spec, iters, ffma):
    """--gemm m,n,k,ta,tb: b2_matrix_multiply (the helpers::Matrix GEMM wrapper) on one shape, operand split kernels
    inside the timed region, with the relative L2 error of 64 rows against float64.  ta/tb are the transpose flags
    of the reference's Matrix::assignProduct on column-major operands: 1,0 = K-major x K-major (input projection
    W^T X); 0,0 = MN-major x K-major (error back-projection W delta); 0,1 = MN-major x MN-major (weight gradient
    X delta^T).  Prints one JSON line; it is a kernel figure for profiles/, not the benchmark value."""
    import numpy as np
    import torch
    import b2lstm
    m, n, k, ta, tb = [int(v) for v in spec.split(",")]
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(1)
    A = torch.randn((k, m) if not ta else (m, k), device=dev, generator=g)
    B = torch.randn((n, k) if not tb else (k, n), device=dev, generator=g)
    Cm = torch.zeros((n, m), device=dev)
    lda, ldb = (m if not ta else k), (k if not tb else n)

    def run():
        b2lstm.matrix_multiply(Cm, m, A, lda, ta, B, ldb, tb, m, n, k, accumulate=False, force_ffma=bool(ffma))
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    rows = min(m, 64)
    want = ((A.T if not ta else A)[:rows].double() @ (B.T if not tb else B).double()).cpu().numpy()
    got = Cm.T[:rows].double().cpu().numpy()
    print(json.dumps({"gemm": {"m": m, "n": n, "k": k, "ta": ta, "tb": tb}, "kernel": "ffma" if ffma else "tcgen05_3xf16",
                      "ms": ms, "tflops": 2.0 * m * n * k / (ms * 1e-3) / 1e12,
                      "rel_l2_err_vs_f64": float(np.linalg.norm(got - want) / np.linalg.norm(want))}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b2lstm", choices=["b2lstm", "reference"])
    ap.add_argument("--workload", default="cfg4", choices=["cfg0", "cfg1", "cfg2", "cfg3", "cfg4"])
    ap.add_argument("--strong", action="store_true", help="accepted for compatibility: cfg4 is always split over the ranks")
    ap.add_argument("--weak", action="store_true", help="cfg4: give every rank a full 256-sequence fraction of its own instead")
    ap.add_argument("--no-check", action="store_true", help="N > 1: skip the correctness record after the timed steps")
    ap.add_argument("--recurrence", type=int, default=1)
    ap.add_argument("--ffma", type=int, default=0)
    ap.add_argument("--cpu-scale", type=float, default=0.0,
                    help="reference arm: frames of its sample as a share of the workload's lengths (0: the fixed per-workload value)")
    ap.add_argument("--frames-scale", type=float, default=1.0,
                    help="shorten every sequence by this factor (profiler captures only; such a line is not a bench value)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="one GPU only: run rank 0's share of a W-way split of the workload, without the all-reduce (kernel tuning; "
                         "such a line is not a bench value)")
    ap.add_argument("--gemm", default="", help="m,n,k,ta,tb: time b2_matrix_multiply on one shape instead of the train step")
    args = ap.parse_args()
    if args.gemm:
        run_gemm_microbench(args.gemm, max(1, args.steps), args.ffma)
        return
    if args.frames_scale == 1.0:
        args.warmup = max(args.warmup, 3) if args.impl == "b2lstm" else max(args.warmup, 1)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import numpy as np
    import torch
    import b2lstm
    from b2lstm import workloads
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    cfg = int(args.workload.replace("cfg", ""))
    c = workloads.CONFIGS[cfg]
    strong = scaling_of(args, world) == "strong"
    if (strong and world > 1) or (world == 1 and args.shard_of > 1):
        full = workloads.build(cfg, scale_frames=args.frames_scale)
        from b2lstm import dp
        idx = dp.shard_indices(c["P"], rank, world if world > 1 else args.shard_of)   # deal the length-sorted sequences in snake order
        wl = dict(full, P=len(idx), lens=full["lens"][idx], x=np.ascontiguousarray(full["x"][:, idx]),
                  tg=np.ascontiguousarray(full["tg"][:, idx]))
        T = int(wl["lens"].max())
        wl["x"], wl["tg"] = wl["x"][:T], wl["tg"][:T]
    else:
        wl = workloads.build(cfg, rank=0 if strong else rank, scale_frames=args.frames_scale)
    layers, P, lens = wl["layers"], wl["P"], wl["lens"]
    T = int(lens.max())
    real_frames = int(lens.sum())

    net = b2lstm.Net(layers, P, T)
    net.set_recurrence_mode(args.recurrence)
    net.set_force_ffma(args.ffma)
    for i, w in wl["weights"].items():
        net.set_weights(i, w)
    if world > 1:
        idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            idt.copy_(torch.frombuffer(bytearray(b2lstm.dp_unique_id()), dtype=torch.uint8))
        dist.broadcast(idt, 0)
        net.dp_attach(rank, world, bytes(idt.cpu().numpy().tobytes()))

    x_host = torch.from_numpy(wl["x"]).pin_memory()
    t_host = torch.from_numpy(wl["tg"]).pin_memory()
    x_dev, t_dev = x_host.cuda(), t_host.cuda()
    lr, mom = 1e-6, 0.9
    ext = torch.cuda.ExternalStream(net.stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(ext)
        for _ in range(steps):
            fn()
        e1.record(ext)
        net.synchronize()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    step_dev = lambda: net.train_step_dev(lens, T, x_dev, t_dev, lr, mom)
    # end to end: the copy of the NEXT step's fraction from pinned host memory is started first (it
    # overlaps this step's kernels on the copy engine), then this step runs on the fraction copied
    # during the previous step and its error is read back to the host
    xh, th = x_host.numpy(), t_host.numpy()


    for _ in range(args.warmup):
        step_dev()
    net.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    l0 = net.launch_count
    ms = timed(step_dev, args.steps)                 # the reported number: no per-phase events inside
    launches = net.launch_count - l0
    # per-phase device times from a second pass over the same steps with CUDA events around every phase
    net.set_profiling(True)
    ms_prof = timed(step_dev, args.steps)
    prof = net.get_profile()
    net.set_profiling(False)
    net.prefetch_fraction(lens, xh, th)
    net.train_step_prefetched(lr, mom, want_error=False)
    net.prefetch_fraction(lens, xh, th)      # the fraction the first timed step will consume
    net.synchronize()

    def step_e2e_timed():
        e = net.train_step_prefetched(lr, mom, want_error=False)   # enqueue this step ...
        net.prefetch_fraction(lens, xh, th)                        # ... start the next copy under it ...
        return e

    def step_sync():
        step_e2e_timed()
        return net.read_error()                                    # ... and read this step's error (synchronises)
    for _ in range(2):
        step_sync()
    ms_e2e = timed(step_sync, args.steps)
    net.train_step_prefetched(lr, mom, want_error=False)           # consume the last prefetch
    net.synchronize()
    sampler.stop_flag = True
    sampler.join(timeout=3)

    frames_all = real_frames
    if world > 1:
        t = torch.tensor([real_frames], device="cuda", dtype=torch.float64)
        dist.all_reduce(t)
        frames_all = int(t.item())
    rec_paths = net.recurrence_paths()
    check = None
    if world > 1 and not args.no_check:
        check = dp_correctness_record(net, wl, full if strong else None, rank, world, dist, torch, args)
    value = frames_all * args.steps / (ms * 1e-3)
    e2e = frames_all * args.steps / (ms_e2e * 1e-3)

    if rank == 0:
        pk = peaks()
        work = phase_work(layers, T, P, real_frames)
        kernels = {}
        for name, (tms, ln) in prof.items():
            per = tms / args.steps
            ent = {"ms_per_step": round(per, 4), "launches_per_step": ln // args.steps, "share": round(tms / ms_prof, 4)}
            if name in work and per > 0:
                kind, amt = work[name]
                if kind == "flops":
                    ent["tflops"] = round(amt / (per * 1e-3) / 1e12, 3)
                else:
                    ent["gbs"] = round(amt / (per * 1e-3) / 1e9, 2)
                    fl = work.get(name + "_flops")
                    if fl:
                        ent["tflops"] = round(fl[1] / (per * 1e-3) / 1e12, 3)
            kernels[name] = ent
        top = max((k for k in kernels if k in work), key=lambda k: kernels[k]["ms_per_step"])
        kind, amt = phase_work(layers, T, P, real_frames, count_padding=False)[top]   # real frames only
        per_launch = kernels[top]["ms_per_step"] * 1e-3
        if kind == "flops":
            peak = pk["bf16"] / 3.0   # fp16 hi/lo split: three MMAs at the 16-bit rate per fp32 product
            roof = {"bound": "tensor", "kernel": top, "achieved": amt / per_launch / 1e12, "peak": peak, "unit": "TFLOP/s",
                    "peak_note": "%s bf16 dense sustained / 3 (fp16 hi/lo split, three MMAs per fp32 product)" % pk["src"]}
        else:
            roof = {"bound": "hbm", "kernel": top, "achieved": amt / per_launch / 1e9, "peak": pk["hbm"], "unit": "GB/s",
                    "peak_note": "%s copy bandwidth" % pk["src"]}
        roof["frac"] = roof["achieved"] / roof["peak"]
        # DRAM bytes (ncu dram__bytes_read.sum + dram__bytes_write.sum) per cell-step of the dominant kernel,
        # per workload and recurrence path, from captures on reduced frame counts; traffic grows in proportion
        # to the frame slots, so it is scaled by units x frame slots of one sweep of one layer.  None where no
        # capture of that kernel on that workload exists.
        path_fwd = sorted(set(v[0] for v in rec_paths.values()))
        path_bwd = sorted(set(v[1] for v in rec_paths.values()))
        per_cell = TRAFFIC_BYTES_PER_CELL_STEP.get((args.workload, top, (path_fwd if "fwd" in top else path_bwd)[0]
                                                    if (path_fwd and path_bwd) else ""))
        lstm_sizes = [l["size"] for l in layers if l["type"] in ("lstm", "blstm")]
        if per_cell and lstm_sizes and not args.ffma:
            roof["traffic"] = per_cell * (sum(lstm_sizes) / len(lstm_sizes)) * T * P
            roof["traffic_note"] = "bytes per sweep of one layer, ncu dram__bytes of a reduced-frames capture scaled by frame slots"
            roof["launches"] = len(lstm_sizes)
        else:
            roof["traffic"] = None
        roof["share_of_step"] = kernels[top]["share"]
        in_b = int(x_host.numel() * 4 + t_host.numel() * 4 + T * P)
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": scaling_of(args, world),
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": c["name"], "parallel_sequences_per_gpu": P, "max_frames": T,
                           "real_frames_per_gpu_step": real_frames, "parallelism": "dp%d" % world,
                           "recurrence_mode_requested": args.recurrence,
                           "recurrence_forward": "+".join(path_fwd), "recurrence_backward": "+".join(path_bwd),
                           "sequences_total": c["P"] if strong else P * world,
                           "gemm": "ffma" if args.ffma else "tcgen05_3xf16",
                           "frames_scale": args.frames_scale, "emulated_shard_of": args.shard_of,
                           "l2": "working set per step (GBs of state buffers) exceeds the 126 MB L2; no flush needed"},
                "e2e": {"value": e2e, "unit": UNIT, "ms_per_step": ms_e2e / args.steps, "h2d_bytes_per_step": in_b,
                        "d2h_bytes_per_step": 8},
                "gpu_launches": launches, "roofline": roof, "kernels": kernels, "clocks": sampler.summary()}
        if check is not None:
            line["dp_check"] = check
        if world == 1 and not args.no_cpu_baseline:
            try:
                out = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--workload", args.workload,
                                      "--steps", "3", "--warmup", "1"],
                                     capture_output=True, text=True, timeout=600)
                ref_line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
                line["cpu_baseline"] = json.loads(ref_line)["cpu_baseline"]
            except Exception as ex:  # the baseline is a reported extra; never lose the GPU line over it
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": "failed: %r" % (ex,)}
        print(json.dumps(line), flush=True)
    net.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
