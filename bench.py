#!/usr/bin/env python
"""Benchmark of the GPT-124M-shaped training step (and the GEMM sweep beside it).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl bmb|reference]
                    [--math tf32|fp32|bf16]

One process per GPU: for N > 1 launch through torchrun
(`python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N`).
Rank 0 prints ONE JSON line.

* `value`   tokens/s of the whole job, batches already resident in HBM, timed
            with CUDA events on the stream the steps run on, max over ranks.
* `e2e`     the same metric with, inside every timed step, the host->device
            copy of the step's token ids from pinned memory and the
            device->host read of the step's loss.
* `roofline` the GEMMs of the step (the dominant kernels): FLOP of every
            GEMM call / its event-timed duration, against the tensor peak
            derived from MEASURED_PEAKS.json (TF32 = BF16 / 2) or, in fp32
            mode, the SIMT peak at the SM clock sampled during the run.
* `cpu_baseline` the CPU oracle's train step (oracle/liborc.so) on a bounded
            sample of the same model, rank 0 at N = 1 only.

`--impl reference` times the reference's own CUDA kernels (the unmodified
sources compiled for sm_100a into oracle/_ref/libbmbref.so) on the same
configuration, in one process with one thread per GPU as its train_gpt does.
The reference has no CPU implementation of any part of this path.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

GPT124M = dict(max_seq_len=1024, vocab_size=50304, padded_vocab=50304, n_layer=12, n_head=12, n_embd=768)
B_PER_GPU, T = 8, 1024
# ncu, one training step: 25.06 GB read + written by the 147 tensor-core GEMM launches; algorithmic (each
# operand and result once, C twice where beta = 1): 21.4 GB
GEMM_DRAM_BYTES_PER_LAUNCH = 170.5e6
GEMM_ALGO_BYTES_PER_LAUNCH = 145.6e6
HP = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, grad_clip=1.0)


def flops_per_step_per_gpu(num_params):
    # the reference's own count, src/train_gpt.cu:361-363
    c = GPT124M
    return 6.0 * B_PER_GPU * T * num_params + 12.0 * c["n_layer"] * c["n_head"] * T * T * (c["n_embd"] // c["n_head"]) * B_PER_GPU


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d.get("hbm_gbs"), bf16=d.get("bf16_tflops"), bf16_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 50 ms while alive.  nvidia-smi takes a few
    tenths of a second to start, about as long as the timed regions of the default run, so it is started
    before the warm-up steps and only the samples stamped inside [mark(), stop()] are used."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.path = "/tmp/bmb_clocks_%d_%d.csv" % (os.getpid(), gpu_index)
        self.proc = None
        self.t_mark = None
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=self.f,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def mark(self):
        """The timed region starts now."""
        self.t_mark = time.time()

    @staticmethod
    def _stamp(text):
        import datetime
        try:
            return datetime.datetime.strptime(text, "%Y/%m/%d %H:%M:%S.%f").timestamp()
        except ValueError:
            return None

    def stop(self):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[])
        if self.proc is None:
            return out
        t_stop = time.time()
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            ts = self._stamp(parts[0])
            if ts is not None and self.t_mark is not None and not (self.t_mark - 0.05 <= ts <= t_stop + 0.05):
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for nm, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if sm:
            out["sm_mhz"] = float(np.median(sm))
            out["sm_max_mhz"] = max(mx)
        out["reasons"] = sorted(reasons)
        out["samples"] = len(sm)
        return out


def gemm_sweep(bmb, torch, peaks, sm_clock_mhz):
    """Square GEMM sweep, fp32 SIMT and TF32: best of 10 after 3 warm-ups (CUDA events)."""
    lib = bmb.lib()
    out = []
    nsm = torch.cuda.get_device_properties(0).multi_processor_count
    simt_peak = 2.0 * 128 * nsm * (sm_clock_mhz or 1965.0) * 1e6 / 1e12
    for n in (1024, 1536, 2048, 4096, 6144, 8192):
        g = torch.Generator(device="cuda").manual_seed(n)
        A = torch.rand(n * n, device="cuda", generator=g) * 2 - 1
        Bm = torch.rand(n * n, device="cuda", generator=g) * 2 - 1
        Cm = torch.zeros(n * n, device="cuda")
        row = dict(n=n)
        for name, fn in (("fp32", lib.bmb_sgemm_simt), ("tf32", lib.bmb_sgemm_tf32)):
            iters = 10 if name == "tf32" or n <= 4096 else 4
            for _ in range(3):
                bmb.check(fn(n, n, n, 1.0, A.data_ptr(), Bm.data_ptr(), 0.0, Cm.data_ptr()))
            best = 1e30
            for _ in range(iters):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                bmb.check(fn(n, n, n, 1.0, A.data_ptr(), Bm.data_ptr(), 0.0, Cm.data_ptr()))
                e1.record()
                e1.synchronize()
                best = min(best, e0.elapsed_time(e1))
            row[name + "_tflops"] = round(2.0 * n ** 3 / (best * 1e-3) / 1e12, 2)
        row["fp32_frac_of_simt_peak"] = round(row["fp32_tflops"] / simt_peak, 3)
        row["tf32_frac_of_tensor_peak"] = round(row["tf32_tflops"] / (peaks["bf16"] / 2.0), 3)
        out.append(row)
        del A, Bm, Cm
    return dict(sizes=out, simt_peak_tflops=round(simt_peak, 1), tf32_peak_tflops=round(peaks["bf16"] / 2.0, 1),
                peak_note="SIMT peak = 2*128*SMs*SM clock sampled in this run; TF32 peak = burst BF16 of "
                          "MEASURED_PEAKS.json / 2 (%s)" % peaks["source"])


def cpu_baseline():
    """The CPU oracle's optimiser step on a bounded sample of the same model:
    the full 124M-parameter network, 1 sequence x 256 tokens, one step."""
    import helpers
    from helpers import _np
    orc = helpers.load_oracle()
    c = GPT124M
    Bc, Tc = 1, 256
    g = orc.orc_gpt_create(c["max_seq_len"], c["vocab_size"], c["padded_vocab"], c["n_layer"], c["n_head"],
                           c["n_embd"], Bc, Tc)
    n = orc.orc_gpt_num_params(g)
    params = np.ctypeslib.as_array(orc.orc_gpt_params(g), shape=(n,))
    rng = np.random.default_rng(1337)
    params[:] = rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)
    tok = rng.integers(0, c["vocab_size"], (Bc, Tc), dtype=np.int32)
    tgt = rng.integers(0, c["vocab_size"], (Bc, Tc), dtype=np.int32)
    orc.orc_gpt_set_batch(g, _np(tok), _np(tgt))
    t0 = time.time()
    loss = orc.orc_gpt_step(g, HP["lr"], HP["beta1"], HP["beta2"], HP["eps"], HP["weight_decay"], HP["grad_clip"], 1)
    dt = time.time() - t0
    orc.orc_gpt_destroy(g)
    return dict(value=round(Bc * Tc / dt, 2), unit="tokens/s", cores=int(orc.orc_num_threads()), kind="port",
                sample="CPU restatement (oracle/bmb_oracle.c, OpenMP), full 124M-parameter model, 1 sequence x %d "
                       "tokens, one optimiser step in %.1f s, loss %.4f; the reference has no CPU path" % (Tc, dt, loss))


def run_bmb(args):
    import torch
    from __graft_entry__ import load_package
    bmb = load_package()
    import importlib
    dist_mod = importlib.import_module("bmb_b200.dist")
    rank, local, world = dist_mod.env_rank()
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus %d needs torchrun with %d processes" % (args.gpus, args.gpus))
    torch.cuda.set_device(local)
    dist_mod.init_process_group("gloo")
    lib = bmb.lib()
    math = {"fp32": bmb.MATH_FP32, "tf32": bmb.MATH_TF32, "bf16": bmb.MATH_BF16}[args.math]
    peaks = measured_peaks()

    tr = bmb.Trainer(seed=1337, B=B_PER_GPU, T=T, use_flash=1, math=math, fused=0 if args.unfused else 1,
                     beta1=HP["beta1"], beta2=HP["beta2"], eps=HP["eps"], weight_decay=HP["weight_decay"],
                     grad_clip=HP["grad_clip"], **GPT124M)
    comm = None
    if world > 1:
        ident = (C.c_ubyte * 128)()
        if rank == 0:
            bmb.check(lib.bmb_comm_unique_id(ident), "bmb_comm_unique_id")
        raw = dist_mod.broadcast_bytes(bytes(ident), 128)
        ident = (C.c_ubyte * 128)(*raw)
        comm = C.c_void_p()
        bmb.check(lib.bmb_comm_create(C.byref(comm), ident, world, rank), "bmb_comm_create")
        tr.attach_comm(comm, world)
        if not args.nccl_dp:
            # fused gradient exchange + optimiser over peer memory: hand every rank's IPC record to every rank
            mine = tr.ipc_export()
            records = b"".join(dist_mod.broadcast_bytes(mine, 192, src=r) for r in range(world))
            try:
                tr.attach_peers(rank, world, records)
                attached = 1.0
            except bmb.BmbError as e:           # e.g. no peer access between two of the GPUs
                sys.stderr.write("rank %d: fused exchange unavailable (%s)\n" % (rank, e))
                attached = 0.0
            if -dist_mod.max_over_ranks(-attached) < 1.0:      # all ranks or none
                tr.attach_peers(rank, world, None)
                args.nccl_dp = True

    PROF_STEPS = 2
    nsteps = args.warmup + 2 * args.steps + PROF_STEPS
    pinned = []
    for s in range(nsteps):
        x, y = dist_mod.synthetic_batch(s, B_PER_GPU * world, T, GPT124M["vocab_size"])
        px = torch.from_numpy(dist_mod.shard_rows(x, rank, world)).pin_memory()
        py = torch.from_numpy(dist_mod.shard_rows(y, rank, world)).pin_memory()
        pinned.append((px, py))
    stream = torch.cuda.ExternalStream(tr.stream)
    step_no = [0]

    def one_step(i, with_io):
        px, py = pinned[i]
        if with_io:
            tr.upload(px, py)
        step_no[0] += 1
        tr.step(HP["lr"], step_no[0])
        if with_io:
            return tr.loss()
        return None

    sampler = ClockSampler(local) if rank == 0 else None
    # warm-up (with IO, so every path has run), then leave a batch resident
    for i in range(args.warmup):
        one_step(i, True)
    tr.upload(*pinned[args.warmup])
    tr.sync()
    dist_mod.barrier()
    if sampler:
        sampler.mark()

    # ---- timed region 1: kernel throughput, inputs resident (forward + backward replayed as a CUDA graph)
    launches_before = lib.bmb_launch_count()
    dist_mod.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record()
    for i in range(args.steps):
        one_step(args.warmup + i, False)
    with torch.cuda.stream(stream):
        e1.record()
    torch.cuda.synchronize()
    dist_mod.barrier()
    ms_dev = dist_mod.max_over_ranks(e0.elapsed_time(e1))
    launches_timed = lib.bmb_launch_count() - launches_before
    loss_last = tr.loss()

    # ---- timed region 2: end to end.  Every step uploads its batch from pinned memory and its loss is
    # copied back to pinned memory; the host reads the loss of step i-1 while step i runs (the way a
    # training loop logs without draining the GPU every step), and the last one before the clock stops.
    host_losses = torch.zeros(args.steps, dtype=torch.float32).pin_memory()
    loss_events = [torch.cuda.Event() for _ in range(args.steps)]
    read_losses = []
    dist_mod.barrier()
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        e0.record()
    t0 = time.time()
    for i in range(args.steps):
        px, py = pinned[args.warmup + args.steps + i]
        tr.upload(px, py)
        step_no[0] += 1
        tr.step(HP["lr"], step_no[0])
        tr.loss_async(host_losses[i:i + 1])
        with torch.cuda.stream(stream):
            loss_events[i].record()
        if i > 0:
            loss_events[i - 1].synchronize()
            read_losses.append(float(host_losses[i - 1]))
    loss_events[args.steps - 1].synchronize()
    read_losses.append(float(host_losses[args.steps - 1]))
    loss_last = read_losses[-1]
    with torch.cuda.stream(stream):
        e1.record()
    torch.cuda.synchronize()
    wall_ms = (time.time() - t0) * 1e3
    dist_mod.barrier()
    ms_e2e = dist_mod.max_over_ranks(max(e0.elapsed_time(e1), wall_ms))
    clocks = sampler.stop() if sampler else None

    # ---- GEMM breakdown: a few more steps launched one kernel at a time with an event pair around
    # every GEMM (not part of either timed region)
    tr.profile(True)
    for i in range(PROF_STEPS):
        one_step(args.warmup + 2 * args.steps + i, False)
    prof = tr.profile_read()
    tr.profile(False)
    prof["steps"] = PROF_STEPS
    prof["launches"] = launches_timed

    tokens_per_step = B_PER_GPU * T * world
    ms_step = ms_dev / args.steps
    value = tokens_per_step / (ms_step * 1e-3)
    e2e_value = tokens_per_step / (ms_e2e / args.steps * 1e-3)
    if rank != 0:
        tr.close()
        return
    achieved = prof["gemm_flop"] / (prof["gemm_ms"] * 1e-3) / 1e12 if prof["gemm_ms"] > 0 else 0.0
    if math == bmb.MATH_FP32:
        nsm = torch.cuda.get_device_properties(local).multi_processor_count
        peak = 2.0 * 128 * nsm * ((clocks or {}).get("sm_mhz") or 1965.0) * 1e6 / 1e12
        bound, peak_note = "fp32-simt", "2*128*SMs*sampled SM clock"
    else:
        scale = 2.0 if math == bmb.MATH_TF32 else 1.0
        peak = peaks["bf16_sustained"] / scale
        bound, peak_note = "tensor", "sustained BF16 of MEASURED_PEAKS.json (%s)%s" % (
            peaks["source"], " / 2 for TF32" if scale == 2.0 else "")
    line = {
        "metric": "GPT-124M train tokens/s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": {0: "fp32", 1: "tf32", 2: "bf16"}[math], "data": "synthetic",
        "config": {"workload": "GPT-2-small-shaped train step: 12 layers, d_model 768, 12 heads, ctx 1024, "
                               "vocab 50304, batch 8 sequences per GPU, AdamW lr 3e-4 betas 0.9/0.95 wd 0.1 clip 1.0",
                   "global_batch": B_PER_GPU * world, "seq_len": T, "parallelism": "dp%d" % world,
                   "gradient_exchange": ("none" if world == 1 else "NCCL all-reduce, full optimiser per rank" if args.nccl_dp
                                         else "fused over peer memory: slice reduce, slice AdamW, parameter broadcast"),
                   "l2": "per-step working set (~10 GB of activations) exceeds the 126 MB L2",
                   "flop_per_step_per_gpu": flops_per_step_per_gpu(tr.num_params)},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 2 * B_PER_GPU * T * 4,
                "d2h_bytes_per_step": 4, "loss_read": "every step, one step late (asynchronous copy to pinned memory)"},
        "gpu_launches": int(prof["launches"]),
        "loss_last_step": round(float(loss_last), 4),
        "model_tflops": round(flops_per_step_per_gpu(tr.num_params) * world / (ms_step * 1e-3) / 1e12, 1),
        "roofline": {"bound": "tensor", "kernel": "GEMMs of the step (%d calls)" % prof["gemm_calls"],
                     "achieved": round(achieved, 1), "peak": round(peak, 1), "unit": "TFLOP/s",
                     "frac": round(achieved / peak, 3) if peak else None,
                     # DRAM bytes per GEMM launch, mean over the 147 launches of one TF32 step, from the ncu
                     # capture summarised in profiles/train_step_gpt124m_tf32_gemm_dram.md (not measured live)
                     "traffic": GEMM_DRAM_BYTES_PER_LAUNCH if (math == bmb.MATH_TF32 and not args.unfused) else None,
                     "algorithmic_bytes_per_launch": GEMM_ALGO_BYTES_PER_LAUNCH,
                     "gemm_ms_per_step": round(prof["gemm_ms"] / prof["steps"], 3), "peak_note": peak_note,
                     "bound_detail": bound},
        "clocks": clocks,
    }
    if world == 1:
        if not args.no_sweep:
            line["gemm"] = gemm_sweep(bmb, torch, peaks, (clocks or {}).get("sm_mhz"))
        tr.close()
        if not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line))


def run_reference(args):
    """The unmodified reference CUDA kernels, one thread per GPU in this process."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import helpers
    from helpers import _np
    ref = helpers.load_reference()
    if ref is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libbmbref.so was not built "
                          "(the reference checkout was absent at build time)"}))
        return
    import torch
    from __graft_entry__ import load_package
    import importlib
    load_package()
    dist_mod = importlib.import_module("bmb_b200.dist")
    n = args.gpus
    if torch.cuda.device_count() < n:
        print(json.dumps({"impl": "reference", "unavailable": "needs %d visible GPUs" % n}))
        return
    if n > 1:
        for i in range(n):
            for j in range(n):
                if i != j and not torch.cuda.can_device_access_peer(i, j):
                    print(json.dumps({"impl": "reference", "unavailable": "the reference's shared static scratch "
                                      "(src/nn.cu:347,362) needs peer access between every GPU pair"}))
                    return
    c = GPT124M
    h = ref.ref_trainer_create(c["max_seq_len"], c["vocab_size"], c["padded_vocab"], c["n_layer"], c["n_head"],
                               c["n_embd"], B_PER_GPU, T, 1, 1337, n, HP["beta1"], HP["beta2"], HP["eps"],
                               HP["weight_decay"], HP["grad_clip"])
    batches = [dist_mod.synthetic_batch(s, B_PER_GPU * n, T, c["vocab_size"]) for s in range(args.warmup + args.steps)]
    step = 0
    for i in range(args.warmup):
        step += 1
        ref.ref_trainer_step(h, _np(batches[i][0]), _np(batches[i][1]), HP["lr"], step)
    sampler = ClockSampler(0)
    torch.cuda.synchronize()
    t0 = time.time()
    loss = 0.0
    for i in range(args.steps):
        step += 1
        loss = ref.ref_trainer_step(h, _np(batches[args.warmup + i][0]), _np(batches[args.warmup + i][1]), HP["lr"], step)
    ms = (time.time() - t0) * 1e3 / args.steps
    clocks = sampler.stop()
    num_params = ref.ref_trainer_num_params(h)
    ref.ref_trainer_destroy(h)
    value = B_PER_GPU * T * n / (ms * 1e-3)
    print(json.dumps({
        "impl": "reference", "metric": "GPT-124M train tokens/s", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": n, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": {"workload": "same GPT-2-small-shaped train step, run by the reference's own gpt_forward / "
                               "gpt_backward / ddp_allreduce / adamw_update compiled for sm_100a",
                   "global_batch": B_PER_GPU * n, "seq_len": T, "parallelism": "dp%d (threads in one process)" % n,
                   "flop_per_step_per_gpu": flops_per_step_per_gpu(num_params)},
        "e2e": {"value": round(value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 2 * B_PER_GPU * T * 4,
                "d2h_bytes_per_step": 8},
        "cpu_baseline": {"value": round(value, 1), "unit": "tokens/s", "cores": 0, "kind": "reference",
                         "sample": "the reference has no CPU implementation; this arm runs its CUDA kernels on the "
                                   "same GPU(s), timed by wall clock around its blocking step (host uploads and "
                                   "loss read-backs are inside every step)"},
        "loss_last_step": round(float(loss), 4), "clocks": clocks}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="bmb", choices=["bmb", "reference"])
    ap.add_argument("--math", default=os.environ.get("BMB_BENCH_MATH", "tf32"), choices=["fp32", "tf32", "bf16"])
    ap.add_argument("--no-sweep", action="store_true", help="skip the square GEMM sweep")
    ap.add_argument("--unfused", action="store_true", help="the reference's op list: separate bias kernels, "
                    "operands rounded by a prepass instead of by their producers")
    ap.add_argument("--nccl-dp", action="store_true", help="N > 1: sum gradients with one NCCL all-reduce and run the "
                    "whole optimiser on every rank, instead of the fused exchange over peer memory")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_bmb(args)


if __name__ == "__main__":
    main()
