#!/usr/bin/env python
"""Benchmark of the GPT-124M-shaped training step, with the GEMM sweep, attention and
batched-GEMM kernels and the CPU baselines beside it.

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
            mode, the SIMT peak at the SM clock sampled during that leg.
* `gemm`, `attention`, `bgemm`   (N = 1) the square GEMM sweep in fp32 and TF32, fused causal
            attention forward / backward at B=8 H=12 T=1024 hs=64, and the attention-shaped
            batched GEMM (batch 96), each as absolute numbers and as a fraction of the
            roofline that bounds it, with the SM clock sampled during that leg.
* `fp32_mode`  (N = 1) a short run of the same training step in fp32 SIMT arithmetic, the
            reference's own precision.
* `cpu_baseline`, `cpu_matmul`  the CPU oracle's train step and fp32 matmul (oracle/liborc.so)
            on bounded samples, rank 0 at N = 1 only, with the thread count.
* `losses_head`  the mean loss of each of the first optimiser steps (at most 20), the same
            batches in both arms; `params_equal_across_ranks` (N > 1) says whether every rank
            ended the run with bit-identical parameters.

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
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

GPT124M = dict(max_seq_len=1024, vocab_size=50304, padded_vocab=50304, n_layer=12, n_head=12, n_embd=768)
B_PER_GPU, T = 8, 1024
# DRAM bytes per tensor-core GEMM launch of one TF32 training step: each of the step's 15 GEMM shapes
# captured alone under a profiler (one launch, DRAM read + write counters), weighted by its launches per
# step (147 in all); and the algorithmic bytes of the same launches (each operand and result once, C
# twice where beta = 1).  Stored constants: this run does not measure DRAM traffic.
GEMM_DRAM_BYTES_PER_LAUNCH = 151.6e6
GEMM_ALGO_BYTES_PER_LAUNCH = 146.2e6
HP = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, grad_clip=1.0)
LOSSES_HEAD = 20
WORKLOAD = ("GPT-2-small-shaped train step: 12 layers, d_model 768, 12 heads, ctx 1024, vocab 50304, "
            "batch 8 sequences per GPU, AdamW lr 3e-4 betas 0.9/0.95 wd 0.1 clip 1.0")


def flops_per_step_per_gpu(num_params):
    # the reference's own count, src/train_gpt.cu:361-363
    c = GPT124M
    return 6.0 * B_PER_GPU * T * num_params + 12.0 * c["n_layer"] * c["n_head"] * T * T * (c["n_embd"] // c["n_head"]) * B_PER_GPU


def config_dict(world, num_params):
    """The same dictionary in both arms: what is run, nothing about how."""
    return {"workload": WORKLOAD, "global_batch": B_PER_GPU * world, "seq_len": T, "parallelism": "dp%d" % world,
            "flop_per_step_per_gpu": flops_per_step_per_gpu(num_params)}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d.get("hbm_gbs"), bf16=d.get("bf16_tflops"), bf16_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class Clocks:
    """SM clock, power and throttle reasons of one GPU, sampled every ~10 ms on a thread
    through NVML (read-only queries) for as long as the object lives; `window(t0, t1)` summarises
    the samples stamped inside a wall-clock interval.  Without NVML it falls back to an
    `nvidia-smi -lms 50` child process (coarser)."""
    REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"), (0x4, "sw_power_cap"))
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, torch, local):
        self.samples = []          # (time, sm MHz, reason bit mask, watts)
        self.max_mhz = None
        self.stop_flag = False
        self.thread = None
        self.proc = None
        self.source = "none"
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(local).uuid)
            try:
                h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByIndex(local)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            self.nv, self.h = pynvml, h
            self.source = "nvml"
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
        except Exception:
            self._start_smi(local)

    def _loop(self):
        nv, h = self.nv, self.h
        while not self.stop_flag:
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                try:
                    watts = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
                except Exception:
                    watts = None
                self.samples.append((time.time(), mhz, mask, watts))
            except Exception:
                pass
            time.sleep(0.010)

    def _start_smi(self, local):
        self.path = "/tmp/bmb_clocks_%d_%d.csv" % (os.getpid(), local)
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(local), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=self.f,
                                         stderr=subprocess.DEVNULL)
            self.source = "nvidia-smi"
        except Exception:
            self.proc = None

    def _smi_samples(self):
        import datetime
        out = []
        try:
            self.f.flush()
            lines = open(self.path).read().splitlines()
        except Exception:
            return out
        for line in lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                mhz = float(parts[1])
                self.max_mhz = max(self.max_mhz or 0.0, float(parts[2]))
            except ValueError:
                continue
            mask = 0
            for (bit, _), v in zip(self.REASONS, parts[5:9]):
                if v.lower().startswith("active"):
                    mask |= bit
            try:
                watts = float(parts[3])
            except ValueError:
                watts = None
            out.append((ts, mhz, mask, watts))
        return out

    def window(self, t0, t1):
        samples = self.samples if self.source == "nvml" else (self._smi_samples() if self.proc else [])
        pad = 0.0 if self.source == "nvml" else 0.05
        sel = [s for s in list(samples) if t0 - pad <= s[0] <= t1 + pad]
        out = dict(sm_mhz=None, sm_max_mhz=self.max_mhz, reasons=[], samples=len(sel), source=self.source)
        if sel:
            out["sm_mhz"] = float(np.median([s[1] for s in sel]))
            mask = 0
            for s in sel:
                mask |= s[2]
            out["reasons"] = sorted(name for bit, name in self.REASONS if mask & bit)
            watts = [s[3] for s in sel if s[3] is not None]
            if watts:
                out["power_w_max"] = round(max(watts), 1)
        return out

    def stop(self):
        self.stop_flag = True
        if self.thread:
            self.thread.join(timeout=1.0)
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            try:
                self.f.close()
                os.remove(self.path)
            except OSError:
                pass


def timed(torch, fn, warmup=5, iters=20):
    """5 warm-up calls, then 20 calls bracketed by CUDA events one at a time: best and median in ms
    (the reference harness's timing, src/bench.cu:75-105)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[0], ts[len(ts) // 2]


def simt_peak_tflops(torch, mhz):
    nsm = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return 2.0 * 128 * nsm * mhz * 1e6 / 1e12


def gemm_sweep(bmb, torch, peaks, clocks):
    """Square GEMM sweep, fp32 SIMT and TF32: 5 warm-ups, 20 timed calls, best and median.  The fp32
    fraction is taken against the SIMT peak at the SM clock sampled while that size's fp32 calls ran."""
    lib = bmb.lib()
    out = []
    tf32_peak = peaks["bf16"] / 2.0
    for n in (1024, 1536, 2048, 4096, 6144, 8192):
        g = torch.Generator(device="cuda").manual_seed(n)
        A = torch.rand(n * n, device="cuda", generator=g) * 2 - 1
        Bm = torch.rand(n * n, device="cuda", generator=g) * 2 - 1
        Cm = torch.zeros(n * n, device="cuda")
        row = dict(n=n)
        for name, fn in (("fp32", lib.bmb_sgemm_simt), ("tf32", lib.bmb_sgemm_tf32)):
            call = lambda: bmb.check(fn(n, n, n, 1.0, A.data_ptr(), Bm.data_ptr(), 0.0, Cm.data_ptr()))
            t0 = time.time()
            best, med = timed(torch, call)
            # small sizes finish before a clock sample lands: keep calling until the window holds a few
            while time.time() - t0 < 0.05:
                call()
            torch.cuda.synchronize()
            ck = clocks.window(t0, time.time())
            row[name + "_tflops"] = round(2.0 * n ** 3 / (best * 1e-3) / 1e12, 2)
            row[name + "_tflops_median"] = round(2.0 * n ** 3 / (med * 1e-3) / 1e12, 2)
            row[name + "_sm_mhz"] = ck["sm_mhz"]
        mhz = row["fp32_sm_mhz"] or clocks.max_mhz or 1965.0
        row["fp32_simt_peak_tflops"] = round(simt_peak_tflops(torch, mhz), 1)
        row["fp32_frac_of_simt_peak"] = round(row["fp32_tflops"] / simt_peak_tflops(torch, mhz), 3)
        row["tf32_frac_of_tensor_peak"] = round(row["tf32_tflops"] / tf32_peak, 3)
        out.append(row)
        del A, Bm, Cm
    return dict(sizes=out, tf32_peak_tflops=round(tf32_peak, 1), timing="5 warm-ups + 20 timed calls, best (and median)",
                peak_note="fp32: SIMT peak = 2*128*SMs*(SM clock sampled during that size's fp32 calls); TF32: burst BF16 of "
                          "MEASURED_PEAKS.json / 2 (%s)" % peaks["source"])


def attention_leg(bmb, torch, peaks, clocks):
    """Fused causal attention at B=8 H=12 T=1024 hs=64: tensor-core (TF32) and fp32 SIMT kernels,
    forward and backward, as time, useful TFLOP/s (4*B*NH*hs*T*(T+1)/2, tools/test_flash.cu:186-187;
    backward 2.5x and the reference's 3.5x count) and fractions of the TF32 tensor peak and of HBM
    bandwidth on the algorithmic bytes (101.1 MB forward, 202.2 MB backward)."""
    lib = bmb.lib()
    B, NH, Tn, hs = 8, 12, 1024, 64
    Cn = NH * hs
    g = torch.Generator(device="cuda").manual_seed(4)
    qkv = torch.randn(B * Tn * 3 * Cn, device="cuda", generator=g)
    dout = torch.randn(B * Tn * Cn, device="cuda", generator=g)
    out, lse = torch.zeros(B * Tn * Cn, device="cuda"), torch.zeros(B * NH * Tn, device="cuda")
    dqkv, dsum = torch.zeros(B * Tn * 3 * Cn, device="cuda"), torch.zeros(B * NH * Tn, device="cuda")
    useful = 4.0 * B * NH * hs * Tn * (Tn + 1) / 2
    fbytes = 4.0 * (B * Tn * 3 * Cn + B * Tn * Cn + B * NH * Tn)
    bbytes = 2.0 * fbytes
    tf32_peak, hbm = peaks["bf16"] / 2.0, peaks["hbm_gbs"]
    res = {"shape": "B=8 H=12 T=1024 hs=64", "useful_flop_fwd": useful, "algorithmic_bytes_fwd": fbytes,
           "algorithmic_bytes_bwd": bbytes, "tf32_peak_tflops": round(tf32_peak, 1), "hbm_peak_gbs": hbm}
    # operands already rounded to TF32, the way the training step hands them over
    qr, dr = qkv.clone(), dout.clone()
    bmb.call("bmb_round_tf32", qr, qr, qr.numel(), None)
    bmb.call("bmb_round_tf32", dr, dr, dr.numel(), None)
    tc_f, tc_b = lib.bmb_flash_num_configs() - 1, lib.bmb_flash_num_bwd_configs() - 1
    t0 = time.time()
    fb, fm = timed(torch, lambda: bmb.call("bmb_flash_attention_forward_ex", tc_f, bmb.FLASH_OPERANDS_ROUNDED, out, lse, qr, B, Tn, Cn, NH))
    bb, bm_ = timed(torch, lambda: bmb.call("bmb_flash_attention_backward_ex", tc_b, bmb.FLASH_OPERANDS_ROUNDED, dqkv, dsum, dr, qr, out, lse, B, Tn, Cn, NH))
    ck = clocks.window(t0, time.time())
    res["tf32"] = {"fwd_us": round(fb * 1e3, 1), "fwd_us_median": round(fm * 1e3, 1), "bwd_us": round(bb * 1e3, 1),
                   "bwd_us_median": round(bm_ * 1e3, 1),
                   "fwd_useful_tflops": round(useful / fb / 1e9, 1), "fwd_frac_of_tf32_peak": round(useful / fb / 1e9 / tf32_peak, 3),
                   "fwd_frac_of_hbm": round(fbytes / fb / 1e6 / hbm, 3),
                   "bwd_tflops_2p5x": round(2.5 * useful / bb / 1e9, 1), "bwd_tflops_3p5x": round(3.5 * useful / bb / 1e9, 1),
                   "bwd_frac_of_tf32_peak_2p5x": round(2.5 * useful / bb / 1e9 / tf32_peak, 3),
                   "bwd_frac_of_hbm": round(bbytes / bb / 1e6 / hbm, 3), "sm_mhz": ck["sm_mhz"],
                   "tokens_per_s_fwd_bwd": round(B * Tn / ((fb + bb) * 1e-3), 0),
                   "kernels": lib.bmb_flash_config_name(tc_f).decode() + " / " + lib.bmb_flash_bwd_config_name(tc_b).decode()}
    t0 = time.time()
    fb, fm = timed(torch, lambda: bmb.call("bmb_flash_attention_forward_cfg", 0, out, lse, qkv, B, Tn, Cn, NH), warmup=3, iters=10)
    bb, bm_ = timed(torch, lambda: bmb.call("bmb_flash_attention_backward_cfg", 0, dqkv, dsum, dout, qkv, out, lse, B, Tn, Cn, NH), warmup=3, iters=10)
    ck = clocks.window(t0, time.time())
    simt = simt_peak_tflops(torch, ck["sm_mhz"] or clocks.max_mhz or 1965.0)
    res["fp32"] = {"fwd_us": round(fb * 1e3, 1), "bwd_us": round(bb * 1e3, 1), "fwd_useful_tflops": round(useful / fb / 1e9, 1),
                   "fwd_frac_of_simt_peak": round(useful / fb / 1e9 / simt, 3),
                   "bwd_tflops_2p5x": round(2.5 * useful / bb / 1e9, 1), "bwd_frac_of_simt_peak_2p5x": round(2.5 * useful / bb / 1e9 / simt, 3),
                   "simt_peak_tflops": round(simt, 1), "sm_mhz": ck["sm_mhz"],
                   "tokens_per_s_fwd_bwd": round(B * Tn / ((fb + bb) * 1e-3), 0)}
    return res


def bgemm_leg(bmb, torch, peaks, clocks):
    """Attention-shaped batched GEMM, batch 96: Q K^T (M=N=1024, K=64) and P V (K=1024, N=64), in
    fp32 SIMT and TF32 modes.  12.9 GFLOP and 453 MB each: the TF32 path is bound by HBM, the fp32
    path by SIMT compute -- both fractions are reported."""
    lib = bmb.lib()
    batch, Tn, hs = 96, 1024, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(batch * Tn * hs, device="cuda", generator=g)
    k = torch.randn(batch * Tn * hs, device="cuda", generator=g)
    att = torch.randn(batch * Tn * Tn, device="cuda", generator=g)
    sc = torch.zeros(batch * Tn * Tn, device="cuda")
    o = torch.zeros(batch * Tn * hs, device="cuda")
    flop = 2.0 * batch * Tn * Tn * hs
    nbytes = 4.0 * batch * (2 * Tn * hs + Tn * Tn)
    cases = (("qk", lambda: bmb.call("bmb_batched_gemm", 0, 1, batch, Tn, Tn, hs, 0.125, q, Tn * hs, k, Tn * hs, 0.0, sc, Tn * Tn, None)),
             ("pv", lambda: bmb.call("bmb_batched_gemm", 0, 0, batch, Tn, hs, Tn, 1.0, att, Tn * Tn, k, Tn * hs, 0.0, o, Tn * hs, None)))
    res = {"shape": "batch 96; Q K^T M=N=1024 K=64; P V M=1024 N=64 K=1024", "flop_each": flop, "algorithmic_bytes_each": nbytes,
           "hbm_peak_gbs": peaks["hbm_gbs"]}
    prev = lib.bmb_get_math_mode()
    try:
        for mode, mname in ((bmb.MATH_FP32, "fp32"), (bmb.MATH_TF32, "tf32")):
            lib.bmb_set_math_mode(mode)
            for tag, fn in cases:
                t0 = time.time()
                best, med = timed(torch, fn)
                ck = clocks.window(t0, time.time())
                ent = {"us": round(best * 1e3, 1), "us_median": round(med * 1e3, 1), "tflops": round(flop / best / 1e9, 2),
                       "gbs": round(nbytes / best / 1e6, 1), "frac_of_hbm": round(nbytes / best / 1e6 / peaks["hbm_gbs"], 3),
                       "sm_mhz": ck["sm_mhz"]}
                if mode == bmb.MATH_FP32:
                    ent["frac_of_simt_peak"] = round(flop / best / 1e9 / simt_peak_tflops(torch, ck["sm_mhz"] or clocks.max_mhz or 1965.0), 3)
                else:
                    ent["frac_of_tf32_peak"] = round(flop / best / 1e9 / (peaks["bf16"] / 2.0), 3)
                res["%s_%s" % (tag, mname)] = ent
    finally:
        lib.bmb_set_math_mode(prev)
    return res


def cpu_matmul():
    """The CPU oracle's fp32 matmul (oracle/bmb_oracle.c, OpenMP) at N = 1024, A and B uniform in
    [-1, 1) from seeds 0 and 1: best of 3."""
    import helpers
    from helpers import _np
    orc = helpers.load_oracle()
    n = 1024
    A, Bm = helpers.uniform(n * n, 0), helpers.uniform(n * n, 1)
    Cm = np.zeros(n * n, np.float32)
    best = 1e30
    for _ in range(3):
        t0 = time.time()
        orc.orc_gemm_fast(0, 0, n, n, n, 1.0, _np(A), _np(Bm), 0.0, _np(Cm))
        best = min(best, time.time() - t0)
    return dict(n=n, gflops=round(2.0 * n ** 3 / best / 1e9, 2), ms=round(best * 1e3, 2), cores=int(orc.orc_num_threads()),
                kind="port", sample="CPU restatement of the fp32 product (the reference has no CPU matmul), M=N=K=1024, best of 3")


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


def note(msg):
    """Progress line on stderr when BMB_BENCH_VERBOSE is set (rank and wall clock in front)."""
    if os.environ.get("BMB_BENCH_VERBOSE"):
        sys.stderr.write("[bench rank %s %.1f] %s\n" % (os.environ.get("RANK", "0"), time.time() % 1000, msg))
        sys.stderr.flush()


def make_trainer(bmb, math, fused):
    return bmb.Trainer(seed=1337, B=B_PER_GPU, T=T, use_flash=1, math=math, fused=fused, beta1=HP["beta1"], beta2=HP["beta2"],
                       eps=HP["eps"], weight_decay=HP["weight_decay"], grad_clip=HP["grad_clip"], **GPT124M)


def fp32_mode_leg(bmb, torch, dist_mod, clocks, steps=5, warmup=3):
    """The same training step in fp32 SIMT arithmetic (the reference's precision): `warmup` untimed steps,
    then `steps` device-timed steps on a resident batch and `steps` more end to end."""
    tr = make_trainer(bmb, bmb.MATH_FP32, 0)
    stream = torch.cuda.ExternalStream(tr.stream)
    batches = []
    for s in range(warmup + 2 * steps):
        x, y = dist_mod.synthetic_batch(s, B_PER_GPU, T, GPT124M["vocab_size"])
        batches.append((torch.from_numpy(x).pin_memory(), torch.from_numpy(y).pin_memory()))
    n = 0
    losses = []
    for i in range(warmup):
        tr.upload(*batches[i]); n += 1
        tr.step(HP["lr"], n)
        losses.append(tr.loss())
    tr.upload(*batches[warmup])
    tr.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    with torch.cuda.stream(stream):
        e0.record()
    for i in range(steps):
        n += 1
        tr.step(HP["lr"], n)
    with torch.cuda.stream(stream):
        e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    ck = clocks.window(t0, time.time())
    host_loss = torch.zeros(1, dtype=torch.float32).pin_memory()
    torch.cuda.synchronize()
    w0 = time.time()
    for i in range(steps):
        tr.upload(*batches[warmup + steps + i]); n += 1
        tr.step(HP["lr"], n)
        tr.loss_async(host_loss)
        tr.sync()
    ms_e2e = (time.time() - w0) * 1e3 / steps
    tr.close()
    simt = simt_peak_tflops(torch, ck["sm_mhz"] or clocks.max_mhz or 1965.0)
    flop = flops_per_step_per_gpu(124475904)
    return dict(dtype="fp32", steps=steps, warmup=warmup, ms_per_step=round(ms, 2), value=round(B_PER_GPU * T / (ms * 1e-3), 1),
                unit="tokens/s", e2e=dict(value=round(B_PER_GPU * T / (ms_e2e * 1e-3), 1), unit="tokens/s",
                                          h2d_bytes_per_step=2 * B_PER_GPU * T * 4, d2h_bytes_per_step=4),
                model_tflops=round(flop / (ms * 1e-3) / 1e12, 1), frac_of_simt_peak=round(flop / (ms * 1e-3) / 1e12 / simt, 3),
                simt_peak_tflops=round(simt, 1), sm_mhz=ck["sm_mhz"], losses_head=[round(float(v), 4) for v in losses])


def dp_selfcheck(bmb, torch, dist_mod, comm, rank, world):
    """N > 1: a small model trained three steps with the gradients summed by one NCCL all-reduce, then with
    the fused exchange over peer memory, from the same seed on the same batches: the largest loss gap, and
    whether the fused run left every rank with bit-identical parameters."""
    import torch.distributed as dist
    cfg = dict(max_seq_len=128, vocab_size=512, padded_vocab=512, n_layer=2, n_head=2, n_embd=128, B=4, T=128)
    rng = np.random.default_rng(99)
    toks = rng.integers(0, 512, (3, 4 * world, 128), dtype=np.int32)
    tgts = rng.integers(0, 512, (3, 4 * world, 128), dtype=np.int32)

    def run(fused):
        tr = bmb.Trainer(seed=1337, use_flash=1, math=bmb.MATH_TF32, fused=1, **cfg)
        tr.attach_comm(comm, world)
        if fused:
            mine = tr.ipc_export()
            tr.attach_peers(rank, world, b"".join(dist_mod.broadcast_bytes(mine, 192, src=r) for r in range(world)))
        losses = []
        for s in range(3):
            tr.upload(dist_mod.shard_rows(toks[s], rank, world), dist_mod.shard_rows(tgts[s], rank, world))
            tr.step(3e-4, s + 1)
            losses.append(tr.loss())
        p = np.empty(tr.num_params, np.float32)
        tr.get_params(p)
        tr.close()
        return np.array(losses), p

    l0, _ = run(False)
    l1, p1 = run(True)
    t = torch.from_numpy(p1)
    lo, hi = t.clone(), t.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    gap = dist_mod.max_over_ranks(float(np.abs(l0 - l1).max()))
    return {"small_model_loss_gap_fused_vs_nccl": float(gap), "small_model_params_equal_across_ranks": bool(torch.equal(lo, hi))}


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

    tr = make_trainer(bmb, math, 0 if args.unfused else 1)
    note("trainer created")
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

    PROF_WARM, PROF_STEPS = 1, 3
    nsteps = args.warmup + 2 * args.steps + PROF_WARM + PROF_STEPS
    pinned = []
    for s in range(nsteps):
        x, y = dist_mod.synthetic_batch(s, B_PER_GPU * world, T, GPT124M["vocab_size"])
        px = torch.from_numpy(dist_mod.shard_rows(x, rank, world)).pin_memory()
        py = torch.from_numpy(dist_mod.shard_rows(y, rank, world)).pin_memory()
        pinned.append((px, py))
    # the batches of the first timed region are staged in HBM before its clock starts
    resident = [(pinned[args.warmup + i][0].cuda(), pinned[args.warmup + i][1].cuda()) for i in range(args.steps)]
    stream = torch.cuda.ExternalStream(tr.stream)
    step_no = [0]
    # every optimiser step's mean loss lands in pinned memory by an asynchronous 4-byte copy
    all_losses = torch.zeros(nsteps, dtype=torch.float32).pin_memory()

    def one_step(i, from_host=True):
        if from_host:
            tr.upload(*pinned[i])
        else:
            tr.upload(*resident[i - args.warmup])      # device-to-device: the batch is already in HBM
        step_no[0] += 1
        tr.step(HP["lr"], step_no[0])
        tr.loss_async(all_losses[step_no[0] - 1:step_no[0]])

    clocks = Clocks(torch, local) if rank == 0 else None
    # warm-up (with IO, so every path has run), then leave a batch resident
    for i in range(args.warmup):
        one_step(i)
        tr.sync()
    torch.cuda.synchronize()
    dist_mod.barrier()
    note("warm-up done")

    # ---- timed region 1: kernel throughput, every batch already resident in HBM (forward + backward
    # replayed as a CUDA graph).  One step streams ~10 GB of activations through the 126 MB L2, so nothing
    # survives in L2 from one use to the next.
    launches_before = lib.bmb_launch_count()
    dist_mod.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_mark = time.time()
    with torch.cuda.stream(stream):
        e0.record()
    for i in range(args.steps):
        one_step(args.warmup + i, from_host=False)
    with torch.cuda.stream(stream):
        e1.record()
    torch.cuda.synchronize()
    dist_mod.barrier()
    ms_dev = dist_mod.max_over_ranks(e0.elapsed_time(e1))
    launches_timed = lib.bmb_launch_count() - launches_before
    note("resident-batch region timed: %.2f ms/step" % (ms_dev / args.steps))

    # ---- timed region 2: end to end.  Every step uploads its batch from pinned memory and its loss is
    # copied back to pinned memory; the host reads the loss of step i-1 while step i runs (the way a
    # training loop logs without draining the GPU every step), and the last one before the clock stops.
    loss_events = [torch.cuda.Event() for _ in range(args.steps)]
    read_losses = []
    dist_mod.barrier()
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        e0.record()
    t0 = time.time()
    first = step_no[0]
    for i in range(args.steps):
        one_step(args.warmup + args.steps + i)
        with torch.cuda.stream(stream):
            loss_events[i].record()
        if i > 0:
            loss_events[i - 1].synchronize()
            read_losses.append(float(all_losses[first + i - 1]))
    loss_events[args.steps - 1].synchronize()
    read_losses.append(float(all_losses[first + args.steps - 1]))
    loss_last = read_losses[-1]
    with torch.cuda.stream(stream):
        e1.record()
    torch.cuda.synchronize()
    wall_ms = (time.time() - t0) * 1e3
    dist_mod.barrier()
    ms_e2e = dist_mod.max_over_ranks(max(e0.elapsed_time(e1), wall_ms))
    step_clocks = clocks.window(t_mark, time.time()) if clocks else None
    note("end-to-end region timed: %.2f ms/step by events, %.2f by the host clock" % (e0.elapsed_time(e1) / args.steps, wall_ms / args.steps))

    # ---- GEMM breakdown: a few more steps launched one kernel at a time with an event pair around
    # every GEMM (not part of either timed region)
    # (the first such step is not counted: the step leaves its CUDA graph for kernel-by-kernel launches there)
    tr.profile(True)
    for i in range(PROF_WARM):
        one_step(args.warmup + 2 * args.steps + i)
    tr.profile(True)                                     # restarts the counters
    for i in range(PROF_STEPS):
        one_step(args.warmup + 2 * args.steps + PROF_WARM + i)
    prof = tr.profile_read()
    tr.profile(False)
    prof["steps"] = PROF_STEPS
    prof["launches"] = launches_timed
    tr.sync()

    note("GEMM breakdown done")
    # losses of the first optimiser steps, averaged over ranks (each rank's loss is its shard's mean)
    head = all_losses[:min(LOSSES_HEAD, nsteps)].clone().double()
    params_equal = None
    dp_check = None
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(head)
        head /= world
        # every rank must hold the same parameters after the run: a float64 sum and sum of squares of the
        # whole buffer plus its first and last 1024 values, compared over ranks
        p = torch.empty(tr.num_params, dtype=torch.float32)
        tr.get_params(p.numpy())
        sig = torch.cat([p.double().sum().reshape(1), (p.double() ** 2).sum().reshape(1), p[:1024].double(), p[-1024:].double()])
        lo, hi = sig.clone(), sig.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        params_equal = bool(torch.equal(lo, hi))
        if not args.nccl_dp and not args.no_dp_check:
            dp_check = dp_selfcheck(bmb, torch, dist_mod, comm, rank, world)

    note("cross-rank checks done: params_equal=%s dp_check=%s" % (params_equal, dp_check))
    tokens_per_step = B_PER_GPU * T * world
    ms_step = ms_dev / args.steps
    value = tokens_per_step / (ms_step * 1e-3)
    e2e_value = tokens_per_step / (ms_e2e / args.steps * 1e-3)
    num_params = tr.num_params

    def finish():
        # every rank leaves together and without a communicator still alive at interpreter exit
        tr.close()
        if comm is not None:
            dist_mod.barrier()
            lib.bmb_comm_destroy(comm)

    if rank != 0:
        finish()
        return
    achieved = prof["gemm_flop"] / (prof["gemm_ms"] * 1e-3) / 1e12 if prof["gemm_ms"] > 0 else 0.0
    if math == bmb.MATH_FP32:
        peak = simt_peak_tflops(torch, (step_clocks or {}).get("sm_mhz") or 1965.0)
        bound, peak_note = "fp32-simt", "2*128*SMs*SM clock sampled during the timed steps"
    else:
        scale = 2.0 if math == bmb.MATH_TF32 else 1.0
        peak = peaks["bf16_sustained"] / scale
        bound, peak_note = "tensor", "sustained BF16 of MEASURED_PEAKS.json (%s)%s" % (
            peaks["source"], " / 2 for TF32" if scale == 2.0 else "")
    stored_traffic = math == bmb.MATH_TF32 and not args.unfused
    line = {
        "metric": "GPT-124M train tokens/s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": {0: "fp32", 1: "tf32", 2: "bf16"}[math], "data": "synthetic",
        "config": config_dict(world, num_params),
        "notes": {"gradient_exchange": ("none" if world == 1 else "NCCL all-reduce, full optimiser per rank" if args.nccl_dp
                                        else ("fused over peer memory: piece-wise reduce, AdamW on the pieces, parameter broadcast; "
                                              + {"1": "three chunks, reduced under backward", "2": "three chunks, under backward and the next forward"}.get(
                                                  os.environ.get("BMB_TRAINER_OVERLAP", "0"), "one chunk after backward"))),
                  "l2": "per-step working set (~10 GB of activations) exceeds the 126 MB L2",
                  "arithmetic": "TF32 tensor-core GEMMs and attention, fp32 everywhere else" if math == bmb.MATH_TF32 else
                                ("fp32 SIMT" if math == bmb.MATH_FP32 else "BF16 tensor-core GEMMs")},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 2 * B_PER_GPU * T * 4,
                "d2h_bytes_per_step": 4, "loss_read": "every step, one step late (asynchronous copy to pinned memory)"},
        "gpu_launches": int(prof["launches"]),
        "loss_last_step": round(float(loss_last), 4),
        "losses_head": [round(float(v), 4) for v in head],
        "model_tflops": round(flops_per_step_per_gpu(num_params) * world / (ms_step * 1e-3) / 1e12, 1),
        "roofline": {"bound": "tensor", "kernel": "GEMMs of the step (%d calls)" % prof["gemm_calls"],
                     "achieved": round(achieved, 1), "peak": round(peak, 1), "unit": "TFLOP/s",
                     "frac": round(achieved / peak, 3) if peak else None,
                     "traffic": GEMM_DRAM_BYTES_PER_LAUNCH if stored_traffic else None,
                     "traffic_source": ("stored constant: each GEMM shape of the step captured alone under a profiler, "
                                        "weighted by launches per step; not measured in this run") if stored_traffic else None,
                     "algorithmic_bytes_per_launch": GEMM_ALGO_BYTES_PER_LAUNCH,
                     "gemm_ms_per_step": round(prof["gemm_ms"] / prof["steps"], 3), "peak_note": peak_note,
                     "bound_detail": bound},
        "clocks": step_clocks,
    }
    if world > 1:
        line["params_equal_across_ranks"] = params_equal
        if dp_check:
            line["dp_check"] = dp_check
    finish()
    torch.cuda.empty_cache()
    if world == 1:
        if not args.no_sweep:
            # the short kernels first: after the large TF32 products the power cap holds the SM clock down
            # for a while, which would be charged to whatever runs next
            time.sleep(0.5)
            line["attention"] = attention_leg(bmb, torch, peaks, clocks)
            line["bgemm"] = bgemm_leg(bmb, torch, peaks, clocks)
            line["gemm"] = gemm_sweep(bmb, torch, peaks, clocks)
            time.sleep(0.5)
            if math != bmb.MATH_FP32:
                line["fp32_mode"] = fp32_mode_leg(bmb, torch, dist_mod, clocks)
        if not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline()
            line["cpu_matmul"] = cpu_matmul()
    if clocks:
        clocks.stop()
    note("printing the line")
    print(json.dumps(line), flush=True)


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
    total = max(args.warmup + args.steps, LOSSES_HEAD)
    batches = [dist_mod.synthetic_batch(s, B_PER_GPU * n, T, c["vocab_size"]) for s in range(total)]
    step = 0
    losses = []
    for i in range(args.warmup):
        step += 1
        losses.append(ref.ref_trainer_step(h, _np(batches[i][0]), _np(batches[i][1]), HP["lr"], step))
    clocks = Clocks(torch, 0)
    torch.cuda.synchronize()
    t0 = time.time()
    for i in range(args.steps):
        step += 1
        losses.append(ref.ref_trainer_step(h, _np(batches[args.warmup + i][0]), _np(batches[args.warmup + i][1]), HP["lr"], step))
    t1 = time.time()
    ms = (t1 - t0) * 1e3 / args.steps
    ck = clocks.window(t0, t1)
    num_params = ref.ref_trainer_num_params(h)
    ref.ref_trainer_destroy(h)
    torch.cuda.set_device(0)
    # The head of the loss curve, untimed, from a fresh replica on the same batches.  Two values per step: what
    # the reference's gpt_forward returned, and the loss recomputed from the probabilities its kernel wrote.  They
    # differ at this vocabulary because the reference's loss kernel reads p[target] without a barrier after the
    # loop that normalises p (src/nn.cu:216-220); the recomputed one is what the formula defines.
    h = ref.ref_trainer_create(c["max_seq_len"], c["vocab_size"], c["padded_vocab"], c["n_layer"], c["n_head"],
                               c["n_embd"], B_PER_GPU, T, 1, 1337, n, HP["beta1"], HP["beta2"], HP["eps"],
                               HP["weight_decay"], HP["grad_clip"])
    head_returned, head = [], []
    for s in range(LOSSES_HEAD):
        head_returned.append(ref.ref_trainer_step(h, _np(batches[s][0]), _np(batches[s][1]), HP["lr"], s + 1))
        head.append(ref.ref_trainer_loss_from_probs(h))
    ref.ref_trainer_destroy(h)
    torch.cuda.set_device(0)
    value = B_PER_GPU * T * n / (ms * 1e-3)
    line = {
        "impl": "reference", "metric": "GPT-124M train tokens/s", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": n, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": config_dict(n, num_params),
        "notes": {"how": "the reference's own gpt_forward / gpt_backward / ddp_allreduce / adamw_update compiled for sm_100a, "
                         "threads in one process as its train_gpt does", "arithmetic": "fp32 SIMT"},
        "e2e": {"value": round(value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 2 * B_PER_GPU * T * 4,
                "d2h_bytes_per_step": 8},
        "cpu_baseline": {"value": round(value, 1), "unit": "tokens/s", "cores": 0, "kind": "reference",
                         "sample": "the reference has no CPU implementation; this arm runs its CUDA kernels on the "
                                   "same GPU(s), timed by wall clock around its blocking step (host uploads and "
                                   "loss read-backs are inside every step)"},
        "loss_last_step": round(float(losses[args.warmup + args.steps - 1]), 4),
        "losses_head": [round(float(v), 4) for v in head],
        "losses_head_as_returned": [round(float(v), 4) for v in head_returned],
        "losses_note": "losses_head is recomputed from the probabilities the reference's kernel wrote; the value its "
                       "gpt_forward returns reads p[target] before every thread has normalised it and is too low at this "
                       "vocabulary", "clocks": ck}
    if n == 1 and not args.no_sweep:
        line.update(reference_kernels(ref, torch, clocks))
    clocks.stop()
    print(json.dumps(line), flush=True)


def reference_kernels(ref, torch, clocks):
    """The reference's own kernels beside its training step: its fused attention at B=8 H=12 T=1024 hs=64 and
    its best fp32 (registry id 8) and tensor-core (id 9) GEMM at N = 8192, timed the same way as this
    repository's (5 warm-ups, best of 20 / of 5 for the long fp32 GEMM)."""
    B, NH, Tn, hs = 8, 12, 1024, 64
    Cn = NH * hs
    g = torch.Generator(device="cuda").manual_seed(4)
    qkv = torch.randn(B * Tn * 3 * Cn, device="cuda", generator=g)
    dout = torch.randn(B * Tn * Cn, device="cuda", generator=g)
    out, lse = torch.zeros(B * Tn * Cn, device="cuda"), torch.zeros(B * NH * Tn, device="cuda")
    dqkv, dsum = torch.zeros(B * Tn * 3 * Cn, device="cuda"), torch.zeros(B * NH * Tn, device="cuda")
    useful = 4.0 * B * NH * hs * Tn * (Tn + 1) / 2
    fb, _ = timed(torch, lambda: ref.ref_flash_attention_forward(out.data_ptr(), lse.data_ptr(), qkv.data_ptr(), B, Tn, Cn, NH), 3, 10)
    bb, _ = timed(torch, lambda: ref.ref_flash_attention_backward(dqkv.data_ptr(), dsum.data_ptr(), dout.data_ptr(), qkv.data_ptr(),
                                                                   out.data_ptr(), lse.data_ptr(), B, Tn, Cn, NH), 3, 10)
    res = {"attention": {"shape": "B=8 H=12 T=1024 hs=64", "fp32": {"fwd_us": round(fb * 1e3, 1), "bwd_us": round(bb * 1e3, 1),
                                                                     "fwd_useful_tflops": round(useful / fb / 1e9, 1),
                                                                     "bwd_tflops_2p5x": round(2.5 * useful / bb / 1e9, 1)}}}
    del qkv, dout, out, lse, dqkv, dsum
    nn = 8192
    A = torch.rand(nn * nn, device="cuda") * 2 - 1
    Bm = torch.rand(nn * nn, device="cuda") * 2 - 1
    Cm = torch.zeros(nn * nn, device="cuda")
    row = dict(n=nn)
    for name, kid, iters in (("fp32", 8, 5), ("tf32", 9, 10)):
        best, _ = timed(torch, lambda: ref.ref_sgemm(kid, nn, nn, nn, 1.0, A.data_ptr(), Bm.data_ptr(), 0.0, Cm.data_ptr()), 2, iters)
        row[name + "_tflops"] = round(2.0 * nn ** 3 / (best * 1e-3) / 1e12, 2)
    res["gemm"] = {"sizes": [row], "kernels": "registry id 8 (dbuffer, fp32) and id 9 (tensorcore, WMMA TF32)"}
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="bmb", choices=["bmb", "reference"])
    ap.add_argument("--math", default=os.environ.get("BMB_BENCH_MATH", "tf32"), choices=["fp32", "tf32", "bf16"])
    ap.add_argument("--no-sweep", action="store_true", help="skip the kernel legs (GEMM sweep, attention, batched GEMM, fp32 mode)")
    ap.add_argument("--unfused", action="store_true", help="the reference's op list: separate bias kernels, "
                    "operands rounded by a prepass instead of by their producers")
    ap.add_argument("--nccl-dp", action="store_true", help="N > 1: sum gradients with one NCCL all-reduce and run the "
                    "whole optimiser on every rank, instead of the fused exchange over peer memory")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs")
    ap.add_argument("--no-dp-check", action="store_true", help="N > 1: skip the small-model comparison of the fused exchange with NCCL")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_bmb(args)


if __name__ == "__main__":
    main()
