"""Per-kernel timings of libbmb.so on one GPU, one JSON line per case.

    python bare-metal-bard_b200/kernel_bench.py [gemm] [bgemm] [flash] [nn] [--small]
    python bare-metal-bard_b200/kernel_bench.py one:tf32:nt:8192x3072x768:rounded      (a single GEMM case)
    python bare-metal-bard_b200/kernel_bench.py registry --csv runs/a.csv [-s 1024,2048]   (the registry sweep as CSV)
    python bare-metal-bard_b200/kernel_bench.py timeline:tf32:nt:8192x3072x768:rounded     (per-CTA timeline, timer build)
    python bare-metal-bard_b200/kernel_bench.py flash_timeline                             (attention forward: work-item stamps and knock-out timings, timer build)
    python bare-metal-bard_b200/kernel_bench.py flash_scan                                 (tensor-core attention at B*T = 8192 for T = 128 .. 4096: fixed cost per CTA against cost per block)

`registry --csv` appends one row per (registry entry, size) in the columns the reference harness writes
(src/bench.cu:238-245, 293-299): kernel_id,kernel,size,gflops_best,gflops_median,cublas_gflops_best,
pct_of_cublas -- so that tools/merge_runs.py and tools/plot_results.py of the reference read the
new numbers unchanged.  The cuBLAS column is torch.matmul in true fp32 on the same operands, the
harness's baseline column; it is not part of the library.

Timing follows the reference harness (src/bench.cu:75-105): 5 warm-up calls,
then 20 calls bracketed by CUDA events one at a time; best and median are
reported.  Work counts are the algorithmic ones:
  GEMM          2*M*N*K FLOP
  flash fwd     4*B*NH*hs*T*(T+1)/2 FLOP ("useful causal", tools/test_flash.cu:186-187)
  flash bwd     2.5x (five products) and the reference's 3.5x count of that
  nn kernels    bytes that must cross HBM once
`--small` shrinks every case so that a profiler capture of one launch ends in
seconds; the shapes stay larger than the 126 MB L2 where DRAM figures matter.
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from __graft_entry__ import load_package  # noqa: E402


def timed(fn, warmup=5, iters=20):
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


def emit(**kw):
    print(json.dumps(kw), flush=True)


def bench_gemm(bmb, small):
    lib = bmb.lib()
    sizes = (1024, 2048) if small else (1024, 1536, 2048, 4096, 6144, 8192)
    for n in sizes:
        A = torch.rand(n * n, device="cuda") * 2 - 1
        B = torch.rand(n * n, device="cuda") * 2 - 1
        Cm = torch.zeros(n * n, device="cuda")
        for name, fn in (("simt_fp32", lib.bmb_sgemm_simt), ("tcgen05_tf32", lib.bmb_sgemm_tf32),
                         ("tcgen05_bf16", lib.bmb_sgemm_bf16)):
            best, med = timed(lambda: bmb.check(fn(n, n, n, 1.0, A.data_ptr(), B.data_ptr(), 0.0, Cm.data_ptr())),
                              iters=8 if (name == "simt_fp32" and n > 4096) else 20)
            emit(kernel=name, M=n, N=n, K=n, best_ms=round(best, 4), median_ms=round(med, 4),
                 tflops_best=round(2.0 * n ** 3 / best / 1e9, 2), tflops_median=round(2.0 * n ** 3 / med / 1e9, 2))
    # the GEMM shapes of the 124M-parameter training step (8192 rows)
    if not small:
        shapes = [("fwd qkv NT", 0, 1, 8192, 2304, 768), ("fwd fc NT", 0, 1, 8192, 3072, 768),
                  ("fwd fcproj NT", 0, 1, 8192, 768, 3072), ("fwd head NT", 0, 1, 8192, 50304, 768),
                  ("dX fc NN", 0, 0, 8192, 768, 3072), ("dW fc TN", 1, 0, 3072, 768, 8192),
                  ("dW head TN", 1, 0, 50304, 768, 8192)]
        for tag, ta, tb, M, N, K in shapes:
            A = torch.rand(M * K, device="cuda") * 2 - 1
            B = torch.rand(K * N, device="cuda") * 2 - 1
            Cm = torch.zeros(M * N, device="cuda")
            for math, mname in ((bmb.MATH_FP32, "simt_fp32"), (bmb.MATH_TF32, "tcgen05_tf32")):
                best, med = timed(lambda: bmb.call("bmb_gemm_ex", math, 0, ta, tb, M, N, K, 1.0, A, B, 0.0, Cm, None),
                                  iters=10)
                emit(kernel=mname, shape=tag, M=M, N=N, K=K, best_ms=round(best, 4), median_ms=round(med, 4),
                     tflops_best=round(2.0 * M * N * K / best / 1e9, 2))
            del A, B, Cm


def bench_bgemm(bmb, small):
    # attention-shaped batched GEMM: batch 96, Q.K^T (M=N=1024, K=64) and P.V (K=1024, N=64)
    batch, T, hs = (24 if small else 96), 1024, 64
    q = torch.randn(batch * T * hs, device="cuda")
    k = torch.randn(batch * T * hs, device="cuda")
    att = torch.zeros(batch * T * T, device="cuda")
    o = torch.zeros(batch * T * hs, device="cuda")
    for tag, fn, flop, nbytes in (
            ("QK^T NT", lambda: bmb.call("bmb_batched_gemm", 0, 1, batch, T, T, hs, 0.125, q, T * hs, k, T * hs, 0.0, att, T * T, None),
             2.0 * batch * T * T * hs, 4.0 * batch * (2 * T * hs + T * T)),
            ("PV NN", lambda: bmb.call("bmb_batched_gemm", 0, 0, batch, T, hs, T, 1.0, att, T * T, k, T * hs, 0.0, o, T * hs, None),
             2.0 * batch * T * T * hs, 4.0 * batch * (2 * T * hs + T * T))):
        prev = bmb.lib().bmb_get_math_mode()
        for mode, name in ((bmb.MATH_FP32, "bgemm_simt_fp32"), (bmb.MATH_TF32, "bgemm_tcgen05_tf32")):
            bmb.lib().bmb_set_math_mode(mode)
            best, med = timed(fn)
            emit(kernel=name, shape=tag, batch=batch, best_ms=round(best, 4), median_ms=round(med, 4),
                 tflops_best=round(flop / best / 1e9, 2), gbs_best=round(nbytes / best / 1e6, 1))
        bmb.lib().bmb_set_math_mode(prev)


def bench_flash(bmb, small):
    lib = bmb.lib()
    B, NH, T, hs = (2 if small else 8), 12, 1024, 64
    C = NH * hs
    qkv = torch.randn(B * T * 3 * C, device="cuda")
    dout = torch.randn(B * T * C, device="cuda")
    out, lse = torch.zeros(B * T * C, device="cuda"), torch.zeros(B * NH * T, device="cuda")
    dqkv, dsum = torch.zeros(B * T * 3 * C, device="cuda"), torch.zeros(B * NH * T, device="cuda")
    useful = 4.0 * B * NH * hs * T * (T + 1) / 2
    fbytes = 4.0 * (B * T * 3 * C + B * T * C + B * NH * T)
    for cfg in range(lib.bmb_flash_num_configs()):
        name = lib.bmb_flash_config_name(cfg).decode()
        best, med = timed(lambda: bmb.call("bmb_flash_attention_forward_cfg", cfg, out, lse, qkv, B, T, C, NH))
        emit(kernel="flash_fwd", config=name, B=B, NH=NH, T=T, hs=hs, best_ms=round(best, 4), median_ms=round(med, 4),
             useful_tflops_best=round(useful / best / 1e9, 2), gbs_best=round(fbytes / best / 1e6, 1))
    # the tensor-core kernels alone, on operands already rounded to TF32 (how the training step runs them)
    tc_fwd = lib.bmb_flash_num_configs() - 1
    qr, dr = qkv.clone(), dout.clone()
    bmb.call("bmb_round_tf32", qr, qr, qr.numel(), None)
    bmb.call("bmb_round_tf32", dr, dr, dr.numel(), None)
    best, med = timed(lambda: bmb.call("bmb_flash_attention_forward_ex", tc_fwd, bmb.FLASH_OPERANDS_ROUNDED, out, lse, qr, B, T, C, NH))
    emit(kernel="flash_fwd", config=lib.bmb_flash_config_name(tc_fwd).decode() + ", operands pre-rounded", B=B, NH=NH, T=T, hs=hs,
         best_ms=round(best, 4), median_ms=round(med, 4), useful_tflops_best=round(useful / best / 1e9, 2),
         gbs_best=round(fbytes / best / 1e6, 1))
    bmb.call("bmb_flash_attention_forward_cfg", 0, out, lse, qkv, B, T, C, NH)
    bbytes = 4.0 * (2 * B * T * 3 * C + 2 * B * T * C + 2 * B * NH * T)
    for cfg in range(lib.bmb_flash_num_bwd_configs()):
        name = lib.bmb_flash_bwd_config_name(cfg).decode()
        best, med = timed(lambda: bmb.call("bmb_flash_attention_backward_cfg", cfg, dqkv, dsum, dout, qkv, out, lse, B, T, C, NH))
        emit(kernel="flash_bwd", config=name, B=B, NH=NH, T=T, hs=hs, best_ms=round(best, 4), median_ms=round(med, 4),
             tflops_2p5x_best=round(2.5 * useful / best / 1e9, 2), tflops_3p5x_best=round(3.5 * useful / best / 1e9, 2),
             gbs_best=round(bbytes / best / 1e6, 1))
    tc_bwd = lib.bmb_flash_num_bwd_configs() - 1
    best, med = timed(lambda: bmb.call("bmb_flash_attention_backward_ex", tc_bwd, bmb.FLASH_OPERANDS_ROUNDED, dqkv, dsum, dr, qr, out, lse, B, T, C, NH))
    emit(kernel="flash_bwd", config=lib.bmb_flash_bwd_config_name(tc_bwd).decode() + ", operands pre-rounded", B=B, NH=NH, T=T, hs=hs,
         best_ms=round(best, 4), median_ms=round(med, 4), tflops_2p5x_best=round(2.5 * useful / best / 1e9, 2),
         tflops_3p5x_best=round(3.5 * useful / best / 1e9, 2), gbs_best=round(bbytes / best / 1e6, 1))


def bench_flash_scan(bmb, small):
    """Tensor-core attention, operands pre-rounded, at a constant B*T: the number of CTAs (work items) stays the same
    while the 128 x 128 blocks they walk grow with T, so a straight line through the times separates the fixed cost per
    CTA (intercept) from the cost per block (slope)."""
    lib = bmb.lib()
    NH, hs = 12, 64
    C = NH * hs
    tc_fwd, tc_bwd = lib.bmb_flash_num_configs() - 1, lib.bmb_flash_num_bwd_configs() - 1
    tokens = 2048 if small else 8192
    for T in (128, 256, 512, 1024, 2048, 4096):
        if T > tokens:
            continue
        B = tokens // T
        qkv, dout = torch.randn(B * T * 3 * C, device="cuda"), torch.randn(B * T * C, device="cuda")
        out, lse = torch.zeros(B * T * C, device="cuda"), torch.zeros(B * NH * T, device="cuda")
        dqkv, dsum = torch.zeros(B * T * 3 * C, device="cuda"), torch.zeros(B * NH * T, device="cuda")
        bmb.call("bmb_round_tf32", qkv, qkv, qkv.numel(), None)
        bmb.call("bmb_round_tf32", dout, dout, dout.numel(), None)
        f, _ = timed(lambda: bmb.call("bmb_flash_attention_forward_ex", tc_fwd, bmb.FLASH_OPERANDS_ROUNDED, out, lse, qkv, B, T, C, NH))
        g, _ = timed(lambda: bmb.call("bmb_flash_attention_backward_ex", tc_bwd, bmb.FLASH_OPERANDS_ROUNDED, dqkv, dsum, dout, qkv, out, lse, B, T, C, NH))
        nb = T // 128
        emit(kernel="flash_scan", B=B, NH=NH, T=T, hs=hs, fwd_us=round(f * 1e3, 1), bwd_us=round(g * 1e3, 1),
             bwd_ctas=2 * B * NH * nb, blocks_128x128=B * NH * nb * (nb + 1) // 2)


def bench_nn(bmb, small):
    N, C, V = (2048 if small else 8192), 768, 50304
    x = torch.randn(N * C, device="cuda")
    w, b = torch.ones(C, device="cuda"), torch.zeros(C, device="cuda")
    y, mean, rstd = torch.zeros(N * C, device="cuda"), torch.zeros(N, device="cuda"), torch.zeros(N, device="cuda")
    dx, dw, db = torch.zeros(N * C, device="cuda"), torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
    cases = [("layernorm_fwd", lambda: bmb.call("bmb_layernorm_forward", y, mean, rstd, x, w, b, N, C), 2.0 * N * C * 4),
             ("layernorm_bwd", lambda: bmb.call("bmb_layernorm_backward", dx, dw, db, y, x, w, mean, rstd, N, C), 4.0 * N * C * 4)]
    h = torch.randn(N * 4 * C, device="cuda")
    g = torch.zeros(N * 4 * C, device="cuda")
    g2 = torch.zeros(N * 4 * C, device="cuda")
    b4 = torch.zeros(4 * C, device="cuda")
    cases += [("gelu_fwd", lambda: bmb.call("bmb_gelu_forward", g, h, N * 4 * C), 2.0 * N * 4 * C * 4),
              ("gelu_bwd", lambda: bmb.call("bmb_gelu_backward", g2, h, g, N * 4 * C), 3.0 * N * 4 * C * 4),
              ("bias_fwd", lambda: bmb.call("bmb_bias_forward", g, b4, N, 4 * C), 2.0 * N * 4 * C * 4),
              ("bias_bwd", lambda: bmb.call("bmb_bias_backward", b4, g, N, 4 * C), 1.0 * N * 4 * C * 4),
              ("residual", lambda: bmb.call("bmb_residual_forward", dx, x, y, N * C), 3.0 * N * C * 4)]
    logits = torch.randn(N * V, device="cuda")
    probs, dlog = torch.zeros(N * V, device="cuda"), torch.zeros(N * V, device="cuda")
    losses = torch.zeros(N, device="cuda")
    tg = torch.randint(0, V, (N,), device="cuda", dtype=torch.int32)
    cases += [("softmax_xent_fwd", lambda: bmb.call("bmb_softmax_crossentropy_forward", probs, losses, logits, tg, N, V, V), 2.0 * N * V * 4),
              ("xent_bwd", lambda: bmb.call("bmb_crossentropy_softmax_backward", dlog, probs, tg, N, V, V, 1.0 / N), 2.0 * N * V * 4)]
    n = 31118976 if small else 124475904
    p, gr, m, v = (torch.zeros(n, device="cuda") for _ in range(4))
    cases += [("adamw", lambda: bmb.call("bmb_adamw_update", p, gr, m, v, n, 3e-4, 0.9, 0.95, 1e-8, 0.1, 1, 1.0), 7.0 * n * 4)]
    sq = torch.zeros(1, device="cuda", dtype=torch.float64)
    cases += [("grad_sumsq", lambda: bmb.call("bmb_grad_sumsq_device", gr, n, sq), 1.0 * n * 4)]
    for name, fn, nbytes in cases:
        best, med = timed(fn)
        emit(kernel=name, best_ms=round(best, 4), median_ms=round(med, 4), algorithmic_MB=round(nbytes / 1e6, 1),
             gbs_best=round(nbytes / best / 1e6, 1), gbs_median=round(nbytes / med / 1e6, 1))


CSV_FIELDS = ["kernel_id", "kernel", "size", "gflops_best", "gflops_median", "cublas_gflops_best", "pct_of_cublas"]


def append_csv(path, rows):
    """Append rows (dicts keyed by CSV_FIELDS) in the reference harness's format: header only when the
    file is new, two decimals (src/bench.cu:244, 297-298)."""
    new = not os.path.exists(path)
    with open(path, "a") as f:
        if new:
            f.write(",".join(CSV_FIELDS) + "\n")
        for r in rows:
            f.write("%d,%s,%d,%.2f,%.2f,%.2f,%.2f\n" % (r["kernel_id"], r["kernel"], r["size"], r["gflops_best"],
                                                       r["gflops_median"], r["cublas_gflops_best"], r["pct_of_cublas"]))


def bench_registry(bmb, csv_path, sizes):
    """Every registry entry over square sizes, 5 warm-ups + 20 timed calls each, with the table the
    reference harness prints and, when asked, its CSV."""
    lib = bmb.lib()
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    table = lib.bmb_kernel_table()
    print("%-4s %-20s %6s %11s %11s %11s %8s" % ("id", "kernel", "size", "best GF/s", "med GF/s", "cuBLAS GF/s", "%cuBLAS"))
    rows = []
    for k in range(lib.bmb_num_kernels()):
        e = table[k]
        fn = getattr(lib, {1: "bmb_sgemm_simt", 2: "bmb_sgemm_tf32", 3: "bmb_sgemm_bf16"}[e.id])
        for n in sizes:
            A = torch.rand(n, n, device="cuda") * 2 - 1
            B = torch.rand(n, n, device="cuda") * 2 - 1
            Cm = torch.zeros(n, n, device="cuda")
            best, med = timed(lambda: bmb.check(fn(n, n, n, 1.0, A.data_ptr(), B.data_ptr(), 0.0, Cm.data_ptr())))
            cb, _ = timed(lambda: torch.matmul(A, B, out=Cm))
            gf, gfm, gfb = (2.0 * n ** 3 / (t * 1e-3) / 1e9 for t in (best, med, cb))
            row = dict(kernel_id=e.id, kernel=e.name.decode(), size=n, gflops_best=gf, gflops_median=gfm,
                       cublas_gflops_best=gfb, pct_of_cublas=100.0 * gf / gfb)
            rows.append(row)
            print("%-4d %-20s %6d %11.1f %11.1f %11.1f %7.1f%%" % (e.id, row["kernel"], n, gf, gfm, gfb, row["pct_of_cublas"]))
            del A, B, Cm
    torch.backends.cuda.matmul.allow_tf32 = prev
    if csv_path:
        append_csv(csv_path, rows)


def bench_one(bmb, spec):
    """One GEMM case, for a profiler capture or a quick comparison:
        one:<math>:<ta><tb>:<M>x<N>x<K>[:rounded][:nosplit][:pair|:nopair][:m128|:m256][:beta1]
    math = fp32 | tf32 | bf16; ta/tb = n or t; `rounded` feeds operands already rounded to TF32
    (what the training step does), `nosplit` keeps every tile on one CTA, `pair` / `nopair` force or forbid
    CTA pairs, `m128` / `m256` force the tile height of single CTAs, `half` plans for half of the SMs, `beta1`
    accumulates into C.  Timed as
    20 back-to-back launches between one pair of events (what a kernel costs inside a stream of kernels)."""
    parts = spec.split(":")
    math = {"fp32": bmb.MATH_FP32, "tf32": bmb.MATH_TF32, "bf16": bmb.MATH_BF16}[parts[1]]
    ta, tb = (1 if ch == "t" else 0 for ch in parts[2])
    M, N, K = (int(x) for x in parts[3].split("x"))
    opts = parts[4:]
    A = torch.rand(M * K, device="cuda") * 2 - 1
    B = torch.rand(K * N, device="cuda") * 2 - 1
    Cm = torch.zeros(M * N, device="cuda")
    flags = 0
    if "rounded" in opts:
        bmb.call("bmb_round_tf32", A, A, M * K, None)
        bmb.call("bmb_round_tf32", B, B, K * N, None)
        flags |= bmb.GEMM_A_ROUNDED | bmb.GEMM_B_ROUNDED
    if "nosplit" in opts:
        flags |= bmb.GEMM_NO_SPLIT
    if "pair" in opts:
        flags |= bmb.GEMM_PAIR
    if "nopair" in opts:
        flags |= bmb.GEMM_NO_PAIR
    if "m128" in opts:
        flags |= bmb.GEMM_TILE_M128
    if "m256" in opts:
        flags |= bmb.GEMM_TILE_M256
    if "half" in opts:
        flags |= bmb.GEMM_HALF_SMS
    beta = 1.0 if "beta1" in opts else 0.0
    call = lambda: bmb.call("bmb_gemm_ex", math, flags, ta, tb, M, N, K, 1.0, A, B, beta, Cm, None)
    best, med = timed(call, warmup=3, iters=5)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        call()
    e1.record()
    e1.synchronize()
    b2b = e0.elapsed_time(e1) / 20
    emit(kernel="gemm_ex", spec=spec, best_ms=round(best, 4), median_ms=round(med, 4),
         tflops_best=round(2.0 * M * N * K / best / 1e9, 2), back_to_back_ms=round(b2b, 4),
         tflops_back_to_back=round(2.0 * M * N * K / b2b / 1e9, 2))


def bench_flash_timeline(bmb, small):
    """flash_timeline -- where the tensor-core attention forward spends its time (B = 8 or, with --small, 2; 12 heads,
    T = 1024, head size 64, operands pre-rounded).  Needs a library built with the developer timers
    (`BMB_NVCC_FLAGS=-DBMB_FLASH_TRACE python bare-metal-bard_b200/build.py -f`).  Printed: per CTA (a sample) the
    nanosecond stamps of its work items (first scores ready, last block folded, output stored) after the first
    CTA's entry; then the back-to-back cost of a launch with parts of the kernel switched off (the results are
    then wrong, only the time means something): 1 no exponentials, 2 no P V load / fold, 4 no maximum, 8 no store
    of P, 16 no score products, 32 no P V products."""
    import ctypes as C
    import numpy as np
    try:
        dbg = C.CDLL(bmb.LIB_PATH)
        dbg.bmb_dbg_flash_trace.argtypes = [C.c_void_p]
        dbg.bmb_dbg_flash_ko.argtypes = [C.c_int]
    except AttributeError:
        raise SystemExit("this libbmb.so has no timers: rebuild with BMB_NVCC_FLAGS=-DBMB_FLASH_TRACE")
    B, NH, T, hs = (2 if small else 8), 12, 1024, 64
    Cd = NH * hs
    qkv = torch.randn(B * T * 3 * Cd, device="cuda")
    out = torch.empty(B * T * Cd, device="cuda")
    lse = torch.empty(B * NH * T, device="cuda")
    bmb.call("bmb_round_tf32", qkv, qkv, qkv.numel(), None)
    run = lambda: bmb.call("bmb_flash_attention_forward_ex", 2, bmb.FLASH_OPERANDS_ROUNDED, out, lse, qkv, B, T, Cd, NH)
    for _ in range(5):
        run()
    torch.cuda.synchronize()
    dbg.bmb_dbg_flash_trace_clear()
    run()
    torch.cuda.synchronize()
    buf = np.zeros((160, 24), dtype=np.uint64)
    dbg.bmb_dbg_flash_trace(buf.ctypes.data)
    t = buf[:148].astype(np.int64)
    t = t[t[:, 0] > 0]
    t0 = t[:, 0].min()
    us = lambda a: round(float(a - t0) / 1000.0, 1)
    rows = []
    for c in sorted(set([0, 8, len(t) // 2, len(t) - 1])):
        items = [[us(t[c][2 + 4 * r]), us(t[c][3 + 4 * r]), us(t[c][4 + 4 * r])] for r in range(5) if t[c][2 + 4 * r]]
        rows.append({"cta": int(c), "items_first_scores_last_fold_stored_us": items, "exit_us": us(t[c][1]),
                     "wait_scores_cycles": int(t[c][22]), "wait_pv_cycles": int(t[c][23])})
    emit(kernel="flash_fwd_timeline", B=B, ctas=int(len(t)), last_exit_us=us(t[:, 1].max()), median_exit_us=us(np.median(t[:, 1])), sample=rows)
    for ko in (0, 1, 2, 15, 16, 32, 48, 63, 0):
        dbg.bmb_dbg_flash_ko(ko)
        for _ in range(5):
            run()
        torch.cuda.synchronize()
        best = 1e9
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(20):
                run()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) / 20 * 1000)
        emit(kernel="flash_fwd_knockout", B=B, switched_off=ko, back_to_back_us=round(best, 1))
    dbg.bmb_dbg_flash_ko(0)


def bench_timeline(bmb, spec):
    """timeline:<math>:<ta><tb>:<M>x<N>x<K>[:rounded][...]  -- where one tensor-core GEMM launch spends its time.
    Needs a library built with the developer timers (`BMB_NVCC_FLAGS=-DBMB_GEMM_TRACE python
    bare-metal-bard_b200/build.py -f`): every CTA then stamps, in nanoseconds of the global timer, its entry,
    set-up done, first copy issued, first K slice landed, last product issued, first accumulator ready, last tile
    stored, stores landed, exit -- and adds up the cycles its issuing thread waited for operand slices and for a free
    accumulator, its producer for a free slot, and one epilogue warp for a finished accumulator.  Printed: min /
    median / max over CTAs of each stamp, in microseconds after the first CTA's entry, the waits (median, max), and
    the event-timed cost of the launch alone and inside 20 back-to-back launches."""
    import ctypes as C
    lib = bmb.lib()
    try:
        dbg = C.CDLL(bmb.LIB_PATH).bmb_dbg_gemm_trace
    except AttributeError:
        raise SystemExit("this libbmb.so has no timers: rebuild with BMB_NVCC_FLAGS=-DBMB_GEMM_TRACE")
    dbg.argtypes = [C.c_void_p]
    parts = spec.split(":")
    math = {"fp32": bmb.MATH_FP32, "tf32": bmb.MATH_TF32, "bf16": bmb.MATH_BF16}[parts[1]]
    ta, tb = (1 if ch == "t" else 0 for ch in parts[2])
    M, N, K = (int(x) for x in parts[3].split("x"))
    opts = parts[4:]
    A = torch.rand(M * K, device="cuda") * 2 - 1
    B = torch.rand(K * N, device="cuda") * 2 - 1
    Cm = torch.zeros(M * N, device="cuda")
    flags = 0
    if "rounded" in opts:
        bmb.call("bmb_round_tf32", A, A, M * K, None)
        bmb.call("bmb_round_tf32", B, B, K * N, None)
        flags |= bmb.GEMM_A_ROUNDED | bmb.GEMM_B_ROUNDED
    for name, bit in (("nosplit", bmb.GEMM_NO_SPLIT), ("pair", bmb.GEMM_PAIR), ("nopair", bmb.GEMM_NO_PAIR),
                      ("m128", bmb.GEMM_TILE_M128), ("m256", bmb.GEMM_TILE_M256), ("half", bmb.GEMM_HALF_SMS)):
        if name in opts:
            flags |= bit
    beta = 1.0 if "beta1" in opts else 0.0
    call = lambda: bmb.call("bmb_gemm_ex", math, flags, ta, tb, M, N, K, 1.0, A, B, beta, Cm, None)
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    buf = np.zeros((256, 16), np.uint64)
    dbg(buf.ctypes.data)                       # clears the device-side stamps
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); call(); e1.record(); e1.synchronize()
    single = e0.elapsed_time(e1) * 1e3
    dbg(buf.ctypes.data)
    t = buf[:, :9].astype(np.float64)
    t = t[t[:, 0] > 0]
    rel = (t - t[:, 0].min()) / 1e3
    names = ["entry", "setup", "copy1", "slice1", "lastmma", "acc1", "laststore", "landed", "exit"]
    e0.record()
    for _ in range(20):
        call()
    e1.record(); e1.synchronize()
    live = buf[:, 0] > 0
    waits = {n: [int(np.median(buf[live, 10 + i])), int(buf[live, 10 + i].max())] for i, n in
             enumerate(["issuer_on_full", "issuer_on_tmem_empty", "producer_on_empty", "epilogue_on_tmem_full"])}
    emit(kernel="gemm_timeline", spec=spec, ctas=int(t.shape[0]), single_us=round(single, 1), wait_cycles_median_max=waits,
         back_to_back_us=round(e0.elapsed_time(e1) * 1e3 / 20, 1),
         us_min_median_max={n: [round(float(rel[:, i].min()), 1), round(float(np.median(rel[:, i])), 1), round(float(rel[:, i].max()), 1)]
                            for i, n in enumerate(names)})


def main():
    argv = sys.argv[1:]
    csv_path, sizes = None, [1024, 1536, 2048, 4096, 6144, 8192]
    for flag in ("--csv", "-s"):
        if flag in argv:
            i = argv.index(flag)
            value = argv[i + 1]
            del argv[i:i + 2]
            if flag == "--csv":
                csv_path = value
            else:
                sizes = [int(x) for x in value.split(",")]
    args = [a for a in argv if not a.startswith("--")]
    small = "--small" in argv
    which = args or ["gemm", "bgemm", "flash", "nn"]
    bmb = load_package()
    torch.cuda.set_device(0)
    if "registry" in which:
        bench_registry(bmb, csv_path, sizes)
        which = [x for x in which if x != "registry"]
        if not which:
            return
    for w in [x for x in which if x.startswith("one:")]:
        bench_one(bmb, w)
    for w in [x for x in which if x.startswith("timeline:")]:
        bench_timeline(bmb, w)
    if "flash_timeline" in which:
        bench_flash_timeline(bmb, small)
    if "flash_scan" in which:
        bench_flash_scan(bmb, small)
    which = [x for x in which if not x.startswith(("one:", "timeline:")) and x not in ("flash_timeline", "flash_scan")]
    for w in which:
        {"gemm": bench_gemm, "bgemm": bench_bgemm, "flash": bench_flash, "nn": bench_nn}[w](bmb, small)


if __name__ == "__main__":
    main()
