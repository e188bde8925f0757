"""Generate tests/golden/*.npz from the reference's own CUDA kernels.

Runs on a machine with a GPU and with oracle/_ref/libbmbref.so built (the
unmodified reference sources compiled for sm_100a; see oracle/Makefile).  Each
fixture stores seeded inputs together with the outputs the reference kernels
produced for them, so that the CPU oracle can be pinned against the reference
on machines without a GPU:

    python tests/golden/make_golden.py [output_dir]      # default: tests/golden

The reference stores no golden vectors of its own; its tests compare two GPU
implementations on the fly (tools/test_gemm.cu, test_flash.cu, test_grad.cu).
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import helpers  # noqa: E402


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


def p(t):
    return t.data_ptr()


def main(out_dir):
    ref = helpers.load_reference()
    orc = helpers.load_oracle()
    assert ref is not None, "build oracle/_ref/libbmbref.so first (make -C oracle ref)"
    os.makedirs(out_dir, exist_ok=True)
    torch.cuda.set_device(0)

    # ---- gemm: the ragged and aligned shapes of tools/test_gemm.cu, alpha .75 beta 1.25
    for (M, N, K) in [(100, 70, 33), (128, 128, 128)]:
        for ta in (0, 1):
            for tb in (0, 1):
                A = helpers.xorshift(M * K, 0x1234, orc)
                B = helpers.xorshift(K * N, 0x9abc, orc)
                C0 = helpers.xorshift(M * N, 0x5555, orc)
                dA, dB, dC = dev(A), dev(B), dev(C0)
                ref.ref_gemm(ta, tb, M, N, K, 0.75, p(dA), p(dB), 1.25, p(dC))
                np.savez_compressed(os.path.join(out_dir, "gemm_%d%d_%dx%dx%d.npz" % (ta, tb, M, N, K)),
                                    kind="gemm", ta=ta, tb=tb, M=M, N=N, K=K, alpha=0.75, beta=1.25,
                                    A=A, B=B, C0=C0, out=host(dC))
    # ---- registry: best fp32 kernel (8) and the TF32 kernel (9), alpha .5 beta 3 (src/bench.cu:261)
    for kid in (8, 9):
        n = 256
        A, B, C0 = (helpers.xorshift(n * n, s, orc) for s in (0x12345678, 0x9abcdef0, 0x0f0f0f0f))
        dA, dB, dC = dev(A), dev(B), dev(C0)
        assert ref.ref_sgemm(kid, n, n, n, 0.5, p(dA), p(dB), 3.0, p(dC)) == 0
        np.savez_compressed(os.path.join(out_dir, "sgemm_k%d_%d.npz" % (kid, n)), kind="sgemm", kid=kid, n=n,
                            alpha=0.5, beta=3.0, A=A, B=B, C0=C0, out=host(dC), tol=ref.ref_kernel_tol(kid))
    # ---- batched gemm, ragged case of tools/test_gemm.cu:122-176
    batch, M, N, K = 8, 100, 48, 33
    A, B, C0 = helpers.xorshift(batch * M * K, 0x1234, orc), helpers.xorshift(batch * K * N, 0x9abc, orc), \
        helpers.xorshift(batch * M * N, 0x5555, orc)
    dA, dB, dC = dev(A), dev(B), dev(C0)
    ref.ref_batched_gemm(0, 1, batch, M, N, K, 0.5, p(dA), M * K, p(dB), K * N, 2.0, p(dC), M * N)
    np.savez_compressed(os.path.join(out_dir, "bgemm_01_ragged.npz"), kind="bgemm", ta=0, tb=1, batch=batch, M=M,
                        N=N, K=K, alpha=0.5, beta=2.0, A=A, B=B, C0=C0, out=host(dC))
    # ---- attention: fused and unfused, a ragged shape of tools/test_flash.cu:336-340
    for (Bn, T, Cc, NH) in [(2, 33, 128, 2), (1, 100, 128, 4)]:
        qkv = helpers.xorshift(Bn * T * 3 * Cc, 1234, orc)
        dout = helpers.xorshift(Bn * T * Cc, 99, orc)
        dq, dd = dev(qkv), dev(dout)
        out, lse = torch.zeros(Bn * T * Cc, device="cuda"), torch.zeros(Bn * NH * T, device="cuda")
        ref.ref_flash_attention_forward(p(out), p(lse), p(dq), Bn, T, Cc, NH)
        dqkv, dsum = torch.zeros(Bn * T * 3 * Cc, device="cuda"), torch.zeros(Bn * NH * T, device="cuda")
        ref.ref_flash_attention_backward(p(dqkv), p(dsum), p(dd), p(dq), p(out), p(lse), Bn, T, Cc, NH)
        uo = torch.zeros(Bn * T * Cc, device="cuda")
        qkvr = torch.zeros(4 * Bn * T * Cc, device="cuda")
        att = torch.zeros(Bn * NH * T * T, device="cuda")
        ref.ref_attention_forward(p(uo), p(qkvr), p(att), p(dq), Bn, T, Cc, NH)
        np.savez_compressed(os.path.join(out_dir, "attention_%d_%d_%d_%d.npz" % (Bn, T, Cc, NH)), kind="attention",
                            B=Bn, T=T, C=Cc, NH=NH, qkv=qkv, dout=dout, out=host(out), lse=host(lse),
                            dqkv=host(dqkv), out_unfused=host(uo))
    # ---- nn kernels
    N, Cc = 12, 96
    x, w, b, dy = (helpers.normal(s, sd) for s, sd in (((N, Cc), 1), (Cc, 2), (Cc, 3), ((N, Cc), 4)))
    dx0, dw0, db0 = helpers.normal((N, Cc), 5), helpers.normal(Cc, 6), helpers.normal(Cc, 7)
    o, mean, rstd = (torch.zeros(n, device="cuda") for n in (N * Cc, N, N))
    dxx, dww, dbb = dev(dx0), dev(dw0), dev(db0)
    tx, tw, tb_, tdy = dev(x), dev(w), dev(b), dev(dy)
    ref.ref_layernorm_forward(p(o), p(mean), p(rstd), p(tx), p(tw), p(tb_), N, Cc)
    ref.ref_layernorm_backward(p(dxx), p(dww), p(dbb), p(tdy), p(tx), p(tw), p(mean), p(rstd), N, Cc)
    g = torch.zeros(N * Cc, device="cuda")
    dg = torch.zeros(N * Cc, device="cuda")
    ref.ref_gelu_forward(p(g), p(tx), N * Cc)
    ref.ref_gelu_backward(p(dg), p(tx), p(tdy), N * Cc)
    dbias = dev(db0)
    ref.ref_bias_backward(p(dbias), p(tdy), N, Cc)
    V, Vp = 65, 128
    logits = helpers.normal((N, Vp), 8, 3.0)
    tg = np.random.default_rng(9).integers(0, V, N, dtype=np.int32)
    tl, tt = dev(logits), dev(tg)
    probs, losses, dlog = torch.zeros(N * Vp, device="cuda"), torch.zeros(N, device="cuda"), torch.zeros(N * Vp, device="cuda")
    ref.ref_softmax_crossentropy_forward(p(probs), p(losses), p(tl), p(tt), N, V, Vp)
    ref.ref_crossentropy_softmax_backward(p(dlog), p(probs), p(tt), N, V, Vp, 1.0 / N)
    np_, ng = helpers.normal(1000, 10), helpers.normal(1000, 11)
    pm, pv = np.abs(helpers.normal(1000, 12, 0.1)), np.abs(helpers.normal(1000, 13, 0.01))
    tp, tgd, tm, tv = dev(np_), dev(ng), dev(pm), dev(pv)
    ref.ref_adamw_update(p(tp), p(tgd), p(tm), p(tv), 1000, 3e-4, 0.9, 0.95, 1e-8, 0.1, 3, 0.5)
    gn = ref.ref_grad_global_norm(p(tgd), 1000)
    np.savez_compressed(os.path.join(out_dir, "nn_ops.npz"), kind="nn", N=N, C=Cc, V=V, Vp=Vp, x=x, w=w, b=b, dy=dy,
                        dx0=dx0, dw0=dw0, db0=db0, ln_out=host(o), ln_mean=host(mean), ln_rstd=host(rstd),
                        ln_dx=host(dxx), ln_dw=host(dww), ln_db=host(dbb), gelu=host(g), dgelu=host(dg),
                        dbias=host(dbias), logits=logits, targets=tg, probs=host(probs), losses=host(losses),
                        dlogits=host(dlog), ad_p0=np_, ad_g=ng, ad_m0=pm, ad_v0=pv, ad_p=host(tp), ad_m=host(tm),
                        ad_v=host(tv), gnorm=gn)
    # ---- train step: 20 optimiser steps, loss trajectory (fused attention path)
    cfg = dict(maxT=32, V=65, Vp=128, L=2, NH=2, C=64, B=2, T=32)
    h = ref.ref_trainer_create(cfg["maxT"], cfg["V"], cfg["Vp"], cfg["L"], cfg["NH"], cfg["C"], cfg["B"], cfg["T"], 1,
                               1337, 1, 0.9, 0.95, 1e-8, 0.1, 1.0)
    n = ref.ref_trainer_num_params(h)
    params0 = np.empty(n, np.float32)
    ref.ref_trainer_get_params(h, helpers._np(params0))
    rng = np.random.default_rng(4242)
    toks = rng.integers(0, cfg["V"], (20, cfg["B"], cfg["T"]), dtype=np.int32)
    tgts = rng.integers(0, cfg["V"], (20, cfg["B"], cfg["T"]), dtype=np.int32)
    grads1 = np.empty(n, np.float32)
    loss_fb = ref.ref_trainer_forward_backward(h, helpers._np(toks[0]), helpers._np(tgts[0]))
    ref.ref_trainer_get_grads(h, helpers._np(grads1))
    losses_t = [ref.ref_trainer_step(h, helpers._np(toks[s]), helpers._np(tgts[s]), 3e-4, s + 1) for s in range(20)]
    params20 = np.empty(n, np.float32)
    ref.ref_trainer_get_params(h, helpers._np(params20))
    ref.ref_trainer_destroy(h)
    np.savez_compressed(os.path.join(out_dir, "train_20steps.npz"), kind="train", params0=params0, tokens=toks,
                        targets=tgts, losses=np.array(losses_t, np.float32), loss_fb=loss_fb,
                        grad_norm1=float(np.linalg.norm(grads1.astype(np.float64))),
                        grads1_sample=grads1[::97].copy(), params20_sample=params20[::97].copy(),
                        lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, clip=1.0, **cfg)
    print("wrote fixtures to", out_dir)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
