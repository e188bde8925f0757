"""GPU parity: every CUDA entry point, called through the C ABI, against the
CPU oracle and (where oracle/_ref/libbmbref.so was built) against the
reference's own kernels on the same seeded inputs.

Bars: fp32 GEMM normwise 1e-6 against the CPU fp32 product; attention and the
nn kernels 1e-5 against the oracle and the reference's fp32 kernels
(tools/test_flash.cu:132); train loss |delta| <= 2e-3 per step over 20 steps.
"""
import ctypes as C

import numpy as np
import pytest

from helpers import _np, normal, normwise, uniform, xorshift

pytestmark = pytest.mark.gpu


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(torch, t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


# ------------------------------------------------------------------- GEMM
SHAPES = [(128, 128, 128), (256, 512, 128), (512, 384, 384), (384, 384, 1024), (100, 70, 33), (65, 65, 65),
          (130, 260, 60), (1, 1, 1), (1, 300, 7)]


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_fp32_vs_oracle(bmb, orc, cuda, ta, tb, M, N, K):
    A, B, C0 = uniform(M * K, 1), uniform(K * N, 2), uniform(M * N, 3)
    want = C0.copy()
    orc.orc_gemm(ta, tb, M, N, K, 0.75, _np(A), _np(B), 1.25, _np(want))
    dA, dB, dC = dev(cuda, A), dev(cuda, B), dev(cuda, C0)
    bmb.call("bmb_gemm_ex", bmb.MATH_FP32, 0, ta, tb, M, N, K, 0.75, dA, dB, 1.25, dC, None)
    assert normwise(host(cuda, dC), want) < 1e-6


def test_gemm_fp32_vs_reference_kernels(bmb, ref, orc, cuda):
    for (M, N, K) in [(256, 512, 128), (100, 70, 33)]:
        for ta in (0, 1):
            for tb in (0, 1):
                A, B, C0 = xorshift(M * K, 0x1234, orc), xorshift(K * N, 0x9abc, orc), xorshift(M * N, 0x5555, orc)
                dA, dB, d1, d2 = dev(cuda, A), dev(cuda, B), dev(cuda, C0), dev(cuda, C0)
                bmb.call("bmb_gemm_ex", bmb.MATH_FP32, 0, ta, tb, M, N, K, 0.75, dA, dB, 1.25, d1, None)
                ref.ref_gemm(ta, tb, M, N, K, 0.75, dA.data_ptr(), dB.data_ptr(), 1.25, d2.data_ptr())
                assert normwise(host(cuda, d1), host(cuda, d2)) < 1e-6


def test_sgemm_1024_seed0_config(bmb, orc, cuda):
    """Single fp32 SGEMM M=N=K=1024, A and B uniform in [-1,1) from seed 0,
    checked against the CPU fp32 product at normwise 1e-6."""
    n = 1024
    A, B = uniform(n * n, 0), uniform(n * n, 1)
    want = np.zeros(n * n, np.float32)
    orc.orc_gemm_fast(0, 0, n, n, n, 1.0, _np(A), _np(B), 0.0, _np(want))
    dA, dB, dC = dev(cuda, A), dev(cuda, B), cuda.full((n * n,), float("nan"), device="cuda")
    bmb.call("bmb_sgemm_simt", n, n, n, 1.0, dA, dB, 0.0, dC)
    err = normwise(host(cuda, dC), want)
    assert err < 1e-6, err
    e = bmb.lib().bmb_find_kernel(1).contents
    assert e.name == b"simt_fp32" and err < e.tol


@pytest.mark.parametrize("ta", [0, 1])
def test_gemm_fp32_tma_fed_kernel_is_bit_identical_to_the_register_staged_one(bmb, orc, cuda, monkeypatch, ta):
    """NN and TN on aligned shapes run on the SIMT kernel whose operand slices arrive by TMA.  Same k order,
    same fused multiply-add: against the CPU oracle's sequential fmaf chain (orc_gemm) the result is exact
    for alpha 1, beta 0, and a long K (many trips round the 3-slot ring) with beta != 0 stays within 1e-6."""
    M, N, K = 256, 384, 2048
    A, B, C0 = uniform(M * K, 21), uniform(K * N, 22), uniform(M * N, 23)
    want = np.zeros(M * N, np.float32)
    orc.orc_gemm(ta, 0, M, N, K, 1.0, _np(A), _np(B), 0.0, _np(want))
    dA, dB = dev(cuda, A), dev(cuda, B)
    dC = cuda.full((M * N,), float("nan"), device="cuda")
    bmb.call("bmb_gemm_ex", bmb.MATH_FP32, 0, ta, 0, M, N, K, 1.0, dA, dB, 0.0, dC, None)
    assert np.array_equal(host(cuda, dC), want)
    want2 = C0.copy()
    orc.orc_gemm(ta, 0, M, N, K, 0.75, _np(A), _np(B), 1.25, _np(want2))
    dC = dev(cuda, C0)
    bmb.call("bmb_gemm_ex", bmb.MATH_FP32, 0, ta, 0, M, N, K, 0.75, dA, dB, 1.25, dC, None)
    assert normwise(host(cuda, dC), want2) < 1e-6


def test_gemm_beta_zero_ignores_garbage_and_k0(bmb, cuda):
    dA, dB = dev(cuda, uniform(128 * 16, 1)), dev(cuda, uniform(16 * 128, 2))
    dC = cuda.full((128 * 128,), float("nan"), device="cuda")
    bmb.call("bmb_gemm", 0, 0, 128, 128, 16, 1.0, dA, dB, 0.0, dC, None)
    assert np.all(np.isfinite(host(cuda, dC)))
    dC = cuda.full((64,), 2.0, device="cuda")
    bmb.call("bmb_gemm", 0, 0, 8, 8, 0, 1.0, dA, dB, 0.5, dC, None)
    assert np.all(host(cuda, dC) == 1.0)
    bmb.call("bmb_gemm", 0, 0, 0, 8, 4, 1.0, dA, dB, 0.5, dC, None)   # empty: no-op


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("batch,M,N,K", [(24, 64, 64, 32), (8, 100, 48, 33), (12, 256, 256, 64), (12, 256, 64, 256),
                                         (3, 128, 256, 96)])   # the last: aligned, NN / TN go to the kernel fed by TMA
def test_batched_gemm_vs_oracle(bmb, orc, cuda, ta, tb, batch, M, N, K):
    A, B, C0 = normal(batch * M * K, 1), normal(batch * K * N, 2), normal(batch * M * N, 3)
    want = C0.copy()
    orc.orc_batched_gemm(ta, tb, batch, M, N, K, 0.5, _np(A), M * K, _np(B), K * N, 2.0, _np(want), M * N)
    dA, dB, dC = dev(cuda, A), dev(cuda, B), dev(cuda, C0)
    prev = bmb.lib().bmb_get_math_mode()
    bmb.lib().bmb_set_math_mode(bmb.MATH_FP32)
    bmb.call("bmb_batched_gemm", ta, tb, batch, M, N, K, 0.5, dA, M * K, dB, K * N, 2.0, dC, M * N, None)
    bmb.lib().bmb_set_math_mode(prev)
    assert normwise(host(cuda, dC), want) < 1e-6


def test_gemm_full_size_linearity_and_sampled_rows(bmb, orc, cuda):
    """N = 4096 (a size of the sweep the oracle cannot finish in seconds):
    linearity in B, plus 8 sampled output rows against the oracle."""
    n = 4096
    A, B1, B2 = uniform(n * n, 10), uniform(n * n, 11), uniform(n * n, 12)
    dA, dB1, dB2 = dev(cuda, A), dev(cuda, B1), dev(cuda, B2)
    c1, c2, c3 = (cuda.zeros(n * n, device="cuda") for _ in range(3))
    bmb.call("bmb_sgemm_simt", n, n, n, 1.0, dA, dB1, 0.0, c1)
    bmb.call("bmb_sgemm_simt", n, n, n, 1.0, dA, dB2, 0.0, c2)
    bmb.call("bmb_sgemm_simt", n, n, n, 1.0, dA, dB1 + dB2, 0.0, c3)
    assert normwise(host(cuda, c1 + c2), host(cuda, c3)) < 1e-5   # three roundings, not one
    rows = [0, 1, 127, 128, 2047, 3000, 4094, 4095]
    Asub = np.ascontiguousarray(A.reshape(n, n)[rows])
    want = np.zeros((len(rows), n), np.float32)
    orc.orc_gemm_fast(0, 0, len(rows), n, n, 1.0, _np(Asub), _np(B1), 0.0, _np(want))
    assert normwise(host(cuda, c1).reshape(n, n)[rows], want) < 1e-6


# -------------------------------------------------------------- attention
ATT_SHAPES = [(2, 64, 128, 2), (3, 100, 384, 6), (2, 33, 384, 6), (1, 1, 384, 6), (2, 129, 256, 8), (5, 200, 128, 4),
              (1, 256, 256, 2)]


@pytest.mark.parametrize("B,T,C,NH", ATT_SHAPES)
def test_flash_forward_backward_vs_oracle(bmb, orc, cuda, B, T, C, NH):
    qkv, dout = normal(B * T * 3 * C, 1234), normal(B * T * C, 99)
    wout, wlse = np.empty(B * T * C, np.float32), np.empty(B * NH * T, np.float32)
    orc.orc_attention_forward(_np(wout), _np(wlse), None, _np(qkv), B, T, C, NH)
    wd = np.empty(B * T * 3 * C, np.float32)
    orc.orc_attention_backward(_np(wd), _np(dout), _np(qkv), B, T, C, NH)
    dq, dd = dev(cuda, qkv), dev(cuda, dout)
    lib = bmb.lib()
    for cfg in range(lib.bmb_flash_num_configs()):
        # outputs poisoned first, as tools/test_flash.cu:103-106
        out = cuda.full((B * T * C,), float("nan"), device="cuda")
        lse = cuda.full((B * NH * T,), float("nan"), device="cuda")
        tensor_core = lib.bmb_flash_config_name(cfg).startswith(b"tcgen05")
        st = lib.bmb_flash_attention_forward_cfg(cfg, out.data_ptr(), lse.data_ptr(), dq.data_ptr(), B, T, C, NH)
        if st == bmb.E_UNSUPPORTED and tensor_core and C // NH != 64:
            continue                      # that config serves head size 64 only
        bmb.check(st, "bmb_flash_attention_forward_cfg")
        tol = 2e-3 if tensor_core else 1e-5     # TF32 products vs fp32 arithmetic
        assert normwise(host(cuda, out), wout) < tol
        assert normwise(host(cuda, lse), wlse) < tol
    # the backward below starts from the fp32 forward's out / lse
    bmb.call("bmb_flash_attention_forward_cfg", 0, out, lse, dq, B, T, C, NH)
    for cfg in range(lib.bmb_flash_num_bwd_configs()):
        dqkv = cuda.full((B * T * 3 * C,), float("nan"), device="cuda")
        dsum = cuda.full((B * NH * T,), float("nan"), device="cuda")
        tensor_core = lib.bmb_flash_bwd_config_name(cfg).startswith(b"tcgen05")
        st = lib.bmb_flash_attention_backward_cfg(cfg, dqkv.data_ptr(), dsum.data_ptr(), dd.data_ptr(), dq.data_ptr(),
                                                  out.data_ptr(), lse.data_ptr(), B, T, C, NH)
        if st == bmb.E_UNSUPPORTED and tensor_core and C // NH != 64:
            continue
        bmb.check(st, "bmb_flash_attention_backward_cfg")
        g, w = host(cuda, dqkv).reshape(B * T, 3, C), wd.reshape(B * T, 3, C)
        for i in range(3):
            # dq, dk, dv separately (tools/test_flash.cu:312-314); the denominator is floored at 5 % of the
            # whole gradient's magnitude (25 % for TF32, whose residue in dP - D scales with dO and v) because at T = 1
            # dq and dk are exactly zero.  fp32: 1e-5, TF32: 5e-3.
            den = max(float(np.max(np.abs(w[:, i]))), (0.25 if tensor_core else 0.05) * float(np.max(np.abs(w))))
            err = float(np.max(np.abs(g[:, i].astype(np.float64) - w[:, i]))) / den
            assert np.all(np.isfinite(g)) and err < (5e-3 if tensor_core else 1e-5), (cfg, i, err)


def test_flash_vs_reference_fused_and_unfused(bmb, ref, orc, cuda):
    """The reference's own comparison (tools/test_flash.cu): default shape
    B16 T256 C384 NH6, xorshift seeds 1234 / 99, normwise < 1e-5."""
    B, T, C, NH = 16, 256, 384, 6
    qkv, dout = xorshift(B * T * 3 * C, 1234, orc), xorshift(B * T * C, 99, orc)
    dq, dd = dev(cuda, qkv), dev(cuda, dout)
    mk = lambda n: cuda.zeros(n, device="cuda")
    o1, l1, o2, l2 = mk(B * T * C), mk(B * NH * T), mk(B * T * C), mk(B * NH * T)
    bmb.call("bmb_flash_attention_forward", o1, l1, dq, B, T, C, NH)
    ref.ref_flash_attention_forward(o2.data_ptr(), l2.data_ptr(), dq.data_ptr(), B, T, C, NH)
    assert normwise(host(cuda, o1), host(cuda, o2)) < 1e-5 and normwise(host(cuda, l1), host(cuda, l2)) < 1e-5
    g1, s1, g2, s2 = mk(B * T * 3 * C), mk(B * NH * T), mk(B * T * 3 * C), mk(B * NH * T)
    bmb.call("bmb_flash_attention_backward", g1, s1, dd, dq, o1, l1, B, T, C, NH)
    ref.ref_flash_attention_backward(g2.data_ptr(), s2.data_ptr(), dd.data_ptr(), dq.data_ptr(), o2.data_ptr(),
                                     l2.data_ptr(), B, T, C, NH)
    a, b = host(cuda, g1).reshape(B * T, 3, C), host(cuda, g2).reshape(B * T, 3, C)
    for i in range(3):
        assert normwise(a[:, i], b[:, i]) < 1e-5
    # the unfused path of both libraries
    qkvr, att, uo = mk(4 * B * T * C), mk(B * NH * T * T), mk(B * T * C)
    bmb.call("bmb_attention_forward", uo, qkvr, att, dq, B, T, C, NH)
    assert normwise(host(cuda, uo), host(cuda, o2)) < 1e-5
    dqkvr, datt, ug = mk(4 * B * T * C), mk(B * NH * T * T), mk(B * T * 3 * C)
    bmb.call("bmb_attention_backward", ug, dqkvr, datt, datt, dd, qkvr, att, B, T, C, NH)
    c = host(cuda, ug).reshape(B * T, 3, C)
    for i in range(3):
        assert normwise(c[:, i], b[:, i]) < 1e-5


def test_flash_full_size_properties(bmb, cuda):
    """B8 H12 T1024 hs64: rows of P sum to one (out of an all-ones V equals one),
    the first token attends only to itself, and fused == unfused."""
    B, T, C, NH = 8, 1024, 768, 12
    qkv = normal(B * T * 3 * C, 7).reshape(B, T, 3, C)
    qkv[:, :, 2, :] = 1.0
    dq = dev(cuda, qkv.reshape(-1))
    out, lse = cuda.zeros(B * T * C, device="cuda"), cuda.zeros(B * NH * T, device="cuda")
    bmb.call("bmb_flash_attention_forward", out, lse, dq, B, T, C, NH)
    assert np.max(np.abs(host(cuda, out) - 1.0)) < 1e-5
    qkv = normal(B * T * 3 * C, 8)
    dq = dev(cuda, qkv)
    bmb.call("bmb_flash_attention_forward", out, lse, dq, B, T, C, NH)
    o = host(cuda, out).reshape(B, T, C)
    assert normwise(o[:, 0, :], qkv.reshape(B, T, 3, C)[:, 0, 2, :]) < 1e-6
    qkvr, att, uo = cuda.zeros(4 * B * T * C, device="cuda"), cuda.zeros(B * NH * T * T, device="cuda"), \
        cuda.zeros(B * T * C, device="cuda")
    bmb.call("bmb_attention_forward", uo, qkvr, att, dq, B, T, C, NH)
    assert normwise(o, host(cuda, uo)) < 1e-5


def test_flash_rejects_unsupported_head_size(bmb, cuda):
    x = cuda.zeros(1024, device="cuda")
    st = bmb.lib().bmb_flash_attention_forward(x.data_ptr(), x.data_ptr(), x.data_ptr(), 1, 2, 48, 1)
    assert st == bmb.E_UNSUPPORTED and b"head size 48" in bmb.lib().bmb_last_error()


# -------------------------------------------------------------- nn kernels
@pytest.mark.parametrize("N,Cc", [(64, 768), (12, 96), (7, 50), (5, 1024), (3, 2052)])
def test_layernorm_vs_oracle(bmb, orc, cuda, N, Cc):
    x, w, b, dy = normal((N, Cc), 1), normal(Cc, 2), normal(Cc, 3), normal((N, Cc), 4)
    o, mean, rstd = np.empty((N, Cc), np.float32), np.empty(N, np.float32), np.empty(N, np.float32)
    orc.orc_layernorm_forward(_np(o), _np(mean), _np(rstd), _np(x), _np(w), _np(b), N, Cc)
    dx, dw, db = normal((N, Cc), 5), normal(Cc, 6), normal(Cc, 7)
    wdx, wdw, wdb = dx.copy(), dw.copy(), db.copy()
    orc.orc_layernorm_backward(_np(wdx), _np(wdw), _np(wdb), _np(dy), _np(x), _np(w), _np(mean), _np(rstd), N, Cc)
    tx, tw, tb, tdy = dev(cuda, x), dev(cuda, w), dev(cuda, b), dev(cuda, dy)
    to, tm, tr = cuda.zeros(N * Cc, device="cuda"), cuda.zeros(N, device="cuda"), cuda.zeros(N, device="cuda")
    bmb.call("bmb_layernorm_forward", to, tm, tr, tx, tw, tb, N, Cc)
    assert normwise(host(cuda, to), o) < 1e-5 and normwise(host(cuda, tm), mean) < 1e-5
    assert normwise(host(cuda, tr), rstd) < 1e-5
    tdx, tdw, tdb = dev(cuda, dx), dev(cuda, dw), dev(cuda, db)
    bmb.call("bmb_layernorm_backward", tdx, tdw, tdb, tdy, tx, tw, tm, tr, N, Cc)
    assert normwise(host(cuda, tdx), wdx) < 1e-5
    assert normwise(host(cuda, tdw), wdw) < 1e-5 and normwise(host(cuda, tdb), wdb) < 1e-5
    # the fused forms the training step uses: residual add + layernorm, and backward + column sums of dinp
    ta, tb2 = dev(cuda, x - dy), dev(cuda, dy)                 # a + b == x up to fp32 rounding of the split
    ts, fo, fm, fr = (cuda.zeros(n, device="cuda") for n in (N * Cc, N * Cc, N, N))
    bmb.call("bmb_residual_layernorm_forward", ts, fo, fm, fr, ta, tb2, tw, tb, N, Cc)
    ssum = ((x - dy) + dy).astype(np.float32)
    assert np.array_equal(host(cuda, ts).reshape(N, Cc), ssum)
    uo, um, ur = cuda.zeros(N * Cc, device="cuda"), cuda.zeros(N, device="cuda"), cuda.zeros(N, device="cuda")
    bmb.call("bmb_layernorm_forward", uo, um, ur, ts, tw, tb, N, Cc)
    assert np.array_equal(host(cuda, fo), host(cuda, uo)) and np.array_equal(host(cuda, fm), host(cuda, um))
    cdx, cdw, cdb, ccs = dev(cuda, dx), dev(cuda, dw), dev(cuda, db), dev(cuda, normal(Cc, 8))
    bmb.call("bmb_layernorm_backward_colsum", cdx, cdw, cdb, ccs, tdy, tx, tw, tm, tr, N, Cc)
    assert np.array_equal(host(cuda, cdx), host(cuda, tdx)) and np.array_equal(host(cuda, cdw), host(cuda, tdw))
    want_cs = normal(Cc, 8).astype(np.float64) + host(cuda, tdx).reshape(N, Cc).astype(np.float64).sum(0)
    assert normwise(host(cuda, ccs), want_cs.astype(np.float32)) < 1e-5


def test_layernorm_backward_is_reproducible(bmb, cuda):
    N, Cc = 4096, 768
    x, w, dy = dev(cuda, normal((N, Cc), 1)), dev(cuda, normal(Cc, 2)), dev(cuda, normal((N, Cc), 4))
    b = cuda.zeros(Cc, device="cuda")
    o, m, r = cuda.zeros(N * Cc, device="cuda"), cuda.zeros(N, device="cuda"), cuda.zeros(N, device="cuda")
    bmb.call("bmb_layernorm_forward", o, m, r, x, w, b, N, Cc)
    res = []
    for _ in range(2):
        dx, dw, db = cuda.zeros(N * Cc, device="cuda"), cuda.zeros(Cc, device="cuda"), cuda.zeros(Cc, device="cuda")
        bmb.call("bmb_layernorm_backward", dx, dw, db, dy, x, w, m, r, N, Cc)
        res.append((host(cuda, dw).copy(), host(cuda, db).copy()))
    assert np.array_equal(res[0][0], res[1][0]) and np.array_equal(res[0][1], res[1][1])


def test_elementwise_bias_encoder_vs_oracle(bmb, orc, cuda):
    N, Cc = 33, 3072
    x, dy, bias = normal((N, Cc), 1, 2.0), normal((N, Cc), 2), normal(Cc, 3)
    g, dg = np.empty(N * Cc, np.float32), np.empty(N * Cc, np.float32)
    orc.orc_gelu_forward(_np(g), _np(x), N * Cc)
    orc.orc_gelu_backward(_np(dg), _np(x), _np(dy), N * Cc)
    tx, tdy, tbias = dev(cuda, x), dev(cuda, dy), dev(cuda, bias)
    tg, tdg = cuda.zeros(N * Cc, device="cuda"), cuda.zeros(N * Cc, device="cuda")
    bmb.call("bmb_gelu_forward", tg, tx, N * Cc)
    bmb.call("bmb_gelu_backward", tdg, tx, tdy, N * Cc)
    assert normwise(host(cuda, tg), g) < 1e-6 and normwise(host(cuda, tdg), dg) < 1e-6
    # fused with the bias gradient of the projection that fed the GELU
    fdg, fcs = cuda.zeros(N * Cc, device="cuda"), dev(cuda, bias)
    bmb.call("bmb_gelu_backward_colsum", fdg, fcs, tx, tdy, N, Cc)
    assert np.array_equal(host(cuda, fdg), host(cuda, tdg))
    want = bias.astype(np.float64) + host(cuda, tdg).reshape(N, Cc).astype(np.float64).sum(0)
    assert normwise(host(cuda, fcs), want.astype(np.float32)) < 1e-5
    r = cuda.zeros(N * Cc, device="cuda")
    bmb.call("bmb_residual_forward", r, tx, tdy, N * Cc)
    assert np.array_equal(host(cuda, r), (x + dy).ravel())
    bmb.call("bmb_add_inplace", r, tx, N * Cc)
    assert np.array_equal(host(cuda, r), ((x + dy) + x).ravel())
    t2 = dev(cuda, x)
    bmb.call("bmb_bias_forward", t2, tbias, N, Cc)
    assert np.array_equal(host(cuda, t2).ravel(), (x + bias).ravel())
    for (n2, c2) in [(N, Cc), (1000, 768), (5, 50)]:
        d = normal((n2, c2), 5)
        db0 = normal(c2, 6)
        want = db0.copy()
        orc.orc_bias_backward(_np(want), _np(d), n2, c2)
        tdb = dev(cuda, db0)
        bmb.call("bmb_bias_backward", tdb, dev(cuda, d), n2, c2)
        assert normwise(host(cuda, tdb), want) < 1e-5
    B, T, V, C2 = 4, 16, 50, 64
    wte, wpe = normal((V, C2), 7), normal((T, C2), 8)
    tok = np.random.default_rng(9).integers(0, V, (B, T), dtype=np.int32)
    enc = np.empty((B, T, C2), np.float32)
    orc.orc_encoder_forward(_np(enc), _np(tok), _np(wte), _np(wpe), B, T, C2)
    te = cuda.zeros(B * T * C2, device="cuda")
    ttok = dev(cuda, tok)
    bmb.call("bmb_encoder_forward", te, ttok, dev(cuda, wte), dev(cuda, wpe), B, T, C2)
    assert np.array_equal(host(cuda, te), enc.ravel())
    d = normal((B, T, C2), 10)
    dwte, dwpe = normal((V, C2), 11), normal((T, C2), 12)
    w1, w2 = dwte.copy(), dwpe.copy()
    orc.orc_encoder_backward(_np(w1), _np(w2), _np(d), _np(tok), B, T, C2)
    t1, t2 = dev(cuda, dwte), dev(cuda, dwpe)
    bmb.call("bmb_encoder_backward", t1, t2, dev(cuda, d), ttok, B, T, C2)
    assert normwise(host(cuda, t1), w1) < 1e-5 and normwise(host(cuda, t2), w2) < 1e-5


@pytest.mark.parametrize("N,V,Vp", [(16, 65, 128), (8, 50257, 50304), (5, 7, 7), (4, 50304, 50304)])
def test_softmax_xent_vs_oracle(bmb, orc, cuda, N, V, Vp):
    logits = normal((N, Vp), 1, 3.0)
    tg = np.random.default_rng(2).integers(0, V, N, dtype=np.int32)
    p, l, d = np.empty(N * Vp, np.float32), np.empty(N, np.float32), np.empty(N * Vp, np.float32)
    orc.orc_softmax_crossentropy_forward(_np(p), _np(l), _np(logits), _np(tg), N, V, Vp)
    orc.orc_crossentropy_softmax_backward(_np(d), _np(p), _np(tg), N, V, Vp, 1.0 / N)
    tp, tl, td = (cuda.full((n,), float("nan"), device="cuda") for n in (N * Vp, N, N * Vp))
    tt = dev(cuda, tg)
    bmb.call("bmb_softmax_crossentropy_forward", tp, tl, dev(cuda, logits), tt, N, V, Vp)
    bmb.call("bmb_crossentropy_softmax_backward", td, tp, tt, N, V, Vp, 1.0 / N)
    assert normwise(host(cuda, tp), p) < 1e-5 and normwise(host(cuda, tl), l) < 1e-5
    assert normwise(host(cuda, td), d) < 1e-5
    assert np.all(host(cuda, tp).reshape(N, Vp)[:, V:] == 0)
    assert abs(host(cuda, tp).reshape(N, Vp).sum(1) - 1).max() < 1e-4      # rows are distributions
    # the one-sweep variant the training step uses gives the same losses and the same gradient
    fl, fd = (cuda.full((n,), float("nan"), device="cuda") for n in (N, N * Vp))
    bmb.call("bmb_softmax_crossentropy_fused", fd, fl, dev(cuda, logits), tt, N, V, Vp, 1.0 / N)
    assert normwise(host(cuda, fl), host(cuda, tl)) < 1e-6   # its row sum is accumulated in a different order
    assert normwise(host(cuda, fd), d) < 1e-5
    assert np.all(host(cuda, fd).reshape(N, Vp)[:, V:] == 0)


def test_adamw_norm_mean_vs_oracle(bmb, orc, cuda):
    n = 100003
    p0, g = normal(n + 1, 1)[:n], normal(n + 1, 2)[:n]
    m0, v0 = np.abs(normal(n + 1, 3, 0.1))[:n], np.abs(normal(n + 1, 4, 0.01))[:n]
    # device buffers stay 16-byte aligned; n itself is not a multiple of 4
    wp, wm, wv = p0.copy(), m0.copy(), v0.copy()
    orc.orc_adamw_update(_np(wp), _np(g.copy()), _np(wm), _np(wv), n, 3e-4, 0.9, 0.95, 1e-8, 0.1, 3, 0.5)
    tp, tg, tm, tv = dev(cuda, p0), dev(cuda, g), dev(cuda, m0), dev(cuda, v0)
    bmb.call("bmb_adamw_update", tp, tg, tm, tv, n, 3e-4, 0.9, 0.95, 1e-8, 0.1, 3, 0.5)
    assert normwise(host(cuda, tp), wp) < 1e-6 and normwise(host(cuda, tm), wm) < 1e-6
    assert normwise(host(cuda, tv), wv) < 1e-6
    out = C.c_float()
    bmb.check(bmb.lib().bmb_grad_global_norm(tg.data_ptr(), n, C.byref(out)))
    assert abs(out.value - np.linalg.norm(g.astype(np.float64))) / np.linalg.norm(g) < 1e-6
    bmb.check(bmb.lib().bmb_reduce_mean(tg.data_ptr(), 8192, C.byref(out)))
    assert abs(out.value - g[:8192].astype(np.float64).mean()) < 1e-6
    # clipped variant: scale derived on the device from the squared norm
    sq = cuda.zeros(1, dtype=cuda.float64, device="cuda")
    bmb.call("bmb_grad_sumsq_device", tg, n, sq)
    gn = np.linalg.norm(g.astype(np.float64)) / 2
    gs = (0.7 / gn if gn > 0.7 else 1.0) / 2
    wp, wm, wv = p0.copy(), m0.copy(), v0.copy()
    orc.orc_adamw_update(_np(wp), _np(g.copy()), _np(wm), _np(wv), n, 3e-4, 0.9, 0.95, 1e-8, 0.1, 5, gs)
    tp, tm, tv = dev(cuda, p0), dev(cuda, m0), dev(cuda, v0)
    sh = cuda.zeros(n + 1, device="cuda")
    bmb.call("bmb_adamw_update_clipped", tp, tg, tm, tv, n, 3e-4, 0.9, 0.95, 1e-8, 0.1, 5, sq, 0.7, 2.0, sh)
    assert normwise(host(cuda, tp), wp) < 1e-6
    rounded = np.empty(n, np.float32)
    orc.orc_round_tf32_n(_np(rounded), _np(host(cuda, tp).copy()), n)
    assert np.array_equal(host(cuda, sh)[:n], rounded)


def test_nn_vs_reference_kernels(bmb, ref, cuda):
    N, Cc = 256, 768
    x, w, b, dy = (dev(cuda, a) for a in (normal((N, Cc), 1), normal(Cc, 2), normal(Cc, 3), normal((N, Cc), 4)))
    mk = lambda n: cuda.zeros(n, device="cuda")
    o1, m1, r1, o2, m2, r2 = mk(N * Cc), mk(N), mk(N), mk(N * Cc), mk(N), mk(N)
    bmb.call("bmb_layernorm_forward", o1, m1, r1, x, w, b, N, Cc)
    ref.ref_layernorm_forward(o2.data_ptr(), m2.data_ptr(), r2.data_ptr(), x.data_ptr(), w.data_ptr(), b.data_ptr(), N, Cc)
    assert normwise(host(cuda, o1), host(cuda, o2)) < 1e-5
    dx1, dw1, db1, dx2, dw2, db2 = mk(N * Cc), mk(Cc), mk(Cc), mk(N * Cc), mk(Cc), mk(Cc)
    bmb.call("bmb_layernorm_backward", dx1, dw1, db1, dy, x, w, m1, r1, N, Cc)
    ref.ref_layernorm_backward(dx2.data_ptr(), dw2.data_ptr(), db2.data_ptr(), dy.data_ptr(), x.data_ptr(),
                               w.data_ptr(), m2.data_ptr(), r2.data_ptr(), N, Cc)
    assert normwise(host(cuda, dx1), host(cuda, dx2)) < 1e-5 and normwise(host(cuda, dw1), host(cuda, dw2)) < 1e-5
    assert normwise(host(cuda, db1), host(cuda, db2)) < 1e-5
    V, Vp = 50257, 50304
    lg = dev(cuda, normal((8, Vp), 5, 3.0))
    tg = dev(cuda, np.random.default_rng(6).integers(0, V, 8, dtype=np.int32))
    p1, l1, p2, l2 = mk(8 * Vp), mk(8), mk(8 * Vp), mk(8)
    bmb.call("bmb_softmax_crossentropy_forward", p1, l1, lg, tg, 8, V, Vp)
    ref.ref_softmax_crossentropy_forward(p2.data_ptr(), l2.data_ptr(), lg.data_ptr(), tg.data_ptr(), 8, V, Vp)
    assert normwise(host(cuda, p1), host(cuda, p2)) < 1e-6 and normwise(host(cuda, l1), host(cuda, l2)) < 1e-6


# -------------------------------------------------------------- all-reduce
def value_of(rank, idx):
    # per-rank pattern of tools/test_ddp.cu:31-34
    return ((idx * 2654435761 + rank * 40503) % 1000).astype(np.float32) * np.float32(0.001) + np.float32(rank)


@pytest.mark.parametrize("n", [1, 2, 3, 4, 8])
def test_ddp_allreduce_matrix(bmb, cuda, n):
    """n in {1,2,3,4,8} x count in {1,3,17,1000,65537,1048576}, ranks placed
    r % ngpu, against a float64 sum, rel < 1e-6 (tools/test_ddp.cu:36-111)."""
    ngpu = cuda.cuda.device_count()
    devs = (C.c_int * n)(*[r % ngpu for r in range(n)])
    h = C.c_void_p()
    bmb.check(bmb.lib().bmb_ddp_create(C.byref(h), n, devs))
    try:
        for count in [1, 3, 17, 1000, 65537, 1048576]:
            idx = np.arange(count, dtype=np.uint64)
            srcs = [value_of(r, idx) for r in range(n)]
            want = np.sum([s.astype(np.float64) for s in srcs], axis=0)
            bufs = [cuda.from_numpy(srcs[r]).to("cuda:%d" % devs[r]) for r in range(n)]
            ptrs = (C.c_void_p * n)(*[b.data_ptr() for b in bufs])
            bmb.check(bmb.lib().bmb_ddp_allreduce(h, ptrs, count))
            for r in range(n):
                got = bufs[r].cpu().numpy().astype(np.float64)
                assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-30)) < 1e-6, (n, count, r)
        t = bmb.DdpTiming()
        bmb.check(bmb.lib().bmb_ddp_timing_get(h, C.byref(t)))
        if n > 1:
            assert t.total_ms > 0 and t.bytes_per_device == 2 * (n - 1) * ((1048576 + n - 1) // n) * 4
    finally:
        bmb.lib().bmb_ddp_destroy(h)
    cuda.cuda.set_device(0)


# ------------------------------------------------------------- train step
TINY = dict(max_seq_len=32, vocab_size=65, padded_vocab=128, n_layer=2, n_head=2, n_embd=64, B=2, T=32)


def _oracle_run(orc, params0, toks, tgts, hp):
    g = orc.orc_gpt_create(TINY["max_seq_len"], TINY["vocab_size"], TINY["padded_vocab"], TINY["n_layer"],
                           TINY["n_head"], TINY["n_embd"], TINY["B"], TINY["T"])
    n = orc.orc_gpt_num_params(g)
    np.ctypeslib.as_array(orc.orc_gpt_params(g), shape=(n,))[:] = params0
    orc.orc_gpt_set_batch(g, _np(toks[0].copy()), _np(tgts[0].copy()))
    orc.orc_gpt_forward(g)
    orc.orc_gpt_backward(g)
    grads = np.ctypeslib.as_array(orc.orc_gpt_grads(g), shape=(n,)).copy()
    losses = []
    for s in range(toks.shape[0]):
        orc.orc_gpt_set_batch(g, _np(toks[s].copy()), _np(tgts[s].copy()))
        losses.append(orc.orc_gpt_step(g, hp["lr"], 0.9, 0.95, 1e-8, 0.1, 1.0, s + 1))
    orc.orc_gpt_destroy(g)
    return grads, np.array(losses)


@pytest.mark.parametrize("use_flash", [1, 0])
def test_train_step_loss_and_gradients_vs_oracle(bmb, orc, cuda, use_flash):
    tr = bmb.Trainer(seed=1337, use_flash=use_flash, math=bmb.MATH_FP32, **TINY)
    n = tr.num_params
    params0 = np.empty(n, np.float32)
    tr.get_params(params0)
    rng = np.random.default_rng(4242)
    toks = rng.integers(0, TINY["vocab_size"], (20, TINY["B"], TINY["T"]), dtype=np.int32)
    tgts = rng.integers(0, TINY["vocab_size"], (20, TINY["B"], TINY["T"]), dtype=np.int32)
    wgrads, wlosses = _oracle_run(orc, params0, toks, tgts, dict(lr=3e-4))
    tr.upload(toks[0], tgts[0])
    tr.forward_backward()
    grads = np.empty(n, np.float32)
    tr.get_grads(grads)
    assert normwise(grads, wgrads) < 1e-4
    losses = []
    for s in range(20):
        tr.upload(toks[s], tgts[s])
        tr.step(3e-4, s + 1)
        losses.append(tr.loss())
    assert np.max(np.abs(np.array(losses) - wlosses)) < 2e-3     # per-step bar over 20 steps
    tr.close()


def test_train_step_vs_reference_trainer(bmb, ref, cuda):
    """Same init (the reference's draw order reproduced), same batches, same
    hyper-parameters: loss per step within 2e-3 of the reference's own
    gpt_forward/gpt_backward/adamw_update, gradients within 1e-4 normwise."""
    c = dict(max_seq_len=64, vocab_size=65, padded_vocab=128, n_layer=2, n_head=4, n_embd=128, B=4, T=64)
    tr = bmb.Trainer(seed=1337, use_flash=1, math=bmb.MATH_FP32, **c)
    h = ref.ref_trainer_create(c["max_seq_len"], c["vocab_size"], c["padded_vocab"], c["n_layer"], c["n_head"],
                               c["n_embd"], c["B"], c["T"], 1, 1337, 1, 0.9, 0.95, 1e-8, 0.1, 1.0)
    n = tr.num_params
    assert n == ref.ref_trainer_num_params(h)
    p1, p2 = np.empty(n, np.float32), np.empty(n, np.float32)
    tr.get_params(p1)
    ref.ref_trainer_get_params(h, _np(p2))
    assert np.array_equal(p1, p2)            # identical initialisation, bit for bit
    rng = np.random.default_rng(4242)
    toks = rng.integers(0, 65, (20, c["B"], c["T"]), dtype=np.int32)
    tgts = rng.integers(0, 65, (20, c["B"], c["T"]), dtype=np.int32)
    tr.upload(toks[0], tgts[0])
    tr.forward_backward()
    g1, g2 = np.empty(n, np.float32), np.empty(n, np.float32)
    tr.get_grads(g1)
    ref.ref_trainer_forward_backward(h, _np(toks[0]), _np(tgts[0]))
    ref.ref_trainer_get_grads(h, _np(g2))
    assert normwise(g1, g2) < 1e-4
    for s in range(20):
        tr.upload(toks[s], tgts[s])
        tr.step(3e-4, s + 1)
        l1 = tr.loss()
        l2 = ref.ref_trainer_step(h, _np(toks[s]), _np(tgts[s]), 3e-4, s + 1)
        assert abs(l1 - l2) < 2e-3, (s, l1, l2)
    ref.ref_trainer_destroy(h)
    tr.close()
    cuda.cuda.set_device(0)


def test_golden_fixtures_on_gpu(bmb, orc, cuda):
    """The committed reference-generated fixtures, through the CUDA path."""
    import glob
    import os
    files = sorted(glob.glob(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "*.npz")))
    if not files:
        pytest.skip("no fixtures committed yet")
    for f in files:
        z = np.load(f)
        kind = str(z["kind"])
        if kind == "gemm":
            M, N, K = int(z["M"]), int(z["N"]), int(z["K"])
            dC = dev(cuda, z["C0"])
            bmb.call("bmb_gemm_ex", bmb.MATH_FP32, 0, int(z["ta"]), int(z["tb"]), M, N, K, float(z["alpha"]),
                     dev(cuda, z["A"]), dev(cuda, z["B"]), float(z["beta"]), dC, None)
            assert normwise(host(cuda, dC), z["out"]) < 1e-6, f
        elif kind == "attention":
            B, T, Cc, NH = int(z["B"]), int(z["T"]), int(z["C"]), int(z["NH"])
            out, lse = cuda.zeros(B * T * Cc, device="cuda"), cuda.zeros(B * NH * T, device="cuda")
            dq = dev(cuda, z["qkv"])
            bmb.call("bmb_flash_attention_forward", out, lse, dq, B, T, Cc, NH)
            assert normwise(host(cuda, out), z["out"]) < 1e-5 and normwise(host(cuda, lse), z["lse"]) < 1e-5, f
            dqkv, dsum = cuda.zeros(B * T * 3 * Cc, device="cuda"), cuda.zeros(B * NH * T, device="cuda")
            bmb.call("bmb_flash_attention_backward", dqkv, dsum, dev(cuda, z["dout"]), dq, out, lse, B, T, Cc, NH)
            g, w = host(cuda, dqkv).reshape(B * T, 3, Cc), z["dqkv"].reshape(B * T, 3, Cc)
            for i in range(3):
                assert normwise(g[:, i], w[:, i]) < 1e-5, f
        elif kind == "train":
            c = dict(max_seq_len=int(z["maxT"]), vocab_size=int(z["V"]), padded_vocab=int(z["Vp"]),
                     n_layer=int(z["L"]), n_head=int(z["NH"]), n_embd=int(z["C"]), B=int(z["B"]), T=int(z["T"]))
            tr = bmb.Trainer(seed=1337, use_flash=1, math=bmb.MATH_FP32, **c)
            p = np.empty(tr.num_params, np.float32)
            tr.get_params(p)
            assert np.array_equal(p, z["params0"]), f
            for s in range(z["tokens"].shape[0]):
                tr.upload(np.ascontiguousarray(z["tokens"][s]), np.ascontiguousarray(z["targets"][s]))
                tr.step(float(z["lr"]), s + 1)
                assert abs(tr.loss() - float(z["losses"][s])) < 2e-3, (f, s)
            tr.close()


def test_fused_data_parallel_step_matches_nccl(cuda):
    """Two ranks (one per GPU) train a small model with the NCCL all-reduce + full optimiser and with
    the fused exchange over peer memory: same losses, same parameters on every rank
    (tests/dp_fused_check.py).  Needs two GPUs."""
    import os
    import subprocess
    import sys
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29577", os.path.join(here, "dp_fused_check.py")],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]

