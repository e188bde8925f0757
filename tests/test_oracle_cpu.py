"""CPU pins for the oracle (oracle/bmb_oracle.c): closed forms, float64 numpy
restatements of the same formulas, finite differences, and the fixtures under
tests/golden/ that were produced by the reference's own CUDA kernels."""
import ctypes as C
import glob
import os

import numpy as np
import pytest

from helpers import _np, normal, normwise, uniform, xorshift

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def gemm_np(ta, tb, alpha, A, B, beta, C0):
    a = A.astype(np.float64).T if ta else A.astype(np.float64)
    b = B.astype(np.float64).T if tb else B.astype(np.float64)
    return alpha * (a @ b) + beta * C0.astype(np.float64)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (100, 70, 33), (65, 65, 65), (130, 260, 60), (1, 1, 1)])
def test_gemm_against_float64(orc, ta, tb, M, N, K):
    # shapes and alpha/beta of tools/test_gemm.cu:50-113; bar: fp32 normwise 1e-6
    A = uniform((K, M) if ta else (M, K), 1)
    B = uniform((N, K) if tb else (K, N), 2)
    C0 = uniform((M, N), 3)
    want = gemm_np(ta, tb, 0.75, A, B, 1.25, C0)
    for fn in (orc.orc_gemm, orc.orc_gemm_fast, orc.orc_gemm_f64):
        c = C0.copy()
        fn(ta, tb, M, N, K, 0.75, _np(A), _np(B), 1.25, _np(c))
        assert normwise(c, want) < 1e-6


def test_gemm_naive_and_fast_agree_bit_for_bit(orc):
    A, B = uniform((96, 200), 5), uniform((200, 72), 6)
    c1, c2 = np.zeros((96, 72), np.float32), np.zeros((96, 72), np.float32)
    orc.orc_gemm(0, 0, 96, 72, 200, 1.0, _np(A), _np(B), 0.0, _np(c1))
    orc.orc_gemm_fast(0, 0, 96, 72, 200, 1.0, _np(A), _np(B), 0.0, _np(c2))
    assert np.array_equal(c1, c2)


def test_gemm_empty_and_k0(orc):
    c = np.full((4, 4), 2.0, np.float32)
    a = np.zeros((4, 0), np.float32)
    orc.orc_gemm(0, 0, 4, 4, 0, 1.0, _np(a), _np(a), 0.5, _np(c))
    assert np.all(c == 1.0)


def test_xorshift_matches_reference_generator(orc):
    # first values of xorshift32 from seed 0x12345678 on the 0.001 grid (src/bench.cu:59-66)
    s, want = 0x12345678, []
    for _ in range(5):
        s ^= (s << 13) & 0xFFFFFFFF
        s ^= s >> 17
        s ^= (s << 5) & 0xFFFFFFFF
        want.append(np.float32((s % 2000) - 1000) / np.float32(1000.0))
    got = xorshift(5, 0x12345678, orc)
    assert np.array_equal(got, np.array(want, np.float32))
    assert np.all(np.abs(xorshift(1000, 0x9abcdef0, orc)) <= 1.0)


def test_tf32_rounding_known_answers(orc):
    cases = {1.0: 1.0, 1.0 + 2.0 ** -11: 1.0 + 2.0 ** -10,   # tie goes away from zero
             1.0 + 2.0 ** -12: 1.0, -(1.0 + 2.0 ** -11): -(1.0 + 2.0 ** -10),
             0.0: 0.0, 3.0e38: np.float32(3.0e38)}
    for x, want in cases.items():
        got = orc.orc_round_tf32(np.float32(x))
        if x == 3.0e38:
            assert abs(got - x) / x < 2.0 ** -10
        else:
            assert got == np.float32(want)
    x = uniform(10000, 9)
    out = np.empty_like(x)
    orc.orc_round_tf32_n(_np(out), _np(x), x.size)
    assert np.all((out.view(np.uint32) & 0x1FFF) == 0)
    assert np.max(np.abs(out - x) / np.maximum(np.abs(x), 1e-30)) <= 2.0 ** -11 * 1.0001
    assert orc.orc_round_bf16(np.float32(1.0 + 2.0 ** -8)) == np.float32(1.0)      # tie to even
    assert orc.orc_round_bf16(np.float32(1.0 + 3 * 2.0 ** -8)) == np.float32(1.0 + 2.0 ** -6)


def attention_np(qkv, B, T, C, NH):
    hs = C // NH
    x = qkv.astype(np.float64).reshape(B, T, 3, NH, hs)
    q, k, v = (x[:, :, i].transpose(0, 2, 1, 3) for i in range(3))
    s = q @ k.transpose(0, 1, 3, 2) / np.sqrt(hs)
    mask = np.tril(np.ones((T, T), bool))
    s = np.where(mask, s, -np.inf)
    m = s.max(-1, keepdims=True)
    e = np.exp(s - m)
    l = e.sum(-1, keepdims=True)
    p = e / l
    out = (p @ v).transpose(0, 2, 1, 3).reshape(B, T, C)
    return out, (m + np.log(l))[..., 0], p


@pytest.mark.parametrize("B,T,C,NH", [(2, 33, 64, 2), (1, 1, 32, 1), (3, 100, 96, 3), (2, 129, 256, 8)])
def test_attention_forward_against_float64(orc, B, T, C, NH):
    # ragged shapes of tools/test_flash.cu:336-340 (scaled down); bar 1e-5 (test_flash.cu:132)
    qkv = normal((B, T, 3 * C), 11)
    out = np.empty((B, T, C), np.float32)
    lse = np.empty((B, NH, T), np.float32)
    att = np.empty((B, NH, T, T), np.float32)
    orc.orc_attention_forward(_np(out), _np(lse), _np(att), _np(qkv), B, T, C, NH)
    wo, wl, wp = attention_np(qkv, B, T, C, NH)
    assert normwise(out, wo) < 1e-5
    assert normwise(lse, wl) < 1e-5
    assert normwise(att, wp) < 1e-5
    assert np.all(att[:, :, np.triu_indices(T, 1)[0], np.triu_indices(T, 1)[1]] == 0.0)


def test_attention_backward_against_finite_differences(orc):
    B, T, C, NH = 1, 9, 16, 2
    qkv = normal((B, T, 3 * C), 21).astype(np.float64)
    dout = normal((B, T, C), 22).astype(np.float64)
    f = lambda x: float((attention_np(x, B, T, C, NH)[0] * dout).sum())
    num = np.zeros_like(qkv)
    eps = 1e-5
    for idx in np.ndindex(*qkv.shape):
        xp, xm = qkv.copy(), qkv.copy()
        xp[idx] += eps
        xm[idx] -= eps
        num[idx] = (f(xp) - f(xm)) / (2 * eps)
    dq = np.empty((B, T, 3 * C), np.float32)
    q32, d32 = qkv.astype(np.float32), dout.astype(np.float32)
    orc.orc_attention_backward(_np(dq), _np(d32), _np(q32), B, T, C, NH)
    assert normwise(dq, num) < 1e-4


def test_layernorm_forward_backward(orc):
    N, C_ = 7, 48
    x, w, b = normal((N, C_), 31), normal(C_, 32), normal(C_, 33)
    out, mean, rstd = np.empty((N, C_), np.float32), np.empty(N, np.float32), np.empty(N, np.float32)
    orc.orc_layernorm_forward(_np(out), _np(mean), _np(rstd), _np(x), _np(w), _np(b), N, C_)
    x64 = x.astype(np.float64)
    mu, var = x64.mean(1, keepdims=True), x64.var(1, keepdims=True)
    want = (x64 - mu) / np.sqrt(var + 1e-5) * w + b
    assert normwise(out, want) < 1e-6
    assert normwise(mean, mu[:, 0]) < 1e-6 and normwise(rstd, 1 / np.sqrt(var[:, 0] + 1e-5)) < 1e-6
    # backward: accumulate semantics + the two mean corrections (src/nn.cu:95-111)
    dy = normal((N, C_), 34)
    dx = np.ones((N, C_), np.float32)
    dw, db = np.full(C_, 2.0, np.float32), np.full(C_, 3.0, np.float32)
    orc.orc_layernorm_backward(_np(dx), _np(dw), _np(db), _np(dy), _np(x), _np(w), _np(mean), _np(rstd), N, C_)
    xh = (x64 - mu) / np.sqrt(var + 1e-5)
    dxh = dy.astype(np.float64) * w
    wdx = 1.0 + (dxh - dxh.mean(1, keepdims=True) - xh * (dxh * xh).mean(1, keepdims=True)) / np.sqrt(var + 1e-5)
    assert normwise(dx, wdx) < 1e-5
    assert normwise(dw, 2.0 + (dy * xh).sum(0)) < 1e-5
    assert normwise(db, 3.0 + dy.astype(np.float64).sum(0)) < 1e-5


def test_gelu_bias_residual_encoder(orc):
    x = normal(1024, 41, 2.0)
    y, g = np.empty_like(x), np.empty_like(x)
    orc.orc_gelu_forward(_np(y), _np(x), x.size)
    x64 = x.astype(np.float64)
    t = np.tanh(0.7978845608028654 * (x64 + 0.044715 * x64 ** 3))
    assert normwise(y, 0.5 * x64 * (1 + t)) < 1e-6
    dy = normal(1024, 42)
    orc.orc_gelu_backward(_np(g), _np(x), _np(dy), x.size)
    eps = 1e-6
    f = lambda z: 0.5 * z * (1 + np.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
    assert normwise(g, dy * (f(x64 + eps) - f(x64 - eps)) / (2 * eps)) < 1e-5
    N, C_ = 5, 12
    o, bias = normal((N, C_), 43), normal(C_, 44)
    o2 = o.copy()
    orc.orc_bias_forward(_np(o2), _np(bias), N, C_)
    assert np.array_equal(o2, o + bias)
    db = np.ones(C_, np.float32)
    orc.orc_bias_backward(_np(db), _np(o), N, C_)
    assert normwise(db, 1 + o.astype(np.float64).sum(0)) < 1e-6
    B, T, V = 2, 3, 7
    wte, wpe = normal((V, C_), 45), normal((T, C_), 46)
    tok = np.array([[1, 6, 1], [0, 1, 2]], np.int32)
    enc = np.empty((B, T, C_), np.float32)
    orc.orc_encoder_forward(_np(enc), _np(tok), _np(wte), _np(wpe), B, T, C_)
    assert np.array_equal(enc, wte[tok] + wpe[None])
    dwte, dwpe = np.zeros_like(wte), np.zeros_like(wpe)
    d = normal((B, T, C_), 47)
    orc.orc_encoder_backward(_np(dwte), _np(dwpe), _np(d), _np(tok), B, T, C_)
    assert normwise(dwpe, d.sum(0)) < 1e-6
    assert normwise(dwte[1], d[0, 0] + d[0, 2] + d[1, 1]) < 1e-6 and np.all(dwte[3] == 0)


def test_softmax_xent_padding_and_gradient(orc):
    N, V, Vp = 4, 65, 128
    logits = normal((N, Vp), 51, 3.0)
    tg = np.array([0, 64, 7, 33], np.int32)
    p, loss = np.empty((N, Vp), np.float32), np.empty(N, np.float32)
    orc.orc_softmax_crossentropy_forward(_np(p), _np(loss), _np(logits), _np(tg), N, V, Vp)
    assert np.all(p[:, V:] == 0.0)                       # padding takes no mass (src/nn.cu:216)
    z = logits[:, :V].astype(np.float64)
    sm = np.exp(z - z.max(1, keepdims=True))
    sm /= sm.sum(1, keepdims=True)
    assert normwise(p[:, :V], sm) < 1e-6
    assert normwise(loss, -np.log(sm[np.arange(N), tg])) < 1e-6
    d = np.empty((N, Vp), np.float32)
    orc.orc_crossentropy_softmax_backward(_np(d), _np(p), _np(tg), N, V, Vp, 0.25)
    want = sm.copy()
    want[np.arange(N), tg] -= 1
    assert normwise(d[:, :V], want * 0.25) < 1e-6 and np.all(d[:, V:] == 0)


def test_adamw_closed_form_and_norm(orc):
    n = 10
    p, g = normal(n, 61), normal(n, 62)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    p0 = p.astype(np.float64)
    orc.orc_adamw_update(_np(p), _np(g), _np(m), _np(v), n, 3e-4, 0.9, 0.95, 1e-8, 0.1, 1, 0.5)
    gs = g.astype(np.float64) * 0.5
    # step 1: mhat = g, vhat = g^2 ; decay on every parameter (src/nn.cu:253)
    want = p0 - 3e-4 * (gs / (np.abs(gs) + 1e-8) + 0.1 * p0)
    assert normwise(p, want) < 1e-6
    assert normwise(m, 0.1 * gs) < 1e-6 and normwise(v, 0.05 * gs * gs) < 1e-5
    assert abs(orc.orc_grad_global_norm(_np(g), n) - np.linalg.norm(g.astype(np.float64))) < 1e-6


def _tiny_gpt(orc, seed=1337):
    cfg = dict(maxT=16, V=29, Vp=32, L=2, NH=2, C=32, B=2, T=16)
    g = orc.orc_gpt_create(cfg["maxT"], cfg["V"], cfg["Vp"], cfg["L"], cfg["NH"], cfg["C"], cfg["B"], cfg["T"])
    n = orc.orc_gpt_num_params(g)
    params = np.ctypeslib.as_array(orc.orc_gpt_params(g), shape=(n,))
    rng = np.random.default_rng(seed)
    params[:] = (rng.standard_normal(n) * 0.05).astype(np.float32)
    tok = rng.integers(0, cfg["V"], (cfg["B"], cfg["T"]), dtype=np.int32)
    tgt = rng.integers(0, cfg["V"], (cfg["B"], cfg["T"]), dtype=np.int32)
    orc.orc_gpt_set_batch(g, _np(tok), _np(tgt))
    return g, n, params, cfg


def test_gpt_gradient_check_like_test_grad(orc):
    # directional finite differences along g/|g| (tools/test_grad.cu:15-27), bar 2e-2
    g, n, params, cfg = _tiny_gpt(orc)
    loss0 = orc.orc_gpt_forward(g)
    assert abs(loss0 - np.log(cfg["V"])) < 0.5
    orc.orc_gpt_backward(g)
    grads = np.ctypeslib.as_array(orc.orc_gpt_grads(g), shape=(n,)).copy()
    base = params.copy()
    gn = np.linalg.norm(grads.astype(np.float64))
    eps = 1e-2
    params[:] = base + eps * (grads / gn).astype(np.float32)
    lp = orc.orc_gpt_forward(g)
    params[:] = base - eps * (grads / gn).astype(np.float32)
    lm = orc.orc_gpt_forward(g)
    assert abs((lp - lm) / (2 * eps) - gn) / gn < 2e-2
    orc.orc_gpt_destroy(g)


def test_gpt_loss_decreases_over_20_steps(orc):
    g, n, params, cfg = _tiny_gpt(orc)
    losses = [orc.orc_gpt_step(g, 3e-3, 0.9, 0.95, 1e-8, 0.1, 1.0, s) for s in range(1, 21)]
    assert all(np.isfinite(losses))
    assert all(b < a for a, b in zip(losses, losses[1:])) and losses[-1] < losses[0] - 0.1
    orc.orc_gpt_destroy(g)


def test_golden_fixtures_from_reference_kernels(orc):
    """Every fixture under tests/golden/ holds inputs plus the outputs the
    reference's own CUDA kernels produced for them; the oracle must reproduce
    those outputs within the reference's tolerances."""
    files = sorted(glob.glob(os.path.join(GOLDEN, "*.npz")))
    if not files:
        pytest.skip("no reference-generated fixtures committed yet")
    import golden_check
    for f in files:
        golden_check.check_fixture_with_oracle(orc, np.load(f), os.path.basename(f))
