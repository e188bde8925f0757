"""GPU parity of the tcgen05 tensor-core GEMM (TF32 and BF16 kinds), through the
C ABI, against the CPU oracle.

Two bars per case:
  * against the fp32 product of the unrounded inputs: normwise 5e-4 for TF32
    (the registry tolerance), 8e-3 for BF16;
  * against the float64 product of the *rounded* inputs: 2e-5.  Only the
    accumulation order differs there, so a wrong descriptor, swizzle or tile
    coordinate cannot hide inside the TF32 tolerance.
"""
import numpy as np
import pytest

from helpers import _np, normal, normwise, uniform

pytestmark = pytest.mark.gpu


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(torch, t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


def rounded(orc, x, kind):
    out = np.empty_like(x)
    if kind == "tf32":
        orc.orc_round_tf32_n(_np(out), _np(x), x.size)
    else:
        u = x.view(np.uint32).astype(np.uint64)
        u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
        out = u.astype(np.uint32).view(np.float32)
    return out


SHAPES = [(128, 256, 32), (128, 256, 128), (256, 512, 96), (384, 768, 200), (1024, 1024, 1024), (300, 515, 77),
          (129, 257, 33), (2304, 768, 512), (768, 2304, 64)]


@pytest.mark.parametrize("kind", ["tf32", "bf16"])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_tensorcore_gemm_vs_oracle(bmb, orc, cuda, kind, ta, tb, M, N, K):
    math = bmb.MATH_TF32 if kind == "tf32" else bmb.MATH_BF16
    A, B, C0 = uniform(M * K, 1), uniform(K * N, 2), uniform(M * N, 3)
    want32 = C0.copy()
    orc.orc_gemm_fast(ta, tb, M, N, K, 0.75, _np(A), _np(B), 1.25, _np(want32))
    want_r = C0.copy()
    Ar, Br = rounded(orc, A, kind), rounded(orc, B, kind)
    orc.orc_gemm_f64(ta, tb, M, N, K, 0.75, _np(Ar), _np(Br), 1.25, _np(want_r))
    dA, dB, dC = dev(cuda, A), dev(cuda, B), dev(cuda, C0)
    bmb.call("bmb_gemm_ex", math, 0, ta, tb, M, N, K, 0.75, dA, dB, 1.25, dC, None)
    got = host(cuda, dC)
    assert normwise(got, want_r) < 2e-5, "layout/descriptor error, not rounding"
    assert normwise(got, want32) < (5e-4 if kind == "tf32" else 8e-3)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 32), (512, 768, 256), (300, 515, 77), (1024, 320, 1024), (2304, 768, 512), (288, 288, 40)])
@pytest.mark.parametrize("split", [0, 1])
def test_pair_kernel_vs_oracle(bmb, orc, cuda, ta, tb, M, N, K, split):
    """The CTA-pair form (one tcgen05.mma.cta_group::2 per 256 rows, each CTA loading half of B) forced by flag:
    all four transposes, ragged edges (a peer CTA whose rows or columns lie outside the matrix), tiles shared
    along K or not, alpha and beta, against the float64 product of the rounded operands (2e-5).  Shapes whose
    M- or N-contiguous operand is not a multiple of 32 wide fall back to single CTAs, which must agree too."""
    A, B, C0 = uniform(M * K, 1), uniform(K * N, 2), uniform(M * N, 3)
    Ar, Br = rounded(orc, A, "tf32"), rounded(orc, B, "tf32")
    want_r = C0.copy()
    orc.orc_gemm_f64(ta, tb, M, N, K, 0.75, _np(Ar), _np(Br), 1.25, _np(want_r))
    dA, dB, dC = dev(cuda, A), dev(cuda, B), dev(cuda, C0)
    flags = bmb.GEMM_PAIR | (0 if split else bmb.GEMM_NO_SPLIT)
    bmb.call("bmb_gemm_ex", bmb.MATH_TF32, flags, ta, tb, M, N, K, 0.75, dA, dB, 1.25, dC, None)
    assert normwise(host(cuda, dC), want_r) < 2e-5
    # beta = 0 on a poisoned C: every element must be written exactly once
    dP = cuda.full((M * N,), float("nan"), device="cuda")
    want0 = np.zeros(M * N, np.float32)
    orc.orc_gemm_f64(ta, tb, M, N, K, 1.0, _np(Ar), _np(Br), 0.0, _np(want0))
    bmb.call("bmb_gemm_ex", bmb.MATH_TF32, flags, ta, tb, M, N, K, 1.0, dA, dB, 0.0, dP, None)
    assert normwise(host(cuda, dP), want0) < 2e-5


@pytest.mark.parametrize("ta,tb,M,N,K,beta", [
    (0, 1, 8192, 3072, 768, 0.0),      # 192-column tiles, whole tiles stored from registers
    (0, 1, 8192, 768, 3072, 0.0),      # last wave shared between CTAs along K
    (0, 0, 8192, 768, 3072, 0.0),      # B MN-major through the 3-d tensor map
    (1, 0, 3072, 768, 8192, 1.0),      # both MN-major, fewer tiles than SMs, accumulate into C
    (1, 0, 768, 768, 8192, 1.0),
    (0, 1, 4096, 160, 512, 0.0),       # 128-column tiles (N < 192)
])
def test_training_step_shapes_at_full_size(bmb, cuda, ta, tb, M, N, K, beta):
    """The GEMM shapes of the 124M training step, operands pre-rounded as the step feeds them,
    against a float64 product on the device (the CPU oracle needs minutes at these sizes):
    2e-5 normwise, which only the accumulation order may use up.  Sharing tiles between CTAs
    must agree with keeping every tile on one CTA to the same bound."""
    g = cuda.Generator(device="cuda").manual_seed(5)
    A = cuda.rand(M * K, device="cuda", generator=g) * 2 - 1
    B = cuda.rand(K * N, device="cuda", generator=g) * 2 - 1
    C0 = cuda.rand(M * N, device="cuda", generator=g)
    bmb.call("bmb_round_tf32", A, A, M * K, None)
    bmb.call("bmb_round_tf32", B, B, K * N, None)
    Am = A.view(K, M).t() if ta else A.view(M, K)
    Bm = B.view(N, K).t() if tb else B.view(K, N)
    want = (Am.double() @ Bm.double() + beta * C0.view(M, N).double())
    outs = []
    # every tile on one CTA / tiles shared along K, on single CTAs and on CTA pairs
    for extra in (bmb.GEMM_NO_PAIR, bmb.GEMM_NO_PAIR | bmb.GEMM_NO_SPLIT, bmb.GEMM_PAIR, bmb.GEMM_PAIR | bmb.GEMM_NO_SPLIT):
        Cm = C0.clone()
        bmb.call("bmb_gemm_ex", bmb.MATH_TF32, bmb.GEMM_A_ROUNDED | bmb.GEMM_B_ROUNDED | extra, ta, tb, M, N, K, 1.0, A, B, beta, Cm, None)
        cuda.cuda.synchronize()
        err = ((Cm.view(M, N).double() - want).norm() / want.norm()).item()
        assert err < 2e-5, (extra, err)
        outs.append(Cm)
    for o in outs[1:]:
        assert ((outs[0] - o).double().norm() / want.norm()).item() < 2e-5


@pytest.mark.parametrize("ta,tb,batch,M,N,K", [
    (0, 1, 12, 256, 256, 64),      # Q K^T of unfused attention: both operands K-major
    (0, 0, 12, 256, 64, 256),      # P V: 64-column tiles, B MN-major
    (1, 0, 6, 256, 64, 128),       # att^T dvaccum: A MN-major
    (0, 1, 5, 200, 136, 96),       # ragged M and N: tiles run past a problem's end
    (0, 0, 3, 128, 64, 40),        # MN-major with K % 32 != 0: stays on the SIMT kernel
])
def test_batched_tensorcore_gemm_vs_oracle(bmb, orc, cuda, ta, tb, batch, M, N, K):
    """batched_gemm (src/gemm.h:26-29) in TF32 mode against the float64 product of the rounded
    operands (2e-5: accumulation order only) and the fp32 product of the raw ones (5e-4)."""
    A, B, C0 = uniform(batch * M * K, 1), uniform(batch * K * N, 2), uniform(batch * M * N, 3)
    Ar, Br = rounded(orc, A, "tf32"), rounded(orc, B, "tf32")
    want_r, want32 = C0.copy(), C0.copy()
    orc.orc_batched_gemm(ta, tb, batch, M, N, K, 0.5, _np(A), M * K, _np(B), K * N, 2.0, _np(want32), M * N)
    for i in range(batch):
        c = want_r[i * M * N:(i + 1) * M * N]
        orc.orc_gemm_f64(ta, tb, M, N, K, 0.5, _np(np.ascontiguousarray(Ar[i * M * K:(i + 1) * M * K])),
                         _np(np.ascontiguousarray(Br[i * K * N:(i + 1) * K * N])), 2.0, _np(c))
    dA, dB, dC = dev(cuda, A), dev(cuda, B), dev(cuda, C0)
    prev = bmb.lib().bmb_get_math_mode()
    bmb.lib().bmb_set_math_mode(bmb.MATH_TF32)
    try:
        bmb.call("bmb_batched_gemm", ta, tb, batch, M, N, K, 0.5, dA, M * K, dB, K * N, 2.0, dC, M * N, None)
        got = host(cuda, dC)
        # beta = 0 leg: C poisoned first
        dP = cuda.full((batch * M * N,), float("nan"), device="cuda")
        bmb.call("bmb_batched_gemm", ta, tb, batch, M, N, K, 1.0, dA, M * K, dB, K * N, 0.0, dP, M * N, None)
        assert np.all(np.isfinite(host(cuda, dP)))
    finally:
        bmb.lib().bmb_set_math_mode(prev)
    on_tensor_cores = ta == 0 and tb == 1 or K % 32 == 0     # else the fp32 kernel serves it, exact in fp32
    if on_tensor_cores:
        assert normwise(got, want_r) < 2e-5
    assert normwise(got, want32) < (5e-4 if on_tensor_cores else 1e-6)


def test_registry_tf32_entry_at_2048(bmb, orc, cuda):
    """Registry entry 2 at the harness's verification setting alpha 0.5, beta 3
    (src/bench.cu:261), inputs uniform [-1,1): normwise below the entry's tol."""
    n = 2048
    A, B, C0 = uniform(n * n, 0), uniform(n * n, 1), uniform(n * n, 2)
    want = C0.copy()
    orc.orc_gemm_fast(0, 0, n, n, n, 0.5, _np(A), _np(B), 3.0, _np(want))
    dA, dB, dC = dev(cuda, A), dev(cuda, B), dev(cuda, C0)
    bmb.call("bmb_sgemm_tf32", n, n, n, 0.5, dA, dB, 3.0, dC)
    e = bmb.lib().bmb_find_kernel(2).contents
    err = normwise(host(cuda, dC), want)
    assert err < e.tol, err
    dC = dev(cuda, C0)
    bmb.call("bmb_sgemm_bf16", n, n, n, 0.5, dA, dB, 3.0, dC)
    assert normwise(host(cuda, dC), want) < bmb.lib().bmb_find_kernel(3).contents.tol


def test_prerounded_operands_are_read_in_place(bmb, orc, cuda):
    """With both operands K-contiguous and flagged as already rounded the kernel
    reads them where they lie; the result equals the prepass route bit for bit."""
    M, N, K = 512, 768, 256
    A, B = rounded(orc, uniform(M * K, 4), "tf32"), rounded(orc, uniform(N * K, 5), "tf32")
    dA, dB = dev(cuda, A), dev(cuda, B)
    c1, c2 = cuda.zeros(M * N, device="cuda"), cuda.zeros(M * N, device="cuda")
    bmb.call("bmb_gemm_ex", bmb.MATH_TF32, 0, 0, 1, M, N, K, 1.0, dA, dB, 0.0, c1, None)
    bmb.call("bmb_gemm_ex", bmb.MATH_TF32, bmb.GEMM_A_ROUNDED | bmb.GEMM_B_ROUNDED, 0, 1, M, N, K, 1.0, dA, dB, 0.0, c2, None)
    assert np.array_equal(host(cuda, c1), host(cuda, c2))


def test_unrounded_operands_show_why_rounding_is_needed(bmb, orc, cuda, capsys):
    """Raw fp32 handed to kind::tf32 (flagged as rounded although it is not):
    records how far truncation lands from the fp32 product.  Informational: the
    only assertion is that rounding first is at least as accurate."""
    M = N = K = 1024
    A, B = uniform(M * K, 6), uniform(N * K, 7)
    want = np.zeros(M * N, np.float32)
    orc.orc_gemm_fast(0, 1, M, N, K, 1.0, _np(A), _np(B), 0.0, _np(want))
    dA, dB = dev(cuda, A), dev(cuda, B)
    c1, c2 = cuda.zeros(M * N, device="cuda"), cuda.zeros(M * N, device="cuda")
    bmb.call("bmb_gemm_ex", bmb.MATH_TF32, 0, 0, 1, M, N, K, 1.0, dA, dB, 0.0, c1, None)
    bmb.call("bmb_gemm_ex", bmb.MATH_TF32, bmb.GEMM_A_ROUNDED | bmb.GEMM_B_ROUNDED, 0, 1, M, N, K, 1.0, dA, dB, 0.0, c2, None)
    e_round, e_raw = normwise(host(cuda, c1), want), normwise(host(cuda, c2), want)
    with capsys.disabled():
        print("\n[tf32] normwise vs fp32 product: rounded operands %.3e, raw operands %.3e" % (e_round, e_raw))
    assert e_round < 5e-4 and e_round <= e_raw * 1.05


ATT_SHAPES = [(2, 64, 128, 2), (1, 256, 128, 2), (2, 300, 192, 3), (3, 100, 384, 6), (2, 33, 384, 6), (1, 1, 384, 6),
              (2, 129, 128, 2), (1, 1024, 128, 2), (2, 513, 64, 1),
              (1, 4224, 64, 1)]       # longer than the 4096 queries whose lse / D the dK/dV kernel parks in shared memory


@pytest.mark.parametrize("B,T,C,NH", ATT_SHAPES)
def test_tensorcore_flash_forward_vs_oracle(bmb, orc, cuda, B, T, C, NH):
    """Forward config 2 (tcgen05, TF32 products, fp32 softmax) against the fp32
    oracle.  TF32 rounding of q, k, p and v bounds the error: out within 2e-3
    normwise (measured about 4e-4), lse within 1e-3 of max|lse|."""
    from helpers import normal
    qkv = normal(B * T * 3 * C, 1234)
    wout, wlse = np.empty(B * T * C, np.float32), np.empty(B * NH * T, np.float32)
    orc.orc_attention_forward(_np(wout), _np(wlse), None, _np(qkv), B, T, C, NH)
    dq = dev(cuda, qkv)
    out = cuda.full((B * T * C,), float("nan"), device="cuda")
    lse = cuda.full((B * NH * T,), float("nan"), device="cuda")
    bmb.call("bmb_flash_attention_forward_cfg", 2, out, lse, dq, B, T, C, NH)
    e_out, e_lse = normwise(host(cuda, out), wout), normwise(host(cuda, lse), wlse)
    assert e_out < 2e-3 and e_lse < 1e-3, (e_out, e_lse)


@pytest.mark.parametrize("B,T,C,NH,ctas", [(1, 640, 64, 1, 1), (1, 1024, 64, 1, 1), (1, 640, 192, 3, 2), (1, 896, 64, 1, 1),
                                           (2, 1000, 192, 3, 4), (3, 300, 128, 2, 3)])
def test_tensorcore_flash_forward_walks_several_items_per_cta(bmb, orc, cuda, monkeypatch, B, T, C, NH, ctas):
    """The forward kernel is persistent: a CTA walks several (head, 256-query) work items, and its warps carry ring
    positions and barrier phases from one item to the next.  At test sizes every CTA gets one item, so the grid is
    capped (BMB_FLASH_FWD_CTAS) to make a few CTAs walk all of them -- including items whose second query tile is
    empty (T = 640, 896, 300), long items followed by short ones, and odd step counts.  Same bars as the one-item
    test; a wrong phase shows as a bounded wait that runs out (BMB_E_TIMEOUT) or as non-finite output."""
    from helpers import normal
    monkeypatch.setenv("BMB_FLASH_FWD_CTAS", str(ctas))
    qkv = normal(B * T * 3 * C, 4321)
    wout, wlse = np.empty(B * T * C, np.float32), np.empty(B * NH * T, np.float32)
    orc.orc_attention_forward(_np(wout), _np(wlse), None, _np(qkv), B, T, C, NH)
    dq = dev(cuda, qkv)
    out = cuda.full((B * T * C,), float("nan"), device="cuda")
    lse = cuda.full((B * NH * T,), float("nan"), device="cuda")
    bmb.call("bmb_flash_attention_forward_cfg", 2, out, lse, dq, B, T, C, NH)
    got_out, got_lse = host(cuda, out), host(cuda, lse)
    assert np.all(np.isfinite(got_out)) and np.all(np.isfinite(got_lse))
    e_out, e_lse = normwise(got_out, wout), normwise(got_lse, wlse)
    assert e_out < 2e-3 and e_lse < 1e-3, (e_out, e_lse)


@pytest.mark.parametrize("B,T,C,NH", ATT_SHAPES)
def test_tensorcore_flash_backward_vs_oracle(bmb, orc, cuda, B, T, C, NH):
    """Backward config 2 (tcgen05 dQ and dK/dV kernels) against the fp32 oracle:
    dq, dk and dv separately, normwise below 5e-3 (TF32 products; measured about 1e-3).
    dqkv starts as NaN: the kernels must overwrite every element."""
    from helpers import normal
    qkv, dout = normal(B * T * 3 * C, 1234), normal(B * T * C, 99)
    wd = np.empty(B * T * 3 * C, np.float32)
    orc.orc_attention_backward(_np(wd), _np(dout), _np(qkv), B, T, C, NH)
    dq, dd = dev(cuda, qkv), dev(cuda, dout)
    out, lse = cuda.zeros(B * T * C, device="cuda"), cuda.zeros(B * NH * T, device="cuda")
    bmb.call("bmb_flash_attention_forward_cfg", 0, out, lse, dq, B, T, C, NH)
    dqkv = cuda.full((B * T * 3 * C,), float("nan"), device="cuda")
    dsum = cuda.full((B * NH * T,), float("nan"), device="cuda")
    bmb.call("bmb_flash_attention_backward_cfg", 2, dqkv, dsum, dd, dq, out, lse, B, T, C, NH)
    g, w = host(cuda, dqkv).reshape(B * T, 3, C), wd.reshape(B * T, 3, C)
    # Normwise per part; the denominator is floored at 25 % of the whole gradient's magnitude because a part
    # can be exactly zero (T = 1: dS = P (dP - D) vanishes, and TF32 leaves a rounding residue there).
    floor = 0.25 * float(np.max(np.abs(w)))
    errs = [float(np.max(np.abs(g[:, i].astype(np.float64) - w[:, i])) / max(float(np.max(np.abs(w[:, i]))), floor))
            for i in range(3)]
    assert np.all(np.isfinite(g)) and max(errs) < 5e-3, errs


def test_tensorcore_flash_reads_prerounded_operands_in_place(bmb, orc, cuda):
    """With BMB_FLASH_OPERANDS_ROUNDED the tensor-core kernels skip their rounding copies; on operands
    that are already TF32-representable the results must equal the copying route bit for bit."""
    B, T, C, NH = 2, 256, 256, 4
    lib = bmb.lib()
    qkv = rounded(orc, normal(B * T * 3 * C, 5), "tf32")
    dout = rounded(orc, normal(B * T * C, 6), "tf32")
    dq, dd = dev(cuda, qkv), dev(cuda, dout)
    fwd, bwd = lib.bmb_flash_num_configs() - 1, lib.bmb_flash_num_bwd_configs() - 1
    o1, l1, o2, l2 = (cuda.zeros(n, device="cuda") for n in (B * T * C, B * NH * T, B * T * C, B * NH * T))
    bmb.call("bmb_flash_attention_forward_cfg", fwd, o1, l1, dq, B, T, C, NH)
    bmb.call("bmb_flash_attention_forward_ex", fwd, bmb.FLASH_OPERANDS_ROUNDED, o2, l2, dq, B, T, C, NH)
    assert np.array_equal(host(cuda, o1), host(cuda, o2)) and np.array_equal(host(cuda, l1), host(cuda, l2))
    g1, g2 = cuda.zeros(B * T * 3 * C, device="cuda"), cuda.zeros(B * T * 3 * C, device="cuda")
    s1, s2 = cuda.zeros(B * NH * T, device="cuda"), cuda.zeros(B * NH * T, device="cuda")
    bmb.call("bmb_flash_attention_backward_cfg", bwd, g1, s1, dd, dq, o1, l1, B, T, C, NH)
    bmb.call("bmb_flash_attention_backward_ex", bwd, bmb.FLASH_OPERANDS_ROUNDED, g2, s2, dd, dq, o1, l1, B, T, C, NH)
    assert np.array_equal(host(cuda, g1), host(cuda, g2))


def test_tensorcore_flash_rejects_other_head_sizes(bmb, cuda):
    x = cuda.zeros(4096, device="cuda")
    st = bmb.lib().bmb_flash_attention_forward_cfg(2, x.data_ptr(), x.data_ptr(), x.data_ptr(), 1, 4, 128, 4)
    assert st == bmb.E_UNSUPPORTED


TINY = dict(max_seq_len=64, vocab_size=300, padded_vocab=384, n_layer=2, n_head=4, n_embd=256, B=4, T=64)


@pytest.mark.parametrize("fused", [0, 1])
def test_train_step_tf32_loss_vs_oracle(bmb, orc, cuda, fused):
    """TF32 GEMMs and attention inside the train step: loss per step within 2e-2
    of the fp32 CPU oracle over 20 steps (shapes large enough to take the
    tensor-core path).  fused = 1 additionally keeps every GEMM / attention
    operand TF32-rounded at its producer and adds the biases in the GEMM epilogue."""
    tr = bmb.Trainer(seed=1337, use_flash=1, math=bmb.MATH_TF32, fused=fused, **TINY)
    n = tr.num_params
    params0 = np.empty(n, np.float32)
    tr.get_params(params0)
    rng = np.random.default_rng(4242)
    toks = rng.integers(0, TINY["vocab_size"], (20, TINY["B"], TINY["T"]), dtype=np.int32)
    tgts = rng.integers(0, TINY["vocab_size"], (20, TINY["B"], TINY["T"]), dtype=np.int32)
    g = orc.orc_gpt_create(TINY["max_seq_len"], TINY["vocab_size"], TINY["padded_vocab"], TINY["n_layer"],
                           TINY["n_head"], TINY["n_embd"], TINY["B"], TINY["T"])
    np.ctypeslib.as_array(orc.orc_gpt_params(g), shape=(n,))[:] = params0
    for s in range(20):
        orc.orc_gpt_set_batch(g, _np(toks[s].copy()), _np(tgts[s].copy()))
        want = orc.orc_gpt_step(g, 3e-4, 0.9, 0.95, 1e-8, 0.1, 1.0, s + 1)
        tr.upload(toks[s], tgts[s])
        tr.step(3e-4, s + 1)
        assert abs(tr.loss() - want) < 2e-2, s
    orc.orc_gpt_destroy(g)
    tr.close()


def test_graph_replay_equals_eager_launches(bmb, cuda, monkeypatch):
    """From its second step on the trainer replays forward + backward from a CUDA graph; with
    BMB_TRAINER_GRAPH=0 it launches kernel by kernel.  Same seeds, same batches: both ways
    must give the same losses up to the run-to-run wobble of the sums that use atomics (the token
    embedding gradient; tiles shared between CTAs in the tensor-core GEMM): 1e-5 fp32, 1e-3 TF32."""
    rng = np.random.default_rng(7)
    toks = rng.integers(0, TINY["vocab_size"], (6, TINY["B"], TINY["T"]), dtype=np.int32)
    tgts = rng.integers(0, TINY["vocab_size"], (6, TINY["B"], TINY["T"]), dtype=np.int32)
    for math, tol in ((bmb.MATH_FP32, 1e-5), (bmb.MATH_TF32, 1e-3)):
        runs = []
        for graph in ("1", "0"):
            monkeypatch.setenv("BMB_TRAINER_GRAPH", graph)
            tr = bmb.Trainer(seed=1337, use_flash=1, math=math, fused=1 if math == bmb.MATH_TF32 else 0, **TINY)
            losses = []
            for s in range(6):
                tr.upload(toks[s], tgts[s])
                tr.step(3e-4, s + 1)
                losses.append(tr.loss())
            tr.close()
            runs.append(losses)
        assert max(abs(a - b) for a, b in zip(*runs)) <= tol, runs



def test_side_by_side_backward_products_equal_one_after_the_other(bmb, cuda, monkeypatch):
    """In the fused TF32 mode the trainer runs the two products of a linear layer's backward (dX and dW) side by
    side, each on half of the SMs, the weight gradient on a second stream forked and joined by events (also
    inside the captured graph).  BMB_TRAINER_SIDE_BY_SIDE=0 runs them one after the other on all SMs: same
    losses up to the run-to-run wobble of the sums that use atomics (1e-3, as for graph replay)."""
    rng = np.random.default_rng(11)
    toks = rng.integers(0, TINY["vocab_size"], (6, TINY["B"], TINY["T"]), dtype=np.int32)
    tgts = rng.integers(0, TINY["vocab_size"], (6, TINY["B"], TINY["T"]), dtype=np.int32)
    runs = []
    for mode in ("1", "0"):
        monkeypatch.setenv("BMB_TRAINER_SIDE_BY_SIDE", mode)
        tr = bmb.Trainer(seed=1337, use_flash=1, math=bmb.MATH_TF32, fused=1, **TINY)
        losses = []
        for s in range(6):
            tr.upload(toks[s], tgts[s])
            tr.step(3e-4, s + 1)
            losses.append(tr.loss())
        tr.close()
        runs.append(losses)
    assert np.all(np.isfinite(runs[0])) and max(abs(a - b) for a, b in zip(*runs)) <= 1e-3, runs


@pytest.mark.parametrize("M,N,K,pad,with_bias", [(512, 768, 256, 0, True), (8192, 3072, 768, 0, True), (300, 516, 77, 0, True),
                                                  (256, 132, 64, 1, False)])
def test_gemm_bias_gelu_equals_the_three_calls(bmb, orc, cuda, M, N, K, pad, with_bias):
    """bmb_gemm_bias_gelu (the activation in the product's epilogue on aligned outputs, a pass of its own otherwise)
    against gemm + bias_forward + gelu_forward on the same operands: C agrees to the last bits that a different
    tile plan may move (no tile is split along K in the fused form), C_gelu is bit-identical to gelu_forward
    applied to the C the fused call returned, and both agree with the oracle's GELU."""
    A, W, bias = rounded(orc, uniform(M * K, 21), "tf32"), rounded(orc, uniform(N * K, 22), "tf32"), uniform(N, 23)
    dA, dW, db = dev(cuda, A), dev(cuda, W), (dev(cuda, bias) if with_bias else None)
    flags = bmb.GEMM_A_ROUNDED | bmb.GEMM_B_ROUNDED
    # pad = 1: outputs that start 4 bytes off a 16-byte boundary (the activation then runs as its own element-wise pass)
    c_f = cuda.full((M * N + 4,), float("nan"), device="cuda")[pad:pad + M * N]
    g_f = cuda.full((M * N + 4,), float("nan"), device="cuda")[pad:pad + M * N]
    bmb.call("bmb_gemm_bias_gelu", bmb.MATH_TF32, flags | bmb.GEMM_AUX_ROUNDED, M, N, K, dA, dW, db, c_f, g_f, None)
    c_s, g_s = cuda.zeros(M * N, device="cuda"), cuda.zeros(M * N, device="cuda")
    bmb.call("bmb_gemm_ex", bmb.MATH_TF32, flags | bmb.GEMM_NO_SPLIT, 0, 1, M, N, K, 1.0, dA, dW, 0.0, c_s, None)
    if with_bias:
        bmb.call("bmb_bias_forward", c_s, db, M, N)
    cf, cs = host(cuda, c_f), host(cuda, c_s)
    assert np.all(np.isfinite(cf)) and normwise(cf, cs) <= 2e-6
    # the activation of exactly what the fused call stored, by the stand-alone kernel, then rounded
    bmb.call("bmb_gelu_forward", g_s, c_f.clone(), M * N)
    bmb.call("bmb_round_tf32", g_s, g_s, M * N, None)
    gf = host(cuda, g_f)
    assert np.array_equal(gf, host(cuda, g_s))
    want = np.empty_like(cf)
    orc.orc_gelu_forward(_np(want), _np(cf), cf.size)
    assert normwise(gf, want) <= 5e-4                            # TF32 rounding of the activation


@pytest.mark.parametrize("M,N,K", [(256, 384, 128), (1024, 3072, 768), (300, 256, 96)])
def test_gemm_bias_gelu_with_the_approximate_tanh(bmb, orc, cuda, M, N, K):
    """BMB_GEMM_AUX_FAST: the activation in the epilogue takes the hardware's approximate tanh.  C is unchanged (equal to
    the accurate variant's bit for bit); C_gelu, unrounded, stays within 1e-3 of max|GELU| of the oracle's activation of
    that C element by element (the approximation's absolute error is about 5e-4 of |x|/2), and within 5e-4 normwise."""
    A, W, bias = rounded(orc, uniform(M * K, 31), "tf32"), rounded(orc, uniform(N * K, 32), "tf32"), uniform(N, 33)
    dA, dW, db = dev(cuda, A), dev(cuda, W), dev(cuda, bias)
    flags = bmb.GEMM_A_ROUNDED | bmb.GEMM_B_ROUNDED
    c_a, g_a = cuda.full((M * N,), float("nan"), device="cuda"), cuda.full((M * N,), float("nan"), device="cuda")
    c_f, g_f = cuda.full((M * N,), float("nan"), device="cuda"), cuda.full((M * N,), float("nan"), device="cuda")
    bmb.call("bmb_gemm_bias_gelu", bmb.MATH_TF32, flags, M, N, K, dA, dW, db, c_a, g_a, None)
    bmb.call("bmb_gemm_bias_gelu", bmb.MATH_TF32, flags | bmb.GEMM_AUX_FAST, M, N, K, dA, dW, db, c_f, g_f, None)
    cf, gf = host(cuda, c_f), host(cuda, g_f)
    assert np.array_equal(cf, host(cuda, c_a)) and np.all(np.isfinite(gf))
    want = np.empty_like(cf)
    orc.orc_gelu_forward(_np(want), _np(cf), cf.size)
    assert float(np.max(np.abs(gf - want))) <= 1e-3 * float(np.max(np.abs(want)))
    assert normwise(gf, want) <= 5e-4
    assert normwise(host(cuda, g_a), want) <= 1e-6               # the accurate variant, for contrast


def test_two_streams_take_turns_on_the_staging_scratch(bmb, cuda):
    """Tensor-core products whose operands are not flagged as rounded first round them into one per-device staging
    block.  Two streams of one device issuing such products at the same time must take turns on it (the library
    orders a slot's users with an event) instead of overwriting each other's operands: every result equals the
    one the same call gives when it runs alone."""
    import ctypes as C
    M, N, K = 1024, 768, 512
    ops = [(cuda.rand(M * K, device="cuda") * 2 - 1, cuda.rand(N * K, device="cuda") * 2 - 1) for _ in range(2)]
    alone = []
    for A, B in ops:
        c = cuda.zeros(M * N, device="cuda")
        bmb.call("bmb_gemm_ex", bmb.MATH_TF32, bmb.GEMM_NO_SPLIT, 0, 1, M, N, K, 1.0, A, B, 0.0, c, None)
        alone.append(host(cuda, c))
    streams = [cuda.cuda.Stream(), cuda.cuda.Stream()]
    outs = [[cuda.zeros(M * N, device="cuda") for _ in range(8)] for _ in range(2)]
    cuda.cuda.synchronize()
    for it in range(8):
        for i, (A, B) in enumerate(ops):
            bmb.call("bmb_gemm_ex", bmb.MATH_TF32, bmb.GEMM_NO_SPLIT, 0, 1, M, N, K, 1.0, A, B, 0.0, outs[i][it],
                     C.c_void_p(streams[i].cuda_stream))
    cuda.cuda.synchronize()
    for i in range(2):
        for it in range(8):
            assert np.array_equal(host(cuda, outs[i][it]), alone[i]), (i, it)


def test_deferred_column_sums_equal_a_launch_per_sum(bmb, cuda, monkeypatch):
    """The trainer defers the final stage of the two-stage parameter-gradient sums (layernorm gains and biases,
    projection biases) to one batched launch at the end of backward.  The batched kernel adds the same partial rows
    in the same order, so in fp32 arithmetic (no tile of a product shared between CTAs) every gradient except the
    token embedding's (atomic adds at colliding tokens) must come out bit for bit as with a launch per sum."""
    cfg = dict(TINY, n_layer=3)
    rng = np.random.default_rng(5)
    toks = rng.integers(0, cfg["vocab_size"], (cfg["B"], cfg["T"]), dtype=np.int32)
    tgts = rng.integers(0, cfg["vocab_size"], (cfg["B"], cfg["T"]), dtype=np.int32)
    grads = []
    for mode in ("1", "0"):
        monkeypatch.setenv("BMB_TRAINER_DEFER_COLSUMS", mode)
        tr = bmb.Trainer(seed=7, use_flash=1, math=bmb.MATH_FP32, fused=0, **cfg)
        tr.upload(toks, tgts)
        for _ in range(2):                       # the second pass replays what the first recorded
            tr.forward_backward()
        g = np.empty(tr.num_params, np.float32)
        tr.get_grads(g)
        tr.close()
        grads.append(g)
    wte = cfg["padded_vocab"] * cfg["n_embd"]
    assert np.all(np.isfinite(grads[0])) and np.abs(grads[0][wte:]).max() > 0
    assert np.array_equal(grads[0][wte:], grads[1][wte:])
    assert normwise(grads[0][:wte], grads[1][:wte]) < 1e-6


def test_qkv_bias_gradient_from_the_attention_backward(bmb, cuda, monkeypatch):
    """In the fused TF32 step the tensor-core attention backward leaves the qkv bias gradient (the column sums of dqkv)
    as partial sums from its own epilogue, instead of another sweep over dqkv.  Against that sweep
    (BMB_TRAINER_QKV_BIAS_IN_ATTENTION=0) on a ragged shape -- T = 200: a second block of 72 rows, quarters of 32, 32,
    8 and 0 valid rows, and three sequences, so that the rows past the end of a sequence inside a tile hold the next
    sequence's values and must be left out -- the bias gradient agrees to summation order, and so does the rest."""
    cfg = dict(max_seq_len=200, vocab_size=300, padded_vocab=384, n_layer=2, n_head=2, n_embd=128, B=3, T=200)
    rng = np.random.default_rng(9)
    toks = rng.integers(0, cfg["vocab_size"], (cfg["B"], cfg["T"]), dtype=np.int32)
    tgts = rng.integers(0, cfg["vocab_size"], (cfg["B"], cfg["T"]), dtype=np.int32)
    grads = []
    # from the epilogue with the sums deferred to the batched launch; from the epilogue with a launch per sum; the sweep
    for mode, defer in (("1", "1"), ("0", "1"), ("1", "0")):
        monkeypatch.setenv("BMB_TRAINER_QKV_BIAS_IN_ATTENTION", mode)
        monkeypatch.setenv("BMB_TRAINER_DEFER_COLSUMS", defer)
        tr = bmb.Trainer(seed=7, use_flash=1, math=bmb.MATH_TF32, fused=1, **cfg)
        tr.upload(toks, tgts)
        for _ in range(2):                       # the second pass replays the recorded job list / the captured graph
            tr.forward_backward()
        g = np.empty(tr.num_params, np.float32)
        tr.get_grads(g)
        tr.close()
        grads.append(g)
    L, C, Vp, maxT = cfg["n_layer"], cfg["n_embd"], cfg["padded_vocab"], cfg["max_seq_len"]
    off = Vp * C + maxT * C + 2 * L * C + L * 3 * C * C          # wte, wpe, ln1 gain and bias, qkv weight (src/gpt.cu:32-51)
    qb = [g[off:off + L * 3 * C] for g in grads]
    assert np.all(np.isfinite(grads[0])) and np.abs(qb[0]).max() > 0
    for other in (1, 2):
        assert normwise(qb[0], qb[other]) < 1e-5, (other, normwise(qb[0], qb[other]))
        assert normwise(grads[0], grads[other]) < 1e-5

