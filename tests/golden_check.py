"""Compare a reference-generated fixture (tests/golden/*.npz) with the CPU
oracle.  Tolerances are the reference's own: 1e-4 normwise for fp32 GEMMs
(src/registry.cu:5-12), the registry tolerance for the TF32 kernel, 1e-5 for
attention (tools/test_flash.cu:132, 226, 314)."""
import numpy as np

from helpers import _np, normwise


def check_fixture_with_oracle(orc, z, name):
    kind = str(z["kind"])
    if kind == "gemm":
        M, N, K = int(z["M"]), int(z["N"]), int(z["K"])
        c = z["C0"].copy()
        orc.orc_gemm(int(z["ta"]), int(z["tb"]), M, N, K, float(z["alpha"]), _np(z["A"].copy()), _np(z["B"].copy()),
                     float(z["beta"]), _np(c))
        assert normwise(c, z["out"]) < 1e-5, name
    elif kind == "sgemm":
        n = int(z["n"])
        c = z["C0"].copy()
        orc.orc_gemm(0, 0, n, n, n, float(z["alpha"]), _np(z["A"].copy()), _np(z["B"].copy()), float(z["beta"]), _np(c))
        assert normwise(c, z["out"]) < float(z["tol"]), name
    elif kind == "bgemm":
        b, M, N, K = int(z["batch"]), int(z["M"]), int(z["N"]), int(z["K"])
        c = z["C0"].copy()
        orc.orc_batched_gemm(int(z["ta"]), int(z["tb"]), b, M, N, K, float(z["alpha"]), _np(z["A"].copy()), M * K,
                             _np(z["B"].copy()), K * N, float(z["beta"]), _np(c), M * N)
        assert normwise(c, z["out"]) < 1e-5, name
    elif kind == "attention":
        B, T, C, NH = int(z["B"]), int(z["T"]), int(z["C"]), int(z["NH"])
        qkv, dout = z["qkv"].copy(), z["dout"].copy()
        out, lse = np.empty(B * T * C, np.float32), np.empty(B * NH * T, np.float32)
        orc.orc_attention_forward(_np(out), _np(lse), None, _np(qkv), B, T, C, NH)
        assert normwise(out, z["out"]) < 1e-5, name
        assert normwise(out, z["out_unfused"]) < 1e-5, name
        assert normwise(lse, z["lse"]) < 1e-5, name
        dqkv = np.empty(B * T * 3 * C, np.float32)
        orc.orc_attention_backward(_np(dqkv), _np(dout), _np(qkv), B, T, C, NH)
        g, w = dqkv.reshape(B * T, 3, C), z["dqkv"].reshape(B * T, 3, C)
        for i in range(3):   # dq, dk, dv separately, as tools/test_flash.cu:312-314
            assert normwise(g[:, i], w[:, i]) < 1e-5, name
    elif kind == "nn":
        N, C, V, Vp = int(z["N"]), int(z["C"]), int(z["V"]), int(z["Vp"])
        x, w, b, dy = (z[k].copy() for k in ("x", "w", "b", "dy"))
        o, mean, rstd = np.empty((N, C), np.float32), np.empty(N, np.float32), np.empty(N, np.float32)
        orc.orc_layernorm_forward(_np(o), _np(mean), _np(rstd), _np(x), _np(w), _np(b), N, C)
        assert normwise(o, z["ln_out"].reshape(N, C)) < 1e-5 and normwise(rstd, z["ln_rstd"]) < 1e-5, name
        dx, dw, db = z["dx0"].copy(), z["dw0"].copy(), z["db0"].copy()
        orc.orc_layernorm_backward(_np(dx), _np(dw), _np(db), _np(dy), _np(x), _np(w), _np(mean), _np(rstd), N, C)
        assert normwise(dx, z["ln_dx"].reshape(N, C)) < 1e-5, name
        assert normwise(dw, z["ln_dw"]) < 1e-5 and normwise(db, z["ln_db"]) < 1e-5, name
        g, dg = np.empty(N * C, np.float32), np.empty(N * C, np.float32)
        orc.orc_gelu_forward(_np(g), _np(x), N * C)
        orc.orc_gelu_backward(_np(dg), _np(x), _np(dy), N * C)
        assert normwise(g, z["gelu"]) < 1e-6 and normwise(dg, z["dgelu"]) < 1e-6, name
        dbias = z["db0"].copy()
        orc.orc_bias_backward(_np(dbias), _np(dy), N, C)
        assert normwise(dbias, z["dbias"]) < 1e-5, name
        p, l, d = np.empty(N * Vp, np.float32), np.empty(N, np.float32), np.empty(N * Vp, np.float32)
        tg = z["targets"].copy()
        orc.orc_softmax_crossentropy_forward(_np(p), _np(l), _np(z["logits"].copy()), _np(tg), N, V, Vp)
        orc.orc_crossentropy_softmax_backward(_np(d), _np(p), _np(tg), N, V, Vp, 1.0 / N)
        assert normwise(p, z["probs"]) < 1e-5 and normwise(l, z["losses"]) < 1e-5, name
        assert normwise(d, z["dlogits"]) < 1e-5, name
        pp, m, v = z["ad_p0"].copy(), z["ad_m0"].copy(), z["ad_v0"].copy()
        orc.orc_adamw_update(_np(pp), _np(z["ad_g"].copy()), _np(m), _np(v), 1000, 3e-4, 0.9, 0.95, 1e-8, 0.1, 3, 0.5)
        assert normwise(pp, z["ad_p"]) < 1e-6 and normwise(m, z["ad_m"]) < 1e-6 and normwise(v, z["ad_v"]) < 1e-6, name
        assert abs(orc.orc_grad_global_norm(_np(z["ad_g"].copy()), 1000) - float(z["gnorm"])) < 1e-4, name
    elif kind == "train":
        g = orc.orc_gpt_create(*(int(z[k]) for k in ("maxT", "V", "Vp", "L", "NH", "C", "B", "T")))
        n = orc.orc_gpt_num_params(g)
        assert n == z["params0"].size, name
        np.ctypeslib.as_array(orc.orc_gpt_params(g), shape=(n,))[:] = z["params0"]
        toks, tgts = z["tokens"], z["targets"]
        orc.orc_gpt_set_batch(g, _np(toks[0].copy()), _np(tgts[0].copy()))
        loss = orc.orc_gpt_forward(g)
        orc.orc_gpt_backward(g)
        grads = np.ctypeslib.as_array(orc.orc_gpt_grads(g), shape=(n,)).copy()
        assert abs(loss - float(z["loss_fb"])) < 1e-4, name
        assert normwise(grads[::97], z["grads1_sample"]) < 1e-4, name
        losses = []
        for s in range(toks.shape[0]):
            orc.orc_gpt_set_batch(g, _np(toks[s].copy()), _np(tgts[s].copy()))
            losses.append(orc.orc_gpt_step(g, float(z["lr"]), float(z["beta1"]), float(z["beta2"]), float(z["eps"]),
                                           float(z["wd"]), float(z["clip"]), s + 1))
        # per-step |loss difference| <= 2e-3 over 20 steps (fp32 path)
        assert np.max(np.abs(np.array(losses) - z["losses"])) < 2e-3, name
        orc.orc_gpt_destroy(g)
    else:
        raise AssertionError("unknown fixture kind %s in %s" % (kind, name))
