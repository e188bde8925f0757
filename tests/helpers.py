"""ctypes views of the two checkers used by the tests: the CPU oracle
(oracle/liborc.so) and the reference's own CUDA kernels (oracle/_ref/libbmbref.so).
Both are test infrastructure; the shipped library never loads them."""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORC_PATH = os.path.join(ORACLE_DIR, "liborc.so")
REF_PATH = os.path.join(ORACLE_DIR, "_ref", "libbmbref.so")

_f, _i, _p, _z, _ll, _d, _u = C.c_float, C.c_int, C.c_void_p, C.c_size_t, C.c_longlong, C.c_double, C.c_uint


def _np(a):
    return a.ctypes.data_as(C.c_void_p)


def load_oracle():
    src = os.path.join(ORACLE_DIR, "bmb_oracle.c")
    if not os.path.exists(ORC_PATH) or os.path.getmtime(ORC_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", ORACLE_DIR, "oracle"], stdout=subprocess.DEVNULL)
    l = C.CDLL(ORC_PATH)
    sig = {
        "orc_num_threads": (_i, []),
        "orc_gemm": (None, [_i, _i, _i, _i, _i, _f, _p, _p, _f, _p]),
        "orc_gemm_fast": (None, [_i, _i, _i, _i, _i, _f, _p, _p, _f, _p]),
        "orc_gemm_f64": (None, [_i, _i, _i, _i, _i, _f, _p, _p, _f, _p]),
        "orc_batched_gemm": (None, [_i, _i, _i, _i, _i, _i, _f, _p, _ll, _p, _ll, _f, _p, _ll]),
        "orc_round_tf32": (_f, [_f]),
        "orc_round_tf32_n": (None, [_p, _p, _z]),
        "orc_round_bf16": (_f, [_f]),
        "orc_normwise": (_d, [_p, _p, _z]),
        "orc_fill_xorshift": (None, [_p, _z, _u]),
        "orc_attention_forward": (None, [_p, _p, _p, _p, _i, _i, _i, _i]),
        "orc_attention_backward": (None, [_p, _p, _p, _i, _i, _i, _i]),
        "orc_encoder_forward": (None, [_p, _p, _p, _p, _i, _i, _i]),
        "orc_encoder_backward": (None, [_p, _p, _p, _p, _i, _i, _i]),
        "orc_layernorm_forward": (None, [_p, _p, _p, _p, _p, _p, _i, _i]),
        "orc_layernorm_backward": (None, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i]),
        "orc_gelu_forward": (None, [_p, _p, _z]),
        "orc_gelu_backward": (None, [_p, _p, _p, _z]),
        "orc_residual_forward": (None, [_p, _p, _p, _z]),
        "orc_bias_forward": (None, [_p, _p, _i, _i]),
        "orc_bias_backward": (None, [_p, _p, _i, _i]),
        "orc_softmax_crossentropy_forward": (None, [_p, _p, _p, _p, _i, _i, _i]),
        "orc_crossentropy_softmax_backward": (None, [_p, _p, _p, _i, _i, _i, _f]),
        "orc_adamw_update": (None, [_p, _p, _p, _p, _z, _f, _f, _f, _f, _f, _i, _f]),
        "orc_grad_global_norm": (_f, [_p, _z]),
        "orc_mean": (_f, [_p, _i]),
        "orc_gpt_create": (_p, [_i] * 8),
        "orc_gpt_destroy": (None, [_p]),
        "orc_gpt_num_params": (_z, [_p]),
        "orc_gpt_params": (C.POINTER(_f), [_p]),
        "orc_gpt_grads": (C.POINTER(_f), [_p]),
        "orc_gpt_set_batch": (None, [_p, _p, _p]),
        "orc_gpt_forward": (_f, [_p]),
        "orc_gpt_backward": (None, [_p]),
        "orc_gpt_step": (_f, [_p, _f, _f, _f, _f, _f, _f, _i]),
    }
    for n, (r, a) in sig.items():
        fn = getattr(l, n)
        fn.restype, fn.argtypes = r, a
    return l


def load_reference():
    if not os.path.exists(REF_PATH):
        return None
    l = C.CDLL(REF_PATH)
    sig = {
        "ref_num_kernels": (_i, []),
        "ref_kernel_tol": (_d, [_i]),
        "ref_sgemm": (_i, [_i, _i, _i, _i, _f, _p, _p, _f, _p]),
        "ref_gemm": (None, [_i, _i, _i, _i, _i, _f, _p, _p, _f, _p]),
        "ref_batched_gemm": (None, [_i, _i, _i, _i, _i, _i, _f, _p, _ll, _p, _ll, _f, _p, _ll]),
        "ref_flash_attention_forward": (None, [_p, _p, _p, _i, _i, _i, _i]),
        "ref_flash_attention_backward": (None, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i]),
        "ref_attention_forward": (None, [_p, _p, _p, _p, _i, _i, _i, _i]),
        "ref_attention_backward": (None, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i]),
        "ref_encoder_forward": (None, [_p, _p, _p, _p, _i, _i, _i]),
        "ref_encoder_backward": (None, [_p, _p, _p, _p, _i, _i, _i]),
        "ref_layernorm_forward": (None, [_p, _p, _p, _p, _p, _p, _i, _i]),
        "ref_layernorm_backward": (None, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i]),
        "ref_gelu_forward": (None, [_p, _p, _i]),
        "ref_gelu_backward": (None, [_p, _p, _p, _i]),
        "ref_residual_forward": (None, [_p, _p, _p, _i]),
        "ref_bias_forward": (None, [_p, _p, _i, _i]),
        "ref_bias_backward": (None, [_p, _p, _i, _i]),
        "ref_softmax_crossentropy_forward": (None, [_p, _p, _p, _p, _i, _i, _i]),
        "ref_crossentropy_softmax_backward": (None, [_p, _p, _p, _i, _i, _i, _f]),
        "ref_adamw_update": (None, [_p, _p, _p, _p, _i, _f, _f, _f, _f, _f, _i, _f]),
        "ref_grad_global_norm": (_f, [_p, _i]),
        "ref_reduce_mean": (_f, [_p, _i]),
        "ref_ddp_create": (_p, [_i, C.POINTER(_i)]),
        "ref_ddp_allreduce": (None, [_p, C.POINTER(_p), _z]),
        "ref_ddp_total_ms": (_d, [_p]),
        "ref_ddp_destroy": (None, [_p]),
        "ref_trainer_create": (_p, [_i] * 9 + [_u, _i] + [_f] * 5),
        "ref_trainer_num_params": (_z, [_p]),
        "ref_trainer_get_params": (None, [_p, _p]),
        "ref_trainer_set_params": (None, [_p, _p]),
        "ref_trainer_get_grads": (None, [_p, _p]),
        "ref_trainer_forward_backward": (_f, [_p, _p, _p]),
        "ref_trainer_step": (_f, [_p, _p, _p, _f, _i]),
        "ref_trainer_loss_from_probs": (_f, [_p]),
        "ref_trainer_destroy": (None, [_p]),
    }
    for n, (r, a) in sig.items():
        fn = getattr(l, n)
        fn.restype, fn.argtypes = r, a
    return l


def normwise(got, ref):
    """max|got-ref| / max|ref| with NaN/Inf failing (src/bench.cu:133-147)."""
    got = np.asarray(got, dtype=np.float64).ravel()
    ref = np.asarray(ref, dtype=np.float64).ravel()
    if not np.all(np.isfinite(got)):
        return float("inf")
    return float(np.max(np.abs(got - ref)) / max(np.max(np.abs(ref)), 1e-30))


def uniform(shape, seed):
    """Uniform [-1, 1) fp32 from a seeded generator."""
    return np.random.default_rng(seed).uniform(-1.0, 1.0, size=shape).astype(np.float32)


def normal(shape, seed, std=1.0):
    return (np.random.default_rng(seed).standard_normal(size=shape) * std).astype(np.float32)


def xorshift(n, seed, orc):
    out = np.empty(n, dtype=np.float32)
    orc.orc_fill_xorshift(_np(out), n, seed)
    return out
