"""ctypes binding of libbmb.so, the sm_100a GEMM / attention / nn / all-reduce
library behind bare-metal-bard's C++ API.

The product is the shared library and the C/C++ headers in ``include/``; this
module exists so that tests and the benchmark can drive the C ABI from Python.
It never computes anything itself and has no CPU fallback: if ``libbmb.so`` is
missing, ``lib()`` raises and says how to build it.

The directory name contains a hyphen, so import it through
``importlib`` (see ``tests/conftest.py``) or ``__graft_entry__.load_package()``.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# BMB_LIB points at another build of the library (e.g. one compiled with the developer timers)
LIB_PATH = os.environ.get("BMB_LIB") or os.path.join(HERE, "libbmb.so")

MATH_FP32, MATH_TF32, MATH_BF16 = 0, 1, 2
GEMM_A_ROUNDED, GEMM_B_ROUNDED, GEMM_C_ROUNDED, GEMM_NO_SPLIT = 1, 2, 4, 8
GEMM_TILE_M128, GEMM_TILE_M256 = 16, 32
GEMM_PAIR, GEMM_NO_PAIR = 64, 128
GEMM_HALF_SMS = 256
GEMM_AUX_ROUNDED = 512
GEMM_AUX_FAST = 1024
FLASH_OPERANDS_ROUNDED = 1
E_UNSUPPORTED = 3
E_TIMEOUT = 4
E_LIMIT = 6

_f, _i, _p, _z, _ll, _d, _u = C.c_float, C.c_int, C.c_void_p, C.c_size_t, C.c_longlong, C.c_double, C.c_uint


class TrainConfig(C.Structure):
    _fields_ = [(n, _i) for n in ("max_seq_len", "vocab_size", "padded_vocab", "n_layer", "n_head", "n_embd",
                                  "B", "T", "use_flash", "math", "fused")] + \
               [(n, _f) for n in ("beta1", "beta2", "eps", "weight_decay", "grad_clip")]


class DdpTiming(C.Structure):
    _fields_ = [("reduce_scatter_ms", _d), ("all_gather_ms", _d), ("total_ms", _d), ("bytes_per_device", _z)]


class KernelEntry(C.Structure):
    _fields_ = [("id", _i), ("name", C.c_char_p), ("fn", _p), ("note", C.c_char_p), ("tol", _d)]


# name -> (restype, argtypes); must list every function include/bmb.h declares.
SIGNATURES = {
    "bmb_last_error": (C.c_char_p, []),
    "bmb_version": (C.c_char_p, []),
    "bmb_launch_count": (_ll, []),
    "bmb_gemm_schedule_check": (_i, [_i, _i, _i, _i, _i, _i, _i, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)]),
    "bmb_kernel_status": (_i, [C.POINTER(_i)]),
    "bmb_kernel_status_clear": (_i, []),
    "bmb_selftest_wait_expiry": (_i, [_ll, C.POINTER(_ll)]),
    "bmb_set_stream": (_i, [_p]),
    "bmb_get_stream": (_p, []),
    "bmb_set_math_mode": (_i, [_i]),
    "bmb_get_math_mode": (_i, []),
    "bmb_num_kernels": (_i, []),
    "bmb_kernel_table": (C.POINTER(KernelEntry), []),
    "bmb_find_kernel": (C.POINTER(KernelEntry), [_i]),
    "bmb_sgemm_simt": (_i, [_i, _i, _i, _f, _p, _p, _f, _p]),
    "bmb_sgemm_tf32": (_i, [_i, _i, _i, _f, _p, _p, _f, _p]),
    "bmb_sgemm_bf16": (_i, [_i, _i, _i, _f, _p, _p, _f, _p]),
    "bmb_gemm": (_i, [_i, _i, _i, _i, _i, _f, _p, _p, _f, _p, _p]),
    "bmb_gemm_ex": (_i, [_i, _i, _i, _i, _i, _i, _i, _f, _p, _p, _f, _p, _p]),
    "bmb_gemm_bias_gelu": (_i, [_i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p]),
    "bmb_batched_gemm": (_i, [_i, _i, _i, _i, _i, _i, _f, _p, _ll, _p, _ll, _f, _p, _ll, _p]),
    "bmb_round_tf32": (_i, [_p, _p, _z, _p]),
    "bmb_flash_attention_forward": (_i, [_p, _p, _p, _i, _i, _i, _i]),
    "bmb_flash_attention_backward": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i]),
    "bmb_flash_num_configs": (_i, []),
    "bmb_flash_config_name": (C.c_char_p, [_i]),
    "bmb_flash_default_config": (_i, []),
    "bmb_flash_attention_forward_cfg": (_i, [_i, _p, _p, _p, _i, _i, _i, _i]),
    "bmb_flash_attention_forward_ex": (_i, [_i, _i, _p, _p, _p, _i, _i, _i, _i]),
    "bmb_flash_num_bwd_configs": (_i, []),
    "bmb_flash_bwd_config_name": (C.c_char_p, [_i]),
    "bmb_flash_default_bwd_config": (_i, []),
    "bmb_flash_attention_backward_cfg": (_i, [_i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i]),
    "bmb_flash_attention_backward_ex": (_i, [_i, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i]),
    "bmb_attention_forward": (_i, [_p, _p, _p, _p, _i, _i, _i, _i]),
    "bmb_attention_backward": (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i]),
    "bmb_encoder_forward": (_i, [_p, _p, _p, _p, _i, _i, _i]),
    "bmb_encoder_backward": (_i, [_p, _p, _p, _p, _i, _i, _i]),
    "bmb_layernorm_forward": (_i, [_p, _p, _p, _p, _p, _p, _i, _i]),
    "bmb_layernorm_backward": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i]),
    "bmb_gelu_backward_colsum": (_i, [_p, _p, _p, _p, _i, _i]),
    "bmb_residual_layernorm_forward": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i]),
    "bmb_layernorm_backward_colsum": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i]),
    "bmb_layernorm_backward_noalloc": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i]),
    "bmb_gelu_forward": (_i, [_p, _p, _i]),
    "bmb_gelu_backward": (_i, [_p, _p, _p, _i]),
    "bmb_residual_forward": (_i, [_p, _p, _p, _i]),
    "bmb_add_inplace": (_i, [_p, _p, _i]),
    "bmb_bias_forward": (_i, [_p, _p, _i, _i]),
    "bmb_bias_backward": (_i, [_p, _p, _i, _i]),
    "bmb_softmax_crossentropy_forward": (_i, [_p, _p, _p, _p, _i, _i, _i]),
    "bmb_crossentropy_softmax_backward": (_i, [_p, _p, _p, _i, _i, _i, _f]),
    "bmb_softmax_crossentropy_fused": (_i, [_p, _p, _p, _p, _i, _i, _i, _f]),
    "bmb_adamw_update": (_i, [_p, _p, _p, _p, _i, _f, _f, _f, _f, _f, _i, _f]),
    "bmb_grad_global_norm": (_i, [_p, _i, C.POINTER(_f)]),
    "bmb_zero_buffer": (_i, [_p, _z]),
    "bmb_reduce_mean": (_i, [_p, _i, C.POINTER(_f)]),
    "bmb_grad_sumsq_device": (_i, [_p, _z, _p]),
    "bmb_reduce_mean_device": (_i, [_p, _i, _p]),
    "bmb_adamw_update_clipped": (_i, [_p, _p, _p, _p, _z, _f, _f, _f, _f, _f, _i, _p, _f, _f, _p]),
    "bmb_ddp_create": (_i, [C.POINTER(_p), _i, C.POINTER(_i)]),
    "bmb_ddp_destroy": (_i, [_p]),
    "bmb_ddp_allreduce": (_i, [_p, C.POINTER(_p), _z]),
    "bmb_ddp_slice": (_i, [_z, _i, _i, C.POINTER(_z), C.POINTER(_z)]),
    "bmb_ddp_timing_get": (_i, [_p, C.POINTER(DdpTiming)]),
    "bmb_ddp_peer_matrix": (_i, [_p, C.POINTER(_i), C.POINTER(_i), C.POINTER(C.c_ubyte)]),
    "bmb_ddp_report_topology": (_i, [_p]),
    "bmb_comm_unique_id": (_i, [C.POINTER(C.c_ubyte)]),
    "bmb_comm_create": (_i, [C.POINTER(_p), C.POINTER(C.c_ubyte), _i, _i]),
    "bmb_comm_destroy": (_i, [_p]),
    "bmb_comm_allreduce": (_i, [_p, _p, _z, _p]),
    "bmb_comm_allreduce_f64": (_i, [_p, _p, _z, _p]),
    "bmb_trainer_create": (_i, [C.POINTER(_p), C.POINTER(TrainConfig), _u]),
    "bmb_trainer_destroy": (_i, [_p]),
    "bmb_trainer_attach_comm": (_i, [_p, _p, _i]),
    "bmb_trainer_ipc_export": (_i, [_p, _p]),
    "bmb_trainer_attach_peers": (_i, [_p, _i, _i, _p]),
    "bmb_trainer_step_plan": (_i, [_p, _i, _p, _p, _p, _p]),
    "bmb_trainer_num_params": (_z, [_p]),
    "bmb_trainer_get_params": (_i, [_p, _p]),
    "bmb_trainer_set_params": (_i, [_p, _p]),
    "bmb_trainer_get_grads": (_i, [_p, _p]),
    "bmb_trainer_upload": (_i, [_p, _p, _p]),
    "bmb_trainer_step": (_i, [_p, _f, _i]),
    "bmb_trainer_forward_backward": (_i, [_p]),
    "bmb_trainer_loss": (_i, [_p, C.POINTER(_f)]),
    "bmb_trainer_loss_async": (_i, [_p, _p]),
    "bmb_trainer_sync": (_i, [_p]),
    "bmb_trainer_memory": (_i, [_p, C.POINTER(_z), C.POINTER(_z), C.POINTER(_z)]),
    "bmb_trainer_grad_norm": (_i, [_p, C.POINTER(_f)]),
    "bmb_trainer_forward_loss": (_i, [_p, C.POINTER(_f)]),
    "bmb_trainer_save": (_i, [_p, C.c_char_p, C.c_char_p, _i, _i, _i]),
    "bmb_checkpoint_header": (_i, [C.c_char_p, C.POINTER(TrainConfig), C.POINTER(_i), C.c_char_p, _i, C.POINTER(_i), C.POINTER(_i)]),
    "bmb_trainer_load": (_i, [_p, C.c_char_p, _i, C.POINTER(_i)]),
    "bmb_trainer_next_token_probs": (_i, [_p, _p, _i, _p]),
    "bmb_trainer_generate": (_i, [_p, _i, _i, _u, _f, _p]),
    "bmb_trainer_stream": (_p, [_p]),
    "bmb_trainer_profile": (_i, [_p, _i]),
    "bmb_trainer_profile_read": (_i, [_p, C.POINTER(_d), C.POINTER(_d), C.POINTER(_ll), C.POINTER(_ll)]),
}

_lib = None


class BmbError(RuntimeError):
    pass


def lib():
    """The loaded library with argument types set.  Raises if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise BmbError("%s is missing: run `python bare-metal-bard_b200/build.py` "
                           "(there is no CPU or PyTorch fallback)" % LIB_PATH)
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib


def check(status, what=""):
    """Raise BmbError with the library's message when a call did not return 0."""
    if status != 0:
        raise BmbError("%s failed (%d): %s" % (what or "bmb call", status, lib().bmb_last_error().decode()))


def ptr(t):
    """Device (or host) address of a torch tensor / numpy array / None."""
    if t is None:
        return None
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    return t.ctypes.data


def call(name, *args):
    """Call a status-returning entry point with tensors turned into pointers."""
    conv = [ptr(a) if (a is None or hasattr(a, "data_ptr") or hasattr(a, "ctypes")) else a for a in args]
    check(getattr(lib(), name)(*conv), name)


class Trainer:
    """Thin owner of a bmb_trainer handle (one GPT replica on the current device)."""

    def __init__(self, seed=1337, **cfg):
        d = dict(max_seq_len=1024, vocab_size=50304, padded_vocab=50304, n_layer=12, n_head=12, n_embd=768,
                 B=8, T=1024, use_flash=1, math=MATH_FP32, fused=0, beta1=0.9, beta2=0.95, eps=1e-8,
                 weight_decay=0.1, grad_clip=1.0)
        d.update(cfg)
        self.cfg = TrainConfig(**d)
        self.h = _p()
        check(lib().bmb_trainer_create(C.byref(self.h), C.byref(self.cfg), seed), "bmb_trainer_create")

    @property
    def num_params(self):
        return lib().bmb_trainer_num_params(self.h)

    def upload(self, tokens, targets):
        check(lib().bmb_trainer_upload(self.h, ptr(tokens), ptr(targets)), "bmb_trainer_upload")

    def step(self, lr, step):
        check(lib().bmb_trainer_step(self.h, lr, step), "bmb_trainer_step")

    def forward_backward(self):
        check(lib().bmb_trainer_forward_backward(self.h), "bmb_trainer_forward_backward")

    def loss(self):
        v = _f()
        check(lib().bmb_trainer_loss(self.h, C.byref(v)), "bmb_trainer_loss")
        return v.value

    def ipc_export(self):
        """This rank's 192-byte record of CUDA IPC handles (gradients, parameters, shadow)."""
        rec = (C.c_ubyte * 192)()
        check(lib().bmb_trainer_ipc_export(self.h, rec), "bmb_trainer_ipc_export")
        return bytes(rec)

    def attach_peers(self, rank, nranks, records):
        """records: the ranks' ipc_export() results concatenated in rank order."""
        buf = (C.c_ubyte * len(records)).from_buffer_copy(records) if records is not None else None
        check(lib().bmb_trainer_attach_peers(self.h, rank, nranks, buf), "bmb_trainer_attach_peers")

    def loss_async(self, pinned_scalar):
        """Enqueue the read of the last step's loss into a pinned float32 tensor / array element."""
        check(lib().bmb_trainer_loss_async(self.h, ptr(pinned_scalar)), "bmb_trainer_loss_async")

    def sync(self):
        check(lib().bmb_trainer_sync(self.h), "bmb_trainer_sync")

    @property
    def stream(self):
        """Raw cudaStream_t the trainer enqueues on."""
        return lib().bmb_trainer_stream(self.h)

    def get_params(self, out):
        check(lib().bmb_trainer_get_params(self.h, ptr(out)), "bmb_trainer_get_params")

    def set_params(self, src):
        check(lib().bmb_trainer_set_params(self.h, ptr(src)), "bmb_trainer_set_params")

    def get_grads(self, out):
        check(lib().bmb_trainer_get_grads(self.h, ptr(out)), "bmb_trainer_get_grads")

    def attach_comm(self, comm, nranks):
        check(lib().bmb_trainer_attach_comm(self.h, comm, nranks), "bmb_trainer_attach_comm")

    def profile(self, on):
        check(lib().bmb_trainer_profile(self.h, 1 if on else 0), "bmb_trainer_profile")

    def profile_read(self):
        fl, ms, calls, launches = _d(), _d(), _ll(), _ll()
        check(lib().bmb_trainer_profile_read(self.h, C.byref(fl), C.byref(ms), C.byref(calls), C.byref(launches)),
              "bmb_trainer_profile_read")
        return dict(gemm_flop=fl.value, gemm_ms=ms.value, gemm_calls=calls.value, launches=launches.value)

    def save(self, path, itos=b"", with_optimizer_state=False, step=0):
        check(lib().bmb_trainer_save(self.h, str(path).encode(), bytes(itos), len(itos), 1 if with_optimizer_state else 0, step),
              "bmb_trainer_save")

    def load(self, path, optimizer_state=False):
        step = _i(0)
        check(lib().bmb_trainer_load(self.h, str(path).encode(), 1 if optimizer_state else 0, C.byref(step)), "bmb_trainer_load")
        return step.value

    def forward_loss(self):
        v = _f()
        check(lib().bmb_trainer_forward_loss(self.h, C.byref(v)), "bmb_trainer_forward_loss")
        return v.value

    def grad_norm(self):
        v = _f()
        check(lib().bmb_trainer_grad_norm(self.h, C.byref(v)), "bmb_trainer_grad_norm")
        return v.value

    def generate(self, start_token, steps, seed, temperature=1.0):
        out = (C.c_int * max(steps, 1))()
        check(lib().bmb_trainer_generate(self.h, start_token, steps, seed, temperature, out), "bmb_trainer_generate")
        return list(out[:steps])

    def close(self):
        if self.h:
            lib().bmb_trainer_destroy(self.h)
            self.h = _p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
