"""The failure paths of the library, exercised without faulting, trapping or hanging anything:

  * a bounded device-side wait that runs out (the kernel gives up, returns, raises the
    per-device status word; later tensor-core calls report BMB_E_TIMEOUT until the word is
    cleared) -- driven by bmb_selftest_wait_expiry, whose one CTA waits a few thousand
    cycles on a barrier nothing arrives on;
  * the all-reduce with every transfer staged through host memory (DDP_NO_P2P, the switch of
    src/ddp.cu:116-120), in a child process because the switch is read when a handle is made.
"""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import normwise, uniform

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_wait_expiry_sets_status_and_clear_recovers(bmb, cuda):
    lib = bmb.lib()
    M = N = K = 256
    A = cuda.from_numpy(uniform(M * K, 1)).cuda()
    B = cuda.from_numpy(uniform(K * N, 2)).cuda()
    Cm = cuda.zeros(M * N, device="cuda")
    args = (bmb.MATH_TF32, 0, 0, 0, M, N, K, 1.0, A.data_ptr(), B.data_ptr(), 0.0, Cm.data_ptr(), None)
    st = C.c_int(-1)
    assert lib.bmb_kernel_status(C.byref(st)) == 0 and st.value == 0
    try:
        waited = C.c_longlong(0)
        bmb.check(lib.bmb_selftest_wait_expiry(20000, C.byref(waited)), "bmb_selftest_wait_expiry")
        # the wait ran out by itself: at least the limit, and nowhere near the two seconds of the real kernels
        assert 20000 <= waited.value < 20000000, waited.value
        assert lib.bmb_kernel_status(C.byref(st)) == 0 and st.value != 0
        rc = lib.bmb_gemm_ex(*args)
        assert rc == bmb.E_TIMEOUT, rc
        assert b"gave up waiting" in lib.bmb_last_error()
    finally:
        bmb.check(lib.bmb_kernel_status_clear(), "bmb_kernel_status_clear")
    assert lib.bmb_kernel_status(C.byref(st)) == 0 and st.value == 0
    bmb.check(lib.bmb_gemm_ex(*args), "bmb_gemm_ex")
    cuda.cuda.synchronize()
    want = (A.view(M, K).double() @ B.view(K, N).double()).cpu().numpy()
    assert normwise(Cm.cpu().numpy(), want) < 5e-4


def test_selftest_rejects_limits_that_could_hold_the_gpu(bmb, cuda):
    assert bmb.lib().bmb_selftest_wait_expiry(10 ** 10, None) != 0
    assert bmb.lib().bmb_selftest_wait_expiry(0, None) != 0


CHILD = r"""
import ctypes as C, os, sys
import numpy as np
sys.path.insert(0, %(tests)r)
from conftest import load_package
import torch
bmb = load_package()
lib = bmb.lib()
ngpu = torch.cuda.device_count()
def value_of(rank, idx):
    return ((idx * 2654435761 + rank * 40503) %% 1000).astype(np.float32) * np.float32(0.001) + np.float32(rank)
for n in (2, 3, 4, 8):
    devs = (C.c_int * n)(*[r %% ngpu for r in range(n)])
    h = C.c_void_p()
    bmb.check(lib.bmb_ddp_create(C.byref(h), n, devs))
    nn, peer = C.c_int(), (C.c_ubyte * (n * n))()
    bmb.check(lib.bmb_ddp_peer_matrix(h, C.byref(nn), None, peer))
    assert nn.value == n and not any(peer), "DDP_NO_P2P must clear every pair"
    for count in (1, 3, 17, 1000, 65537, 1048576):
        idx = np.arange(count, dtype=np.uint64)
        srcs = [value_of(r, idx) for r in range(n)]
        want = np.sum([s.astype(np.float64) for s in srcs], axis=0)
        bufs = [torch.from_numpy(srcs[r]).to("cuda:%%d" %% devs[r]) for r in range(n)]
        ptrs = (C.c_void_p * n)(*[b.data_ptr() for b in bufs])
        bmb.check(lib.bmb_ddp_allreduce(h, ptrs, count))
        for r in range(n):
            got = bufs[r].cpu().numpy().astype(np.float64)
            assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-30)) < 1e-6, (n, count, r)
    bmb.check(lib.bmb_ddp_destroy(h))
print("staged all-reduce ok")
"""


def test_allreduce_staged_through_host_memory(cuda, tmp_path):
    """tools/test_ddp.cu's matrix (n x count against a float64 sum, rel < 1e-6) with DDP_NO_P2P=1."""
    script = tmp_path / "staged.py"
    script.write_text(CHILD % {"tests": HERE})
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, DDP_NO_P2P="1"))
    assert r.returncode == 0 and "staged all-reduce ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
    assert "DDP_NO_P2P set" in r.stdout
