"""bmb_layernorm_backward_noalloc: the layernorm backward for callers that cannot allocate
(a training loop whose device memory is fully handed out at start-up, where a lazy
cudaMalloc inside a step could fail or stall the device).  Its scratch is a fixed array in
the library image, so the check is that it gives what bmb_layernorm_backward gives and what
the CPU oracle (src/nn.cu:85-113 restated) gives -- on two calls in a row, because the array
keeps the previous call's contents -- and that it refuses rows wider than the array was sized
for.  Collected last on purpose."""
import numpy as np
import pytest

from helpers import _np, normal, normwise

pytestmark = pytest.mark.gpu


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run(bmb, torch, name, args_np, N, C):
    x, w, dy, mean, rstd, dx0, dw0, db0 = (dev(torch, a) for a in args_np)
    bmb.call(name, dx0, dw0, db0, dy, x, w, mean, rstd, N, C)
    torch.cuda.synchronize()
    return dx0.cpu().numpy(), dw0.cpu().numpy(), db0.cpu().numpy()


@pytest.mark.parametrize("N,C", [(8192, 768), (100, 64), (33, 1024)])
def test_noalloc_layernorm_backward_matches_the_allocating_entry_point(bmb, orc, cuda, N, C):
    for call in range(2):                     # second call meets the first call's leftovers in the array
        x, w, dy = normal((N, C), 10 + call), normal(C, 20 + call), normal((N, C), 30 + call)
        b = np.zeros(C, np.float32)
        tx, tw, tb = dev(cuda, x), dev(cuda, w), dev(cuda, b)
        out, mean, rstd = cuda.zeros(N * C, device="cuda"), cuda.zeros(N, device="cuda"), cuda.zeros(N, device="cuda")
        bmb.call("bmb_layernorm_forward", out, mean, rstd, tx, tw, tb, N, C)
        cuda.cuda.synchronize()
        args = (x, w, dy, mean.cpu().numpy(), rstd.cpu().numpy(), normal((N, C), 40 + call), normal(C, 50 + call),
                normal(C, 60 + call))
        want = run(bmb, cuda, "bmb_layernorm_backward", args, N, C)
        got = run(bmb, cuda, "bmb_layernorm_backward_noalloc", args, N, C)
        for g, wnt in zip(got, want):
            assert normwise(g, wnt) < 1e-5     # the bar of the other layernorm tests
        # and against the CPU oracle, started from the same dinp / dweight / dbias (all three accumulate)
        odx, odw, odb = args[5].copy(), args[6].copy(), args[7].copy()
        orc.orc_layernorm_backward(_np(odx), _np(odw), _np(odb), _np(dy), _np(x), _np(w), _np(args[3]), _np(args[4]), N, C)
        # the oracle sums the N rows one after another in fp32: its own rounding grows with N
        bar = 1e-5 if N <= 1024 else 1e-4
        for g, wnt in zip(got, (odx, odw, odb)):
            assert normwise(g, wnt) < bar


def test_noalloc_layernorm_backward_rejects_rows_beyond_its_array(bmb, cuda):
    N, C = 4, 2048
    z = cuda.zeros(N * C, device="cuda")
    st = bmb.lib().bmb_layernorm_backward_noalloc(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(),
                                                  z.data_ptr(), z.data_ptr(), z.data_ptr(), N, C)
    assert st == bmb.E_LIMIT and b"C <= 1024" in bmb.lib().bmb_last_error()
