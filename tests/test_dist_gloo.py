"""World-size-2 rehearsal, on CPU with the gloo backend, of the launcher-side
logic the multi-GPU benchmark uses: unique-id hand-off, batch sharding,
max-over-ranks timing.  Also checks, with numpy standing in for the device,
that reduce-scatter + all-gather over bmb_ddp_slice's partition is a sum."""
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys, ctypes as C
import numpy as np
sys.path.insert(0, os.path.join(%(root)r, "tests"))
from conftest import load_package
bmb = load_package()
import importlib
dist_mod = importlib.import_module("bmb_b200.dist")
rank, local, world = dist_mod.env_rank()
dist_mod.init_process_group("gloo")
payload = bytes(range(128)) if rank == 0 else bytes(128)
got = dist_mod.broadcast_bytes(payload, 128)
assert got == bytes(range(128)), "id hand-off"
assert dist_mod.max_over_ranks(10.0 + rank) == 10.0 + world - 1
x, y = dist_mod.synthetic_batch(3, 4 * world, 16, 100)
mine = dist_mod.shard_rows(x, rank, world)
assert mine.shape == (4, 16) and np.array_equal(mine, x[rank * 4:(rank + 1) * 4])
# two-phase sum over the library's own partition, numpy in place of the GPU
import torch, torch.distributed as td
count = 1003
lib = bmb.lib()
buf = (np.arange(count) * (rank + 1)).astype(np.float32)
allbufs = [torch.zeros(count) for _ in range(world)]
td.all_gather(allbufs, torch.from_numpy(buf))
off, ln = C.c_size_t(), C.c_size_t()
lib.bmb_ddp_slice(count, world, rank, C.byref(off), C.byref(ln))
mine = sum(b[off.value:off.value + ln.value].numpy().astype(np.float64) for b in allbufs)
pieces = [None] * world
td.all_gather_object(pieces, (off.value, mine))
out = np.zeros(count)
for o, p in pieces:
    out[o:o + len(p)] = p
assert np.array_equal(out, np.arange(count) * sum(range(1, world + 1)))
dist_mod.barrier()
print("rank", rank, "ok")
"""


def test_world_size_two_on_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % {"root": ROOT})
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29517", str(script)],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.count("ok") == 2
