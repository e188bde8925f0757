"""Run under torchrun with 2..8 ranks (one per GPU): trains a small model for a few steps twice --
gradients summed by NCCL and every rank running the whole optimiser, then the fused exchange over
peer memory, in one chunk after backward and in three chunks overlapped with backward (and, in a third
run, also with the next forward) -- from the same seed on the same batches, and checks that the losses agree, that
every rank ends with the same parameters, and that the ways end with the same parameters up
to the reassociation of the gradient sum.  Exit status 0 = ok.  Used by test_gpu_parity.py."""
import ctypes as C
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from __graft_entry__ import load_package  # noqa: E402

bmb = load_package()
import importlib
dist_mod = importlib.import_module("bmb_b200.dist")


def main():
    rank, local, world = dist_mod.env_rank()
    torch.cuda.set_device(local)
    dist_mod.init_process_group("gloo")
    lib = bmb.lib()
    cfg = dict(max_seq_len=128, vocab_size=512, padded_vocab=512, n_layer=4, n_head=2, n_embd=128, B=4, T=128)   # four layers: all three chunks of the overlapped exchange hold something
    steps = 6
    rng = np.random.default_rng(99)
    toks = rng.integers(0, 512, (steps, 4 * world, 128), dtype=np.int32)
    tgts = rng.integers(0, 512, (steps, 4 * world, 128), dtype=np.int32)

    def run(fused, overlap=0):
        os.environ["BMB_TRAINER_OVERLAP"] = str(overlap)                 # read when the trainer is created
        tr = bmb.Trainer(seed=1337, use_flash=1, math=bmb.MATH_TF32, fused=1, **cfg)
        ident = (C.c_ubyte * 128)()
        if rank == 0:
            bmb.check(lib.bmb_comm_unique_id(ident), "bmb_comm_unique_id")
        raw = dist_mod.broadcast_bytes(bytes(ident), 128)
        comm = C.c_void_p()
        bmb.check(lib.bmb_comm_create(C.byref(comm), (C.c_ubyte * 128)(*raw), world, rank), "bmb_comm_create")
        tr.attach_comm(comm, world)
        if fused:
            mine = tr.ipc_export()
            recs = b"".join(dist_mod.broadcast_bytes(mine, 192, src=r) for r in range(world))
            tr.attach_peers(rank, world, recs)
        losses = []
        for s in range(steps):
            tr.upload(dist_mod.shard_rows(toks[s], rank, world), dist_mod.shard_rows(tgts[s], rank, world))
            tr.step(3e-4, s + 1)
            losses.append(tr.loss())
        params = np.empty(tr.num_params, np.float32)
        tr.get_params(params)
        tr.close()
        bmb.check(lib.bmb_comm_destroy(comm), "bmb_comm_destroy")
        return np.array(losses), params

    l0, p0 = run(False)
    l0b, p0b = run(False)
    l1, p1 = run(True, overlap=2)          # three chunks, under backward and the next forward
    l2, p2 = run(True, overlap=0)          # one chunk after backward
    l3, p3 = run(True, overlap=1)          # three chunks, reduces under backward
    ok = True
    if max(np.abs(l0 - l1).max(), np.abs(l0 - l2).max(), np.abs(l0 - l3).max()) > 1e-4:
        print("rank %d: losses differ %s %s %s %s" % (rank, l0, l1, l2, l3)); ok = False
    # Sums that use atomics (token-embedding gradient, GEMM tiles shared between CTAs) wobble from run to
    # run, and AdamW's g / sqrt(v) magnifies that where v is tiny: the bar is the gap between two runs
    # of the SAME way.
    norm = np.linalg.norm(p0.astype(np.float64))
    wobble = np.linalg.norm(p0.astype(np.float64) - p0b) / norm
    rel = max(np.linalg.norm(p0.astype(np.float64) - p) / norm for p in (p1, p2, p3))
    if rel > 5 * wobble + 1e-6:
        print("rank %d: parameters differ between the two ways: %.3e (run-to-run wobble %.3e)" % (rank, rel, wobble)); ok = False
    # every rank must hold the same parameters after the fused steps
    import torch.distributed as dist
    for name, p in (("overlapped", p1), ("one chunk", p2), ("reduces overlapped", p3)):
        t = torch.from_numpy(p.copy())
        ref = t.clone()
        dist.broadcast(ref, src=0)
        if not torch.equal(t, ref):
            print("rank %d: parameters differ from rank 0 after the fused steps (%s)" % (rank, name)); ok = False
    flag = torch.tensor([0 if ok else 1])
    dist.all_reduce(flag)
    if rank == 0:
        print("fused data-parallel step vs NCCL: %s (max loss gap %.2e, parameter gap %.2e, run-to-run wobble %.2e)" % ("ok" if flag.item() == 0 else "MISMATCH", np.abs(l0 - l1).max(), rel, wobble))
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
