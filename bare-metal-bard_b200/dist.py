"""Launcher-side plumbing for the one-process-per-GPU form: rank discovery from
the torchrun environment, the hand-off of the NCCL unique id, batch sharding
and max-over-ranks timing.  torch.distributed is used for this plumbing only;
the gradient all-reduce itself runs inside libbmb.so (bmb_comm_allreduce).
"""
import os

import numpy as np


def env_rank():
    """(rank, local_rank, world_size) from the torchrun environment, else (0, 0, 1)."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def init_process_group(backend=None):
    """Join the rendezvous torchrun described (MASTER_ADDR/PORT); no-op at world size 1."""
    import torch.distributed as dist
    rank, _, world = env_rank()
    if world == 1 or dist.is_initialized():
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group(backend=backend or "gloo", rank=rank, world_size=world)


def broadcast_bytes(payload, nbytes, src=0):
    """Every rank returns the `nbytes` bytes rank `src` passed as `payload`."""
    import torch
    import torch.distributed as dist
    rank, _, world = env_rank()
    if world == 1:
        return bytes(payload)
    buf = torch.zeros(nbytes, dtype=torch.uint8)
    if rank == src:
        buf.copy_(torch.frombuffer(bytearray(payload), dtype=torch.uint8))
    dist.broadcast(buf, src=src)
    return bytes(buf.numpy().tobytes())


def max_over_ranks(value):
    """Largest `value` (a float) over all ranks."""
    import torch
    import torch.distributed as dist
    _, _, world = env_rank()
    if world == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier():
    import torch.distributed as dist
    if env_rank()[2] > 1:
        dist.barrier()


def shard_rows(global_rows, rank, world):
    """Rows [rank*B, (rank+1)*B) of a (world*B, T) batch: the split the reference
    makes at src/train_gpt.cu:405 (contiguous shards in rank order)."""
    n = global_rows.shape[0]
    if n % world:
        raise ValueError("global batch %d is not divisible by %d ranks" % (n, world))
    b = n // world
    return np.ascontiguousarray(global_rows[rank * b:(rank + 1) * b])


def synthetic_batch(step, global_batch, T, vocab, seed=4242):
    """Token ids and targets uniform over the vocabulary, one generator per step
    so that every rank can rebuild the same global batch without communication."""
    rng = np.random.default_rng(seed + step)
    x = rng.integers(0, vocab, size=(global_batch, T), dtype=np.int32)
    y = rng.integers(0, vocab, size=(global_batch, T), dtype=np.int32)
    return x, y
