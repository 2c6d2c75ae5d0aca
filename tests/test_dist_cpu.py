"""world_size-2 gloo tests (CPU) of the multi-rank host logic: row sharding and the
data-parallel gradient exchange (sum of per-shard gradients scaled by 1/global_batch equals
the single-process gradient).  The per-rank math is done by the CPU oracle here; on GPUs the
same exchange runs over NCCL in tensotron_b200/mlp.py."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from tensotron_b200.mlp import layer_layout, shard_rows


def test_shard_rows_partitions_exactly():
    for total in (0, 1, 7, 8192, 16384, 1000):
        for world in (1, 2, 3, 4, 8):
            blocks = [shard_rows(total, world, r) for r in range(world)]
            assert blocks[0][0] == 0 and blocks[-1][1] == total
            for (s0, e0), (s1, e1) in zip(blocks, blocks[1:]):
                assert e0 == s1 and s0 <= e0
    assert shard_rows(16384, 8, 3) == (6144, 8192)


def test_layer_layout_is_aligned_and_disjoint():
    offs, total = layer_layout([784, 4096, 4096, 4096, 10])
    assert total >= 36818954 and total % 4 == 0
    prev_end = 0
    dims = [784, 4096, 4096, 4096, 10]
    for i, (w, b) in enumerate(offs):
        assert w % 4 == 0 and w >= prev_end and b == w + dims[i + 1] * dims[i]
        prev_end = b + dims[i + 1]


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(0)                      # identical data on every rank
        dims = [12, 16, 8, 4]
        ws = [(rng.uniform(-1, 1, (dims[i + 1], dims[i])) / np.sqrt(dims[i])).astype(np.float32) for i in range(3)]
        bs = [rng.uniform(-0.1, 0.1, dims[i + 1]).astype(np.float32) for i in range(3)]
        batch = 30
        x = rng.standard_normal((batch, dims[0])).astype(np.float32)
        y = rng.integers(0, dims[-1], batch).astype(np.int32)
        s, e = shard_rows(batch, world, rank)
        # local forward/backward on the shard, loss scaled by 1/global batch
        mlp = oracle.MlpOracle(ws, bs)
        acts, zs = [x[s:e]], []
        for i in range(3):
            z, a = oracle.linear_fwd(acts[-1], mlp.w[i], mlp.b[i], 1 if i < 2 else 0)
            zs.append(z)
            acts.append(a)
        loss, g = oracle.cross_entropy(acts[-1], y[s:e], scale=1.0 / batch)
        grads = [None] * 6
        for i in reversed(range(3)):
            dx, dw, db, _ = oracle.linear_bwd(acts[i], mlp.w[i], zs[i], acts[i + 1], g, 1 if i < 2 else 0, need_dx=i > 0)
            grads[i], grads[3 + i] = dw, db
            g = dx
        flat = torch.from_numpy(np.concatenate([t.reshape(-1) for t in grads]))
        lt = torch.tensor([loss], dtype=torch.float64)
        dist.all_reduce(flat)                                # the one exchange step
        dist.all_reduce(lt)
        if rank == 0:
            full = oracle.MlpOracle(ws, bs)
            lfull = full.step(x, y, apply_update=False)
            ref = np.concatenate([t.reshape(-1) for t in full.grads])
            q.put((float(np.abs(flat.numpy() - ref).max()), abs(lt.item() - lfull)))
    finally:
        dist.destroy_process_group()


def test_data_parallel_gradients_equal_single_process_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    gerr, lerr = q.get(timeout=10)
    assert gerr <= 1e-6 and lerr <= 1e-6
