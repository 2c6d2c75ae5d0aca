"""One rank of the two-GPU peer-exchange test (launched by test_peer_multi_gpu.py through
torch.distributed.run; gloo carries the IPC handles, the gradients travel over peer memory)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np
import torch
import torch.distributed as dist

from tensotron_b200.mlp import MlpTrainer, shard_rows
from tensotron_b200.runtime import TensorRuntime


def main():
    mode = int(sys.argv[1])
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dims, batch = [512, 2048, 1024, 10], 1024
    rng = np.random.default_rng(7)
    x = torch.from_numpy(rng.standard_normal((batch, dims[0])).astype(np.float32)).cuda()
    y = torch.from_numpy(rng.integers(0, dims[-1], batch).astype(np.int32)).cuda()
    lo, hi = shard_rows(batch, world, rank)
    tr = MlpTrainer(dims, rt=TensorRuntime(local), device=local, lr=1e-3, seed=5, math_mode=mode,
                    process_group=dist.group.WORLD, exchange="peer")
    ref = MlpTrainer(dims, rt=TensorRuntime(local), device=local, lr=1e-3, seed=5, math_mode=mode)
    dist.barrier()
    for step in range(4):
        tr.step(x[lo:hi].contiguous(), y[lo:hi].contiguous(), global_batch=batch)
        ref.step(x, y)
        tr.rt.Check()
        assert tr.fused[:2] == [True, True], tr.fused
        d = (tr.params - ref.params).abs()
        assert float(d.max()) <= 2.1e-3 * (step + 1), float(d.max())
        assert float(d.mean()) <= (0.02 if mode == 0 else 0.2) * 1e-3, float(d.mean())
        # every rank must hold the same bits
        mine = tr.params.cpu()
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        for g in gathered:
            assert torch.equal(g, mine)
    tr.close()
    dist.barrier()
    if rank == 0:
        print("PEER_OK mode %d world %d" % (mode, world))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
