"""GPU parity of the MLP training step (forward, cross-entropy, backward, Adam) against the
CPU oracle's restatement of the reference op sequence."""
import numpy as np
import pytest
import torch

import oracle
from tensotron_b200.mlp import MlpTrainer

pytestmark = pytest.mark.gpu


def _oracle_from(tr):
    ws = [tr.weight(i).cpu().numpy().copy() for i in range(tr.L)]
    bs = [tr.bias(i).cpu().numpy().copy() for i in range(tr.L)]
    return oracle.MlpOracle(ws, bs, lr=tr.lr)


@pytest.mark.parametrize("dims,batch", [([20, 32, 48, 5], 64), ([784, 256, 256, 256, 10], 512), ([33, 17, 9], 50)])
def test_mlp_steps_match_oracle(rt, dims, batch):
    tr = MlpTrainer(dims, rt=rt, lr=1e-3, seed=5)
    ref = _oracle_from(tr)
    rng = np.random.default_rng(0)
    x = rng.standard_normal((batch, dims[0])).astype(np.float32)
    y = rng.integers(0, dims[-1], batch).astype(np.int32)
    xd, yd = torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()
    for step in range(3):
        loss = tr.step(xd, yd).item()
        lo = ref.step(x, y)
        rt.Check()
        assert abs(loss - lo) <= 2e-5 * max(1.0, abs(lo)), (step, loss, lo)
        # gradients of this step (strict-FP32 bound on the largest contraction, K = batch)
        for i in range(tr.L):
            gw = tr.weight(i, tr.grads).cpu().numpy()
            assert np.abs(gw - ref.grads[i]).max() <= 1e-5 * np.sqrt(batch) * max(1.0, np.abs(x).max()) * 0.5 + 1e-6
            gb = tr.bias(i, tr.grads).cpu().numpy()
            assert np.abs(gb - ref.grads[tr.L + i]).max() <= 1e-5
        # parameters after Adam: lr * O(1) steps, so compare tightly relative to lr
        for i in range(tr.L):
            assert np.abs(tr.weight(i).cpu().numpy() - ref.w[i]).max() <= 0.05 * tr.lr + 1e-6
            assert np.abs(tr.bias(i).cpu().numpy() - ref.b[i]).max() <= 0.05 * tr.lr + 1e-6
    assert tr.adv[0].item() == 3


def test_mlp_loss_decreases_and_is_bitwise_repeatable(rt):
    dims = [64, 128, 128, 10]
    rng = np.random.default_rng(1)
    x = torch.from_numpy(rng.standard_normal((256, 64)).astype(np.float32)).cuda()
    y = torch.from_numpy(rng.integers(0, 10, 256).astype(np.int32)).cuda()
    runs = []
    for _ in range(2):
        tr = MlpTrainer(dims, rt=rt, lr=1e-2, seed=9)
        losses = [tr.step(x, y).item() for _ in range(15)]
        runs.append((losses, tr.params.clone()))
    assert runs[0][0][-1] < runs[0][0][0]
    assert runs[0][0] == runs[1][0]
    assert torch.equal(runs[0][1], runs[1][1])
