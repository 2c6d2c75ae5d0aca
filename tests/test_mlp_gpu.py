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
        # After the first update the two sides may differ by up to 2*lr in parameters whose
        # gradient is at noise level (see below), so only step 0 is compared tightly.
        assert abs(loss - lo) <= (2e-5 if step == 0 else 2e-3) * max(1.0, abs(lo)), (step, loss, lo)
        # gradients of the first step (strict-FP32 bound on the largest contraction, K = batch)
        for i in range(tr.L if step == 0 else 0):
            gw = tr.weight(i, tr.grads).cpu().numpy()
            assert np.abs(gw - ref.grads[i]).max() <= 1e-5 * np.sqrt(batch) * max(1.0, np.abs(x).max()) * 0.5 + 1e-6
            gb = tr.bias(i, tr.grads).cpu().numpy()
            assert np.abs(gb - ref.grads[tr.L + i]).max() <= 1e-4
        # Parameters after Adam.  Adam normalises each gradient element, so an element whose
        # gradient is at rounding-noise level may take a +lr step on one side and -lr on the
        # other: those are bounded by 2*lr per step; everything else must agree closely.
        for i in range(tr.L):
            for got, want in ((tr.weight(i).cpu().numpy(), ref.w[i]), (tr.bias(i).cpu().numpy(), ref.b[i])):
                d = np.abs(got - want)
                assert d.max() <= 2.1 * tr.lr * (step + 1)
                assert np.mean(d) <= 0.02 * tr.lr
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


def test_mlp_step_replays_from_a_cuda_graph(rt):
    """The whole step (forward, loss, backward, Adam with its device-resident step counter)
    records into one CUDA graph and replays: the reference's captured-step contract
    (src/Tensotron/TensorRuntime.cs:596-698; tests/Tensotron.Tests/TraceReplayTests.cs:134-194
    for the Adam bias correction advancing across replays)."""
    dims = [8, 64, 64, 2]          # an RL-policy sized network
    rng = np.random.default_rng(2)
    x = torch.from_numpy(rng.standard_normal((64, 8)).astype(np.float32)).cuda()
    y = torch.from_numpy(rng.integers(0, 2, 64).astype(np.int32)).cuda()
    eager = MlpTrainer(dims, rt=rt, lr=1e-2, seed=4)
    eager_losses = [eager.step(x, y).item() for _ in range(6)]

    tr = MlpTrainer(dims, rt=rt, lr=1e-2, seed=4)
    losses = [tr.step(x, y).item()]                 # step 1 eagerly (also the warm-up)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        tr.step(x, y)                               # recorded, not executed
    for _ in range(5):
        graph.replay()
        torch.cuda.synchronize()
        losses.append(tr.loss.item())
    assert tr.adv[0].item() == 6                    # the step counter advanced on the device
    assert losses == eager_losses
    assert torch.equal(tr.params, eager.params)
