"""The one-launch training step for small MLPs (tt_mlp_train_step) against the CPU oracle's
restatement of the reference step it replaces: Sequential(Linear, Tanh, Linear, Tanh, Linear) +
MseLoss + Backward + ClipGradNorm + Adam.Step (examples/Tensotron.Examples/BenchExample.cs:163-176;
network sizes of showcase/Tensotron.Showcase/Rl/ActorCritic.cs:21-32 and the replay sweep at
BenchExample.cs:140-146), plus the layer-by-layer entries it falls back to (tt_mse_loss,
tt_clip_grad_norm)."""
import numpy as np
import pytest
import torch

import oracle
from tensotron_b200.mlp import MlpTrainer
from tensotron_b200.runtime import TensotronGemmError

pytestmark = pytest.mark.gpu


def _oracle_from(tr, **kw):
    ws = [tr.weight(i).cpu().numpy().copy() for i in range(tr.L)]
    bs = [tr.bias(i).cpu().numpy().copy() for i in range(tr.L)]
    return oracle.MlpOracle(ws, bs, lr=tr.lr, **kw)


def _data(dims, batch, loss, seed):
    rng = np.random.default_rng(seed)
    x = (rng.random((batch, dims[0])) - 0.5).astype(np.float32)          # the reference's rand - 0.5 inputs
    if loss == "mse":
        t = (0.1 * rng.standard_normal((batch, dims[-1]))).astype(np.float32)
    else:
        t = rng.integers(0, dims[-1], batch).astype(np.int32)
    return x, t


CASES = [
    # dims, batch, act, loss, max_grad_norm
    ([8, 64, 64, 2], 1, "tanh", "mse", 0.5),       # ctrl-net-b1
    ([8, 64, 64, 2], 64, "tanh", "mse", 0.01),     # clip active
    ([8, 64, 64, 2], 512, "tanh", "mse", 0.5),     # ppo-b512 (a cluster of 16 CTAs)
    ([4, 32, 32, 1], 64, "tanh", "mse", 0.0),      # the critic; no clip
    ([4, 32, 32, 1], 100, "tanh", "mse", 0.02),    # rows do not divide evenly over the cluster
    ([20, 33, 47, 5], 50, "relu", "ce", 0.05),     # odd widths, cross-entropy
    ([10, 64, 64, 64, 7], 200, "relu", "ce", 0.0), # four layers
    ([6, 3], 17, "tanh", "mse", 0.0),              # a single layer
]


@pytest.mark.parametrize("case", CASES)
def test_fused_step_matches_oracle(rt, case):
    dims, batch, act, loss, clip = case
    tr = MlpTrainer(dims, rt=rt, lr=1e-2, seed=7, act=act, loss=loss, max_grad_norm=clip, fused=True)
    ref = _oracle_from(tr, act={"relu": 1, "tanh": 2}[act], loss=loss, max_grad_norm=clip)
    x, t = _data(dims, batch, loss, seed=batch)
    xd, td = torch.from_numpy(x).cuda(), torch.from_numpy(t).cuda()
    for step in range(3):
        rt.ResetCounters()
        got = tr.step(xd, td).item()
        rt.Check()
        assert tr.last_step_fused and rt.Stats()["launches"] == 1      # the whole step is one launch
        lo = ref.step(x, t)
        assert abs(got - lo) <= 2e-5 * max(1.0, abs(lo)) + 1e-7, (step, got, lo)
        if step == 0:
            # (clipped) gradients of the first step, element by element
            for i in range(tr.L):
                scale = max(np.abs(ref.grads[i]).max(), 1e-6)
                assert np.abs(tr.weight(i, tr.grads).cpu().numpy() - ref.grads[i]).max() <= 2e-5 * scale + 1e-7, i
                assert np.abs(tr.bias(i, tr.grads).cpu().numpy() - ref.grads[tr.L + i]).max() <= 2e-5 * scale + 1e-7, i
        # Parameters after Adam.  An element whose gradient is at rounding-noise level may step
        # +lr on one side and -lr on the other; everything else agrees closely.
        for i in range(tr.L):
            for a, b in ((tr.weight(i).cpu().numpy(), ref.w[i]), (tr.bias(i).cpu().numpy(), ref.b[i])):
                d = np.abs(a - b)
                assert d.max() <= 2.1 * tr.lr * (step + 1)
                assert np.mean(d) <= 0.02 * tr.lr
    assert tr.adv[0].item() == 3


def test_fused_step_equals_the_layer_by_layer_step_closely_and_repeats_bitwise(rt):
    dims, batch = [8, 64, 64, 2], 512
    x, t = _data(dims, batch, "mse", seed=3)
    xd, td = torch.from_numpy(x).cuda(), torch.from_numpy(t).cuda()
    runs = []
    for fused in (True, True, False):
        tr = MlpTrainer(dims, rt=rt, lr=1e-3, seed=11, act="tanh", loss="mse", max_grad_norm=0.5, fused=fused)
        losses = [tr.step(xd, td).item() for _ in range(10)]
        rt.Check()
        runs.append((losses, tr.params.clone(), tr.last_step_fused))
    assert runs[0][2] and runs[1][2] and not runs[2][2]
    assert runs[0][0] == runs[1][0] and torch.equal(runs[0][1], runs[1][1])       # bit-stable
    assert np.allclose(runs[0][0], runs[2][0], rtol=1e-4, atol=1e-7)
    assert float((runs[0][1] - runs[2][1]).abs().max()) <= 2.1e-3 * 10
    assert runs[0][0][-1] < runs[0][0][0]


def test_fused_step_replays_from_a_cuda_graph(rt):
    dims, batch = [8, 64, 64, 2], 64
    x, t = _data(dims, batch, "mse", seed=4)
    xd, td = torch.from_numpy(x).cuda(), torch.from_numpy(t).cuda()
    eager = MlpTrainer(dims, rt=rt, lr=1e-2, seed=5, act="tanh", loss="mse", max_grad_norm=0.5, fused=True)
    eager_losses = [eager.step(xd, td).item() for _ in range(6)]
    tr = MlpTrainer(dims, rt=rt, lr=1e-2, seed=5, act="tanh", loss="mse", max_grad_norm=0.5, fused=True)
    losses = [tr.step(xd, td).item()]
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        tr.step(xd, td)
    for _ in range(5):
        graph.replay()
        torch.cuda.synchronize()
        losses.append(tr.loss.item())
    assert tr.adv[0].item() == 6
    assert losses == eager_losses
    assert torch.equal(tr.params, eager.params)


def test_networks_outside_one_cluster_fall_back_or_say_so(rt):
    dims, batch = [128, 256, 256, 10], 256          # the reference's mlp-b256 sweep entry: too wide
    x, t = _data(dims, batch, "mse", seed=6)
    xd, td = torch.from_numpy(x).cuda(), torch.from_numpy(t).cuda()
    tr = MlpTrainer(dims, rt=rt, lr=1e-3, seed=1, act="tanh", loss="mse", max_grad_norm=0.5, fused=True)
    with pytest.raises(TensotronGemmError) as e:
        tr.step(xd, td)
    assert e.value.status == 3
    auto = MlpTrainer(dims, rt=rt, lr=1e-3, seed=1, act="tanh", loss="mse", max_grad_norm=0.5, fused="auto")
    ref = _oracle_from(auto, act=2, loss="mse", max_grad_norm=0.5)
    got = auto.step(xd, td).item()
    rt.Check()
    assert not auto.last_step_fused
    lo = ref.step(x, t)
    assert abs(got - lo) <= 2e-5 * max(1.0, abs(lo))
    for i in range(auto.L):
        d = np.abs(auto.weight(i).cpu().numpy() - ref.w[i])
        assert d.max() <= 2.1e-3 and d.mean() <= 2e-5


def test_mse_loss_and_clip_grad_norm_entries(rt):
    rng = np.random.default_rng(8)
    a = rng.standard_normal((300, 7)).astype(np.float32)
    b = rng.standard_normal((300, 7)).astype(np.float32)
    ad, bd = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    d, loss = torch.empty_like(ad), torch.zeros(1, device="cuda")
    rt.LaunchMseLoss(ad, bd, d, loss, a.size)
    lo, do = oracle.mse_loss(a, b)
    assert abs(loss.item() - lo) <= 1e-6 * max(1.0, abs(lo))
    np.testing.assert_allclose(d.cpu().numpy(), do, rtol=1e-6, atol=1e-9)
    for n, max_norm in ((100003, 5.0), (1000, 1e9), (5, 0.1)):
        g = rng.standard_normal(n).astype(np.float32)
        gd = torch.from_numpy(g).cuda()
        norm = torch.zeros(1, device="cuda")
        rt.LaunchClipGradNorm(gd, n, max_norm, 1e-6, norm)
        go = [g.copy()]
        total = oracle.clip_grad_norm(go, max_norm, 1e-6)
        assert abs(norm.item() - total) <= 1e-5 * total
        np.testing.assert_allclose(gd.cpu().numpy(), go[0], rtol=2e-5, atol=1e-9)
        gd2 = torch.from_numpy(g).cuda()
        rt.LaunchClipGradNorm(gd2, n, max_norm, 1e-6, None)
        assert torch.equal(gd, gd2)                                   # fixed-order sum: bit-stable
    rt.Check()
