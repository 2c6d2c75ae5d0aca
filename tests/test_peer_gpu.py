"""GPU suite (one GPU): the peer-memory gradient exchange.  Several ranks are emulated inside
one process on one device: every rank has its own runtime handle and buffers, and the ranks'
calls are issued phase by phase on one stream, so each flag is set before the kernel that
waits for it runs (no kernel ever waits for a later launch)."""
import numpy as np
import pytest
import torch

from tensotron_b200.mlp import MlpTrainer, layer_layout, shard_rows
from tensotron_b200.peer import PeerGroup, exchange_plan
from tensotron_b200.runtime import TT_MATH_FP32, TT_MATH_TF32, TensorRuntime, TensotronGemmError

pytestmark = pytest.mark.gpu

DIMS = [512, 2048, 1024, 10]      # two partitioned layers (>= 1M weights), one replicated


def _data(batch, seed=0):
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.standard_normal((batch, DIMS[0])).astype(np.float32)).cuda()
    y = torch.from_numpy(rng.integers(0, DIMS[-1], batch).astype(np.int32)).cuda()
    return x, y


def _emulated_trainers(world, mode, variant=0):
    rts = [TensorRuntime(0) for _ in range(world)]
    for r in rts:
        r.SetVariant(variant)
    total = layer_layout(DIMS)[1]
    groups = PeerGroup.emulate(rts, total)
    return [MlpTrainer(DIMS, rt=rts[r], lr=1e-3, seed=5, math_mode=mode, exchange="peer", peer_group=groups[r])
            for r in range(world)]


def _emulated_step(trs, x, y, check=True):
    """One step of all emulated ranks, phase by phase in the order MlpTrainer.step() uses."""
    world, batch, L = len(trs), x.shape[0], trs[0].L
    shard = [x[slice(*shard_rows(batch, world, r))] for r in range(world)]
    for r, t in enumerate(trs):
        lo, hi = shard_rows(batch, world, r)
        t.forward(shard[r], y[lo:hi], batch)
    assert trs[0].pipelined
    for i in reversed(range(L)):
        for r, t in enumerate(trs):
            t.peer_backward_layer(shard[r], i)
            t.peer_push(i)
        if i + 1 < L:
            for t in trs:
                t.peer_update(i + 1)
    for t in trs:
        t.peer_update(0)
    for t in trs:
        t.peer_sync()
    for t in trs if check else []:
        t.rt.Check()


@pytest.mark.parametrize("mode,variant,fused", [(TT_MATH_FP32, 0, True), (TT_MATH_TF32, 0, True), (TT_MATH_FP32, 1, False)])
def test_scattered_weight_gradient_lands_in_the_owners_slots(mode, variant, fused):
    """After the backward phase, slot s on owner o holds rank s's gradient rows that o owns:
    compared with the same rank's whole gradient from the plain backward pass."""
    world, batch = 2, 512
    x, y = _data(batch)
    trs = _emulated_trainers(world, mode, variant)
    own_rows, owned, _ = exchange_plan(DIMS, world)
    try:
        for r, t in enumerate(trs):
            lo, hi = shard_rows(batch, world, r)
            t.forward(x[lo:hi], y[lo:hi], batch)
            for i in reversed(range(t.L)):
                t.peer_backward_layer(x[lo:hi], i)
            assert t.fused == [fused, fused, False]
        torch.cuda.synchronize()
        for r in range(world):
            lo, hi = shard_rows(batch, world, r)
            plain = MlpTrainer(DIMS, rt=trs[r].rt, lr=1e-3, seed=5, math_mode=mode)
            plain.step(x[lo:hi], y[lo:hi], global_batch=batch, apply_update=False)
            for o in range(world):
                slot = trs[o].peer.stage[r]              # what owner o received from rank r
                for off, ln in [s for lay in owned[o] for s in lay]:
                    got, want = slot[off:off + ln], plain.grads[off:off + ln]
                    tol = (1e-6 if mode == TT_MATH_FP32 else 2e-4) * float(want.abs().max())
                    assert float((got - want).abs().max()) <= tol
            trs[r].rt.Check()
    finally:
        for t in trs:
            t.close()


@pytest.mark.parametrize("mode", [TT_MATH_FP32, TT_MATH_TF32])
@pytest.mark.parametrize("world", [1, 2, 4])
def test_emulated_ranks_agree_bitwise_and_match_one_rank(mode, world):
    batch = 512
    x, y = _data(batch, seed=3)
    trs = _emulated_trainers(world, mode)
    ref = MlpTrainer(DIMS, rt=TensorRuntime(0), lr=1e-3, seed=5, math_mode=mode)
    try:
        for step in range(3):
            _emulated_step(trs, x, y)
            ref.step(x, y)
            for t in trs[1:]:
                assert torch.equal(t.params, trs[0].params)          # bit-identical on every rank
            d = (trs[0].params - ref.params).abs()
            # same bound as against the oracle: Adam may flip the sign of a noise-level gradient
            assert float(d.max()) <= 2.1 * 1e-3 * (step + 1)
            assert float(d.mean()) <= (0.02 if mode == TT_MATH_FP32 else 0.2) * 1e-3
            loss = sum(t.loss.item() for t in trs)
            assert abs(loss - ref.loss.item()) <= 2e-3 * max(1.0, abs(ref.loss.item()))
        assert all(t.adv[0].item() == 3 for t in trs)
    finally:
        for t in trs:
            t.close()


def test_world_one_peer_step_equals_plain_adam_bitwise_on_replicated_segments():
    """With one rank the reduce+Adam kernel does the arithmetic of the plain Adam kernel."""
    x, y = _data(256, seed=4)
    dims = [64, 128, 10]              # everything replicated: gradients come from the same kernels
    a = MlpTrainer(dims, rt=TensorRuntime(0), lr=1e-2, seed=9, exchange="peer")
    b = MlpTrainer(dims, rt=TensorRuntime(0), lr=1e-2, seed=9)
    try:
        for _ in range(5):
            a.step(x[:, :64].contiguous(), y)
            b.step(x[:, :64].contiguous(), y)
        assert torch.equal(a.params, b.params)
        assert a.loss.item() == b.loss.item()
    finally:
        a.close()


def test_a_wait_for_a_rank_that_never_signals_gives_up_with_an_error_code():
    x, y = _data(256, seed=5)
    trs = _emulated_trainers(2, TT_MATH_FP32)
    try:
        trs[0].peer.set_wait_limit(200)       # milliseconds
        trs[0].forward(x[:128], y[:128], 256)
        top = trs[0].L - 1
        trs[0].peer_backward_layer(x[:128], top)
        trs[0].peer_push(top)
        torch.cuda.synchronize()
        before = [t.clone() for t in (trs[0].params, trs[1].params, trs[0].m, trs[0].v, trs[0].adv)]
        trs[0].peer_update(top)               # rank 1 never pushed: the wait for its flag runs out
        with pytest.raises(TensotronGemmError) as e:
            trs[0].rt.Check()
        assert e.value.status == 5
        trs[0].rt.Check()                     # the status word was cleared; the context is still usable
        # the step that timed out touched nothing: no sum over a slot that never arrived, no Adam,
        # no store into any rank's parameters, no advance of the bias corrections
        after = (trs[0].params, trs[1].params, trs[0].m, trs[0].v, trs[0].adv)
        for b, a in zip(before, after):
            assert torch.equal(b, a)
    finally:
        for t in trs:
            t.close()


def test_exchange_step_replays_from_a_cuda_graph():
    """The step counter of the exchange lives in device memory, so a captured step (all phases of
    two emulated ranks on one stream) can be replayed: same bits as issuing the steps eagerly."""
    x, y = _data(512, seed=6)
    eager = _emulated_trainers(2, TT_MATH_FP32)
    graphed = _emulated_trainers(2, TT_MATH_FP32)
    try:
        for _ in range(4):
            _emulated_step(eager, x, y)
        _emulated_step(graphed, x, y)                      # warm-up: buffers allocated, step 1 done
        torch.cuda.synchronize()
        import gc
        gc.collect()                                       # no handle of an earlier test dies (and frees) mid-capture
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            _emulated_step(graphed, x, y, check=False)     # recorded, not run
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        for t in graphed:
            t.rt.Check()
        assert torch.equal(graphed[0].params, eager[0].params)
        assert torch.equal(graphed[1].params, graphed[0].params)
        assert graphed[0].adv[0].item() == 4
    finally:
        for t in eager + graphed:
            t.close()
