"""Conv2d through the batched GEMM engine (tt_conv2d_fwd / tt_conv2d_bwd) against the reference's
own conv fixtures (tests/Tensotron.Tests/Fixtures/conv.json: forward and all gradients at the
reference tolerance) and against the CPU oracle's restatement of Im2Col + batched matmul + bias
(src/Tensotron/TensorOps.Conv.cs:60-80) on larger seeded cases."""
import numpy as np
import pytest
import torch

import oracle
from conftest import fixture_close, fp32_bound
from tensotron_b200 import ops
from tensotron_b200.runtime import TT_MATH_FP32, TT_MATH_TF32, TensorRuntime, TensotronGemmError

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


def _arr(t):
    return np.asarray(t["data"], dtype=np.float32).reshape(t["shape"])


def test_reference_conv_fixtures_forward_and_grads(rt, reference_fixtures):
    for c in reference_fixtures["groups"]["conv2d"]:
        cfg = c["meta"]["config"]
        ins = [_arr(t) for t in c["inputs"]]
        x, w = dev(ins[0]), dev(ins[1])
        b = dev(ins[2]) if len(ins) > 2 else None
        kw = dict(stride=cfg["stride"], padding=cfg["padding"], dilation=cfg["dilation"])
        y = ops.Conv2d(x, w, b, **kw)
        assert list(y.shape) == c["output"]["shape"], c["name"]
        fixture_close(y.cpu().numpy(), c["output"]["data"])
        dx, dw, db = ops.Conv2dBackward(x, w, dev(_arr(c["grad_output"])), has_bias=b is not None, **kw)
        rt.Check()
        fixture_close(dx.cpu().numpy(), c["grads"][0]["data"])
        fixture_close(dw.cpu().numpy(), c["grads"][1]["data"])
        if b is not None:
            fixture_close(db.cpu().numpy(), c["grads"][2]["data"])


CASES = [
    # n, c, h, w, o, k, stride, pad, dil
    (8, 16, 28, 28, 32, 3, 1, 1, 1),     # L = 784: the TMA-fed kernels serve every product
    (4, 3, 33, 31, 10, 5, 2, 2, 1),      # odd sizes, L = 255: the any-stride kernel
    (2, 8, 16, 16, 24, 3, 1, 2, 2),      # dilation
    (16, 1, 28, 28, 8, 3, 1, 0, 1),      # one input channel (K = 9)
]


@pytest.mark.parametrize("case", CASES)
def test_conv2d_matches_oracle(rt, case):
    n, c, h, w, o, k, stride, pad, dil = case
    rng = np.random.default_rng(n * 1000 + c * 100 + o)
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wt = (rng.uniform(-1, 1, (o, c, k, k)) / np.sqrt(c * k * k)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, o).astype(np.float32)
    xd, wd, bd = dev(x), dev(wt), dev(b)
    rt.ResetCounters()
    y = ops.Conv2d(xd, wd, bd, stride, pad, dil)
    assert rt.Stats()["launches"] <= 4            # im2col, weight packing, one batched GEMM (+ a transposition)
    yo = oracle.conv2d_fwd(x, wt, b, stride, pad, dil)
    K = c * k * k
    assert y.shape == yo.shape
    assert np.abs(y.cpu().numpy() - yo).max() <= fp32_bound(K + 1, x, wt) + 1e-6
    g = rng.standard_normal(yo.shape).astype(np.float32)
    dx, dw, db = ops.Conv2dBackward(xd, wd, dev(g), stride, pad, dil)
    rt.Check()
    dxo, dwo, dbo = oracle.conv2d_bwd(x, wt, g, stride, pad, dil)
    L = yo.shape[2] * yo.shape[3]
    assert np.abs(dx.cpu().numpy() - dxo).max() <= k * k * fp32_bound(o, g, wt) + 1e-6
    assert np.abs(dw.cpu().numpy() - dwo).max() <= fp32_bound(n * L, g, x)
    assert np.abs(db.cpu().numpy() - dbo).max() <= fp32_bound(n * L, g, 1.0)
    # fixed summation orders everywhere (no atomics): a second run gives the same bits
    dx2, dw2, db2 = ops.Conv2dBackward(xd, wd, dev(g), stride, pad, dil)
    assert torch.equal(dx, dx2) and torch.equal(dw, dw2) and torch.equal(db, db2)
    # without a bias and without dx
    y0 = ops.Conv2d(xd, wd, None, stride, pad, dil)
    assert np.abs(y0.cpu().numpy() - oracle.conv2d_fwd(x, wt, None, stride, pad, dil)).max() <= fp32_bound(K, x, wt) + 1e-6
    _, dw3, none = ops.Conv2dBackward(xd, wd, dev(g), stride, pad, dil, need_dx=False, has_bias=False)
    assert none is None and torch.equal(dw3, dw)


def test_conv2d_in_tf32_mode_and_argument_errors(rt):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((8, 16, 28, 28)).astype(np.float32)
    wt = (rng.uniform(-1, 1, (32, 16, 3, 3)) / 12).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, 32).astype(np.float32)
    yo = oracle.conv2d_fwd(x, wt, b, 1, 1, 1)
    rt.SetCuBlasMathMode(TT_MATH_TF32)
    try:
        rt.ResetCounters()
        y = ops.Conv2d(dev(x), dev(wt), dev(b), 1, 1, 1)
        rt.Check()
        assert rt.Stats()["tcgen05"] == 1
    finally:
        rt.SetCuBlasMathMode(TT_MATH_FP32)
    assert np.abs(y.cpu().numpy() - yo).max() <= 2e-3 * np.sqrt(145) * np.abs(x).max() * np.abs(wt).max()
    with pytest.raises(TensotronGemmError):
        ops.Conv2d(dev(x), dev(wt[:, :8]), None)                     # channel mismatch
    with pytest.raises(TensotronGemmError):
        ops.Conv2d(dev(x[:, :, :2, :2]), dev(wt), None)              # kernel larger than the image
    small = TensorRuntime(0, 1 << 20)                                 # 1 MiB workspace: the columns do not fit
    try:
        from tensotron_b200.runtime import Conv2dDesc
        d = Conv2dDesc(8, 16, 28, 28, 32, 3, 3, 1, 1, 1)
        assert TensorRuntime.Conv2dWorkspace(d) > (1 << 20)
        with pytest.raises(TensotronGemmError) as e:
            small.LaunchConv2dForward(d, dev(x), dev(wt), None, torch.empty((8, 32, 28, 28), device="cuda"))
        assert e.value.status == 4
    finally:
        small.Dispose()
