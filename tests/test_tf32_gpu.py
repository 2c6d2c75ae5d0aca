"""GPU parity of the tensor-core modes (tcgen05): AllowTf32 (math mode 3) and 3xTF32
(math mode 4) against the CPU oracle.  Tolerances are stated here, separately from the
strict-FP32 bound:
  TF32   : max|err| <= 2e-3 * sqrt(K) * max|A| * max|B|   (inputs truncated to a 10-bit mantissa)
  3xTF32 : max|err| <= 1e-5 * sqrt(K) * max|A| * max|B|  +  (3K/8) * 2^-23 * max|C|
           The first term is the strict-FP32 bound.  The second covers the tensor core's
           accumulator, which truncates (rounds toward zero) once per MMA instruction
           (K = 8 per instruction, three instructions per k-step), so that part of the error
           grows linearly in K instead of like sqrt(K).
"""
import numpy as np
import pytest
import torch

import oracle
from tensotron_b200.runtime import TT_MATH_3XTF32, TT_MATH_FP32, TT_MATH_TF32

pytestmark = pytest.mark.gpu

TOL = {TT_MATH_TF32: 2e-3, TT_MATH_3XTF32: 1e-5}


def bound(mode, K, a, b, exp):
    t = TOL[mode] * np.sqrt(K) * np.abs(a).max() * np.abs(b).max()
    if mode == TT_MATH_3XTF32:
        t += (3 * K / 8) * 2.0 ** -23 * np.abs(exp).max()
    return t


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


def strides(layout, M, N, K):
    aMs, aKs = (K, 1) if layout[0] == "N" else (1, M)
    bKs, bNs = (N, 1) if layout[1] == "N" else (1, K)
    return aMs, aKs, bKs, bNs


def run(rt, mode, variant, a, b, M, N, K, st):
    c = torch.full((M, N), float("nan"), device="cuda")
    rt.SetCuBlasMathMode(mode)
    rt.SetVariant(variant)
    try:
        rt.ResetCounters()
        rt.LaunchMatMul(dev(a), dev(b), c, M, N, K, *st)
        rt.Check()
        stats = rt.Stats()
    finally:
        rt.SetCuBlasMathMode(TT_MATH_FP32)
        rt.SetVariant(0)
    return c.cpu().numpy(), stats


SHAPES = [(128, 256, 32), (256, 256, 512), (512, 384, 1024), (136, 264, 40), (1000, 520, 72),
          (64, 64, 128), (4, 8, 8), (300, 1028, 2056)]


@pytest.mark.parametrize("mode", [TT_MATH_TF32, TT_MATH_3XTF32])
@pytest.mark.parametrize("variant", [4, 5])
@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
@pytest.mark.parametrize("shape", SHAPES)
def test_tensor_core_modes_match_oracle(rt, shape, layout, variant, mode):
    M, N, K = shape
    rng = np.random.default_rng(M * 7919 + N * 31 + K + ["NN", "NT", "TN"].index(layout))
    a = rng.uniform(-1, 1, M * K).astype(np.float32)
    b = rng.uniform(-1, 1, K * N).astype(np.float32)
    st = strides(layout, M, N, K)
    got, stats = run(rt, mode, variant, a, b, M, N, K, st)
    exp = oracle.matmul2d_f64(a, b, M, N, K, *st)
    assert not np.isnan(got).any()
    err = np.abs(got - exp).max()
    assert err <= bound(mode, K, a, b, exp), err
    aligned = (M % 4 == 0 or layout[0] == "N") and (N % 4 == 0 or layout[1] == "T") and K % 4 == 0
    if aligned:
        assert stats["tcgen05"] == 1, stats


def test_tf32_is_really_reduced_precision_and_3x_recovers(rt):
    """TF32 error is far above the FP32 error on the same inputs; 3xTF32 is back near it."""
    rng = np.random.default_rng(11)
    M = N = 512
    K = 2048
    a = rng.uniform(-1, 1, M * K).astype(np.float32)
    b = rng.uniform(-1, 1, K * N).astype(np.float32)
    st = (K, 1, N, 1)
    exp = oracle.matmul2d_f64(a, b, M, N, K, *st)
    e32 = np.abs(run(rt, TT_MATH_FP32, 0, a, b, M, N, K, st)[0] - exp).max()
    etf = np.abs(run(rt, TT_MATH_TF32, 0, a, b, M, N, K, st)[0] - exp).max()
    e3x = np.abs(run(rt, TT_MATH_3XTF32, 0, a, b, M, N, K, st)[0] - exp).max()
    print("max|err| fp32 %.3g  tf32 %.3g  3xtf32 %.3g" % (e32, etf, e3x))
    assert etf > 20 * e32
    assert e3x < etf / 20


def test_tensor_core_bitwise_repeatable(rt):
    rng = np.random.default_rng(12)
    M, N, K = 384, 512, 1024
    a = rng.standard_normal(M * K).astype(np.float32)
    b = rng.standard_normal(K * N).astype(np.float32)
    for mode in (TT_MATH_TF32, TT_MATH_3XTF32):
        r1, _ = run(rt, mode, 0, a, b, M, N, K, (K, 1, N, 1))
        r2, _ = run(rt, mode, 0, a, b, M, N, K, (K, 1, N, 1))
        assert np.array_equal(r1, r2)


def test_tensor_core_batched_and_linear(rt):
    from tensotron_b200 import ops
    rng = np.random.default_rng(13)
    a = rng.uniform(-1, 1, (3, 1, 128, 64)).astype(np.float32)
    b = rng.uniform(-1, 1, (1, 2, 64, 256)).astype(np.float32)
    rt.SetCuBlasMathMode(TT_MATH_TF32)
    try:
        rt.ResetCounters()
        c = ops.MatMul(dev(a), dev(b))
        x = rng.standard_normal((256, 128)).astype(np.float32)
        w = (rng.uniform(-1, 1, (512, 128)) / np.sqrt(128)).astype(np.float32)
        bias = rng.uniform(-0.1, 0.1, 512).astype(np.float32)
        lin = ops.Linear(128, 512, act="relu")
        lin.Weight, lin.Bias = dev(w), dev(bias)
        y = lin.Forward(dev(x))
        rt.Check()
        assert rt.Stats()["tcgen05"] == 2
    finally:
        rt.SetCuBlasMathMode(TT_MATH_FP32)
    exp = (a.astype(np.float64) @ b.astype(np.float64))
    assert np.abs(c.cpu().numpy() - exp).max() <= 2e-3 * np.sqrt(64)
    _, yo = oracle.linear_fwd(x, w, bias, 1)
    assert np.abs(y.cpu().numpy() - yo).max() <= 2e-3 * np.sqrt(128) * np.abs(x).max() * np.abs(w).max()
