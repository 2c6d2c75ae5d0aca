"""GPU parity at the sizes the benchmark numbers are quoted on, in the spirit of the reference's
naive-loop checks of its large tiers (tests/Tensotron.Tests/TiledMatMulTests.cs:34-75,
tests/Tensotron.Tests/BatchedCuBlasMatMulTests.cs:55-118).

The small-shape parity tests run every CTA through exactly one output tile.  The persistent
kernels carry state from tile to tile (stage ring and phase bits, the accumulator double
buffer, the staging blocks of the TMA-store epilogue, stream-K hand-over), so these cases use
grids where every CTA gets several tiles and compare
  * a sample of rows (all columns) with the CPU oracle on the same inputs, at the bound of the
    math mode (strict FP32: 1e-5*sqrt(K)*max|A|*max|B|; TF32: 2e-3*...; 3xTF32: FP32 bound +
    (3K/8)*2^-23*max|C|), and
  * the WHOLE output of the tensor-core modes with the strict-FP32 kernel's output (itself
    oracle-checked) on the device, and a second run bit for bit.
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import fp32_bound
from tensotron_b200.runtime import TT_MATH_3XTF32, TT_MATH_FP32, TT_MATH_TF32, TensorRuntime

pytestmark = pytest.mark.gpu

TF32_TOL = 2e-3


@pytest.fixture(scope="module")
def big_rt(gemm_lib):
    """A handle with the benchmark's workspace (2.5 GiB): the pre-transposed copies of 16384^2
    operands and the hi/lo planes of 8192^2 operands live there."""
    rt = TensorRuntime(0, 2560 << 20)
    yield rt
    rt.Dispose()


def _uniform(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.rand(shape, generator=g, device="cuda") * 2 - 1


def _sample_rows(M, count=64):
    """Rows spread over every part of M: the first and last rows, tile edges, and a seeded spread."""
    rng = np.random.default_rng(M)
    fixed = [0, 1, 127, 128, 255, 256, M - 257, M - 129, M - 2, M - 1]
    fixed = [r for r in fixed if 0 <= r < M]
    rest = rng.choice(M, size=max(0, count - len(fixed)), replace=False).tolist()
    return np.array(sorted(set(fixed + rest)), dtype=np.int64)


def _mode_bound(mode, K, amax, bmax, cmax):
    if mode == TT_MATH_FP32:
        return 1e-5 * np.sqrt(K) * amax * bmax
    if mode == TT_MATH_TF32:
        return TF32_TOL * np.sqrt(K) * amax * bmax
    return 1e-5 * np.sqrt(K) * amax * bmax + (3 * K / 8) * 2.0 ** -23 * cmax


def _launch(rt, mode, variant, a, b, c, M, N, K, st):
    rt.SetCuBlasMathMode(mode)
    rt.SetVariant(variant)
    try:
        rt.ResetCounters()
        rt.LaunchMatMul(a, b, c, M, N, K, *st)
        rt.Check()
        return rt.Stats()
    finally:
        rt.SetCuBlasMathMode(TT_MATH_FP32)
        rt.SetVariant(0)


def _strides(layout, M, N, K):
    aMs, aKs = (K, 1) if layout[0] == "N" else (1, M)
    bKs, bNs = (N, 1) if layout[1] == "N" else (1, K)
    return aMs, aKs, bKs, bNs


def _rows_of_a(a_store, layout, rows):
    """The sampled rows of the logical (M, K) operand as a contiguous (rows, K) host array."""
    t = a_store[rows] if layout[0] == "N" else a_store[:, rows].t()
    return t.contiguous().cpu().numpy()


def _b_logical(b_store, layout):
    """The logical (K, N) operand as a contiguous host array."""
    t = b_store if layout[1] == "N" else b_store.t()
    return t.contiguous().cpu().numpy()


def _check_rows(got_rows, a_rows, b_kn, mode, K):
    """got_rows (r, N) against the oracle on those rows."""
    r, N = got_rows.shape
    if mode == TT_MATH_FP32:
        exp = oracle.matmul2d(a_rows, b_kn, r, N, K, K, 1, N, 1)
    else:
        exp = oracle.matmul2d_f64(a_rows, b_kn, r, N, K, K, 1, N, 1)
    err = float(np.abs(got_rows - exp).max())
    bound = _mode_bound(mode, K, np.abs(a_rows).max(), np.abs(b_kn).max(), np.abs(exp).max())
    assert not np.isnan(got_rows).any()
    assert err <= bound, (err, bound)
    return err, bound


# ---- tensor-core kernel on grids with several tiles per CTA ---------------------------------

# (M, N, K): with 128x256 tiles 1152 / 1353 tiles, with 256x256 tiles 576 / 693, on 148 CTAs
MULTI_WAVE = [(6144, 6144, 256), (5124, 8200, 520)]


@pytest.mark.parametrize("mode", [TT_MATH_TF32, TT_MATH_3XTF32])
@pytest.mark.parametrize("variant", [4, 5])
@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
@pytest.mark.parametrize("shape", MULTI_WAVE)
def test_tensor_core_kernel_over_several_tiles_per_cta(big_rt, shape, layout, variant, mode):
    rt = big_rt
    M, N, K = shape
    a = _uniform((M, K) if layout[0] == "N" else (K, M), 1000 + M)
    b = _uniform((K, N) if layout[1] == "N" else (N, K), 2000 + N)
    st = _strides(layout, M, N, K)
    c = torch.full((M, N), float("nan"), device="cuda")
    stats = _launch(rt, mode, variant, a, b, c, M, N, K, st)
    assert stats["tcgen05"] == 1, stats
    # sampled rows against the oracle
    rows = _sample_rows(M)
    _check_rows(c[rows].cpu().numpy(), _rows_of_a(a, layout, rows), _b_logical(b, layout), mode, K)
    # the whole output against the strict-FP32 kernel (oracle-checked itself, below and in
    # test_gemm_gpu.py), compared on the device
    c32 = torch.full((M, N), float("nan"), device="cuda")
    stats32 = _launch(rt, TT_MATH_FP32, 0, a, b, c32, M, N, K, st)
    assert stats32["tcgen05"] == 0
    _check_rows(c32[rows].cpu().numpy(), _rows_of_a(a, layout, rows), _b_logical(b, layout), TT_MATH_FP32, K)
    cmax = float(c32.abs().max())
    diff = float((c - c32).abs().max())
    assert not torch.isnan(c).any()
    assert diff <= _mode_bound(mode, K, 1.0, 1.0, cmax) + _mode_bound(TT_MATH_FP32, K, 1.0, 1.0, cmax), diff
    # bit-stable from run to run
    c2 = torch.empty_like(c)
    _launch(rt, mode, variant, a, b, c2, M, N, K, st)
    assert torch.equal(c, c2)


@pytest.mark.parametrize("mode", [TT_MATH_TF32, TT_MATH_3XTF32])
def test_bmm_config3_in_the_tensor_core_modes(big_rt, mode):
    """Benchmark config 3, A [32,1,384,256] x B [1,16,256,192] -> [32,16,384,192], one launch in
    TF32 / 3xTF32: sampled batch entries against the oracle, the whole output against strict
    FP32, the transposed-B storage variant, and a bitwise repeat."""
    rt = big_rt
    a = _uniform((32, 1, 384, 256), 0)
    b = _uniform((1, 16, 256, 192), 1)
    c = torch.full((32, 16, 384, 192), float("nan"), device="cuda")
    dims, aBs, bBs = [32, 16], [98304, 0], [0, 49152]

    def launch(m, b_store, bKs, bNs, out):
        rt.SetCuBlasMathMode(m)
        try:
            rt.ResetCounters()
            rt.LaunchMatMulBatched(a, b_store, out, 512, 384, 192, 256, 256, 1, bKs, bNs, dims, aBs, bBs)
            rt.Check()
            return rt.Stats()
        finally:
            rt.SetCuBlasMathMode(TT_MATH_FP32)

    stats = launch(mode, b, 192, 1, c)
    assert stats["tcgen05"] == 1 and stats["launches"] == (3 if mode == TT_MATH_3XTF32 else 1), stats
    an, bn = a.cpu().numpy(), b.cpu().numpy()
    for (i, j) in [(0, 0), (31, 15), (7, 3), (16, 9), (30, 1), (1, 14)]:
        exp = oracle.matmul2d_f64(an[i, 0], bn[0, j], 384, 192, 256, 256, 1, 192, 1)
        err = np.abs(c[i, j].cpu().numpy() - exp).max()
        assert err <= _mode_bound(mode, 256, 1.0, 1.0, np.abs(exp).max()), (i, j, err)
    c32 = torch.empty_like(c)
    launch(TT_MATH_FP32, b, 192, 1, c32)
    assert not torch.isnan(c).any()
    cmax = float(c32.abs().max())
    assert float((c - c32).abs().max()) <= _mode_bound(mode, 256, 1.0, 1.0, cmax) + _mode_bound(TT_MATH_FP32, 256, 1.0, 1.0, cmax)
    bt = b.transpose(-1, -2).contiguous()
    ct = torch.full_like(c, float("nan"))
    launch(mode, bt, 1, 256, ct)
    assert float((ct - c32).abs().max()) <= _mode_bound(mode, 256, 1.0, 1.0, cmax) + _mode_bound(TT_MATH_FP32, 256, 1.0, 1.0, cmax)
    c2 = torch.empty_like(c)
    launch(mode, b, 192, 1, c2)
    assert torch.equal(c, c2)


# ---- the benchmark's own calls ----------------------------------------------------------------

@pytest.mark.parametrize("mode", [TT_MATH_FP32, TT_MATH_TF32, TT_MATH_3XTF32])
def test_sgemm_8192_cubed_row_slab(big_rt, mode):
    """8192^3 (the size the north-star fractions are quoted on) in every math mode, automatic
    variant, as the benchmark calls it: sampled rows against the oracle."""
    rt = big_rt
    n = 8192
    a, b = _uniform((n, n), 11), _uniform((n, n), 12)
    c = torch.full((n, n), float("nan"), device="cuda")
    stats = _launch(rt, mode, 0, a, b, c, n, n, n, (n, 1, n, 1))
    assert (stats["tcgen05"] == 1) == (mode != TT_MATH_FP32), stats
    rows = _sample_rows(n)
    b_host = b.cpu().numpy()
    _check_rows(c[rows].cpu().numpy(), a[rows].cpu().numpy(), b_host, mode, n)
    # every row block holds finite numbers of the right magnitude (a missed tile would stay NaN)
    assert not torch.isnan(c).any()
    c2 = torch.empty_like(c)
    _launch(rt, mode, 0, a, b, c2, n, n, n, (n, 1, n, 1))
    assert torch.equal(c, c2)


@pytest.mark.parametrize("rows_per_gpu", [16384, 2048])
def test_headline_16384_wide_call_row_slab(big_rt, rows_per_gpu):
    """The headline call: C = A.B with A (rows, 16384), B 16384^2, strict FP32, automatic variant
    (A transposed once into the workspace, 256x128 whole tiles).  rows = 16384 is the 1-GPU
    step, 2048 the 8-GPU rank's shard."""
    rt = big_rt
    n, M = 16384, rows_per_gpu
    a, b = _uniform((M, n), 21), _uniform((n, n), 22)
    c = torch.full((M, n), float("nan"), device="cuda")
    stats = _launch(rt, TT_MATH_FP32, 0, a, b, c, M, n, n, (n, 1, n, 1))
    assert stats["simt_tma"] == 1, stats
    rows = _sample_rows(M, 48)
    _check_rows(c[rows].cpu().numpy(), a[rows].cpu().numpy(), b.cpu().numpy(), TT_MATH_FP32, n)
    assert not torch.isnan(c).any()


def test_mlp_step_at_full_width_1024_rows(big_rt):
    """One training step of the benchmark network 784-4096-4096-4096-10 on 1024 rows (the 8-GPU
    rank's share of the 8192 batch: stream-K GEMMs and the tiny-N kernels) against the oracle's
    restatement of the reference op sequence."""
    from tensotron_b200.mlp import MlpTrainer
    rt = big_rt
    dims, batch = [784, 4096, 4096, 4096, 10], 1024
    tr = MlpTrainer(dims, rt=rt, lr=1e-3, seed=2)
    ws = [tr.weight(i).cpu().numpy().copy() for i in range(tr.L)]
    bs = [tr.bias(i).cpu().numpy().copy() for i in range(tr.L)]
    ref = oracle.MlpOracle(ws, bs, lr=1e-3)
    oracle.set_threads("auto")
    rng = np.random.default_rng(0)
    x = rng.standard_normal((batch, dims[0])).astype(np.float32)
    y = rng.integers(0, 10, batch).astype(np.int32)
    loss = tr.step(torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()).item()
    rt.Check()
    lo = ref.step(x, y)
    assert abs(loss - lo) <= 2e-5 * max(1.0, abs(lo)), (loss, lo)
    # Yardstick for the gradients: the oracle against itself with another SIMD width (4 lanes
    # instead of 8), i.e. the same arithmetic in another summation order.  At initialisation the
    # gradients nearly cancel, rounding differences are handed down through three 4096-wide
    # layers, and a pre-activation within an ulp of zero may pass the ReLU on one side and not on
    # the other (one g element then changes by its full value), so the strict-FP32 bound of a
    # single product does not apply to the deep layers.  The CUDA path must differ from the
    # oracle by no more than a small multiple of what the oracle differs from itself.
    alt = oracle.MlpOracle(ws, bs, lr=1e-3)
    oracle.lib().oracle_set_vector_width(4)
    try:
        alt.step(x, y, apply_update=False)
    finally:
        oracle.lib().oracle_set_vector_width(8)
    for i in range(tr.L):
        g_i, a_i = ref.gs[i], ref.acts[i]
        loose = 2 * float(np.abs(g_i).max() * np.abs(a_i).max())       # one flipped ReLU
        for got, want, other in ((tr.weight(i, tr.grads).cpu().numpy(), ref.grads[i], alt.grads[i]),
                                 (tr.bias(i, tr.grads).cpu().numpy(), ref.grads[tr.L + i], alt.grads[tr.L + i])):
            d = np.abs(got - want)
            noise = float(np.abs(other - want).mean())
            single = fp32_bound(batch, g_i, a_i)                        # bound of this one product
            assert d.max() <= loose, (i, d.max(), loose)
            assert d.mean() <= 4 * noise + single, (i, float(d.mean()), noise, single)
        for got, want in ((tr.weight(i).cpu().numpy(), ref.w[i]), (tr.bias(i).cpu().numpy(), ref.b[i])):
            d = np.abs(got - want)
            # Adam normalises each element: one whose gradient is at rounding-noise level may step
            # +lr on one side and -lr on the other; everything else agrees closely
            assert d.max() <= 2.1 * tr.lr
            assert np.mean(d) <= 0.02 * tr.lr
    tr.close()
