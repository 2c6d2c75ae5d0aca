"""GPU parity: every product goes through the C-ABI library and is compared with the
CPU oracle on the same seeded inputs (strict FP32: max|err| <= 1e-5*sqrt(K)*max|A|*max|B|),
with the reference's golden fixtures, and -- at full benchmark sizes -- through
size-independent properties."""
import numpy as np
import pytest
import torch

import oracle
from conftest import fixture_close, fp32_bound
from tensotron_b200 import ops
from tensotron_b200.runtime import TensotronGemmError

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).cuda()


def _arr(t):
    return np.asarray(t["data"], dtype=np.float32).reshape(t["shape"])


def layout_strides(layout, M, N, K):
    aMs, aKs = (K, 1) if layout[0] == "N" else (1, M)
    bKs, bNs = (N, 1) if layout[1] == "N" else (1, K)
    return aMs, aKs, bKs, bNs


def run_matmul(rt, a, b, M, N, K, strides, variant=0):
    c = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    rt.SetVariant(variant)
    try:
        rt.LaunchMatMul(dev(a), dev(b), c, M, N, K, *strides)
        rt.Check()
    finally:
        rt.SetVariant(0)
    return c.cpu().numpy()


# ---- golden fixtures of the reference ------------------------------------------------

@pytest.mark.parametrize("group", ["matmul", "matmul_nd"])
def test_reference_fixtures_forward_and_grads(rt, reference_fixtures, group):
    for c in reference_fixtures["groups"][group]:
        a, b = (dev(_arr(t)) for t in c["inputs"])
        g = dev(_arr(c["grad_output"]))
        if c.get("meta") and c["meta"].get("op") == "outer":
            out = ops.Outer(a, b)
            dA, dB = ops.MatMulBackward(a.reshape(-1, 1), b.reshape(1, -1), g)
            dA, dB = dA.reshape(a.shape), dB.reshape(b.shape)
        else:
            out = ops.MatMul(a, b)
            dA, dB = ops.MatMulBackward(a, b, g)
        assert list(out.shape) == c["output"]["shape"], c["name"]
        fixture_close(out.cpu().numpy(), c["output"]["data"])
        fixture_close(dA.cpu().numpy(), c["grads"][0]["data"])
        fixture_close(dB.cpu().numpy(), c["grads"][1]["data"])


def test_seeded_golden_cases(rt, seeded_cases):
    """Shapes of TiledMatMulTests / MatMulNtOpTests / BatchedCuBlasMatMulTests."""
    idx, arrays = seeded_cases
    for c in idx["matmul"]:
        a, b = (dev(arrays[n]) for n in c["inputs"])
        g = dev(arrays[c["grad_output"]])
        if c["layout"] == "NT":
            out = ops.MatMulNT(a, b)
            dA, dB = ops.MatMulNTBackward(a, b, g)
        else:
            out = ops.MatMul(a, b)
            dA, dB = ops.MatMulBackward(a, b, g)
        np.testing.assert_allclose(out.cpu().numpy(), arrays[c["output"]], atol=2e-3, rtol=2e-3)
        np.testing.assert_allclose(dA.cpu().numpy(), arrays[c["grads"][0]], atol=3e-3, rtol=3e-3)
        np.testing.assert_allclose(dB.cpu().numpy(), arrays[c["grads"][1]], atol=3e-3, rtol=3e-3)


# ---- strict-FP32 parity with the oracle ---------------------------------------------

SHAPES = [(256, 256, 512),   # benchmark config 1
          (128, 128, 32), (129, 131, 36), (96, 112, 80), (64, 64, 128), (300, 260, 1000),
          (1, 512, 512), (512, 1, 512), (512, 512, 4), (8, 64, 64), (1, 1, 1), (5, 3, 7), (2, 4, 3)]


@pytest.mark.parametrize("variant", [0, 1, 2, 3, 7])
@pytest.mark.parametrize("layout", ["NN", "NT", "TN", "TT"])
@pytest.mark.parametrize("shape", SHAPES)
def test_matmul_matches_oracle(rt, shape, layout, variant):
    M, N, K = shape
    rng = np.random.default_rng(M * 1000003 + N * 1009 + K * 31 + ["NN", "NT", "TN", "TT"].index(layout))
    a = rng.uniform(-1, 1, M * K).astype(np.float32)
    b = rng.uniform(-1, 1, K * N).astype(np.float32)
    strides = layout_strides(layout, M, N, K)
    got = run_matmul(rt, a, b, M, N, K, strides, variant)
    exp = oracle.matmul2d(a, b, M, N, K, *strides)
    assert not np.isnan(got).any()
    assert np.abs(got - exp).max() <= fp32_bound(K, a, b)


def test_config1_uniform_seed0(rt):
    """A 256x512, B 512x256, uniform[-1,1) from seed 0, row-major (benchmark config 1)."""
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (256, 512)).astype(np.float32)
    b = rng.uniform(-1, 1, (512, 256)).astype(np.float32)
    exp = oracle.matmul2d(a, b, 256, 256, 512, 512, 1, 256, 1)
    for variant in (0, 1, 2, 3, 7):
        got = run_matmul(rt, a, b, 256, 256, 512, (512, 1, 256, 1), variant)
        assert np.abs(got - exp).max() <= fp32_bound(512, a, b)


@pytest.mark.parametrize("shape", [(256, 256, 512), (64, 64, 128), (64, 128, 64), (200, 36, 1000), (512, 512, 512), (100, 300, 4096)])
@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
def test_small_outputs_cut_k_across_a_cluster_in_one_launch(rt, shape, layout):
    """A few output tiles and a long K (benchmark config 1; the GEMMs of the small networks): the
    any-stride kernel cuts K across the CTAs of a thread-block cluster, which add their partial
    tiles through distributed shared memory in ascending k -- one launch, and the same bits as the
    two-launch form that adds the ranges through the workspace (variant 8)."""
    M, N, K = shape
    rng = np.random.default_rng(M + 2 * N + 3 * K)
    a = rng.uniform(-1, 1, M * K).astype(np.float32)
    b = rng.uniform(-1, 1, K * N).astype(np.float32)
    st = layout_strides(layout, M, N, K)
    rt.ResetCounters()
    one = run_matmul(rt, a, b, M, N, K, st, 0)
    stats = rt.Stats()
    assert stats["generic"] == 1 and stats["launches"] == 1, stats
    two = run_matmul(rt, a, b, M, N, K, st, 8)
    assert np.array_equal(one, two)
    exp = oracle.matmul2d(a, b, M, N, K, *st)
    assert np.abs(one - exp).max() <= fp32_bound(K, a, b)
    again = run_matmul(rt, a, b, M, N, K, st, 0)
    assert np.array_equal(one, again)


def test_tma_kernel_serves_aligned_shapes(rt):
    rng = np.random.default_rng(1)
    a = rng.uniform(-1, 1, (1024, 256)).astype(np.float32)
    b = rng.uniform(-1, 1, (256, 768)).astype(np.float32)
    rt.ResetCounters()
    run_matmul(rt, a, b, 1024, 768, 256, (256, 1, 768, 1))
    s = rt.Stats()
    # one GEMM launch, plus the split-K reduction when the plan cut K
    assert s["simt_tma"] == 1 and s["generic"] == 0 and s["launches"] == 1 + s["splitk"]


def test_bitwise_repeatable_and_grid_independent(rt):
    """Same inputs, two runs -> identical bits; forcing the other FP32 kernel keeps the
    result inside the bound (different tile shapes, same ascending-k order per output)."""
    rng = np.random.default_rng(2)
    M, N, K = 640, 384, 2048
    a = rng.standard_normal(M * K).astype(np.float32)
    b = rng.standard_normal(K * N).astype(np.float32)
    r1 = run_matmul(rt, a, b, M, N, K, (K, 1, N, 1), 2)
    r2 = run_matmul(rt, a, b, M, N, K, (K, 1, N, 1), 2)
    assert np.array_equal(r1, r2)
    r3 = run_matmul(rt, a, b, M, N, K, (K, 1, N, 1), 3)   # 128x128-tile kernel
    assert np.array_equal(r1, r3)  # both: one accumulator per output, ascending k, fused multiply-add
    # the any-stride kernel cuts K for this small grid (fixed-order partial sums): same bound, other bits
    r4 = run_matmul(rt, a, b, M, N, K, (K, 1, N, 1), 1)
    exp = oracle.matmul2d(a, b, M, N, K, K, 1, N, 1)
    assert np.abs(r4 - exp).max() <= fp32_bound(K, a, b)
    # without a cut along K (short K) the any-stride kernel also reproduces the bits
    a2, b2 = a[:M * 64].copy(), b[:64 * N].copy()
    assert np.array_equal(run_matmul(rt, a2, b2, M, N, 64, (64, 1, N, 1), 2),
                          run_matmul(rt, a2, b2, M, N, 64, (64, 1, N, 1), 1))


@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
@pytest.mark.parametrize("shape", [(256, 256, 2048), (128, 384, 4096), (512, 512, 1024), (130, 260, 1000), (1024, 1024, 1024)])
def test_split_k_matches_oracle_and_is_repeatable(rt, shape, layout):
    """Small M x N with long K: the automatic plan cuts K into ranges whose partial tiles are
    reduced in a fixed order by the last CTA of each tile (no atomics on data)."""
    M, N, K = shape
    rng = np.random.default_rng(M + 3 * N + 7 * K)
    a = rng.uniform(-1, 1, M * K).astype(np.float32)
    b = rng.uniform(-1, 1, K * N).astype(np.float32)
    st = layout_strides(layout, M, N, K)
    rt.ResetCounters()
    r1 = run_matmul(rt, a, b, M, N, K, st, 0)
    used_split = rt.Stats()["splitk"]
    r2 = run_matmul(rt, a, b, M, N, K, st, 0)
    assert np.array_equal(r1, r2)
    exp = oracle.matmul2d(a, b, M, N, K, *st)
    assert np.abs(r1 - exp).max() <= fp32_bound(K, a, b)
    if (M, N, K) == (256, 256, 2048) and M % 4 == 0:
        assert used_split == 1


@pytest.mark.parametrize("case", [
    # (M, N, K, aMs, aKs, bKs, bNs): the last MLP layer's backward (10 classes): leading
    # dimensions of 10 floats cannot be described by TMA, so the any-stride kernel serves them
    (8192, 4096, 10, 10, 1, 4096, 1),      # dx = g (8192x10) . W (10x4096)
    (10, 4096, 8192, 1, 10, 4096, 1),      # dW = g^T (10x8192) . x (8192x4096): split-K
    (64, 64, 4096, 4096, 1, 64, 1),        # one tile, long K
    (7, 5, 3000, 3000, 1, 1, 3000),        # ragged NT
])
def test_any_stride_kernel_skinny_and_split_k(rt, case):
    M, N, K, aMs, aKs, bKs, bNs = case
    rng = np.random.default_rng(M + N + K)
    a = rng.uniform(-1, 1, M * K).astype(np.float32)
    b = rng.uniform(-1, 1, K * N).astype(np.float32)
    r1 = run_matmul(rt, a, b, M, N, K, (aMs, aKs, bKs, bNs), 1)
    r2 = run_matmul(rt, a, b, M, N, K, (aMs, aKs, bKs, bNs), 1)
    assert np.array_equal(r1, r2)
    exp = oracle.matmul2d(a, b, M, N, K, aMs, aKs, bKs, bNs)
    assert np.abs(r1 - exp).max() <= fp32_bound(K, a, b)


@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
@pytest.mark.parametrize("shape", [(1024, 2048, 2048), (1000, 2052, 1028), (2048, 2048, 1024), (3072, 1536, 1056)])
def test_stream_k_matches_oracle_and_is_repeatable(rt, shape, layout):
    """Grids that would leave SMs idle in a partial last wave deal tiles x k-tiles units evenly
    to the CTAs; a tile shared by several CTAs is finished by the CTA that holds its first
    k-tiles, which adds the others' partial tiles in ascending k (one launch, no atomics)."""
    M, N, K = shape
    rng = np.random.default_rng(M + 3 * N + 7 * K)
    a = rng.uniform(-1, 1, M * K).astype(np.float32)
    b = rng.uniform(-1, 1, K * N).astype(np.float32)
    st = layout_strides(layout, M, N, K)
    rt.ResetCounters()
    r1 = run_matmul(rt, a, b, M, N, K, st, 6)      # 256x128 tiles, stream-K pinned
    stats = rt.Stats()
    assert stats["simt_tma"] == 1 and stats["splitk"] == 1 and stats["launches"] == 1, stats
    r2 = run_matmul(rt, a, b, M, N, K, st, 6)
    assert np.array_equal(r1, r2)
    r0 = run_matmul(rt, a, b, M, N, K, st, 0)      # whatever the plan picks
    oracle.set_threads("auto")
    exp = oracle.matmul2d(a, b, M, N, K, *st)
    oracle.set_threads(1)
    assert np.abs(r1 - exp).max() <= fp32_bound(K, a, b)
    assert np.abs(r0 - exp).max() <= fp32_bound(K, a, b)


@pytest.mark.parametrize("variant,shape", [
    (6, (512, 11392, 256)),     # 178 tiles of 256x128: less than half a wave behind the first one -> all of it dealt out as units
    (6, (1024, 12672, 256)),    # 396 tiles: two whole waves round-robin, 100 tiles dealt out as units
    (6, (1024, 10112, 264)),    # 316 tiles: one whole wave, 168 tiles as units (a tile and a bit per CTA); ragged K
    (9, (1024, 1024, 1024)),    # 64 tiles of 128x128 over 148 CTAs: up to three CTAs per tile
    (9, (900, 1156, 520)),      # ragged, 80 tiles
    (9, (2048, 2304, 512)),     # 288 tiles of 128x128: one whole wave + 140 tiles as units
])
def test_stream_k_behind_whole_waves(rt, variant, shape):
    """Multi-wave grids in stream-K mode: whole waves of tiles first (round-robin, as in the whole-tile
    mode), then the k-tile units of the remaining tiles in equal contiguous ranges.  Compared with
    the oracle on sampled rows and with the whole-tile kernel everywhere; bit-stable from run to run."""
    M, N, K = shape
    rng = np.random.default_rng(M + 3 * N + 7 * K)
    a = rng.uniform(-1, 1, M * K).astype(np.float32)
    b = rng.uniform(-1, 1, K * N).astype(np.float32)
    st = layout_strides("TN", M, N, K)             # both operands MN-major: no pre-transposition involved
    rt.ResetCounters()
    r1 = run_matmul(rt, a, b, M, N, K, st, variant)
    stats = rt.Stats()
    assert stats["simt_tma"] == 1 and stats["splitk"] == 1 and stats["launches"] == 1, stats
    r2 = run_matmul(rt, a, b, M, N, K, st, variant)
    assert np.array_equal(r1, r2)
    whole = run_matmul(rt, a, b, M, N, K, st, 2 if variant == 6 else 3)
    assert np.abs(r1 - whole).max() <= fp32_bound(K, a, b)
    rows = np.unique(np.concatenate([[0, M - 1], rng.integers(0, M, 24)]))
    am = a.reshape(K, M)[:, rows]                   # "T": stored (K, M)
    exp = am.T.astype(np.float64) @ b.reshape(K, N).astype(np.float64)
    assert np.abs(r1[rows] - exp).max() <= fp32_bound(K, a, b)
    rt.Check()


@pytest.mark.parametrize("layout,shape", [("NN", (1028, 1540, 1032)), ("NT", (2564, 1540, 1028)), ("NT", (1028, 1540, 1032)),
                                          ("NT", (508, 1540, 1032)), ("NT", (1028, 508, 1032)), ("NN", (300, 508, 1032))])
def test_large_k_major_operands_are_transposed_once_without_changing_a_bit(rt, layout, shape):
    """A large K-major operand is copied MN-major into the workspace before the FMA kernel runs
    (A when N >= 512, B when M >= 512, operands of at least 2^19 elements): one extra launch per
    transposed operand, same sums in the same order, so the result equals the untransposed run
    bit for bit."""
    M, N, K = shape
    rng = np.random.default_rng(M + N + K)
    a = rng.uniform(-1, 1, M * K).astype(np.float32)
    b = rng.uniform(-1, 1, K * N).astype(np.float32)
    st = layout_strides(layout, M, N, K)
    pinned = run_matmul(rt, a, b, M, N, K, st, 2)          # pinned variant: no pre-transposition
    rt.ResetCounters()
    auto = run_matmul(rt, a, b, M, N, K, st, 0)
    stats = rt.Stats()
    transposed = (1 if (N >= 512 and M * K >= 2 ** 19) else 0) + \
                 (1 if (layout == "NT" and M >= 512 and N * K >= 2 ** 19) else 0)
    # the transpositions, the GEMM, and the reduction kernel when the plan cut K (stream-K has none)
    assert stats["simt_tma"] == 1 and stats["launches"] - transposed in ((1, 2) if stats["splitk"] else (1,)), stats
    if not stats["splitk"]:
        assert np.array_equal(auto, pinned)                # stream-K / split-K would regroup the partial sums
    oracle.set_threads("auto")
    exp = oracle.matmul2d(a, b, M, N, K, *st)
    oracle.set_threads(1)
    assert np.abs(auto - exp).max() <= fp32_bound(K, a, b)


@pytest.mark.parametrize("case", [
    # (M, N, K, strides, expected launches): the 10-class output layer of the MLP config
    (8192, 10, 4096, (4096, 1, 1, 4096), 1),     # forward  y = x . W^T          (tiny N)
    (10, 4096, 8192, (1, 10, 4096, 1), 2),       # dW = g^T . x                   (tiny M, K cut into ranges)
    (1000, 1, 516, (516, 1, 1, 516), 1),         # matrix-vector
    (3, 260, 300, (300, 1, 260, 1), 1),          # tiny M, one k range
])
def test_tiny_dimension_kernels(rt, case):
    M, N, K, st, launches = case
    rng = np.random.default_rng(M * 3 + N * 5 + K * 7)
    a = rng.uniform(-1, 1, M * K).astype(np.float32)
    b = rng.uniform(-1, 1, K * N).astype(np.float32)
    rt.ResetCounters()
    r1 = run_matmul(rt, a, b, M, N, K, st, 0)
    stats = rt.Stats()
    assert stats["skinny"] == 1 and stats["launches"] <= 2, stats   # the tiny-M form may add its range reduction
    r2 = run_matmul(rt, a, b, M, N, K, st, 0)
    assert np.array_equal(r1, r2)
    exp = oracle.matmul2d(a, b, M, N, K, *st)
    assert np.abs(r1 - exp).max() <= fp32_bound(K, a, b)


@pytest.mark.parametrize("shape", [(8192, 10, 4096), (5000, 3, 1000), (4200, 16, 260), (9000, 12, 516), (6000, 1, 2048),
                                   (16384, 7, 128)])
def test_tall_tiny_n_stream_kernel(rt, shape):
    """Tall products with N <= 16 (at least half a wave of 56-row units) run on the TMA-fed stream:
    a persistent CTA per SM, A through a shared-memory ring.  Ragged M, K that is not a multiple of the
    128-k chunk, N = 1; against the oracle, the K-cut form (variant 10), and itself (bit-stable)."""
    M, N, K = shape
    rng = np.random.default_rng(M + 5 * N + 11 * K)
    a = rng.uniform(-1, 1, M * K).astype(np.float32)
    b = rng.uniform(-1, 1, K * N).astype(np.float32)
    st = (K, 1, 1, K)                                   # A (M, K) row-major, B stored (N, K)
    rt.ResetCounters()
    r1 = run_matmul(rt, a, b, M, N, K, st, 0)
    stats = rt.Stats()
    assert stats["skinny"] == 1 and stats["launches"] == 1, stats
    assert np.array_equal(r1, run_matmul(rt, a, b, M, N, K, st, 0))
    exp = oracle.matmul2d(a, b, M, N, K, *st)
    assert np.abs(r1 - exp).max() <= fp32_bound(K, a, b)
    cut = run_matmul(rt, a, b, M, N, K, st, 10)
    assert np.abs(r1 - cut).max() <= fp32_bound(K, a, b)


@pytest.mark.parametrize("case", [
    # (M, N, K, strides)
    (10, 4096, 8192, (1, 10, 4096, 1)),        # dW of the 10-class layer: g stored (K, 10), x (K, N)
    (16, 1024, 3000, (3000, 1, 1024, 1)),      # A stored (M, K); K not a multiple of the 32-k tile
    (3, 260, 300, (300, 1, 260, 1)),           # N just above one 256-column block
    (7, 772, 1000, (1, 7, 772, 1)),
    (12, 2048, 16384, (1, 12, 2048, 1)),       # k ranges capped by the slice buffer: more CTAs than one wave
])
def test_tiny_m_stream_kernel(rt, case):
    """Products with M <= 16 and a large K x N operand run on the TMA-fed stream (B through a
    shared-memory ring, the small operand's slice resident); against the oracle, the plain-load
    form (variant 10), and itself (bit-stable)."""
    M, N, K, st = case
    rng = np.random.default_rng(M * 3 + N * 5 + K * 7)
    a = rng.uniform(-1, 1, M * K).astype(np.float32)
    b = rng.uniform(-1, 1, K * N).astype(np.float32)
    rt.ResetCounters()
    r1 = run_matmul(rt, a, b, M, N, K, st, 0)
    stats = rt.Stats()
    assert stats["skinny"] == 1 and stats["launches"] <= 2, stats
    assert np.array_equal(r1, run_matmul(rt, a, b, M, N, K, st, 0))
    exp = oracle.matmul2d(a, b, M, N, K, *st)
    assert np.abs(r1 - exp).max() <= fp32_bound(K, a, b)
    plain = run_matmul(rt, a, b, M, N, K, st, 10)
    assert np.abs(r1 - plain).max() <= fp32_bound(K, a, b)


@pytest.mark.parametrize("case", [
    # (M, N, K, strides)
    (8192, 4096, 10, (10, 1, 4096, 1)),        # dX of the 10-class layer: g (M, 10) . W (10, N)
    (1000, 260, 3, (3, 1, 260, 1)),
    (64, 256, 16, (1, 64, 256, 1)),            # A stored (K, M)
    (5000, 1028, 7, (7, 1, 1028, 1)),
])
def test_tiny_k_kernel(rt, case):
    """Products with K <= 16 are bound by the write of C: one streaming kernel, B in registers,
    the A tile in shared memory.  Against the oracle and the any-stride kernel (variant 1); bit-stable."""
    M, N, K, st = case
    rng = np.random.default_rng(M * 3 + N * 5 + K * 7)
    a = rng.uniform(-1, 1, M * K).astype(np.float32)
    b = rng.uniform(-1, 1, K * N).astype(np.float32)
    rt.ResetCounters()
    r1 = run_matmul(rt, a, b, M, N, K, st, 0)
    stats = rt.Stats()
    assert stats["skinny"] == 1 and stats["launches"] == 1, stats
    assert np.array_equal(r1, run_matmul(rt, a, b, M, N, K, st, 0))
    exp = oracle.matmul2d(a, b, M, N, K, *st)
    assert np.abs(r1 - exp).max() <= fp32_bound(K, a, b)
    assert np.array_equal(r1, run_matmul(rt, a, b, M, N, K, st, 1))     # same sums in the same order


def test_nan_propagates_like_reference(rt):
    a = np.zeros((128, 64), dtype=np.float32)
    b = np.ones((64, 128), dtype=np.float32)
    b[5, 7] = np.nan
    for variant in (1, 2, 3):
        c = run_matmul(rt, a, b, 128, 128, 64, (64, 1, 128, 1), variant)
        assert np.isnan(c[:, 7]).all() and not np.isnan(c[:, 0]).any()


def test_empty_and_degenerate(rt):
    z = torch.zeros(16, device="cuda")
    rt.LaunchMatMul(z, z, z, 0, 4, 4, 4, 1, 4, 1)
    rt.LaunchMatMul(z, z, z, 4, 0, 4, 4, 1, 0, 1)
    c = torch.full((4, 4), 7.0, device="cuda")
    rt.LaunchMatMul(z, z, c, 4, 4, 0, 0, 1, 4, 1)   # K = 0 -> zeros
    rt.Check()
    assert (c == 0).all()
    with pytest.raises(TensotronGemmError):
        rt.LaunchMatMul(z, z, z, -1, 4, 4, 4, 1, 4, 1)
    with pytest.raises(TensotronGemmError):
        rt.LaunchMatMul(None, z, z, 4, 4, 4, 4, 1, 4, 1)
    with pytest.raises(TensotronGemmError):
        ops.MatMul(torch.zeros(2, 3, device="cuda"), torch.zeros(4, 5, device="cuda"))
    with pytest.raises(TensotronGemmError):
        ops.Bmm(torch.zeros(2, 3, 4, device="cuda"), torch.zeros(3, 4, 5, device="cuda"))


def test_unaligned_subview_goes_generic(rt):
    """An operand pointer that is not 16-byte aligned cannot use TMA: the any-stride kernel serves it."""
    rng = np.random.default_rng(4)
    M, N, K = 128, 128, 128
    abuf = dev(rng.uniform(-1, 1, M * K + 1))
    b = rng.uniform(-1, 1, K * N).astype(np.float32)
    c = torch.empty((M, N), device="cuda")
    rt.ResetCounters()
    rt.SetVariant(2)
    rt.LaunchMatMul(abuf.data_ptr() + 4, dev(b), c, M, N, K, K, 1, N, 1)
    rt.SetVariant(0)
    rt.Check()
    assert rt.Stats()["generic"] == 1
    a = abuf.cpu().numpy()[1:]
    exp = oracle.matmul2d(a, b, M, N, K, K, 1, N, 1)
    assert np.abs(c.cpu().numpy() - exp).max() <= fp32_bound(K, a, b)


# ---- batched ---------------------------------------------------------------------------

BATCH_CASES = [
    # (a shape, b shape, transposed-B storage)
    ((4, 2, 3), (4, 3, 5), False),
    ((3, 64, 64), (3, 64, 80), False),
    ((2, 1, 130, 36), (1, 3, 36, 132), False),
    ((2, 1, 128, 64), (1, 3, 64, 128), True),
    ((2, 3, 2, 40, 32), (3, 1, 32, 48), False),
    ((5, 128, 128), (128, 128), False),
]


@pytest.mark.parametrize("variant", [0, 1, 2, 3, 7])
@pytest.mark.parametrize("case", BATCH_CASES)
def test_batched_matches_scalar_oracle(rt, case, variant):
    a_shape, b_shape, bt = case
    rng = np.random.default_rng(len(a_shape) * 100 + a_shape[-1])
    a = rng.uniform(-1, 1, a_shape).astype(np.float32)
    b = rng.uniform(-1, 1, b_shape).astype(np.float32)
    M, K = a_shape[-2:]
    N = b_shape[-1]
    strides = lambda s: [int(np.prod(s[i + 1:])) for i in range(len(s))]
    from tensotron_b200.runtime import broadcast_batch
    dims, aBs, bBs = broadcast_batch(a_shape[:-2], strides(a_shape)[:-2], b_shape[:-2], strides(b_shape)[:-2])
    if bt:
        b_store = np.ascontiguousarray(np.swapaxes(b, -1, -2))   # stored [.., N, K]
        bKs, bNs = 1, K
    else:
        b_store, bKs, bNs = b, N, 1
    count = int(np.prod(dims))
    c = torch.full(tuple(dims) + (M, N), float("nan"), device="cuda")
    rt.SetVariant(variant)
    try:
        rt.LaunchMatMulBatched(dev(a), dev(b_store), c, count, M, N, K, K, 1, bKs, bNs, dims, aBs, bBs)
        rt.Check()
    finally:
        rt.SetVariant(0)
    exp = oracle.matmul_batched(a, b_store, M, N, K, K, 1, bKs, bNs, dims, aBs, bBs)
    assert np.abs(c.cpu().numpy() - exp).max() <= fp32_bound(K, a, b)


def test_bmm_config3_full_size_properties(rt):
    """A [32,1,384,256] x B [1,16,256,192] (benchmark config 3) at full size.  The scalar
    oracle checks a sample of batch entries; the whole output is checked through
    linearity in A and through the transposed-B variant giving identical bits."""
    g = torch.Generator(device="cpu").manual_seed(0)
    a = (torch.rand((32, 1, 384, 256), generator=g) * 2 - 1).cuda()
    g.manual_seed(1)
    b = (torch.rand((1, 16, 256, 192), generator=g) * 2 - 1).cuda()
    rt.ResetCounters()
    c = ops.MatMul(a, b)
    rt.Check()
    assert tuple(c.shape) == (32, 16, 384, 192)
    stats = rt.Stats()
    # one GEMM launch, not 512 library calls (plus the one-off transposition of the stacked A)
    assert stats["simt_tma"] == 1 and stats["launches"] <= 2, stats
    an, bn, cn = a.cpu().numpy(), b.cpu().numpy(), c.cpu().numpy()
    for (i, j) in [(0, 0), (31, 15), (7, 3), (16, 9)]:
        exp = oracle.matmul2d(an[i, 0], bn[0, j], 384, 192, 256, 256, 1, 192, 1)
        assert np.abs(cn[i, j] - exp).max() <= fp32_bound(256, an, bn)
    # transposed-B storage [1,16,192,256] read with bKs=1, bNs=256: same products, same k order
    bt = b.transpose(-1, -2).contiguous()
    ct = torch.empty_like(c)
    rt.LaunchMatMulBatched(a, bt, ct, 512, 384, 192, 256, 256, 1, 1, 256, [32, 16], [98304, 0], [0, 49152])
    rt.Check()
    assert torch.equal(c, ct)
    # linearity: (2A) B == 2 (A B) exactly in binary floating point
    c2 = ops.MatMul(a * 2, b)
    assert torch.equal(c2, c * 2)


@pytest.mark.parametrize("shapes", [
    ((6, 1, 130, 36), (1, 5, 36, 72)),          # each operand broadcast along one axis
    ((4, 96, 64), (64, 80)),                    # b has no batch axes: dB sums the whole batch
    ((3, 2, 1, 40, 32), (2, 4, 32, 48)),        # summed axis in the middle / leading
    ((2, 1, 3, 1, 16, 8), (1, 4, 1, 5, 8, 12)), # summed axes do not merge: unfused fallback
])
def test_broadcast_backward_fuses_the_batch_reduction(rt, shapes):
    """dA / dB of a broadcast matmul: RawBmm + ReduceGradToShape
    (src/Tensotron/TensorOps.MatMulND.cs:80-103) as one launch that sums the broadcast axis inside
    the k loop, in a fixed order."""
    a_shape, b_shape = shapes
    rng = np.random.default_rng(sum(a_shape) + sum(b_shape))
    a = rng.uniform(-1, 1, a_shape).astype(np.float32)
    b = rng.uniform(-1, 1, b_shape).astype(np.float32)
    out_shape = np.broadcast_shapes(a_shape[:-2], b_shape[:-2]) + (a_shape[-2], b_shape[-1])
    g = rng.uniform(-1, 1, out_shape).astype(np.float32)
    ad, bd_, gd = dev(a), dev(b), dev(g)
    rt.ResetCounters()
    dA, dB = ops.MatMulBackward(ad, bd_, gd)
    launches = rt.Stats()["launches"]
    rt.Check()
    dA2, dB2 = ops.MatMulBackward(ad, bd_, gd)
    assert torch.equal(dA, dA2) and torch.equal(dB, dB2)
    ta = torch.tensor(a, dtype=torch.float64, requires_grad=True)
    tb = torch.tensor(b, dtype=torch.float64, requires_grad=True)
    (ta @ tb).backward(torch.tensor(g, dtype=torch.float64))
    n_red_a = int(np.prod(out_shape[:-2])) // max(1, int(np.prod(a_shape[:-2])))
    n_red_b = int(np.prod(out_shape[:-2])) // max(1, int(np.prod(b_shape[:-2])))
    assert tuple(dA.shape) == a_shape and tuple(dB.shape) == b_shape
    assert np.abs(dA.cpu().numpy() - ta.grad.numpy()).max() <= fp32_bound(b_shape[-1] * n_red_a, g, b)
    assert np.abs(dB.cpu().numpy() - tb.grad.numpy()).max() <= fp32_bound(a_shape[-2] * n_red_b, a, g)
    if len(a_shape) < 6:
        assert launches == 2          # one fused launch per gradient, no full-batch temporary


# ---- Linear forward + backward -----------------------------------------------------------

def test_linear_golden_cases(rt, seeded_cases):
    """nn.Linear fwd+bwd, batch 64, 128 -> 64 (benchmark config 2): NN/NT/TN GEMMs + bias grad."""
    idx, arrays = seeded_cases
    for c in idx["linear"]:
        x, w, b = (arrays[n] for n in c["inputs"])
        lin = ops.Linear(128, 64, act=c["act"])
        lin.Weight, lin.Bias = dev(w), dev(b)
        xd, dy = dev(x), dev(arrays[c["grad_output"]])
        rt.ResetCounters()
        y = lin.Forward(xd)
        assert rt.Stats()["launches"] == 1       # Linear + bias + activation = one launch
        rt.ResetCounters()
        dx, dw, db = lin.Backward(xd, y, dy)
        rt.Check()
        assert rt.Stats()["launches"] == 1       # activation backward + bias gradient + dX + dW = one launch
        np.testing.assert_allclose(y.cpu().numpy(), arrays[c["output"]], atol=1e-4, rtol=1e-4)
        np.testing.assert_allclose(dx.cpu().numpy(), arrays[c["grads"][0]], atol=2e-4, rtol=2e-4)
        np.testing.assert_allclose(dw.cpu().numpy(), arrays[c["grads"][1]], atol=2e-4, rtol=2e-4)
        np.testing.assert_allclose(db.cpu().numpy(), arrays[c["grads"][2]], atol=2e-4, rtol=2e-4)
        # and against the oracle's restatement of the reference op sequence
        act = {"none": 0, "relu": 1, "tanh": 2}[c["act"]]
        z, yo = oracle.linear_fwd(x, w, b, act)
        dxo, dwo, dbo, _ = oracle.linear_bwd(x, w, z, yo, arrays[c["grad_output"]], act)
        assert np.abs(y.cpu().numpy() - yo).max() <= fp32_bound(128, x, w) + 1e-6
        assert np.abs(dw.cpu().numpy() - dwo).max() <= fp32_bound(64, arrays[c["grad_output"]], x)
        assert np.abs(db.cpu().numpy() - dbo).max() <= fp32_bound(64, arrays[c["grad_output"]], 1.0)


@pytest.mark.parametrize("shape", [(256, 512, 384, "relu"), (100, 36, 52, "tanh"), (33, 7, 5, "relu"), (1024, 10, 4096, "none"),
                                   (8192, 10, 512, "tanh"),      # tall, 10 outputs: the TMA-fed stream with bias + activation
                                   (256, 512, 10, "relu"),       # 10 inputs: the output-streaming kernel with bias + activation
                                   (16, 1024, 2048, "relu")])    # 16 rows: the tiny-M stream, epilogue in its range sum
def test_linear_matches_oracle(rt, shape):
    M, N, K, act = shape
    rng = np.random.default_rng(M + N + K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.uniform(-1, 1, (N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, N).astype(np.float32)
    dy = rng.standard_normal((M, N)).astype(np.float32)
    lin = ops.Linear(K, N, act=act)
    lin.Weight, lin.Bias = dev(w), dev(b)
    xd = dev(x)
    y = lin.Forward(xd)
    dx, dw, db = lin.Backward(xd, y, dev(dy))
    rt.Check()
    a = {"none": 0, "relu": 1, "tanh": 2}[act]
    z, yo = oracle.linear_fwd(x, w, b, a)
    dxo, dwo, dbo, g = oracle.linear_bwd(x, w, z, yo, dy, a)
    assert np.abs(y.cpu().numpy() - yo).max() <= fp32_bound(K, x, w) + 2e-6
    # backward uses the GPU's y; for tanh the oracle's y differs in the last ulp, covered by the bound
    assert np.abs(dx.cpu().numpy() - dxo).max() <= fp32_bound(N, g, w) + 1e-5
    assert np.abs(dw.cpu().numpy() - dwo).max() <= fp32_bound(M, g, x) + 1e-5
    assert np.abs(db.cpu().numpy() - dbo).max() <= fp32_bound(M, g, 1.0) + 1e-5
    # fixed-order bias gradient: bitwise repeatable
    _, _, db2 = lin.Backward(xd, y, dev(dy))
    assert torch.equal(db, db2)


# ---- MLP-step support ops -----------------------------------------------------------------

def test_cross_entropy_and_adam_reference_fixtures(rt, reference_fixtures):
    g = reference_fixtures["groups"]
    for c in g["cross_entropy"]:
        x = dev(_arr(c["inputs"][0]))
        labels = torch.tensor(c["meta"]["index"], dtype=torch.int32, device="cuda")
        scale = 1.0 / x.shape[0] if c["meta"]["reduction"] == "mean" else 1.0
        d = torch.empty_like(x)
        loss = torch.zeros(1, device="cuda")
        rt.LaunchSoftmaxCrossEntropy(x, labels, d, loss, x.shape[0], x.shape[1], scale)
        fixture_close(loss.cpu().numpy(), c["output"]["data"])
        go = float(np.asarray(c["grad_output"]["data"]).reshape(-1)[0])
        fixture_close(d.cpu().numpy() * go, c["grads"][0]["data"])
    for c in g["adam"]:
        cfg = c["meta"]["config"]
        p = dev(_arr(c["inputs"][0]))
        tgt = dev(_arr(c["inputs"][1]))
        m, v = torch.zeros_like(p), torch.zeros_like(p)
        adv = torch.zeros(3, device="cuda")
        for _ in range(int(cfg["steps"])):
            grad = p - tgt
            rt.LaunchAdam(p, grad, m, v, adv, p.numel(), lr=cfg["lr"], coupledWd=cfg.get("weight_decay", 0.0))
        fixture_close(p.cpu().numpy(), c["output"]["data"], atol=1e-3, rtol=1e-3)
        assert adv[0].item() == cfg["steps"]


def test_cross_entropy_large_matches_oracle(rt):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((8192, 10)).astype(np.float32) * 3
    y = rng.integers(0, 10, 8192).astype(np.int32)
    d = torch.empty((8192, 10), device="cuda")
    loss = torch.zeros(1, device="cuda")
    rt.LaunchSoftmaxCrossEntropy(dev(x), torch.from_numpy(y).cuda(), d, loss, 8192, 10, 1.0 / 8192)
    lo, do = oracle.cross_entropy(x, y)
    assert abs(loss.item() - lo) <= 1e-5 * max(1.0, abs(lo))
    np.testing.assert_allclose(d.cpu().numpy(), do, atol=1e-9, rtol=2e-5)


def test_cross_entropy_label_outside_the_classes_is_an_error_code_not_a_stray_read(rt):
    """The reference indexes with host int[] targets and throws on a bad one; here labels are on
    the device, so a label outside [0, classes) is never used as an index: the loss turns NaN
    and tt_check reports status 7."""
    from tensotron_b200 import runtime
    rng = np.random.default_rng(10)
    x = dev(rng.standard_normal((64, 10)) * 2)
    for bad in (10, -1, 2 ** 30):
        y = rng.integers(0, 10, 64).astype(np.int32)
        y[17] = bad
        yd = torch.from_numpy(y).cuda()
        d = torch.empty((64, 10), device="cuda")
        loss = torch.zeros(1, device="cuda")
        rt.LaunchSoftmaxCrossEntropy(x, yd, d, loss, 64, 10, 1.0 / 64)
        with pytest.raises(TensotronGemmError) as e:
            rt.Check()
        assert e.value.status == 7
        rt.Check()                                  # reported once, then cleared
        assert np.isnan(loss.item())
        assert torch.isfinite(d).all()              # the gradient is the plain softmax on that row
        # the allocation-free entry has no handle to report through: NaN loss only
        l2 = torch.zeros(1, device="cuda")
        runtime.softmax_cross_entropy_static(x, yd, None, l2, 64, 10, 1.0 / 64)
        torch.cuda.synchronize()
        assert np.isnan(l2.item())


def test_add_into(rt):
    a = torch.arange(1003, dtype=torch.float32, device="cuda")
    b = torch.ones(1003, device="cuda")
    rt.LaunchAddInto(a, b, 1003)
    assert torch.equal(a, torch.arange(1003, dtype=torch.float32, device="cuda") + 1)


def test_tensor_map_descriptors_are_cached_per_buffer_and_shape(rt):
    """The TMA descriptors of a call are a function of (pointer, dims, strides, box): the second
    call on the same buffers re-encodes nothing, another buffer or shape does."""
    M, N, K = 1024, 768, 256
    a = torch.randn(M, K, device="cuda")
    b = torch.randn(K, N, device="cuda")
    c = torch.empty(M, N, device="cuda")
    rt.LaunchMatMul(a, b, c, M, N, K, K, 1, N, 1)
    rt.ResetCounters()
    rt.LaunchMatMul(a, b, c, M, N, K, K, 1, N, 1)
    s = rt.Stats()
    assert s["simt_tma"] == 1 and s["tensor_map_misses"] == 0 and s["tensor_map_hits"] == 2, s
    # the same product read through another leading dimension: a new descriptor for A only
    a2 = torch.randn(M, K + 72, device="cuda")
    rt.LaunchMatMul(a2, b, c, M, N, K, K + 72, 1, N, 1)
    s = rt.Stats()
    assert s["tensor_map_misses"] == 1 and s["tensor_map_hits"] == 3, s
    rt.Check()
    a2h = a2.cpu().numpy()
    exp = oracle.matmul2d(a2h, b.cpu().numpy(), M, N, K, K + 72, 1, N, 1)
    assert np.abs(c.cpu().numpy() - exp).max() <= fp32_bound(K, a2h, b.cpu().numpy())


# ---- stream capture (the reference's native-graph contract) --------------------------------

def test_graph_capture_replays_with_new_inputs(rt):
    """TraceReplayTests.Native_cuda_graph_captures_cublas_gemm (batch/in/out = 128): the
    call records into a CUDA graph and replays against new buffer contents."""
    M = N = K = 128
    a = torch.randn(M, K, device="cuda")
    b = torch.randn(K, N, device="cuda")
    c = torch.empty(M, N, device="cuda")
    y = torch.empty(M, N, device="cuda")
    bias = torch.randn(N, device="cuda")
    rt.LaunchMatMul(a, b, c, M, N, K, K, 1, N, 1)       # warm-up outside capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        rt.LaunchMatMul(a, b, c, M, N, K, K, 1, N, 1)
        rt.LaunchLinearForward(c, b, bias, y, M, N, K, "relu")
    for _ in range(2):
        a.copy_(torch.randn(M, K, device="cuda"))
        graph.replay()
        torch.cuda.synchronize()
        exp = oracle.matmul2d(a.cpu().numpy(), b.cpu().numpy(), M, N, K, K, 1, N, 1)
        assert np.abs(c.cpu().numpy() - exp).max() <= fp32_bound(K, a.cpu().numpy(), b.cpu().numpy())
        _, yo = oracle.linear_fwd(c.cpu().numpy(), b.cpu().numpy(), bias.cpu().numpy(), 1)
        assert np.abs(y.cpu().numpy() - yo).max() <= fp32_bound(K, c.cpu().numpy(), b.cpu().numpy()) + 1e-5
