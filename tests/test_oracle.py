"""CPU suite: pins the oracle against the reference's golden fixtures and checks its
internal consistency (path choice, threading, batched decode)."""
import numpy as np
import pytest

import oracle
from conftest import fixture_close, fp32_bound
from oracle_ops import matmul, matmul_backward


def _arr(t):
    return np.asarray(t["data"], dtype=np.float32).reshape(t["shape"])


@pytest.mark.parametrize("group", ["matmul", "matmul_nd"])
def test_oracle_matches_reference_matmul_fixtures(reference_fixtures, gemm_lib, group):
    cases = reference_fixtures["groups"][group]
    assert len(cases) == (4 if group == "matmul" else 6)
    for c in cases:
        a, b = (_arr(t) for t in c["inputs"])
        if c.get("meta") and c["meta"].get("op") == "outer":
            out = matmul(a.reshape(-1, 1), b.reshape(1, -1))
            dA, dB = matmul_backward(a.reshape(-1, 1), b.reshape(1, -1), _arr(c["grad_output"]))
            dA, dB = dA.reshape(a.shape), dB.reshape(b.shape)
        else:
            out = matmul(a, b)
            dA, dB = matmul_backward(a, b, _arr(c["grad_output"]))
        assert list(out.shape) == c["output"]["shape"], c["name"]
        fixture_close(out, c["output"]["data"])
        fixture_close(dA, c["grads"][0]["data"])
        fixture_close(dB, c["grads"][1]["data"])


def test_oracle_seeded_cases(seeded_cases, gemm_lib):
    idx, arrays = seeded_cases
    for c in idx["matmul"]:
        a, b = (arrays[n] for n in c["inputs"])
        g = arrays[c["grad_output"]]
        if c["layout"] == "NT":
            M, K = a.shape
            N = b.shape[0]
            out = oracle.matmul2d(a, b, M, N, K, K, 1, 1, K)
            dA = oracle.matmul2d(g, b, M, K, N, N, 1, K, 1)
            dB = oracle.matmul2d(g, a, N, K, M, 1, N, K, 1)
        else:
            out = matmul(a, b)
            dA, dB = matmul_backward(a, b, g)
        # tolerances of the reference's own tolerance tests (2e-3 abs is their loosest common one)
        np.testing.assert_allclose(out, arrays[c["output"]], atol=2e-3, rtol=2e-3)
        np.testing.assert_allclose(dA, arrays[c["grads"][0]], atol=3e-3, rtol=3e-3)
        np.testing.assert_allclose(dB, arrays[c["grads"][1]], atol=3e-3, rtol=3e-3)


def test_oracle_linear_cases(seeded_cases):
    idx, arrays = seeded_cases
    for c in idx["linear"]:
        x, w, b = (arrays[n] for n in c["inputs"])
        act = {"none": 0, "relu": 1, "tanh": 2}[c["act"]]
        z, y = oracle.linear_fwd(x, w, b, act)
        np.testing.assert_allclose(y, arrays[c["output"]], atol=1e-4, rtol=1e-4)
        dx, dw, db, _ = oracle.linear_bwd(x, w, z, y, arrays[c["grad_output"]], act)
        np.testing.assert_allclose(dx, arrays[c["grads"][0]], atol=2e-4, rtol=2e-4)
        np.testing.assert_allclose(dw, arrays[c["grads"][1]], atol=2e-4, rtol=2e-4)
        np.testing.assert_allclose(db, arrays[c["grads"][2]], atol=2e-4, rtol=2e-4)


@pytest.mark.parametrize("layout", ["NN", "NT", "TN", "TT"])
@pytest.mark.parametrize("shape", [(5, 7, 3), (33, 70, 65), (96, 112, 80), (1, 1, 1), (2, 3, 100)])
def test_oracle_paths_agree_with_f64(layout, shape):
    """Dot (NT), Axpy (NN/TN) and the scalar fallback (TT) all stay inside the FP32 bound."""
    M, N, K = shape
    rng = np.random.default_rng(M * 1000 + N * 10 + K)
    a = rng.uniform(-1, 1, M * K).astype(np.float32)
    b = rng.uniform(-1, 1, K * N).astype(np.float32)
    aMs, aKs = (K, 1) if layout[0] == "N" else (1, M)
    bKs, bNs = (N, 1) if layout[1] == "N" else (1, K)
    c = oracle.matmul2d(a, b, M, N, K, aMs, aKs, bKs, bNs)
    c64 = oracle.matmul2d_f64(a, b, M, N, K, aMs, aKs, bKs, bNs)
    assert np.abs(c - c64).max() <= fp32_bound(K, a, b)


def test_oracle_threaded_equals_serial_bitwise():
    """Row-parallel matmul is bit-identical to serial (src/Tensotron/CpuKernels.cs:413-415)."""
    rng = np.random.default_rng(3)
    M, N, K = 257, 130, 190
    a = rng.standard_normal(M * K).astype(np.float32)
    b = rng.standard_normal(K * N).astype(np.float32)
    for strides in ((K, 1, N, 1), (K, 1, 1, K), (1, M, N, 1)):
        oracle.set_threads(1)
        s = oracle.matmul2d(a, b, M, N, K, *strides)
        oracle.set_threads(4)
        t = oracle.matmul2d(a, b, M, N, K, *strides)
        oracle.set_threads(1)
        assert np.array_equal(s, t)


def test_oracle_batched_decode_and_fast_variant():
    rng = np.random.default_rng(5)
    a = rng.uniform(-1, 1, (3, 1, 6, 5)).astype(np.float32)
    b = rng.uniform(-1, 1, (1, 4, 5, 7)).astype(np.float32)
    dims, aBs, bBs = [3, 4], [30, 0], [0, 35]
    c = oracle.matmul_batched(a, b, 6, 7, 5, 5, 1, 7, 1, dims, aBs, bBs)
    np.testing.assert_allclose(c, a @ b, atol=1e-5)
    cf = oracle.matmul_batched(a, b, 6, 7, 5, 5, 1, 7, 1, dims, aBs, bBs, fast=True)
    np.testing.assert_allclose(cf, c, atol=1e-5)
    # empty batch / empty matrix
    assert oracle.matmul_batched(a, b, 0, 7, 5, 5, 1, 7, 1, dims, aBs, bBs).shape == (3, 4, 0, 7)
    assert oracle.matmul2d(a, b, 0, 3, 5, 5, 1, 3, 1).shape == (0, 3)


def test_oracle_nan_is_not_skipped():
    """0 * NaN must stay NaN on the Axpy path (src/Tensotron/CpuKernels.cs:525-526)."""
    a = np.zeros((2, 3), dtype=np.float32)
    b = np.ones((3, 4), dtype=np.float32)
    b[1, 2] = np.nan
    c = oracle.matmul2d(a, b, 2, 4, 3, 3, 1, 4, 1)
    assert np.isnan(c[:, 2]).all() and not np.isnan(c[:, 0]).any()


def test_oracle_support_ops_match_reference_fixtures(reference_fixtures):
    g = reference_fixtures["groups"]
    c = g["bias_add"][0]
    x, bias = (_arr(t) for t in c["inputs"])
    z, _ = oracle.linear_fwd(np.eye(3, dtype=np.float32)[:0].reshape(0, 3), np.zeros((3, 3), np.float32), None, 0)
    out = np.empty(x.size, dtype=np.float32)
    oracle.lib().oracle_bias_add(oracle._p(oracle._flat(x)), oracle._p(oracle._flat(bias)), oracle._p(out), *x.shape)
    fixture_close(out, c["output"]["data"])
    db = np.empty(3, dtype=np.float32)
    go = _arr(c["grad_output"])
    oracle.lib().oracle_colsum(oracle._p(oracle._flat(go)), oracle._p(db), *go.shape)
    fixture_close(db, c["grads"][1]["data"])

    for c in g["activation"]:
        act = 1 if c["meta"]["op"] == "relu" else 2
        x = _arr(c["inputs"][0])
        y = oracle.act_fwd(x, act)
        fixture_close(y, c["output"]["data"])
        gx = np.empty(x.size, dtype=np.float32)
        oracle.lib().oracle_act_bwd(oracle._p(oracle._flat(x)), oracle._p(y), oracle._p(oracle._flat(_arr(c["grad_output"]))),
                                    oracle._p(gx), x.size, act)
        fixture_close(gx, c["grads"][0]["data"])

    for c in g["cross_entropy"]:
        x = _arr(c["inputs"][0])
        labels = np.asarray(c["meta"]["index"], dtype=np.int32)
        scale = 1.0 / x.shape[0] if c["meta"]["reduction"] == "mean" else 1.0
        loss, d = oracle.cross_entropy(x, labels, scale)
        fixture_close([loss], c["output"]["data"])
        go = float(np.asarray(c["grad_output"]["data"]).reshape(-1)[0])
        fixture_close(d * go, c["grads"][0]["data"])

    for c in g["adam"]:
        cfg = c["meta"]["config"]
        p = _arr(c["inputs"][0]).copy()
        tgt = _arr(c["inputs"][1])
        m, v, adv = np.zeros_like(p), np.zeros_like(p), np.zeros(3, dtype=np.float32)
        for _ in range(int(cfg["steps"])):
            grad = p - tgt
            oracle.adam_step(p, grad, m, v, adv, lr=cfg["lr"], wd=cfg.get("weight_decay", 0.0))
        fixture_close(p, c["output"]["data"], atol=1e-3, rtol=1e-3)  # OptimizerTests.cs:24-50 tolerance


def test_mlp_oracle_step_decreases_loss():
    rng = np.random.default_rng(0)
    dims = [20, 32, 32, 5]
    ws = [rng.uniform(-1, 1, (dims[i + 1], dims[i])).astype(np.float32) / np.sqrt(dims[i]) for i in range(3)]
    bs = [np.zeros(dims[i + 1], dtype=np.float32) for i in range(3)]
    mlp = oracle.MlpOracle(ws, bs, lr=1e-2)
    x = rng.standard_normal((64, 20)).astype(np.float32)
    y = rng.integers(0, 5, 64).astype(np.int32)
    losses = [mlp.step(x, y) for _ in range(20)]
    assert losses[-1] < losses[0]
