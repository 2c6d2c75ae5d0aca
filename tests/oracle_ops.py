"""numpy + oracle emulation of the reference's matmul op surface (test infrastructure).

Same promotion / broadcast / backward logic as src/Tensotron/TensorOps.cs:211-279 and
src/Tensotron/TensorOps.MatMulND.cs:11-108, with every product computed by the CPU
oracle.  BroadcastBatch goes through the C-ABI host function so that logic is tested
without a GPU.
"""
import numpy as np

import oracle
from tensotron_b200.runtime import broadcast_batch


def _strides(shape):
    s, acc = [], 1
    for d in reversed(shape):
        s.append(acc)
        acc *= d
    return list(reversed(s))


def _mm2d(a, b):
    M, K = a.shape
    N = b.shape[1]
    return oracle.matmul2d(a, b, M, N, K, K, 1, N, 1)


def _mm2d_bwd(a, b, g):
    M, K = a.shape
    N = b.shape[1]
    dA = oracle.matmul2d(g, b, M, K, N, N, 1, 1, N)
    dB = oracle.matmul2d(a, g, K, N, M, 1, K, N, 1)
    return dA, dB


def _nd(a, b):
    M, K = a.shape[-2:]
    N = b.shape[-1]
    dims, aBs, bBs = broadcast_batch(a.shape[:-2], _strides(a.shape)[:-2], b.shape[:-2], _strides(b.shape)[:-2])
    return oracle.matmul_batched(a, b, M, N, K, K, 1, N, 1, dims, aBs, bBs)


def _reduce_to(g, shape):
    shape = tuple(shape)
    if g.shape == shape:
        return g.copy()
    r = g.ndim
    axes = tuple(j for j in range(r)
                 if (shape[j - (r - len(shape))] if j - (r - len(shape)) >= 0 else 1) != g.shape[j])
    return g.sum(axis=axes, keepdims=True, dtype=np.float32).reshape(shape)


def _nd_bwd(a, b, g):
    M, K = a.shape[-2:]
    N = b.shape[-1]
    a_s, b_s, g_s = _strides(a.shape), _strides(b.shape), _strides(g.shape)
    bd, gBs, bBs = broadcast_batch(g.shape[:-2], g_s[:-2], b.shape[:-2], b_s[:-2])
    dA = oracle.matmul_batched(g, b, M, K, N, g_s[-2], g_s[-1], b_s[-1], b_s[-2], bd, gBs, bBs)
    bd, aBs, gBs = broadcast_batch(a.shape[:-2], a_s[:-2], g.shape[:-2], g_s[:-2])
    dB = oracle.matmul_batched(a, g, K, N, M, a_s[-1], a_s[-2], g_s[-2], g_s[-1], bd, aBs, gBs)
    return _reduce_to(dA, a.shape), _reduce_to(dB, b.shape)


def matmul(a, b):
    if a.ndim == 2 and b.ndim == 2:
        return _mm2d(a, b)
    if a.ndim == 1 and b.ndim == 2:
        return _mm2d(a.reshape(1, -1), b).reshape(b.shape[1])
    if a.ndim == 2 and b.ndim == 1:
        return _mm2d(a, b.reshape(-1, 1)).reshape(a.shape[0])
    if a.ndim == 1 and b.ndim == 1:
        return _mm2d(a.reshape(1, -1), b.reshape(-1, 1)).reshape(())
    if a.ndim == 1:
        r = _nd(a.reshape(1, -1), b)
        return r.reshape(r.shape[:-2] + r.shape[-1:])
    if b.ndim == 1:
        r = _nd(a, b.reshape(-1, 1))
        return r.reshape(r.shape[:-1])
    return _nd(a, b)


def matmul_backward(a, b, g):
    if a.ndim == 2 and b.ndim == 2:
        return _mm2d_bwd(a, b, g)
    if a.ndim == 1 and b.ndim == 2:
        dA, dB = _mm2d_bwd(a.reshape(1, -1), b, g.reshape(1, -1))
        return dA.reshape(a.shape), dB
    if a.ndim == 2 and b.ndim == 1:
        dA, dB = _mm2d_bwd(a, b.reshape(-1, 1), g.reshape(-1, 1))
        return dA, dB.reshape(b.shape)
    if a.ndim == 1 and b.ndim == 1:
        dA, dB = _mm2d_bwd(a.reshape(1, -1), b.reshape(-1, 1), g.reshape(1, 1))
        return dA.reshape(a.shape), dB.reshape(b.shape)
    if a.ndim == 1:
        dA, dB = _nd_bwd(a.reshape(1, -1), b, np.ascontiguousarray(g.reshape(g.shape[:-1] + (1, g.shape[-1]))))
        return dA.reshape(a.shape), dB
    if b.ndim == 1:
        dA, dB = _nd_bwd(a, b.reshape(-1, 1), np.ascontiguousarray(g.reshape(g.shape + (1,))))
        return dA, dB.reshape(b.shape)
    return _nd_bwd(a, b, g)
