"""CPU oracle for the matmul hot path -- TEST INFRASTRUCTURE, not product code.

Only the tests, the smoke check and the benchmark's CPU-baseline leg import this
package.  It wraps oracle/cpu_matmul.c (a C restatement of the reference's
CpuKernels.MatMul2D / MatMulBatched, src/Tensotron/CpuKernels.cs:406-572) with
numpy-facing helpers, and composes the reference's op sequences for Linear
(src/Tensotron/Module.cs:100-105, src/Tensotron/TensorOps.LinearNT.cs:13-51) and
the MLP training step out of them.

Parity pinning: the C# reference cannot be built here, so the restatement is
pinned against the reference's torch golden fixtures (tests/golden/), not against
a run of the reference itself.
"""
import ctypes
import os

import numpy as np

from . import build as _build

_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_i32p = ctypes.POINTER(ctypes.c_int)
_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.build()
        L = ctypes.CDLL(path)
        L.oracle_matmul2d.argtypes = [_f32p, _f32p, _f32p] + [ctypes.c_int] * 7
        L.oracle_matmul2d_f64.argtypes = [_f32p, _f32p, _f64p] + [ctypes.c_int] * 7
        bat = [_f32p, _f32p, _f32p] + [ctypes.c_int] * 9 + [_i32p, _i32p, _i32p]
        L.oracle_matmul_batched.argtypes = bat
        L.oracle_matmul_batched_fast.argtypes = bat
        L.oracle_set_threads.argtypes = [ctypes.c_int]
        L.oracle_get_threads.restype = ctypes.c_int
        L.oracle_set_min_flops.argtypes = [ctypes.c_longlong]
        L.oracle_set_vector_width.argtypes = [ctypes.c_int]
        L.oracle_bias_add.argtypes = [_f32p, _f32p, _f32p, ctypes.c_int, ctypes.c_int]
        L.oracle_act_fwd.argtypes = [_f32p, _f32p, ctypes.c_longlong, ctypes.c_int]
        L.oracle_act_bwd.argtypes = [_f32p, _f32p, _f32p, _f32p, ctypes.c_longlong, ctypes.c_int]
        L.oracle_colsum.argtypes = [_f32p, _f32p, ctypes.c_int, ctypes.c_int]
        L.oracle_add_into.argtypes = [_f32p, _f32p, ctypes.c_longlong]
        L.oracle_cross_entropy.argtypes = [_f32p, _i32p, _f32p, ctypes.c_int, ctypes.c_int, ctypes.c_float]
        L.oracle_cross_entropy.restype = ctypes.c_float
        L.oracle_adam_step.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, ctypes.c_longlong] + \
            [ctypes.c_float] * 6 + [ctypes.c_int]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(_f32p)


def _ip(a):
    return a.ctypes.data_as(_i32p)


def _flat(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a.reshape(-1)


def set_threads(t):
    """TENSOTRON_CPU_THREADS (src/Tensotron/CpuSimdRuntime.cs:19-38): 'auto'/'max'
    resolve to the logical CPU count off Windows (src/Tensotron/CpuTopology.cs:19-30)."""
    if t in ("auto", "max"):
        t = os.cpu_count() or 1
    lib().oracle_set_threads(int(t))
    return lib().oracle_get_threads()


def matmul2d(a, b, M, N, K, aMs, aKs, bKs, bNs):
    """LaunchMatMul contract on flat float32 arrays -> C (M,N)."""
    a, b = _flat(a), _flat(b)
    c = np.empty(M * N, dtype=np.float32)
    if M * N:
        lib().oracle_matmul2d(_p(a), _p(b), _p(c), M, N, K, aMs, aKs, bKs, bNs)
    return c.reshape(M, N)


def matmul2d_f64(a, b, M, N, K, aMs, aKs, bKs, bNs):
    a, b = _flat(a), _flat(b)
    c = np.empty(M * N, dtype=np.float64)
    if M * N:
        lib().oracle_matmul2d_f64(_p(a), _p(b), c.ctypes.data_as(_f64p), M, N, K, aMs, aKs, bKs, bNs)
    return c.reshape(M, N)


def matmul_batched(a, b, M, N, K, aMs, aKs, bKs, bNs, batchDims, aBs, bBs, fast=False):
    """LaunchMatMulBatched contract -> C (batch..., M, N)."""
    a, b = _flat(a), _flat(b)
    bd = np.asarray(batchDims, dtype=np.int32).reshape(-1)
    abs_ = np.asarray(aBs, dtype=np.int32).reshape(-1)
    bbs_ = np.asarray(bBs, dtype=np.int32).reshape(-1)
    count = int(np.prod(bd)) if bd.size else 1
    c = np.empty(count * M * N, dtype=np.float32)
    fn = lib().oracle_matmul_batched_fast if fast else lib().oracle_matmul_batched
    if c.size:
        fn(_p(a), _p(b), _p(c), count, M, N, K, aMs, aKs, bKs, bNs, bd.size, _ip(bd), _ip(abs_), _ip(bbs_))
    return c.reshape(tuple(int(d) for d in bd) + (M, N))


def act_fwd(x, act):
    x = _flat(x)
    y = np.empty_like(x)
    lib().oracle_act_fwd(_p(x), _p(y), x.size, act)
    return y


def linear_fwd(x, w, bias, act):
    """Linear.Forward then the Activation module: MatMulNT (K,1,1,K) + Add(bias) + act.
    Returns (pre-activation z, output y), both (M,N)."""
    M, K = x.shape
    N = w.shape[0]
    z = matmul2d(x, w, M, N, K, K, 1, 1, K)
    if bias is not None:
        zb = np.empty(M * N, dtype=np.float32)
        lib().oracle_bias_add(_p(_flat(z)), _p(_flat(bias)), _p(zb), M, N)
        z = zb.reshape(M, N)
    y = act_fwd(z, act).reshape(M, N) if act else z
    return z, y


def linear_bwd(x, w, z, y, dy, act, need_dx=True):
    """Backward of act(Linear(x)): activation backward, bias grad (column sum in
    row order), dX = g.W (NN, TensorOps.LinearNT.cs:36), dW = g^T.X (TN, :44)."""
    M, K = x.shape
    N = w.shape[0]
    dy = _flat(dy)
    if act:
        g = np.empty(M * N, dtype=np.float32)
        lib().oracle_act_bwd(_p(_flat(z)), _p(_flat(y)), _p(dy), _p(g), M * N, act)
    else:
        g = dy
    db = np.empty(N, dtype=np.float32)
    lib().oracle_colsum(_p(g), _p(db), M, N)
    dx = matmul2d(g, w, M, K, N, N, 1, K, 1) if need_dx else None
    dw = matmul2d(g, x, N, K, M, 1, N, K, 1)
    return dx, dw, db, g.reshape(M, N)


def cross_entropy(logits, labels, scale=None):
    rows, classes = logits.shape
    lg = _flat(logits)
    lb = np.ascontiguousarray(labels, dtype=np.int32)
    d = np.empty(rows * classes, dtype=np.float32)
    if scale is None:
        scale = 1.0 / rows
    loss = lib().oracle_cross_entropy(_p(lg), _ip(lb), _p(d), rows, classes, scale)
    return float(loss), d.reshape(rows, classes)


def mse_loss(pred, target):
    """MseLoss, mean reduction (src/Tensotron/TensorOps.Losses.cs:29-61): per = (in - tgt)^2,
    loss = Sum(per) * (1 / count); backward with upstream gradient 1: (2 / count) * (in - tgt)."""
    pred = np.ascontiguousarray(pred, dtype=np.float32)
    target = np.ascontiguousarray(target, dtype=np.float32)
    diff = pred - target
    count = diff.size
    loss = np.float32(np.sum(diff * diff, dtype=np.float32) * np.float32(1.0 / count))
    return float(loss), (np.float32(2.0 / count) * diff).astype(np.float32)


def clip_grad_norm(grads, max_norm, eps=1e-6):
    """GradUtils.ClipGradNorm (src/Tensotron/Optimizers.cs:394-422), in place on a list of float32
    arrays: sumSq = sum over tensors of Sum(Square(g)); total = sqrt(sumSq);
    coef = clamp(maxNorm / (total + eps), 0, 1); every g *= coef (unconditionally).  Returns total."""
    sum_sq = None
    for g in grads:
        s = np.sum(np.square(g, dtype=np.float32), dtype=np.float32)
        sum_sq = s if sum_sq is None else np.float32(sum_sq + s)
    if sum_sq is None:
        return 0.0
    total = np.float32(np.sqrt(sum_sq))
    coef = np.float32(min(max(np.float32(max_norm) / (total + np.float32(eps)), np.float32(0.0)), np.float32(1.0)))
    for g in grads:
        g *= coef
    return float(total)


def _conv_out(size, k, stride, pad, dil):
    """ConvOutSize (src/Tensotron/TensorOps.Conv.cs:5-6)."""
    return (size + 2 * pad - dil * (k - 1) - 1) // stride + 1


def im2col(x, kh, kw, stride, pad, dil):
    """Kernels.Im2Col (src/Tensotron/Kernels.cs:784-801): (N,C,H,W) -> (N, C*kh*kw, Ho*Wo), padding
    positions read 0."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, c, h, w = x.shape
    ho, wo = _conv_out(h, kh, stride, pad, dil), _conv_out(w, kw, stride, pad, dil)
    col = np.zeros((n, c * kh * kw, ho * wo), dtype=np.float32)
    oh, ow = np.meshgrid(np.arange(ho), np.arange(wo), indexing="ij")
    for ci in range(c):
        for ki in range(kh):
            for kj in range(kw):
                ih = (oh * stride - pad + ki * dil).reshape(-1)
                iw = (ow * stride - pad + kj * dil).reshape(-1)
                ok = (ih >= 0) & (ih < h) & (iw >= 0) & (iw < w)
                k = (ci * kh + ki) * kw + kj
                col[:, k, ok] = x[:, ci, ih[ok], iw[ok]]
    return col


def col2im(gcol, shape, kh, kw, stride, pad, dil):
    """Kernels.Col2Im (src/Tensotron/Kernels.cs:803-814): scatter-add each column gradient back
    to its input pixel (the reference uses atomics; here every pixel adds its windows in k order)."""
    n, c, h, w = shape
    ho, wo = _conv_out(h, kh, stride, pad, dil), _conv_out(w, kw, stride, pad, dil)
    gx = np.zeros(shape, dtype=np.float32)
    oh, ow = np.meshgrid(np.arange(ho), np.arange(wo), indexing="ij")
    for ci in range(c):
        for ki in range(kh):
            for kj in range(kw):
                ih = (oh * stride - pad + ki * dil).reshape(-1)
                iw = (ow * stride - pad + kj * dil).reshape(-1)
                ok = (ih >= 0) & (ih < h) & (iw >= 0) & (iw < w)
                k = (ci * kh + ki) * kw + kj
                np.add.at(gx[:, ci], (slice(None), ih[ok], iw[ok]), gcol[:, k, ok])
    return gx


def conv2d_fwd(x, w, bias, stride=1, pad=0, dil=1):
    """TensorOps.Conv2d (src/Tensotron/TensorOps.Conv.cs:60-80): Im2Col, then the batched matmul of
    the weight (1, O, K) against the columns (N, K, L), then the broadcast bias add."""
    n = x.shape[0]
    o, c, kh, kw = w.shape
    col = im2col(x, kh, kw, stride, pad, dil)
    K, L = col.shape[1], col.shape[2]
    out = matmul_batched(w.reshape(o, K), col, o, L, K, K, 1, L, 1, [n], [0], [K * L], fast=True)
    if bias is not None:
        out = out + np.asarray(bias, dtype=np.float32).reshape(1, o, 1)
    ho, wo = _conv_out(x.shape[2], kh, stride, pad, dil), _conv_out(x.shape[3], kw, stride, pad, dil)
    return out.astype(np.float32).reshape(n, o, ho, wo)


def conv2d_bwd(x, w, dy, stride=1, pad=0, dil=1):
    """The gradients the reference's autograd chain produces for Conv2d: through the bias add
    (sum over batch and positions), the broadcast batched matmul (dW summed over the batch,
    src/Tensotron/TensorOps.MatMulND.cs:80-103) and Im2Col's backward (Col2Im)."""
    n = x.shape[0]
    o, c, kh, kw = w.shape
    col = im2col(x, kh, kw, stride, pad, dil)
    K, L = col.shape[1], col.shape[2]
    g = np.ascontiguousarray(dy, dtype=np.float32).reshape(n, o, L)
    dbias = g.sum(axis=(0, 2), dtype=np.float32)
    # dW[o][k] = sum_n sum_l g[n][o][l] * col[n][k][l]
    dw_n = matmul_batched(g, col, o, K, L, L, 1, 1, L, [n], [o * L], [K * L], fast=True)
    dw = dw_n.sum(axis=0, dtype=np.float32).reshape(w.shape)
    # dcol[n][k][l] = sum_o W[o][k] * g[n][o][l]
    dcol = matmul_batched(w.reshape(o, K), g, K, L, o, 1, K, L, 1, [n], [0], [o * L], fast=True)
    dx = col2im(dcol, x.shape, kh, kw, stride, pad, dil)
    return dx, dw, dbias


def adam_step(p, g, m, v, adv, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.0):
    """In place on float32 numpy arrays (all contiguous); adv = [t, ibc1, ibc2]."""
    lib().oracle_adam_step(_p(p.reshape(-1)), _p(_flat(g)), _p(m.reshape(-1)), _p(v.reshape(-1)),
                           _p(adv), p.size, b1, b2, lr, eps, wd, 1.0, 1)


class MlpOracle:
    """The reference's op sequence for a Sequential of Linear+ReLU layers with a
    final Linear, CrossEntropy(mean) and Adam: one training step on the CPU."""

    def __init__(self, weights, biases, lr=1e-3, act=1, loss="ce", max_grad_norm=0.0, clip_eps=1e-6):
        """act: 1 ReLU / 2 Tanh between the layers; loss "ce" (int labels) or "mse" (float
        target, the reference's captured step: examples/Tensotron.Examples/BenchExample.cs:163-176);
        max_grad_norm > 0: ClipGradNorm before the Adam step."""
        self.act, self.loss_kind = act, loss
        self.max_grad_norm, self.clip_eps = max_grad_norm, clip_eps
        self.w = [np.array(w, dtype=np.float32, copy=True) for w in weights]
        self.b = [np.array(b, dtype=np.float32, copy=True) for b in biases]
        self.lr = lr
        self.state = [(np.zeros_like(t), np.zeros_like(t), np.zeros(3, dtype=np.float32))
                      for t in self.w + self.b]

    def step(self, x, labels, apply_update=True):
        L = len(self.w)
        acts, zs = [np.ascontiguousarray(x, dtype=np.float32)], []
        for i in range(L):
            z, y = linear_fwd(acts[-1], self.w[i], self.b[i], self.act if i < L - 1 else 0)
            zs.append(z)
            acts.append(y)
        loss, g = cross_entropy(acts[-1], labels) if self.loss_kind == "ce" else mse_loss(acts[-1], labels)
        dws, dbs, gs = [None] * L, [None] * L, [None] * L
        for i in reversed(range(L)):
            dx, dw, db, gm = linear_bwd(acts[i], self.w[i], zs[i], acts[i + 1], g,
                                        self.act if i < L - 1 else 0, need_dx=i > 0)
            dws[i], dbs[i], gs[i] = dw, db, gm
            g = dx
        self.grads = dws + dbs
        self.acts, self.gs = acts, gs      # layer inputs and masked upstream gradients, for error bounds
        self.grad_norm = clip_grad_norm(self.grads, self.max_grad_norm, self.clip_eps) if self.max_grad_norm > 0 else None
        if apply_update:
            for t, gr, (m, v, adv) in zip(self.w + self.b, self.grads, self.state):
                adam_step(t, gr, m, v, adv, lr=self.lr)
        return loss
