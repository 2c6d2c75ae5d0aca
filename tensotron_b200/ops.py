"""Host-side mirror of the reference's matmul op surface, on top of TensorRuntime.

Follows src/Tensotron/TensorOps.cs:211-279 (MatMul rank promotion, MatMul2D and its
stride-swap backward), src/Tensotron/TensorOps.MatMulND.cs:11-132 (batch broadcast,
RawBmm, batched backward, Bmm/Mv/Dot/Outer), src/Tensotron/TensorOps.LinearNT.cs:13-51
(MatMulNT) and src/Tensotron/Module.cs:82-112 (Linear).  Tensors are contiguous
float32 torch CUDA tensors used purely as device buffers; every product goes through
the C-ABI library.  Backward functions return the gradients the reference's GradNode
closures would hand to AddGrad.
"""
import math

import torch

from .runtime import ACT, Conv2dDesc, TensorRuntime, TensotronGemmError, broadcast_batch

_runtime = {}


def runtime(device=None):
    """Process-wide runtime per device (TensorRuntime.Instance, src/Tensotron/TensorRuntime.cs:49-50)."""
    if device is None:
        device = torch.cuda.current_device()
    if device not in _runtime:
        _runtime[device] = TensorRuntime(device)
    return _runtime[device]


def _strides(shape):
    s, acc = [], 1
    for d in reversed(shape):
        s.append(acc)
        acc *= d
    return list(reversed(s))


def _check(t):
    if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
        raise TensotronGemmError(1, "operands must be contiguous float32 CUDA tensors")


# ---- 2-D ---------------------------------------------------------------------------

def _matmul2d(a, b):
    M, K = a.shape
    K2, N = b.shape
    if K != K2:
        raise TensotronGemmError(1, "MatMul inner dims differ: %s @ %s." % (list(a.shape), list(b.shape)))
    out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    runtime(a.device.index).LaunchMatMul(a, b, out, M, N, K, K, 1, N, 1)
    return out


def _matmul2d_backward(a, b, g):
    M, K = a.shape
    N = b.shape[1]
    rt = runtime(a.device.index)
    dA = torch.empty((M, K), dtype=torch.float32, device=a.device)
    rt.LaunchMatMul(g, b, dA, M, K, N, N, 1, 1, N)      # dA = g . B^T  (TensorOps.cs:264)
    dB = torch.empty((K, N), dtype=torch.float32, device=a.device)
    rt.LaunchMatMul(a, g, dB, K, N, M, 1, K, N, 1)      # dB = A^T . g  (TensorOps.cs:272)
    return dA, dB


# ---- N-D ---------------------------------------------------------------------------

def _raw_bmm(a, b, M, N, K, aMs, aKs, bKs, bNs, batch_dims, aBs, bBs):
    count = 1
    for d in batch_dims:
        count *= d
    out = torch.empty(tuple(batch_dims) + (M, N), dtype=torch.float32, device=a.device)
    runtime(a.device.index).LaunchMatMulBatched(a, b, out, count, M, N, K, aMs, aKs, bKs, bNs,
                                                batch_dims, aBs, bBs)
    return out


def _reduce_grad_to_shape(g, shape):
    """ReduceGradToShape (src/Tensotron/TensorOps.cs:76-100): sum over broadcast axes.  Only
    reached when the broadcast axes cannot be fused into the batched GEMM (they do not merge
    into one strided axis); then a fixed-order reduction kernel behind the C ABI does the sum."""
    shape = tuple(shape)
    if tuple(g.shape) == shape:
        return g.clone()
    r = g.dim()
    reduce_axis = []
    for j in range(r):
        axt = j - (r - len(shape))
        dt = shape[axt] if axt >= 0 else 1
        reduce_axis.append(1 if dt != g.shape[j] else 0)
    out = torch.empty(shape, dtype=torch.float32, device=g.device)
    runtime(g.device.index).LaunchReduceSumAxes(g, out, list(g.shape), reduce_axis)
    return out


def _bmm_reduced(x, y, M, N, K, xMs, xKs, yKs, yNs, batch_dims, xBs, yBs, target_shape):
    """RawBmm followed by ReduceGradToShape(., target_shape), fused into one launch when the
    broadcast axes merge into one (src/Tensotron/TensorOps.MatMulND.cs:80-103); otherwise the
    unfused pair."""
    r = len(batch_dims)
    tb = tuple(target_shape[:-2])
    reduce_axis = []
    for j in range(r):
        axt = j - (r - len(tb))
        dt = tb[axt] if axt >= 0 else 1
        reduce_axis.append(1 if dt != batch_dims[j] else 0)
    if any(reduce_axis):
        out = torch.empty(tuple(target_shape), dtype=torch.float32, device=x.device)
        try:
            runtime(x.device.index).LaunchMatMulBatchedReduce(x, y, out, M, N, K, xMs, xKs, yKs, yNs,
                                                              batch_dims, xBs, yBs, reduce_axis)
            return out
        except TensotronGemmError as e:
            if e.status != 3:
                raise
    full = _raw_bmm(x, y, M, N, K, xMs, xKs, yKs, yNs, batch_dims, xBs, yBs)
    return _reduce_grad_to_shape(full, target_shape)


def _matmul_nd(a, b):
    ar, br = a.dim(), b.dim()
    M, K = a.shape[-2], a.shape[-1]
    K2, N = b.shape[-2], b.shape[-1]
    if K != K2:
        raise TensotronGemmError(1, "MatMul inner dims differ: %s @ %s." % (list(a.shape), list(b.shape)))
    a_str, b_str = _strides(a.shape), _strides(b.shape)
    dims, aBs, bBs = broadcast_batch(a.shape[:-2], a_str[:-2], b.shape[:-2], b_str[:-2])
    return _raw_bmm(a, b, M, N, K, K, 1, N, 1, dims, aBs, bBs)


def _matmul_nd_backward(a, b, g):
    ar, br = a.dim(), b.dim()
    M, K = a.shape[-2], a.shape[-1]
    N = b.shape[-1]
    a_str, b_str, g_str = _strides(a.shape), _strides(b.shape), _strides(g.shape)
    gMs, gNs = g_str[-2], g_str[-1]
    # dA[.,m,k] = sum_n g[.,m,n] * B[.,k,n]   (TensorOps.MatMulND.cs:80-91)
    bd, gBs2, bBs2 = broadcast_batch(g.shape[:-2], g_str[:-2], b.shape[:-2], b_str[:-2])
    dA = _bmm_reduced(g, b, M, K, N, gMs, gNs, b_str[-1], b_str[-2], bd, gBs2, bBs2, a.shape)
    # dB[.,k,n] = sum_m A[.,m,k] * g[.,m,n]   (TensorOps.MatMulND.cs:92-103)
    bd, aBs2, gBs3 = broadcast_batch(a.shape[:-2], a_str[:-2], g.shape[:-2], g_str[:-2])
    dB = _bmm_reduced(a, g, K, N, M, a_str[-1], a_str[-2], gMs, gNs, bd, aBs2, gBs3, b.shape)
    return dA, dB


# ---- public surface -----------------------------------------------------------------

def MatMul(a, b):
    """TensorOps.MatMul (src/Tensotron/TensorOps.cs:211-240): torch matmul promotion rules."""
    _check(a), _check(b)
    if a.dim() == 2 and b.dim() == 2:
        return _matmul2d(a, b)
    if a.dim() == 1 and b.dim() == 2:
        return _matmul2d(a.reshape(1, -1), b).reshape(b.shape[1])
    if a.dim() == 2 and b.dim() == 1:
        return _matmul2d(a, b.reshape(-1, 1)).reshape(a.shape[0])
    if a.dim() == 1 and b.dim() == 1:
        return _matmul2d(a.reshape(1, -1), b.reshape(-1, 1)).reshape(())
    if a.dim() == 1:
        res = _matmul_nd(a.reshape(1, -1), b)
        return res.reshape(res.shape[:-2] + res.shape[-1:])
    if b.dim() == 1:
        res = _matmul_nd(a, b.reshape(-1, 1))
        return res.reshape(res.shape[:-1])
    return _matmul_nd(a, b)


def MatMulBackward(a, b, g):
    """The (dA, dB) the MatMul GradNode closures produce for upstream gradient g."""
    _check(a), _check(b), _check(g)
    if a.dim() == 2 and b.dim() == 2:
        return _matmul2d_backward(a, b, g)
    if a.dim() == 1 and b.dim() == 2:
        dA, dB = _matmul2d_backward(a.reshape(1, -1), b, g.reshape(1, -1))
        return dA.reshape(a.shape), dB
    if a.dim() == 2 and b.dim() == 1:
        dA, dB = _matmul2d_backward(a, b.reshape(-1, 1), g.reshape(-1, 1))
        return dA, dB.reshape(b.shape)
    if a.dim() == 1 and b.dim() == 1:
        dA, dB = _matmul2d_backward(a.reshape(1, -1), b.reshape(-1, 1), g.reshape(1, 1))
        return dA.reshape(a.shape), dB.reshape(b.shape)
    if a.dim() == 1:
        a2 = a.reshape(1, -1)
        g2 = g.reshape(g.shape[:-1] + (1, g.shape[-1]))
        dA, dB = _matmul_nd_backward(a2, b, g2.contiguous())
        return dA.reshape(a.shape), dB
    if b.dim() == 1:
        b2 = b.reshape(-1, 1)
        g2 = g.reshape(g.shape + (1,))
        dA, dB = _matmul_nd_backward(a, b2, g2.contiguous())
        return dA, dB.reshape(b.shape)
    return _matmul_nd_backward(a, b, g)


def Bmm(a, b):
    """TensorOps.Bmm (src/Tensotron/TensorOps.MatMulND.cs:110-118)."""
    if a.dim() != 3 or b.dim() != 3:
        raise TensotronGemmError(1, "bmm expects 3D tensors, got %s and %s." % (list(a.shape), list(b.shape)))
    if a.shape[0] != b.shape[0]:
        raise TensotronGemmError(1, "bmm batch sizes differ: %d vs %d." % (a.shape[0], b.shape[0]))
    _check(a), _check(b)
    return _matmul_nd(a, b)


def Mv(mat, vec):
    return MatMul(mat, vec)


def Dot(a, b):
    return MatMul(a, b)


def Outer(a, b):
    """TensorOps.Outer (src/Tensotron/TensorOps.MatMulND.cs:126-131)."""
    if a.dim() != 1 or b.dim() != 1:
        raise TensotronGemmError(1, "outer expects 1D tensors, got %s and %s." % (list(a.shape), list(b.shape)))
    return MatMul(a.reshape(-1, 1), b.reshape(1, -1))


def MatMulNT(a, b):
    """y = a . b^T without materialising b^T (src/Tensotron/TensorOps.LinearNT.cs:13-25)."""
    if a.dim() != 2 or b.dim() != 2:
        raise TensotronGemmError(1, "MatMulNT expects 2D operands, got %s and %s." % (list(a.shape), list(b.shape)))
    _check(a), _check(b)
    M, K = a.shape
    N, K2 = b.shape
    if K != K2:
        raise TensotronGemmError(1, "MatMulNT inner dims differ: %s . %s^T." % (list(a.shape), list(b.shape)))
    out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    runtime(a.device.index).LaunchMatMul(a, b, out, M, N, K, K, 1, 1, K)
    return out


def MatMulNTBackward(a, b, g):
    """da = g . b (NN), db = g^T . a (TN) (src/Tensotron/TensorOps.LinearNT.cs:27-48)."""
    M, K = a.shape
    N = b.shape[0]
    rt = runtime(a.device.index)
    dA = torch.empty((M, K), dtype=torch.float32, device=a.device)
    rt.LaunchMatMul(g, b, dA, M, K, N, N, 1, K, 1)
    dB = torch.empty((N, K), dtype=torch.float32, device=a.device)
    rt.LaunchMatMul(g, a, dB, N, K, M, 1, N, K, 1)
    return dA, dB


def _conv_desc(x, weight, stride, padding, dilation):
    if x.dim() != 4:
        raise TensotronGemmError(1, "Conv2d expects (N,C,H,W), got %s." % list(x.shape))
    if weight.dim() != 4:
        raise TensotronGemmError(1, "Conv2d weight must be (O,C,kh,kw), got %s." % list(weight.shape))
    if weight.shape[1] != x.shape[1]:
        raise TensotronGemmError(1, "Conv2d channel mismatch: input %d vs weight %d." % (x.shape[1], weight.shape[1]))
    d = Conv2dDesc()
    d.n, d.c, d.h, d.w = (int(v) for v in x.shape)
    d.o, d.kh, d.kw = int(weight.shape[0]), int(weight.shape[2]), int(weight.shape[3])
    d.stride, d.padding, d.dilation = int(stride), int(padding), int(dilation)
    ho = (d.h + 2 * d.padding - d.dilation * (d.kh - 1) - 1) // d.stride + 1
    wo = (d.w + 2 * d.padding - d.dilation * (d.kw - 1) - 1) // d.stride + 1
    if ho <= 0 or wo <= 0:
        raise TensotronGemmError(1, "Im2Col: non-positive output size (%dx%d) for %s." % (ho, wo, list(x.shape)))
    return d, ho, wo


def Conv2d(x, weight, bias=None, stride=1, padding=0, dilation=1):
    """TensorOps.Conv2d (src/Tensotron/TensorOps.Conv.cs:60-80): im2col + batched matmul + bias, on
    the batched GEMM engine.  The handle workspace must hold the columns
    (TensorRuntime.Conv2dWorkspace)."""
    _check(x), _check(weight)
    d, ho, wo = _conv_desc(x, weight, stride, padding, dilation)
    y = torch.empty((d.n, d.o, ho, wo), dtype=torch.float32, device=x.device)
    runtime(x.device.index).LaunchConv2dForward(d, x, weight, bias, y)
    return y


def Conv2dBackward(x, weight, g, stride=1, padding=0, dilation=1, need_dx=True, has_bias=True):
    """(dx, dW, dbias) for upstream gradient g of Conv2d's output: what the reference's autograd
    chain (bias add, broadcast matmul, Im2Col) hands to AddGrad."""
    _check(x), _check(weight), _check(g)
    d, _, _ = _conv_desc(x, weight, stride, padding, dilation)
    dx = torch.empty_like(x) if need_dx else None
    dw = torch.empty_like(weight)
    db = torch.empty((d.o,), dtype=torch.float32, device=x.device) if has_bias else None
    runtime(x.device.index).LaunchConv2dBackward(d, x, weight, g, dx, dw, db)
    return dx, dw, db


class Linear:
    """y = act(x . W^T + b): Linear (src/Tensotron/Module.cs:82-112) with the Activation
    module that follows it fused into the GEMM epilogue.  Weight is (out, in)."""

    def __init__(self, in_features, out_features, bias=True, act=None, device="cuda", generator=None):
        bound = 1.0 / math.sqrt(in_features)  # Kaiming-uniform a=sqrt(5) (src/Tensotron/Init.cs:54-58)
        self.Weight = (torch.rand((out_features, in_features), generator=generator) * 2 - 1).mul_(bound).to(device)
        self.Bias = ((torch.rand((out_features,), generator=generator) * 2 - 1).mul_(bound).to(device)
                     if bias else None)
        self.act = ACT[act]

    def Forward(self, x):
        _check(x)
        M, K = x.shape
        N = self.Weight.shape[0]
        y = torch.empty((M, N), dtype=torch.float32, device=x.device)
        runtime(x.device.index).LaunchLinearForward(x, self.Weight, self.Bias, y, M, N, K, self.act)
        return y

    def Backward(self, x, y, dy, need_dx=True):
        """Returns (dx, dW, dbias) for upstream gradient dy of the activated output y."""
        M, K = x.shape
        N = self.Weight.shape[0]
        dx = torch.empty((M, K), dtype=torch.float32, device=x.device) if need_dx else None
        dw = torch.empty((N, K), dtype=torch.float32, device=x.device)
        db = torch.empty((N,), dtype=torch.float32, device=x.device) if self.Bias is not None else None
        runtime(x.device.index).LaunchLinearBackward(x, self.Weight, y, dy, dx, dw, db, M, N, K, self.act)
        return dx, dw, db
