"""ctypes binding of libtensotron_gemm.so and a mirror of the reference runtime
surface for the matmul path (src/Tensotron/TensorRuntime.cs:242-254: LaunchMatMul,
LaunchMatMulBatched; :158-159, :332-338: AllowTf32 / SetCuBlasMathMode).

Buffers are torch CUDA tensors (device memory plumbing only) or raw integer device
addresses.  Errors follow the reference: a non-zero native status raises
(InvalidOperationException there, TensotronGemmError here).
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("TENSOTRON_GEMM_LIB", os.path.join(_HERE, "libtensotron_gemm.so"))

TT_MATH_FP32, TT_MATH_TF32, TT_MATH_3XTF32 = 0, 3, 4
TT_ACT_NONE, TT_ACT_RELU, TT_ACT_TANH = 0, 1, 2
ACT = {None: 0, "none": 0, "relu": 1, "tanh": 2, 0: 0, 1: 1, 2: 2}

EXPORTS = [
    "tt_version", "tt_create", "tt_destroy", "tt_last_error", "tt_set_math_mode", "tt_get_math_mode",
    "tt_matmul", "tt_matmul_batched", "tt_matmul_batched_reduce", "tt_linear_fwd", "tt_linear_bwd", "tt_softmax_cross_entropy",
    "tt_adam_step", "tt_add_into", "tt_broadcast_batch", "tt_get_stats", "tt_reset_stats", "tt_check",
    "tt_set_variant", "tt_softmax_cross_entropy_static", "tt_mse_loss", "tt_clip_grad_norm", "tt_mlp_train_step", "tt_reduce_sum_axes",
    "tt_conv2d_workspace", "tt_conv2d_fwd", "tt_conv2d_bwd", "tt_shard_range",
    "tt_peer_alloc", "tt_peer_free", "tt_peer_export", "tt_peer_open", "tt_peer_close", "tt_peer_group_create",
    "tt_peer_group_destroy", "tt_peer_linear_bwd", "tt_peer_push", "tt_peer_adam_step", "tt_peer_sync",
    "tt_peer_set_wait_limit",
]


class TensotronGemmError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("tensotron_gemm status %d: %s" % (status, message))
        self.status = status


TT_LOSS_MSE, TT_LOSS_CE = 0, 1
LOSS = {"mse": 0, "ce": 1, 0: 0, 1: 1}
MLP_MAX_LAYERS = 4


class MlpDesc(ctypes.Structure):
    """tt_mlp_desc: a small MLP for tt_mlp_train_step."""
    _fields_ = [("n_layers", ctypes.c_int), ("dims", ctypes.c_int * (MLP_MAX_LAYERS + 1)),
                ("act", ctypes.c_int), ("loss", ctypes.c_int)]


class Conv2dDesc(ctypes.Structure):
    """tt_conv2d_desc."""
    _fields_ = [(n, ctypes.c_int) for n in ("n", "c", "h", "w", "o", "kh", "kw", "stride", "padding", "dilation")]


class Stats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_longlong) for n in
                ("launches", "calls", "simt_tma", "tcgen05", "generic", "splitk", "skinny", "workspace_bytes",
                 "tensor_map_hits", "tensor_map_misses")]


_lib = None


def load_library(path=None):
    """Loads the CUDA library.  No fallback: a missing library is an error."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    path = path or LIB_PATH
    if not os.path.exists(path):
        raise ImportError(
            "%s is missing: build it with `python -m tensotron_b200.build` "
            "(there is no CPU or cuBLAS fallback on this path)" % path)
    L = ctypes.CDLL(path)
    vp, i, f, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
    ip = ctypes.POINTER(ctypes.c_int)
    L.tt_version.restype = ctypes.c_char_p
    L.tt_last_error.restype = ctypes.c_char_p
    L.tt_last_error.argtypes = [vp]
    L.tt_create.argtypes = [i, ctypes.c_size_t, ctypes.POINTER(vp)]
    L.tt_destroy.argtypes = [vp]
    L.tt_set_math_mode.argtypes = [vp, i]
    L.tt_get_math_mode.argtypes = [vp, ip]
    L.tt_matmul.argtypes = [vp, vp, vp, vp, vp] + [i] * 7
    L.tt_matmul_batched.argtypes = [vp, vp, vp, vp, vp] + [i] * 9 + [ip, ip, ip]
    L.tt_matmul_batched_reduce.argtypes = [vp, vp, vp, vp, vp] + [i] * 8 + [ip, ip, ip, ip]
    L.tt_linear_fwd.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i]
    L.tt_linear_bwd.argtypes = [vp, vp] + [vp] * 7 + [i, i, i, i]
    L.tt_softmax_cross_entropy.argtypes = [vp, vp, vp, vp, vp, vp, i, i, f]
    L.tt_softmax_cross_entropy_static.argtypes = [vp, vp, vp, vp, vp, i, i, f]
    L.tt_adam_step.argtypes = [vp, vp, vp, vp, vp, vp, vp, ll, f, f, f, f, f, f, i]
    L.tt_reduce_sum_axes.argtypes = [vp, vp, vp, vp, i, ip, ip]
    cd = ctypes.POINTER(Conv2dDesc)
    L.tt_conv2d_workspace.argtypes = [cd, i]
    L.tt_conv2d_workspace.restype = ctypes.c_size_t
    L.tt_conv2d_fwd.argtypes = [vp, vp, cd, vp, vp, vp, vp]
    L.tt_conv2d_bwd.argtypes = [vp, vp, cd, vp, vp, vp, vp, vp, vp]
    L.tt_mse_loss.argtypes = [vp, vp, vp, vp, vp, vp, ll]
    L.tt_clip_grad_norm.argtypes = [vp, vp, vp, ll, f, f, vp]
    L.tt_mlp_train_step.argtypes = [vp, vp, ctypes.POINTER(MlpDesc), vp, vp, vp, vp, vp, vp, vp, vp, i, f, f, f, f, f, f]
    L.tt_add_into.argtypes = [vp, vp, vp, vp, ll]
    L.tt_broadcast_batch.argtypes = [i, ip, ip, i, ip, ip, ip, ip, ip, ip]
    L.tt_get_stats.argtypes = [vp, ctypes.POINTER(Stats)]
    L.tt_reset_stats.argtypes = [vp]
    L.tt_check.argtypes = [vp, vp]
    L.tt_set_variant.argtypes = [vp, i]
    for name in EXPORTS:
        if getattr(L, name).restype is ctypes.c_int:
            pass
    if path == LIB_PATH:
        _lib = L
    return L


def _ptr(x):
    """Device address of a torch CUDA float32/int32 tensor, or a raw integer / None."""
    if x is None:
        return None
    if isinstance(x, int):
        return ctypes.c_void_p(x)
    if not x.is_cuda:
        raise TypeError("expected a CUDA tensor")
    return ctypes.c_void_p(x.data_ptr())


def _iarr(v):
    v = [int(t) for t in v]
    return (ctypes.c_int * max(1, len(v)))(*v)


STATIC_CE_MAX_ROWS = 65536


def softmax_cross_entropy_static(logits, labels, dlogits, loss, rows, classes, scale, stream=None):
    """tt_softmax_cross_entropy_static: cross-entropy for callers that may not allocate device
    memory (no handle, scratch built into the library).  Runs on torch's current device."""
    import torch
    L = load_library()
    st = ctypes.c_void_p(stream if isinstance(stream, int) else
                         (stream.cuda_stream if stream is not None else torch.cuda.current_stream().cuda_stream))
    rc = L.tt_softmax_cross_entropy_static(st, _ptr(logits), _ptr(labels), _ptr(dlogits), _ptr(loss),
                                           rows, classes, scale)
    if rc == 6:
        raise TensotronGemmError(rc, "rows %d exceed the built-in scratch (%d rows)" % (rows, STATIC_CE_MAX_ROWS))
    if rc:
        raise TensotronGemmError(rc, "tt_softmax_cross_entropy_static failed")


def shard_range(total, world, rank):
    """tt_shard_range: the contiguous block [start, start + count) of `total` units that `rank` of
    `world` owns (ceil-sized blocks)."""
    L = load_library()
    L.tt_shard_range.argtypes = [ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                                 ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_longlong)]
    s, c = ctypes.c_longlong(0), ctypes.c_longlong(0)
    rc = L.tt_shard_range(total, world, rank, ctypes.byref(s), ctypes.byref(c))
    if rc:
        raise TensotronGemmError(rc, "bad shard arguments")
    return s.value, c.value


def broadcast_batch(a_dims, a_strides, b_dims, b_strides):
    """BroadcastBatch (src/Tensotron/TensorOps.MatMulND.cs:11-31) through the C ABI."""
    L = load_library()
    ra, rb = len(a_dims), len(b_dims)
    r = max(ra, rb)
    dims, a_bs, b_bs = _iarr([0] * r), _iarr([0] * r), _iarr([0] * r)
    rank = ctypes.c_int(0)
    rc = L.tt_broadcast_batch(ra, _iarr(a_dims), _iarr(a_strides), rb, _iarr(b_dims), _iarr(b_strides),
                              ctypes.byref(rank), dims, a_bs, b_bs)
    if rc:
        raise TensotronGemmError(rc, "Cannot broadcast batch dims %s with %s" % (list(a_dims), list(b_dims)))
    return list(dims)[:r], list(a_bs)[:r], list(b_bs)[:r]


_parked = []     # handles whose owner was collected during a stream capture: destroyed later


def _capturing():
    try:
        import torch
        return torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()
    except Exception:
        return False


class TensorRuntime:
    """The CUDA-backend runtime surface of the matmul path, one handle per device."""

    def __init__(self, device=0, workspace_bytes=0):
        self._L = load_library()
        self._h = ctypes.c_void_p()
        self.device = device
        rc = self._L.tt_create(device, workspace_bytes, ctypes.byref(self._h))
        if rc:
            raise TensotronGemmError(rc, "tt_create failed (needs a sm_100 device)")
        self._stream = None

    # -- lifetime ---------------------------------------------------------------
    def Dispose(self):
        if self._h:
            self._L.tt_destroy(self._h)
            self._h = ctypes.c_void_p()
        while _parked and not _capturing():
            L, h = _parked.pop()
            L.tt_destroy(h)

    def __del__(self):
        # The garbage collector may run this at any point, also while some stream of the process is
        # being captured into a CUDA graph -- and tt_destroy frees device memory, which invalidates a
        # capture in progress.  So a handle that dies during a capture is parked and destroyed with
        # the next one that dies (or is disposed) outside a capture.
        try:
            if self._h and _capturing():
                _parked.append((self._L, self._h))
                self._h = ctypes.c_void_p()
                return
            self.Dispose()
        except Exception:
            pass

    def _ck(self, rc):
        if rc:
            raise TensotronGemmError(rc, self._L.tt_last_error(self._h).decode())

    def _st(self, stream):
        """CUstream for the call: explicit, else torch's current stream on this device."""
        if stream is not None:
            return ctypes.c_void_p(stream if isinstance(stream, int) else stream.cuda_stream)
        import torch
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    # -- math mode (src/Tensotron/TensorRuntime.cs:158-159, :332-338) --------------
    @property
    def AllowTf32(self):
        return self.GetMathMode() == TT_MATH_TF32

    @AllowTf32.setter
    def AllowTf32(self, value):
        self.SetCuBlasMathMode(TT_MATH_TF32 if value else TT_MATH_FP32)

    def SetCuBlasMathMode(self, mode):
        self._ck(self._L.tt_set_math_mode(self._h, int(mode)))

    def GetMathMode(self):
        m = ctypes.c_int(0)
        self._ck(self._L.tt_get_math_mode(self._h, ctypes.byref(m)))
        return m.value

    def SetVariant(self, variant):
        self._ck(self._L.tt_set_variant(self._h, int(variant)))

    # -- launches ----------------------------------------------------------------
    def LaunchMatMul(self, a, b, c, M, N, K, aMs, aKs, bKs, bNs, stream=None):
        self._ck(self._L.tt_matmul(self._h, self._st(stream), _ptr(a), _ptr(b), _ptr(c),
                                   M, N, K, aMs, aKs, bKs, bNs))

    def LaunchMatMulBatched(self, a, b, c, batchCount, M, N, K, aMs, aKs, bKs, bNs,
                            batchDims, aBatchStrides, bBatchStrides, stream=None):
        self._ck(self._L.tt_matmul_batched(
            self._h, self._st(stream), _ptr(a), _ptr(b), _ptr(c), batchCount, M, N, K,
            aMs, aKs, bKs, bNs, len(batchDims), _iarr(batchDims), _iarr(aBatchStrides),
            _iarr(bBatchStrides)))

    def LaunchMatMulBatchedReduce(self, a, b, c, M, N, K, aMs, aKs, bKs, bNs,
                                  batchDims, aBatchStrides, bBatchStrides, reduceAxis, stream=None):
        """RawBmm + ReduceGradToShape in one launch; raises status 3 when the summed axes do
        not merge (the caller then reduces separately)."""
        self._ck(self._L.tt_matmul_batched_reduce(
            self._h, self._st(stream), _ptr(a), _ptr(b), _ptr(c), M, N, K, aMs, aKs, bKs, bNs,
            len(batchDims), _iarr(batchDims), _iarr(aBatchStrides), _iarr(bBatchStrides),
            _iarr(reduceAxis)))

    @staticmethod
    def Conv2dWorkspace(desc, backward=False):
        return load_library().tt_conv2d_workspace(ctypes.byref(desc), 1 if backward else 0)

    def LaunchConv2dForward(self, desc, x, w, bias, y, stream=None):
        """Conv2d = Im2Col + batched matmul + bias (src/Tensotron/TensorOps.Conv.cs:60-80)."""
        self._ck(self._L.tt_conv2d_fwd(self._h, self._st(stream), ctypes.byref(desc), _ptr(x), _ptr(w), _ptr(bias), _ptr(y)))

    def LaunchConv2dBackward(self, desc, x, w, dy, dx, dw, dbias, stream=None):
        self._ck(self._L.tt_conv2d_bwd(self._h, self._st(stream), ctypes.byref(desc), _ptr(x), _ptr(w), _ptr(dy),
                                       _ptr(dx), _ptr(dw), _ptr(dbias)))

    def LaunchReduceSumAxes(self, src, dst, dims, reduceAxis, stream=None):
        """ReduceGradToShape's sum over the marked axes (src/Tensotron/TensorOps.cs:76-100), fixed order."""
        self._ck(self._L.tt_reduce_sum_axes(self._h, self._st(stream), _ptr(src), _ptr(dst), len(dims),
                                            _iarr(dims), _iarr(reduceAxis)))

    def LaunchLinearForward(self, x, w, bias, y, M, N, K, act=0, stream=None):
        self._ck(self._L.tt_linear_fwd(self._h, self._st(stream), _ptr(x), _ptr(w), _ptr(bias),
                                       _ptr(y), M, N, K, ACT[act]))

    def LaunchLinearBackward(self, x, w, y, dy, dx, dw, dbias, M, N, K, act=0, stream=None):
        self._ck(self._L.tt_linear_bwd(self._h, self._st(stream), _ptr(x), _ptr(w), _ptr(y), _ptr(dy),
                                       _ptr(dx), _ptr(dw), _ptr(dbias), M, N, K, ACT[act]))

    def LaunchSoftmaxCrossEntropy(self, logits, labels, dlogits, loss, rows, classes, scale, stream=None):
        self._ck(self._L.tt_softmax_cross_entropy(self._h, self._st(stream), _ptr(logits), _ptr(labels),
                                                  _ptr(dlogits), _ptr(loss), rows, classes, scale))

    def LaunchAdam(self, p, g, m, v, adv, n, b1=0.9, b2=0.999, lr=1e-3, eps=1e-8,
                   coupledWd=0.0, decoupledFactor=1.0, advance=True, stream=None):
        self._ck(self._L.tt_adam_step(self._h, self._st(stream), _ptr(p), _ptr(g), _ptr(m), _ptr(v),
                                      _ptr(adv), n, b1, b2, lr, eps, coupledWd, decoupledFactor,
                                      1 if advance else 0))

    def LaunchMseLoss(self, input, target, dinput, loss, count, stream=None):
        """MseLoss(mean) forward + backward (src/Tensotron/TensorOps.Losses.cs:29-61)."""
        self._ck(self._L.tt_mse_loss(self._h, self._st(stream), _ptr(input), _ptr(target), _ptr(dinput),
                                     _ptr(loss), count))

    def LaunchClipGradNorm(self, grads, n, max_norm, eps=1e-6, norm_out=None, stream=None):
        """GradUtils.ClipGradNorm over a flat gradient span (src/Tensotron/Optimizers.cs:383-422)."""
        self._ck(self._L.tt_clip_grad_norm(self._h, self._st(stream), _ptr(grads), n, max_norm, eps, _ptr(norm_out)))

    def LaunchMlpTrainStep(self, dims, act, loss_kind, params, m, v, adv, grads_out, x, target, loss, batch,
                           lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, max_grad_norm=0.0, clip_eps=1e-6, stream=None):
        """tt_mlp_train_step: forward + loss + backward + clip + Adam of a small MLP as one launch.
        Raises status 3 when the network or the batch does not fit one cluster."""
        d = MlpDesc()
        d.n_layers = len(dims) - 1
        if not 1 <= d.n_layers <= MLP_MAX_LAYERS:
            raise TensotronGemmError(3, "the one-launch MLP step takes 1..%d layers" % MLP_MAX_LAYERS)
        for i, w in enumerate(dims):
            d.dims[i] = int(w)
        d.act, d.loss = ACT[act], LOSS[loss_kind]
        self._ck(self._L.tt_mlp_train_step(self._h, self._st(stream), ctypes.byref(d), _ptr(params), _ptr(m), _ptr(v),
                                           _ptr(adv), _ptr(grads_out), _ptr(x), _ptr(target), _ptr(loss), batch,
                                           lr, b1, b2, eps, max_grad_norm, clip_eps))

    def LaunchAddInto(self, target, source, n, stream=None):
        self._ck(self._L.tt_add_into(self._h, self._st(stream), _ptr(target), _ptr(source), n))

    # -- counters / checks ---------------------------------------------------------
    def Stats(self):
        s = Stats()
        self._ck(self._L.tt_get_stats(self._h, ctypes.byref(s)))
        return {n: getattr(s, n) for n, _ in Stats._fields_}

    def ResetCounters(self):
        self._ck(self._L.tt_reset_stats(self._h))

    def Check(self, stream=None):
        """Synchronises and raises if a bounded device-side wait gave up."""
        self._ck(self._L.tt_check(self._h, self._st(stream)))
