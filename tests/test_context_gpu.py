"""The library binds to the CUDA context of its caller.

The reference's accelerator layer creates its own driver-API context and hands that context's
buffers and streams to native libraries (the cuBLAS handle is created next to it,
src/Tensotron/TensorRuntime.cs:505-511; its default stream is the NULL stream, :308-317).  This
test plays that host: it creates a context with cuCtxCreate through libcuda, allocates every
buffer with cuMemAlloc in it, and drives tt_create / tt_matmul / tt_linear_bwd /
tt_softmax_cross_entropy(_static) on stream 0 and on a created stream, against the oracle.
torch is not involved in any allocation here (it only holds the primary context of the same
device, which is what the library must NOT fall back to).
"""
import ctypes

import numpy as np
import pytest

import oracle
from conftest import fp32_bound

pytestmark = pytest.mark.gpu

vp, u64 = ctypes.c_void_p, ctypes.c_uint64


class DriverContext:
    """A driver-API context with a few typed helpers (all calls checked)."""

    def __init__(self):
        self.cu = ctypes.CDLL("libcuda.so.1")
        self._ck(self.cu.cuInit(0))
        dev = ctypes.c_int()
        self._ck(self.cu.cuDeviceGet(ctypes.byref(dev), 0))
        self.prev = vp()
        self._ck(self.cu.cuCtxGetCurrent(ctypes.byref(self.prev)))
        self.ctx = vp()
        self._ck(self.cu.cuCtxCreate_v2(ctypes.byref(self.ctx), 0, dev))   # also makes it current
        self.allocs, self.streams = [], []

    @staticmethod
    def _ck(rc):
        assert rc == 0, "CUDA driver call failed with %d" % rc

    def current(self):
        c = vp()
        self._ck(self.cu.cuCtxGetCurrent(ctypes.byref(c)))
        return c.value

    def set_current(self, ctx):
        self._ck(self.cu.cuCtxSetCurrent(ctx))

    def alloc(self, nbytes):
        p = u64()
        self._ck(self.cu.cuMemAlloc_v2(ctypes.byref(p), ctypes.c_size_t(nbytes)))
        self.allocs.append(p.value)
        return p.value

    def upload(self, arr):
        arr = np.ascontiguousarray(arr)
        p = self.alloc(arr.nbytes)
        self._ck(self.cu.cuMemcpyHtoD_v2(u64(p), arr.ctypes.data_as(vp), ctypes.c_size_t(arr.nbytes)))
        return p

    def filled(self, shape, dtype=np.float32):
        return self.upload(np.full(shape, np.nan, dtype=dtype))

    def download(self, p, shape, dtype=np.float32):
        out = np.empty(shape, dtype=dtype)
        self._ck(self.cu.cuMemcpyDtoH_v2(out.ctypes.data_as(vp), u64(p), ctypes.c_size_t(out.nbytes)))
        return out

    def stream(self):
        s = vp()
        self._ck(self.cu.cuStreamCreate(ctypes.byref(s), 0))
        self.streams.append(s)
        return s

    def sync(self):
        self._ck(self.cu.cuCtxSynchronize())

    def close(self):
        self.set_current(self.ctx)
        self.sync()
        for s in self.streams:
            self.cu.cuStreamDestroy_v2(s)
        for p in self.allocs:
            self.cu.cuMemFree_v2(u64(p))
        self._ck(self.cu.cuCtxDestroy_v2(self.ctx))
        self.set_current(self.prev)            # back to what the process had (torch's primary context)


@pytest.fixture()
def driver_ctx(gemm_lib):
    import torch
    assert torch.cuda.is_available()
    torch.zeros(1, device="cuda")              # the primary context exists and is current, as in a torch host
    d = DriverContext()
    try:
        yield d
    finally:
        d.close()


def _create(L, workspace=64 << 20):
    h = vp()
    assert L.tt_create(0, workspace, ctypes.byref(h)) == 0
    return h


def test_handle_lives_in_the_callers_driver_context(gemm_lib, driver_ctx):
    L, d = gemm_lib, driver_ctx
    assert d.current() == d.ctx.value and d.ctx.value != d.prev.value
    h = _create(L)
    assert d.current() == d.ctx.value          # tt_create did not replace the current context
    rng = np.random.default_rng(0)
    M, N, K = 384, 320, 512
    a = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    exp = oracle.matmul2d(a, b, M, N, K, K, 1, N, 1)
    da, db = d.upload(a), d.upload(b)
    try:
        for stream in (vp(None), d.stream()):      # the NULL stream and a created stream
            dc = d.filled((M, N))
            rc = L.tt_matmul(h, stream, vp(da), vp(db), vp(dc), M, N, K, K, 1, N, 1)
            assert rc == 0, L.tt_last_error(h)
            assert L.tt_check(h, stream) == 0
            got = d.download(dc, (M, N))
            assert np.abs(got - exp).max() <= fp32_bound(K, a, b)
        # Linear backward (activation mask + bias gradient in the handle's workspace, dX, dW)
        x = rng.standard_normal((M, K)).astype(np.float32)
        w = (rng.uniform(-1, 1, (N, K)) / np.sqrt(K)).astype(np.float32)
        bias = rng.uniform(-0.1, 0.1, N).astype(np.float32)
        dy = rng.standard_normal((M, N)).astype(np.float32)
        z, y = oracle.linear_fwd(x, w, bias, 1)
        dxo, dwo, dbo, g = oracle.linear_bwd(x, w, z, y, dy, 1)
        st = d.stream()
        px, pw, pb, pdy = d.upload(x), d.upload(w), d.upload(bias), d.upload(dy)
        py, pdx, pdw, pdb = d.filled((M, N)), d.filled((M, K)), d.filled((N, K)), d.filled((N,))
        assert L.tt_linear_fwd(h, st, vp(px), vp(pw), vp(pb), vp(py), M, N, K, 1) == 0
        assert L.tt_linear_bwd(h, st, vp(px), vp(pw), vp(py), vp(pdy), vp(pdx), vp(pdw), vp(pdb), M, N, K, 1) == 0
        assert L.tt_check(h, st) == 0
        assert np.abs(d.download(py, (M, N)) - y).max() <= fp32_bound(K, x, w) + 2e-6
        assert np.abs(d.download(pdx, (M, K)) - dxo).max() <= fp32_bound(N, g, w) + 1e-5
        assert np.abs(d.download(pdw, (N, K)) - dwo).max() <= fp32_bound(M, g, x) + 1e-5
        assert np.abs(d.download(pdb, (N,)) - dbo).max() <= fp32_bound(M, g, 1.0) + 1e-5
        # cross-entropy, handle entry and the allocation-free entry, in this context
        rows, classes = 1000, 10
        lg = (rng.standard_normal((rows, classes)) * 3).astype(np.float32)
        lb = rng.integers(0, classes, rows).astype(np.int32)
        lo, do = oracle.cross_entropy(lg, lb)
        plg, plb = d.upload(lg), d.upload(lb)
        for static in (False, True):
            pd, pl = d.filled((rows, classes)), d.filled((1,))
            if static:
                rc = L.tt_softmax_cross_entropy_static(st, vp(plg), vp(plb), vp(pd), vp(pl), rows, classes, 1.0 / rows)
            else:
                rc = L.tt_softmax_cross_entropy(h, st, vp(plg), vp(plb), vp(pd), vp(pl), rows, classes, 1.0 / rows)
            assert rc == 0
            assert L.tt_check(h, st) == 0
            assert abs(d.download(pl, (1,))[0] - lo) <= 1e-5 * max(1.0, abs(lo))
            np.testing.assert_allclose(d.download(pd, (rows, classes)), do, atol=1e-9, rtol=2e-5)
        # With ANOTHER context current on the thread (here: the process's primary context), a call
        # still runs in the handle's context and leaves the thread's current context alone.
        dc = d.filled((M, N))
        d.set_current(d.prev)
        assert L.tt_matmul(h, vp(None), vp(da), vp(db), vp(dc), M, N, K, K, 1, N, 1) == 0
        assert L.tt_check(h, vp(None)) == 0
        assert d.current() == d.prev.value
        d.set_current(d.ctx)
        assert np.abs(d.download(dc, (M, N)) - exp).max() <= fp32_bound(K, a, b)
    finally:
        d.set_current(d.ctx)
        assert L.tt_destroy(h) == 0
