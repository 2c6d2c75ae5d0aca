"""Gradient exchange between the GPUs of one node over peer memory (the tt_peer_* part of the
C ABI): the multi-GPU form of the reference's Linear backward + Adam step
(src/Tensotron/TensorOps.LinearNT.cs:31-52, src/Tensotron/Optimizers.cs:144-193), which the
reference itself only runs on one GPU.

Every rank owns a block of rows of each large weight matrix.  A rank's weight-gradient GEMM
stores each finished tile straight into the owner's memory (NVLink store from the epilogue),
the owner sums the per-rank copies in rank order, runs Adam on its rows and stores the new
rows into every rank's parameters.  Small segments (biases, narrow layers) are replicated.
torch.distributed only carries the 64-byte IPC handles at set-up.
"""
import ctypes

from .runtime import _ptr

MAX_PEERS = 8
MAX_SEGMENTS = 16
CHANNELS = 8                 # independent parts of a step's exchange (one per layer)
FLAG_WORDS = 256
ROW_BLOCK = 256              # ownership granularity = tallest GEMM tile
MIN_PARTITIONED = 1 << 20    # weight matrices below this many elements are replicated


def exchange_plan(dims, world, offs=None):
    """Which rank owns what, layer by layer.  dims: layer widths; offs: (w_off, b_off) per layer
    as laid out by mlp.layer_layout (computed when omitted).  Returns (own_rows, owned, replicated):
    own_rows[i]       rows of W_i per owner (0 = the layer is replicated),
    owned[r][i]       list of (offset, length) float segments of layer i owned by rank r,
    replicated[i]     list of (offset, length) segments of layer i that every rank reduces and
                      updates itself (the bias, or the whole layer when it is replicated).
    Segments are multiples of 4 floats; together they cover the flat buffer exactly once."""
    from .mlp import layer_layout
    if offs is None:
        offs, total = layer_layout(dims)
    else:
        total = layer_layout(dims)[1]
    L = len(dims) - 1
    own_rows, owned, repl = [], [[[] for _ in range(L)] for _ in range(world)], [[] for _ in range(L)]
    for i in range(L):
        fan_in, fan_out = dims[i], dims[i + 1]
        w_off, b_off = offs[i]
        end = offs[i + 1][0] if i + 1 < L else total      # padded end of this layer
        rows = 0
        if fan_out * fan_in >= MIN_PARTITIONED and (fan_in % 4 == 0):
            per = -(-fan_out // world)
            rows = -(-per // ROW_BLOCK) * ROW_BLOCK
        own_rows.append(rows)
        if rows:
            for r in range(world):
                lo, hi = min(fan_out, r * rows), min(fan_out, (r + 1) * rows)
                if hi > lo:
                    owned[r][i].append((w_off + lo * fan_in, (hi - lo) * fan_in))
            repl[i].append((b_off, end - b_off))
        else:
            repl[i].append((w_off, end - w_off))
        for off, ln in repl[i] + [s for r in range(world) for s in owned[r][i]]:
            assert off % 4 == 0 and ln % 4 == 0
    return own_rows, owned, repl


def merge_segments(segs):
    """Sorts (offset, length) segments and joins the adjacent ones."""
    out = []
    for off, ln in sorted(segs):
        if ln <= 0:
            continue
        if out and out[-1][0] + out[-1][1] == off:
            out[-1] = (out[-1][0], out[-1][1] + ln)
        else:
            out.append((off, ln))
    if len(out) > MAX_SEGMENTS:
        raise ValueError("more than %d exchange segments" % MAX_SEGMENTS)
    return out


class _DeviceBuffer:
    """A raw device allocation that torch can view (`torch.as_tensor(buf, device=...)`)."""

    def __init__(self, ptr, n_floats, typestr="<f4"):
        self.ptr = ptr
        self.__cuda_array_interface__ = {"shape": (n_floats,), "typestr": typestr, "data": (ptr, False),
                                         "version": 2}


def _larr(v):
    v = [int(t) for t in v]
    return (ctypes.c_longlong * max(1, len(v)))(*v)


class PeerGroup:
    """Peer-mapped staging, parameter and flag buffers of all ranks + the native group handle."""

    def __init__(self, rt, n_floats, process_group=None, _emulated=None):
        import torch.distributed as dist
        self.rt, L, h = rt, rt._L, rt._h
        self._declare(L)
        self.pg = process_group
        if _emulated is not None:
            self.world, self.rank = _emulated
        else:
            self.world = dist.get_world_size(process_group) if process_group is not None else 1
            self.rank = dist.get_rank(process_group) if process_group is not None else 0
        if self.world > MAX_PEERS:
            raise ValueError("at most %d ranks" % MAX_PEERS)
        self.n = n_floats
        self._sizes = {"stage": 4 * self.world * n_floats, "params": 4 * n_floats, "flags": 4 * FLAG_WORDS}
        self._own, self._opened, self._g = {}, [], None
        try:
            for name, nbytes in self._sizes.items():
                p = ctypes.c_void_p()
                rt._ck(L.tt_peer_alloc(h, nbytes, ctypes.byref(p)))
                self._own[name] = p.value
        except Exception:
            # a failed allocation must not leave the earlier buffers of this group behind
            for p in self._own.values():
                L.tt_peer_free(h, ctypes.c_void_p(p))
            self._own = {}
            raise
        if _emulated is not None:
            return                      # emulate() connects the ranks
        maps = {name: [None] * self.world for name in self._sizes}
        for name in self._sizes:
            maps[name][self.rank] = self._own[name]
        if self.world > 1:
            mine = {}
            for name in self._sizes:
                buf = (ctypes.c_ubyte * 64)()
                rt._ck(L.tt_peer_export(h, ctypes.c_void_p(self._own[name]), buf))
                mine[name] = bytes(buf)
            everyone = [None] * self.world
            dist.all_gather_object(everyone, mine, group=process_group)
            for r in range(self.world):
                if r == self.rank:
                    continue
                for name in self._sizes:
                    p = ctypes.c_void_p()
                    hb = (ctypes.c_ubyte * 64).from_buffer_copy(everyone[r][name])
                    rt._ck(L.tt_peer_open(h, hb, ctypes.byref(p)))
                    maps[name][r] = p.value
                    self._opened.append(p.value)
        self._connect(maps)

    def _connect(self, maps):
        import torch
        rt, n = self.rt, self.n
        arr = lambda name: (ctypes.c_void_p * self.world)(*maps[name])
        self._g = ctypes.c_void_p()
        rt._ck(rt._L.tt_peer_group_create(rt._h, self.world, self.rank, n, arr("stage"), arr("params"),
                                          arr("flags"), ctypes.byref(self._g)))
        dev = torch.device("cuda", rt.device)
        self._views = [_DeviceBuffer(self._own["params"], n),
                       _DeviceBuffer(self._own["stage"] + 4 * self.rank * n, n),
                       _DeviceBuffer(self._own["stage"], self.world * n)]
        self.params = torch.as_tensor(self._views[0], device=dev)     # flat parameters (local copy)
        self.grads = torch.as_tensor(self._views[1], device=dev)      # this rank's own slot
        self.stage = torch.as_tensor(self._views[2], device=dev).view(self.world, n)

    @classmethod
    def emulate(cls, rts, n_floats):
        """len(rts) ranks inside this process, one runtime handle each, buffers shared by address
        (no IPC).  For tests on one GPU: the caller issues the ranks' calls phase by phase on one
        stream (all backward passes, all pushes, all optimizer steps, all syncs), so every flag
        is already set when its wait kernel runs and no kernel ever waits for a later one."""
        world = len(rts)
        groups = [cls(rt, n_floats, None, _emulated=(world, r)) for r, rt in enumerate(rts)]
        maps = {name: [g._own[name] for g in groups] for name in groups[0]._sizes}
        for g in groups:
            g._connect(maps)
        return groups

    @staticmethod
    def _declare(L):
        if getattr(L, "_peer_declared", False):
            return
        vp, i, f, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
        pvp, pll = ctypes.POINTER(vp), ctypes.POINTER(ll)
        L.tt_peer_alloc.argtypes = [vp, ctypes.c_size_t, pvp]
        L.tt_peer_free.argtypes = [vp, vp]
        L.tt_peer_export.argtypes = [vp, vp, ctypes.c_void_p]
        L.tt_peer_open.argtypes = [vp, ctypes.c_void_p, pvp]
        L.tt_peer_close.argtypes = [vp, vp]
        L.tt_peer_group_create.argtypes = [vp, i, i, ll, pvp, pvp, pvp, pvp]
        L.tt_peer_group_destroy.argtypes = [vp]
        L.tt_peer_linear_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, ll, ll, i, i, i, i, i, ctypes.POINTER(i)]
        L.tt_peer_push.argtypes = [vp, vp, vp, i, i, i, pll, pll]
        L.tt_peer_adam_step.argtypes = [vp, vp, vp, i, i, pll, pll, i, pll, pll, vp, vp, vp, f, f, f, f, f, f, i]
        L.tt_peer_sync.argtypes = [vp, vp, vp, i]
        L.tt_peer_set_wait_limit.argtypes = [vp, i]
        L._peer_declared = True

    # -- the three calls of a step ------------------------------------------------------------
    def linear_bwd(self, x, w, y, dy, dx, w_off, b_off, M, N, K, act, own_rows, stream=None):
        """tt_peer_linear_bwd; returns True when the GEMM epilogue did the scatter."""
        fused = ctypes.c_int(0)
        rt = self.rt
        rt._ck(rt._L.tt_peer_linear_bwd(rt._h, rt._st(stream), self._g, _ptr(x), _ptr(w), _ptr(y), _ptr(dy),
                                        _ptr(dx), w_off, b_off, M, N, K, act, own_rows, ctypes.byref(fused)))
        return bool(fused.value)

    def push(self, segments, channel=0, new_step=True, stream=None):
        rt = self.rt
        rt._ck(rt._L.tt_peer_push(rt._h, rt._st(stream), self._g, channel, 1 if new_step else 0, len(segments),
                                  _larr([s[0] for s in segments]), _larr([s[1] for s in segments])))

    def adam_step(self, owned, replicated, m, v, adv, channel=0, b1=0.9, b2=0.999, lr=1e-3, eps=1e-8,
                  coupledWd=0.0, decoupledFactor=1.0, advance=True, stream=None):
        rt = self.rt
        rt._ck(rt._L.tt_peer_adam_step(
            rt._h, rt._st(stream), self._g, channel, len(owned), _larr([s[0] for s in owned]),
            _larr([s[1] for s in owned]), len(replicated), _larr([s[0] for s in replicated]),
            _larr([s[1] for s in replicated]), _ptr(m), _ptr(v), _ptr(adv), b1, b2, lr, eps, coupledWd,
            decoupledFactor, 1 if advance else 0))

    def set_wait_limit(self, milliseconds):
        self.rt._ck(self.rt._L.tt_peer_set_wait_limit(self._g, int(milliseconds)))

    def sync(self, n_channels=1, stream=None):
        rt = self.rt
        rt._ck(rt._L.tt_peer_sync(rt._h, rt._st(stream), self._g, n_channels))

    # -- lifetime -------------------------------------------------------------------------------
    def close(self):
        """Unmaps the other ranks' buffers, then (after everybody has) frees this rank's."""
        if self._g is None:
            return
        import torch
        torch.cuda.synchronize(self.rt.device)
        rt, L = self.rt, self.rt._L
        self.params = self.grads = self.stage = None
        L.tt_peer_group_destroy(self._g)
        self._g = None
        via_ipc = bool(self._opened)
        for p in self._opened:
            L.tt_peer_close(rt._h, ctypes.c_void_p(p))
        self._opened = []
        if via_ipc:
            import torch.distributed as dist
            dist.barrier(group=self.pg)
        for p in self._own.values():
            L.tt_peer_free(rt._h, ctypes.c_void_p(p))
        self._own = {}
