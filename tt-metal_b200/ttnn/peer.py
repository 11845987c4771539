"""Peer-memory plumbing for the matmul whose epilogue is the all-gather (ttb_matmul_peer in include/ttb.h).

One process per GPU. Every rank allocates one arena with the same layout, exports it with CUDA IPC, and maps the other
ranks' arenas; the handles travel through torch.distributed (any backend). The arena holds a ring of gather points:
per point a pair of counters (`arrived`, written by every rank over NVLink, and `expected`, written only by its owner) and a
buffer for the gathered tensor. All ranks take the points of the ring in the same order, so a point's buffer is reused
only `slots` gathering launches later, long after every rank has consumed it.

Replaces the ring topology set-up of the reference's AllGather
(tt_eager/tt_dnn/op_library/all_gather/all_gather_op.cpp:18-104) for the decode path."""
import ctypes

from .runtime import lib as _rt

MAX_RANKS = 8
_vp, _i32, _i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64


class PeerGather(ctypes.Structure):
    """ttb_peer_gather."""
    _fields_ = [("ranks", _i32), ("rank", _i32), ("out", _vp * MAX_RANKS), ("arrived", _vp * MAX_RANKS), ("expected", _vp)]


class PeerWait(ctypes.Structure):
    """ttb_peer_wait_t."""
    _fields_ = [("arrived", _vp), ("expected", _vp)]


def _declare(cdll):
    cdll.ttb_malloc.argtypes = [ctypes.POINTER(_vp), ctypes.c_size_t]
    cdll.ttb_free.argtypes = [_vp]
    cdll.ttb_memset.argtypes = [_vp, _i32, ctypes.c_size_t, _vp]
    cdll.ttb_device_synchronize.argtypes = []
    cdll.ttb_ipc_export.argtypes = [_vp, _vp]
    cdll.ttb_ipc_open.argtypes = [_vp, ctypes.POINTER(_vp)]
    cdll.ttb_ipc_close.argtypes = [_vp]
    cdll.ttb_peer_wait.argtypes = [_vp, _vp]
    cdll.ttb_matmul_peer_workspace_bytes.argtypes = [_i32, _i64, _i64, _i64, _i64]
    cdll.ttb_matmul_peer_workspace_bytes.restype = _i64
    cdll.ttb_matmul_peer.argtypes = [_vp, _i32, _vp, _i32, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _i32, _i32, _vp, _i64, _vp, _vp, _vp]
    cdll.ttb_matmul_multi_workspace_bytes.argtypes = [_i32, _i64, _i64, _i64, _i32, _vp]
    cdll.ttb_matmul_multi_workspace_bytes.restype = _i64
    cdll.ttb_matmul_multi.argtypes = [_vp, _i32, _i32, _vp, _i32, _vp, _vp, _i32, _i64, _i64, _i64, _vp, _i32, _i32, _vp, _i64, _vp, _vp, _vp]


_declare(_rt.cdll)


def _check(rc):
    if rc != 0:
        raise RuntimeError(_rt.cdll.ttb_last_error().decode())


_COUNTER_STRIDE = 256          # bytes per gather point in the counter area: arrived at +0, expected at +128
_ALIGN = 4096


def ring_layout(slots, slot_bytes):
    """Pure layout arithmetic: (counter area bytes, rounded slot bytes, arena bytes)."""
    if slots < 2:
        raise RuntimeError("a gather ring needs at least two points: consecutive gathers must not share a buffer")
    counters = (slots * _COUNTER_STRIDE + _ALIGN - 1) // _ALIGN * _ALIGN
    slot = (slot_bytes + _ALIGN - 1) // _ALIGN * _ALIGN
    return counters, slot, counters + slots * slot


class GatherRing:
    """A ring of `slots` gather points of `slot_bytes` each, identical on every rank of `group`."""

    def __init__(self, rank, world, slot_bytes, slots=4, group=None):
        import torch.distributed as dist
        if not 2 <= world <= MAX_RANKS:
            raise RuntimeError(f"the gather epilogue serves 2..{MAX_RANKS} ranks, got {world}")
        self.rank, self.world, self.slots = rank, world, slots
        self.counter_bytes, self.slot_bytes, self.arena_bytes = ring_layout(slots, slot_bytes)
        base = _vp()
        _check(_rt.cdll.ttb_malloc(ctypes.byref(base), self.arena_bytes))
        self._own = base.value
        _check(_rt.cdll.ttb_memset(self._own, 0, self.arena_bytes, None))
        _check(_rt.cdll.ttb_device_synchronize())
        handle = ctypes.create_string_buffer(64)
        _check(_rt.cdll.ttb_ipc_export(self._own, handle))
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self.bases = []
        for r in range(world):
            if r == rank:
                self.bases.append(self._own)
                continue
            ptr = _vp()
            buf = ctypes.create_string_buffer(handles[r], 64)
            _check(_rt.cdll.ttb_ipc_open(buf, ctypes.byref(ptr)))
            self.bases.append(ptr.value)
        dist.barrier(group=group)      # every arena is zeroed and mapped before anyone's kernels touch a peer
        self._next = 0
        self._gathers = [self._make_gather(s) for s in range(slots)]
        self._waits = [self._make_wait(s) for s in range(slots)]
        # the same ring for the C++ host layer (ttnn.linear_multi / linear_all_gather): it takes the points in its own order,
        # so one ring object serves either the ctypes callers (take / gather / wait below) or the host layer, not both
        from . import _ttnn
        self.native = _ttnn.GatherRing(rank, [int(b) for b in self.bases], slots, self.counter_bytes, self.slot_bytes)

    def _make_gather(self, s):
        g = PeerGather()
        g.ranks, g.rank = self.world, self.rank
        for r, b in enumerate(self.bases):
            g.out[r] = b + self.counter_bytes + s * self.slot_bytes
            g.arrived[r] = b + s * _COUNTER_STRIDE
        g.expected = self._own + s * _COUNTER_STRIDE + 128
        return g

    def _make_wait(self, s):
        w = PeerWait()
        w.arrived = self._own + s * _COUNTER_STRIDE
        w.expected = self._own + s * _COUNTER_STRIDE + 128
        return w

    def take(self, nbytes):
        """Next point of the ring (every rank calls this in the same order)."""
        if nbytes > self.slot_bytes:
            raise RuntimeError(f"gathered tensor of {nbytes} bytes exceeds the ring's {self.slot_bytes}-byte buffers")
        s = self._next
        self._next = (s + 1) % self.slots
        return s

    def gather(self, s):
        return self._gathers[s]

    def wait(self, s):
        return self._waits[s]

    def out_ptr(self, s):
        return self._own + self.counter_bytes + s * self.slot_bytes

    def stream_wait(self, s, stream=None):
        """Holds `stream` until point `s` is complete on this rank (for consumers other than ttb_matmul_peer)."""
        _check(_rt.cdll.ttb_peer_wait(ctypes.byref(self._waits[s]), stream))

    def close(self):
        """Unmaps the peers' arenas and frees this rank's. Only after every rank has stopped launching into this ring (the
        mesh replaces a ring behind a barrier), since peers store into this rank's arena."""
        for r, b in enumerate(self.bases):
            if r != self.rank and b:
                _rt.cdll.ttb_ipc_close(b)
        if self._own:
            _rt.cdll.ttb_free(self._own)
        self.bases, self._own, self.native = [], None, None

    def __del__(self):
        try:
            if getattr(self, "_own", None):
                _rt.cdll.ttb_device_synchronize()
                self.close()
        except Exception:
            pass
