"""The communicator entry points (ttb_comm_*) against a fake of the collective library, on the host: argument checks, a
peer that never joins (initialisation stays "in progress" -> time limit -> the half-built communicator is aborted), an
asynchronous error reported while polling, and the orderly path. No GPU is involved: the failures are produced by the
fake's return codes (ttb_comm_set_backend), never by a device."""
import ctypes

import pytest

import cabi

OK, IN_PROGRESS, REMOTE_ERROR = 0, 7, 6
_vp, _int = ctypes.c_void_p, ctypes.c_int


class Backend(ctypes.Structure):
    """ttb_comm_backend of include/ttb.h."""
    _fields_ = [("get_unique_id", ctypes.CFUNCTYPE(_int, _vp)),
                ("init_rank_config", ctypes.CFUNCTYPE(_int, ctypes.POINTER(_vp), _int, _vp, _int, _vp)),
                ("get_async_error", ctypes.CFUNCTYPE(_int, _vp, ctypes.POINTER(_int))),
                ("all_gather", ctypes.CFUNCTYPE(_int, _vp, _vp, ctypes.c_size_t, _int, _vp, _vp)),
                ("abort", ctypes.CFUNCTYPE(_int, _vp)),
                ("destroy", ctypes.CFUNCTYPE(_int, _vp)),
                ("error_string", ctypes.CFUNCTYPE(_vp, _int)),
                ("user", _vp)]


class Fake:
    """A collective library whose communicator stays in `state` (settable) and that records what was called."""

    def __init__(self, state=OK, ready_after=0):
        self.state, self.ready_after, self.polls, self.calls = state, ready_after, 0, []
        self._msg = ctypes.create_string_buffer(b"fake error")
        F = dict(Backend._fields_)
        self.table = Backend(
            F["get_unique_id"](self._uid), F["init_rank_config"](self._init), F["get_async_error"](self._poll),
            F["all_gather"](self._gather), F["abort"](self._abort), F["destroy"](self._destroy),
            F["error_string"](lambda code: ctypes.addressof(self._msg)), None)

    def _uid(self, ptr):
        ctypes.memset(ptr, 0x5A, 128)
        return OK

    def _init(self, comm_out, ranks, uid, rank, user):
        self.calls.append(("init", ranks, rank, ctypes.string_at(uid, 4)))
        comm_out[0] = 0x1234
        return IN_PROGRESS

    def _poll(self, comm, state_out):
        self.polls += 1
        state_out[0] = OK if (self.ready_after and self.polls > self.ready_after) else self.state
        return OK

    def _gather(self, src, dst, count, dtype, comm, stream):
        self.calls.append(("all_gather", src, dst, count, dtype))
        return OK

    def _abort(self, comm):
        self.calls.append(("abort", comm))
        return OK

    def _destroy(self, comm):
        self.calls.append(("destroy", comm))
        return OK


@pytest.fixture
def lib():
    lib = cabi.load()
    yield lib
    lib.cdll.ttb_comm_set_backend(None)


def _init(lib, ranks, rank, timeout_ms):
    comm = _vp()
    uid = ctypes.create_string_buffer(128)
    lib.check(lib.cdll.ttb_comm_unique_id(uid))
    return lib.cdll.ttb_comm_init(ctypes.byref(comm), ranks, rank, uid, timeout_ms), comm


def test_arguments_are_checked_before_the_library_is_touched(lib):
    fake = Fake()
    lib.check(lib.cdll.ttb_comm_set_backend(ctypes.byref(fake.table)))
    for ranks, rank in ((0, 0), (9, 0), (2, 2), (2, -1)):
        rc, comm = _init(lib, ranks, rank, 100)
        assert rc == -1 and not comm.value
    assert not [c for c in fake.calls if c[0] == "init"]
    assert lib.cdll.ttb_comm_init(None, 2, 0, None, 10) == -1
    assert lib.cdll.ttb_all_gather(None, 1, 2, 16, None) == -1


def test_a_peer_that_never_joins_ends_in_a_timeout_and_an_abort(lib):
    fake = Fake(state=IN_PROGRESS)
    lib.check(lib.cdll.ttb_comm_set_backend(ctypes.byref(fake.table)))
    rc, comm = _init(lib, 2, 0, 50)
    assert rc == -5 and b"not complete after 50 ms" in lib.cdll.ttb_last_error()
    assert not comm.value                                   # nothing usable is handed out
    assert fake.polls > 10 and ("abort", 0x1234) in fake.calls and not [c for c in fake.calls if c[0] == "destroy"]


def test_an_asynchronous_error_is_reported_and_abort_is_the_way_out(lib):
    fake = Fake(state=IN_PROGRESS, ready_after=3)           # joins after a few polls
    lib.check(lib.cdll.ttb_comm_set_backend(ctypes.byref(fake.table)))
    rc, comm = _init(lib, 2, 1, 1000)
    assert rc == 0 and comm.value
    assert fake.calls[0] == ("init", 2, 1, b"ZZZZ")         # the unique id travelled
    lib.check(lib.cdll.ttb_all_gather(comm, 0x1000, 0x2000, 4096, None))
    assert ("all_gather", 0x1000, 0x2000, 4096, 1) in fake.calls   # bytes: element type uint8
    assert lib.cdll.ttb_comm_check(comm, 100) == 0
    fake.ready_after, fake.state = 0, REMOTE_ERROR          # a peer died
    assert lib.cdll.ttb_comm_check(comm, 100) == -2 and b"asynchronous error" in lib.cdll.ttb_last_error()
    lib.check(lib.cdll.ttb_comm_abort(comm))
    assert fake.calls[-1] == ("abort", 0x1234)


def test_orderly_release(lib):
    fake = Fake(state=OK)
    lib.check(lib.cdll.ttb_comm_set_backend(ctypes.byref(fake.table)))
    rc, comm = _init(lib, 1, 0, 100)
    assert rc == 0
    assert lib.cdll.ttb_all_gather(comm, None, 0x2000, 16, None) == -1
    lib.check(lib.cdll.ttb_comm_destroy(comm))
    assert fake.calls[-1] == ("destroy", 0x1234)
    assert lib.cdll.ttb_comm_destroy(None) == 0 and lib.cdll.ttb_comm_abort(None) == 0
