"""Direct ctypes access to the few libttb entry points the Python layer calls itself."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))


class _Lib:
    def __init__(self):
        path = os.path.join(os.path.dirname(_HERE), "lib", "libttb.so")
        self.cdll = ctypes.CDLL(path)
        self.cdll.ttb_last_error.restype = ctypes.c_char_p
        self.cdll.ttb_gather_interleave.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int64,
                                                    ctypes.c_int64, ctypes.c_void_p]

    def gather_interleave(self, src, dst, ranks, rows, row_bytes):
        rc = self.cdll.ttb_gather_interleave(src, dst, 1, ranks, rows, row_bytes, None)
        if rc != 0:
            raise RuntimeError(self.cdll.ttb_last_error().decode())


lib = _Lib()
