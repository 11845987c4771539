"""CPU oracle for the block-float weight path. TEST INFRASTRUCTURE ONLY.

Two checkers, both reached through ctypes and numpy arrays:

* ``port``  - ``libbfp_oracle.so``, the plain-C restatement in ``bfp_oracle.c``;
* ``ref``   - ``_ref/libttref.so``, the reference's own host headers compiled out of tree
  (present only where the reference tree was available at build time, or where a prebuilt
  copy travelled with the repository).

Only the tests, the smoke check and the bench's CPU-baseline leg may import this package.
The product (the ``ttnn`` package and ``libttb.so``) never does.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
BFP8_B, BFP4_B = 0, 1
TILE_BYTES = {BFP8_B: 1088, BFP4_B: 576}

_i64, _int, _vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p


def build(reference_root="/root/reference"):
    """Compile the C restatement and, when the reference tree exists, the reference wrapper."""
    subprocess.check_call(["make", "-s", "-C", _HERE, f"REF={reference_root}"])


def _ptr(a):
    return a.ctypes.data_as(_vp)


class _Port:
    def __init__(self):
        path = os.path.join(_HERE, "libbfp_oracle.so")
        if not os.path.exists(path):
            build()
        self.lib = ctypes.CDLL(path)
        L = self.lib
        L.orc_tilize.argtypes = [_vp, _vp, _int, _i64, _i64, _i64]
        L.orc_untilize.argtypes = [_vp, _vp, _int, _i64, _i64, _i64]
        L.orc_pack_bfp.argtypes = [_vp, _vp, _int, _i64, _int]
        L.orc_unpack_bfp.argtypes = [_vp, _vp, _int, _i64, _int]
        L.orc_from_torch_bfp.argtypes = [_vp, _vp, _int, _i64, _i64, _i64, _vp]
        L.orc_to_torch_bfp.argtypes = [_vp, _vp, _int, _i64, _i64, _i64, _vp]
        for f in (L.orc_tilize, L.orc_untilize, L.orc_pack_bfp, L.orc_unpack_bfp, L.orc_from_torch_bfp,
                  L.orc_to_torch_bfp):
            f.restype = None

    def tilize(self, x, outer, H, W):
        """x: contiguous array of outer*H*W elements of 2 or 4 bytes; returns the tiled array."""
        x = np.ascontiguousarray(x)
        out = np.empty_like(x)
        self.lib.orc_tilize(_ptr(x), _ptr(out), x.dtype.itemsize, outer, H, W)
        return out

    def untilize(self, x, outer, H, W):
        x = np.ascontiguousarray(x)
        out = np.empty_like(x)
        self.lib.orc_untilize(_ptr(x), _ptr(out), x.dtype.itemsize, outer, H, W)
        return out

    def pack(self, x, fmt, in_tile_row_major=False):
        """x: fp32 (or uint32 bit patterns), size a multiple of 1024; returns the packed bytes."""
        bits = np.ascontiguousarray(x).reshape(-1).view(np.uint32)
        nt = bits.size // 1024
        out = np.empty(nt * TILE_BYTES[fmt], np.uint8)
        self.lib.orc_pack_bfp(_ptr(bits), _ptr(out), fmt, nt, int(in_tile_row_major))
        return out

    def unpack(self, packed, fmt, in_tile_row_major=False):
        """packed: uint8 tiles; returns fp32 values (viewable as uint32 bit patterns)."""
        p = np.ascontiguousarray(packed).reshape(-1).view(np.uint8)
        nt = p.size // TILE_BYTES[fmt]
        out = np.empty(nt * 1024, np.uint32)
        self.lib.orc_unpack_bfp(_ptr(p), _ptr(out), fmt, nt, int(in_tile_row_major))
        return out.view(np.float32)

    def from_torch(self, x, fmt, outer, H, W):
        bits = np.ascontiguousarray(x).reshape(-1).view(np.uint32)
        n = outer * H * W
        out = np.empty(n // 1024 * TILE_BYTES[fmt], np.uint8)
        scratch = np.empty(8 * n + out.size + 64, np.uint8)
        self.lib.orc_from_torch_bfp(_ptr(bits), _ptr(out), fmt, outer, H, W, _ptr(scratch))
        return out

    def to_torch(self, packed, fmt, outer, H, W):
        p = np.ascontiguousarray(packed).reshape(-1).view(np.uint8)
        n = outer * H * W
        out = np.empty(n, np.uint32)
        scratch = np.empty(8 * n + p.size + 64, np.uint8)
        self.lib.orc_to_torch_bfp(_ptr(p), _ptr(out), fmt, outer, H, W, _ptr(scratch))
        return out.view(np.float32)


class _Ref:
    def __init__(self):
        path = os.path.join(_HERE, "_ref", "libttref.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = ctypes.CDLL(path)
        L = self.lib
        L.ref_tilize_f32.argtypes = [_vp, _vp, _i64, _i64, _i64]
        L.ref_untilize_f32.argtypes = [_vp, _vp, _i64, _i64, _i64]
        L.ref_pack_bfp.argtypes = [_vp, _vp, _int, _i64, _int]
        L.ref_unpack_bfp.argtypes = [_vp, _vp, _int, _i64, _int]
        L.ref_from_torch_bfp.argtypes = [_vp, _vp, _int, _i64, _i64, _i64]
        L.ref_to_torch_bfp.argtypes = [_vp, _vp, _int, _i64, _i64, _i64]
        for f in (L.ref_tilize_f32, L.ref_untilize_f32, L.ref_pack_bfp, L.ref_unpack_bfp, L.ref_from_torch_bfp,
                  L.ref_to_torch_bfp):
            f.restype = None

    def tilize(self, x, outer, H, W):
        x = np.ascontiguousarray(x).view(np.float32)
        out = np.empty_like(x)
        self.lib.ref_tilize_f32(_ptr(x), _ptr(out), outer, H, W)
        return out

    def untilize(self, x, outer, H, W):
        x = np.ascontiguousarray(x).view(np.float32)
        out = np.empty_like(x)
        self.lib.ref_untilize_f32(_ptr(x), _ptr(out), outer, H, W)
        return out

    def pack(self, x, fmt, in_tile_row_major=False):
        x = np.ascontiguousarray(x).reshape(-1).view(np.float32)
        nt = x.size // 1024
        out = np.empty(nt * TILE_BYTES[fmt], np.uint8)
        self.lib.ref_pack_bfp(_ptr(x), _ptr(out), fmt, nt, int(in_tile_row_major))
        return out

    def unpack(self, packed, fmt, in_tile_row_major=False):
        p = np.ascontiguousarray(packed).reshape(-1).view(np.uint8)
        nt = p.size // TILE_BYTES[fmt]
        out = np.empty(nt * 1024, np.float32)
        self.lib.ref_unpack_bfp(_ptr(p), _ptr(out), fmt, nt, int(in_tile_row_major))
        return out

    def from_torch(self, x, fmt, outer, H, W):
        x = np.ascontiguousarray(x).reshape(-1).view(np.float32)
        out = np.empty(outer * H * W // 1024 * TILE_BYTES[fmt], np.uint8)
        self.lib.ref_from_torch_bfp(_ptr(x), _ptr(out), fmt, outer, H, W)
        return out

    def to_torch(self, packed, fmt, outer, H, W):
        p = np.ascontiguousarray(packed).reshape(-1).view(np.uint8)
        out = np.empty(outer * H * W, np.float32)
        self.lib.ref_to_torch_bfp(_ptr(p), _ptr(out), fmt, outer, H, W)
        return out


_port = None
_ref = None


def port():
    global _port
    if _port is None:
        _port = _Port()
    return _port


def ref():
    """The compiled reference, or None where it is not available."""
    global _ref
    if _ref is None:
        try:
            _ref = _Ref()
        except (FileNotFoundError, OSError):
            return None
    return _ref


def comp_pcc(golden, calculated):
    """Pearson correlation as the reference's tests compute it (models/utility_functions.py:544-596):
    both-all-NaN counts as 1, one-all-NaN or one-all-zero as 0, NaN/Inf are replaced by 0, equal
    tensors give 1, otherwise the smallest entry of the 2x2 correlation matrix of the flattened data."""
    g = np.asarray(golden, np.float64).reshape(-1).copy()
    c = np.asarray(calculated, np.float64).reshape(-1).copy()
    if np.all(np.isnan(g)) and np.all(np.isnan(c)):
        return 1.0
    if np.all(np.isnan(g)) or np.all(np.isnan(c)):
        return 0.0
    if bool(np.any(g != 0)) != bool(np.any(c != 0)):
        return 0.0
    g[~np.isfinite(g)] = 0
    c[~np.isfinite(c)] = 0
    if np.array_equal(g, c):
        return 1.0
    r = np.min(np.ma.corrcoef(np.ma.masked_invalid(g), np.ma.masked_invalid(c)))
    if isinstance(r, np.ma.core.MaskedConstant):
        return 1.0
    return float(r)
