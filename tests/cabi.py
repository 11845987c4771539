"""ctypes view of libttb.so for the tests: every entry point of include/ttb.h with its argument types.

The GPU parity tests call the library through this module only, i.e. through the C ABI, with torch
tensors providing device memory (their data_ptr())."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(ROOT, "tt-metal_b200", "lib", "libttb.so")
HEADER = os.path.join(ROOT, "include", "ttb.h")

BFLOAT16, FLOAT32, UINT32, BFLOAT8_B, BFLOAT4_B, UINT16 = 0, 1, 2, 3, 4, 6
ACT_NONE, ACT_RELU, ACT_GELU, ACT_SILU = 0, 1, 2, 3
MM_A_ROW_MAJOR, MM_OUT_ROW_MAJOR, MM_FORCE_GENERIC, MM_WORKSPACE_ZEROED, MM_DECODE_TMEM_OPERAND, MM_DETERMINISTIC = 1, 2, 4, 8, 16, 32
MM_WEIGHTS_RESIDENT = 64
MM_DECODE_SMEM_OPERAND = 128
MM_GATED = 256
TILE_BYTES = {BFLOAT8_B: 1088, BFLOAT4_B: 576}

_vp, _i32, _i64, _sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_size_t

_SIGS = {
    "ttb_last_error": (ctypes.c_char_p, []),
    "ttb_version": (_i32, []),
    "ttb_device_count": (_i32, [ctypes.POINTER(_i32)]),
    "ttb_set_device": (_i32, [_i32]),
    "ttb_get_device": (_i32, [ctypes.POINTER(_i32)]),
    "ttb_malloc": (_i32, [ctypes.POINTER(_vp), _sz]),
    "ttb_free": (_i32, [_vp]),
    "ttb_host_alloc": (_i32, [ctypes.POINTER(_vp), _sz]),
    "ttb_host_free": (_i32, [_vp]),
    "ttb_memcpy_h2d": (_i32, [_vp, _vp, _sz, _vp]),
    "ttb_memcpy_d2h": (_i32, [_vp, _vp, _sz, _vp]),
    "ttb_memcpy_d2d": (_i32, [_vp, _vp, _sz, _vp]),
    "ttb_memset": (_i32, [_vp, _i32, _sz, _vp]),
    "ttb_stream_synchronize": (_i32, [_vp]),
    "ttb_device_synchronize": (_i32, []),
    "ttb_nvtx_push": (_i32, [ctypes.c_char_p]),
    "ttb_nvtx_pop": (_i32, []),
    "ttb_buffer_bytes": (_i64, [_i32, _i64, _i64, _i64]),
    "ttb_tilize": (_i32, [_vp, _vp, _i32, _i64, _i64, _i64, _vp]),
    "ttb_untilize": (_i32, [_vp, _vp, _i32, _i64, _i64, _i64, _vp]),
    "ttb_pad": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, ctypes.c_uint32, _vp]),
    "ttb_unpad": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, _vp]),
    "ttb_mul_bf16": (_i32, [_vp, _vp, _vp, _i64, _vp]),
    "ttb_pack_bfp": (_i32, [_vp, _i32, _vp, _i32, _i64, _i64, _i64, _i32, _i32, _vp]),
    "ttb_unpack_bfp": (_i32, [_vp, _i32, _vp, _i32, _i64, _i64, _i64, _i32, _i32, _vp]),
    "ttb_matmul_workspace_bytes": (_i64, [_i32, _i64, _i64, _i64, _i64, _i32]),
    "ttb_matmul_plan": (_i32, [_i32, _i64, _i64, _i64, _i64, _i32, _vp, _i32]),
    "ttb_matmul": (_i32, [_vp, _i32, _vp, _i32, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _i32, _i32, _vp, _i64, _vp]),
    "ttb_bmm": (_i32, [_vp, _i32, _vp, _i32, _vp, _i32, _i64, _i64, _i64, _i64, _vp]),
    "ttb_matmul_decode_static": (_i32, [_vp, _i32, _vp, _i32, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _i32, _i32, _vp]),
    "ttb_matmul_decode_static_scratch_bytes": (_i64, [_i32, _i64, _i64, _i64, _i64]),
    "ttb_check_status": (_i32, [_vp]),
    "ttb_set_wait_limit_cycles": (_i32, [_i64]),
    "ttb_mem_info": (_i32, [ctypes.POINTER(_i64), ctypes.POINTER(_i64)]),
    "ttb_gather_interleave": (_i32, [_vp, _vp, _i32, _i32, _i64, _i64, _vp]),
    "ttb_matmul_peer_workspace_bytes": (_i64, [_i32, _i64, _i64, _i64, _i64]),
    "ttb_matmul_peer": (_i32, [_vp, _i32, _vp, _i32, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _i32, _i32, _vp, _i64, _vp, _vp, _vp]),
    "ttb_peer_wait": (_i32, [_vp, _vp]),
    "ttb_matmul_decode_plan": (_i32, [_i32, _i64, _i64, _i64, _i32, _vp, _vp, _i32]),
    "ttb_matmul_gated_workspace_bytes": (_i64, [_i32, _i64, _i64, _i64, _i64]),
    "ttb_matmul_multi_workspace_bytes": (_i64, [_i32, _i64, _i64, _i64, _i32, _vp]),
    "ttb_matmul_multi": (_i32, [_vp, _i32, _i32, _vp, _i32, _vp, _vp, _i32, _i64, _i64, _i64, _vp, _i32, _i32, _vp, _i64, _vp, _vp, _vp]),
    "ttb_matmul_sequence_workspace_bytes": (_i64, [_i32, _i64, _i64, _vp, _i32]),
    "ttb_matmul_sequence": (_i32, [_vp, _i32, _i32, _i32, _i64, _i64, _i32, _vp, _i64, _vp]),
    "ttb_comm_unique_id": (_i32, [_vp]),
    "ttb_comm_init": (_i32, [ctypes.POINTER(_vp), _i32, _i32, _vp, _i64]),
    "ttb_comm_check": (_i32, [_vp, _i64]),
    "ttb_all_gather": (_i32, [_vp, _vp, _vp, _i64, _vp]),
    "ttb_comm_abort": (_i32, [_vp]),
    "ttb_comm_destroy": (_i32, [_vp]),
    "ttb_comm_set_backend": (_i32, [_vp]),
    "ttb_ipc_export": (_i32, [_vp, _vp]),
    "ttb_ipc_open": (_i32, [_vp, ctypes.POINTER(_vp)]),
    "ttb_ipc_close": (_i32, [_vp]),
}

MAX_RANKS = 8


class PeerGather(ctypes.Structure):
    """ttb_peer_gather of include/ttb.h."""
    _fields_ = [("ranks", _i32), ("rank", _i32), ("out", _vp * MAX_RANKS), ("arrived", _vp * MAX_RANKS), ("expected", _vp)]


class PeerWait(ctypes.Structure):
    """ttb_peer_wait_t of include/ttb.h."""
    _fields_ = [("arrived", _vp), ("expected", _vp)]


MAX_GROUP, MAX_STAGES = 4, 4


class MatmulStage(ctypes.Structure):
    """ttb_matmul_stage of include/ttb.h."""
    _fields_ = [("a", _vp), ("count", _i32), ("w", _vp * MAX_GROUP), ("bias", _vp * MAX_GROUP), ("out", _vp * MAX_GROUP),
                ("out_dtype", _i32), ("K", _i64), ("N", _i64 * MAX_GROUP), ("activation", _i32), ("flags", _i32),
                ("gather", ctypes.POINTER(PeerGather)), ("wait", ctypes.POINTER(PeerWait)), ("input_from", _i32)]


def matmul_stage(a, ws, outs, K, Ns, biases=None, out_dtype=BFLOAT16, act=ACT_NONE, flags=0, gather=None, wait=None, input_from=-1):
    """One stage from device addresses (ints); `gather` / `wait` are PeerGather / PeerWait objects the caller keeps alive."""
    st = MatmulStage()
    st.a, st.count, st.out_dtype, st.K, st.activation, st.flags, st.input_from = a, len(ws), out_dtype, K, act, flags, input_from
    for j, w in enumerate(ws):
        st.w[j], st.out[j], st.N[j] = w, outs[j], Ns[j]
        st.bias[j] = biases[j] if biases else None
    if gather is not None:
        st.gather = ctypes.pointer(gather)
    if wait is not None:
        st.wait = ctypes.pointer(wait)
    return st


def peer_gather(rank, outs, arrived, uses):
    g = PeerGather()
    g.ranks, g.rank = len(outs), rank
    for r, (o, a) in enumerate(zip(outs, arrived)):
        g.out[r], g.arrived[r] = o, a
    g.expected = uses
    return g


def peer_wait(arrived, expected):
    w = PeerWait()
    w.arrived, w.expected = arrived, expected
    return w


def declared_symbols():
    """Names of all functions declared in include/ttb.h."""
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ttb_[a-z0-9_]+)\s*\(", text)))


class TtbError(RuntimeError):
    pass


class Lib:
    def __init__(self, path=LIB_PATH):
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` first")
        self.cdll = ctypes.CDLL(path)
        for name, (res, args) in _SIGS.items():
            if hasattr(self.cdll, name):
                fn = getattr(self.cdll, name)
                fn.restype, fn.argtypes = res, args

    def check(self, rc):
        if rc != 0:
            raise TtbError(f"libttb status {rc}: {self.cdll.ttb_last_error().decode()}")

    def __getattr__(self, name):
        return getattr(self.cdll, "ttb_" + name)

    # ---- conveniences over torch CUDA tensors (device memory only) --------------------------------
    def pack(self, src, fmt, outer, H, W, row_major=True, two_pass=False):
        import torch
        Hp, Wp = (H + 31) // 32 * 32, (W + 31) // 32 * 32
        out = torch.empty(outer * Hp * Wp // 1024 * TILE_BYTES[fmt], dtype=torch.uint8, device=src.device)
        sd = FLOAT32 if src.dtype == torch.float32 else BFLOAT16
        self.check(self.pack_bfp(src.data_ptr(), sd, out.data_ptr(), fmt, outer, H, W, int(row_major), int(two_pass), None))
        return out

    def unpack(self, packed, fmt, outer, H, W, row_major=True, two_pass=False, dtype=None):
        import torch
        dtype = dtype or torch.float32
        n = outer * H * W if row_major else outer * ((H + 31) // 32 * 32) * ((W + 31) // 32 * 32)
        out = torch.empty(n, dtype=dtype, device=packed.device)
        dd = FLOAT32 if dtype == torch.float32 else BFLOAT16
        self.check(self.unpack_bfp(packed.data_ptr(), fmt, out.data_ptr(), dd, outer, H, W, int(row_major), int(two_pass), None))
        return out

    def tilize(self, src, outer, H, W):
        import torch
        Hp, Wp = (H + 31) // 32 * 32, (W + 31) // 32 * 32
        out = torch.empty(outer * Hp * Wp, dtype=src.dtype, device=src.device)
        self.check(self.cdll.ttb_tilize(src.data_ptr(), out.data_ptr(), src.element_size(), outer, H, W, None))
        return out

    def untilize(self, src, outer, H, W):
        import torch
        out = torch.empty(outer * H * W, dtype=src.dtype, device=src.device)
        self.check(self.cdll.ttb_untilize(src.data_ptr(), out.data_ptr(), src.element_size(), outer, H, W, None))
        return out

    def matmul(self, a, w, w_dtype, batch, M, K, N, bias=None, act=ACT_NONE, flags=0, out_fp32=False):
        """a: bf16 device tensor (tiled unless MM_A_ROW_MAJOR), w: packed/tiled weight bytes; returns the output tensor."""
        import torch
        out = torch.empty(batch * M * N, dtype=torch.float32 if out_fp32 else torch.bfloat16, device=a.device)
        ws_bytes = self.matmul_workspace_bytes(w_dtype, batch, M, K, N, flags)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=a.device) if ws_bytes else None
        self.check(self.cdll.ttb_matmul(a.data_ptr(), BFLOAT16, w.data_ptr(), w_dtype, bias.data_ptr() if bias is not None else None,
                                        out.data_ptr(), FLOAT32 if out_fp32 else BFLOAT16, batch, M, K, N, act, flags,
                                        ws.data_ptr() if ws is not None else None, ws_bytes, None))
        self.check(self.check_status(None))
        return out


_lib = None


def load():
    global _lib
    if _lib is None:
        _lib = Lib()
    return _lib
