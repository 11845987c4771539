"""ttnn.all_gather (mirrors ttnn/ttnn/operations/ccl.py:26-39 and the AllGather op,
tt_eager/tt_dnn/op_library/all_gather/all_gather_op.cpp:18-104): every rank ends up with the concatenation of all
ranks' shards along `dim`, dtype and layout preserved. The ethernet ring of the reference is replaced by an NCCL
all-gather over NVLink (torch.distributed, one process per GPU)."""
import torch

from .. import _ttnn
from .. import types as T
from ..multi_device import MultiDeviceTensor

_BYTES = {T.bfloat16: 2, T.uint16: 2, T.float32: 4, T.uint32: 4}


class _DeviceBytes:
    """Zero-copy torch view of raw device memory through the CUDA array interface."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _as_torch_bytes(tensor, device_index):
    return torch.as_tensor(_DeviceBytes(tensor.buffer_address(), tensor.buffer_bytes()), device=torch.device("cuda", device_index))


def gather_plan(dims, padded, dtype, layout, dim, n):
    """Pure shape logic of the all-gather: how the rank-major concatenation an NCCL all-gather leaves relates to the
    result tensor. Returns (interleave, rows, row_bytes, out_dims, out_padded): when `interleave` is set the result is
    rows x [n shards x row_bytes] and a device kernel re-orders the staged buffer; otherwise the staged buffer already
    is the result."""
    rank = len(dims)
    d = dim if dim >= 0 else dim + rank
    if not 0 <= d < rank:
        raise RuntimeError(f"ttnn.all_gather: dim {dim} is out of range for a rank-{rank} tensor")
    tiled = layout == T.TILE_LAYOUT
    if tiled and rank < 2:
        raise RuntimeError("ttnn.all_gather: tiled tensors have at least two dimensions")
    outer_rows = 1
    for i in range(rank - (2 if tiled else 1)):
        outer_rows *= padded[i]
    if tiled:
        rows = outer_rows * (padded[-2] // 32)
        tile_bytes = {T.bfloat8_b: 1088, T.bfloat4_b: 576}.get(dtype) or 1024 * _BYTES[dtype]
        row_bytes = (padded[-1] // 32) * tile_bytes     # one tile row of this rank's shard
    else:
        rows = outer_rows
        row_bytes = padded[-1] * _BYTES[dtype]
    if d == rank - 1:
        interleave = rows > 1
    elif tiled and d == rank - 2 and outer_rows == 1:
        if dims[d] != padded[d]:
            raise RuntimeError("ttnn.all_gather: cannot concatenate padded tile rows")
        interleave = False   # shards are whole contiguous blocks: the rank-major concatenation is the result
    elif all(x == 1 for x in padded[:d]):
        interleave = False
    else:
        raise RuntimeError(f"ttnn.all_gather: gathering along dim {dim} of a rank-{rank} tensor is not supported")
    out_dims, out_padded = list(dims), list(padded)
    out_dims[d] *= n
    out_padded[d] *= n
    return interleave, rows, row_bytes, out_dims, out_padded


def all_gather(multidevice_tensor, dim: int, num_links: int = 1, *, memory_config: T.MemoryConfig = T.DRAM_MEMORY_CONFIG):
    if not isinstance(multidevice_tensor, MultiDeviceTensor):
        raise RuntimeError("ttnn.all_gather requires input tensors to be multi-device tensor")
    mesh = multidevice_tensor.mesh
    t = multidevice_tensor.local
    n = mesh.get_num_devices()
    if n == 1:
        return multidevice_tensor
    if t.storage_type() != T.StorageType.DEVICE:
        raise RuntimeError("ttnn.all_gather: the tensor must be on device")
    interleave, rows, row_bytes, out_dims, out_padded = gather_plan(list(t.shape), list(t.shape.padded), t.dtype, t.layout, dim, n)
    import torch.distributed as dist
    dev = t.device()
    src = _as_torch_bytes(t, dev.id())
    staged = torch.empty(n * src.numel(), dtype=torch.uint8, device=src.device)
    dist.all_gather_into_tensor(staged, src, group=mesh.process_group)
    if interleave:
        out = torch.empty_like(staged)
        from ..runtime import lib
        lib.gather_interleave(staged.data_ptr(), out.data_ptr(), n, rows, row_bytes)
    else:
        out = staged
    result = _ttnn.wrap_device_memory(out.data_ptr(), T.Shape(out_dims, out_padded), t.dtype, t.layout, dev)
    wrapped = MultiDeviceTensor(result, mesh)
    wrapped._keepalive = out     # the torch allocation owns the memory
    return wrapped


# ---- linear with the all-gather in its epilogue, and several linears of one activation in one launch ---------------------
_ACT = {None: 0, "relu": 1, "gelu": 2, "silu": 3}
_DTYPE_CODE = {T.bfloat16: 0, T.float32: 1, T.bfloat8_b: 3, T.bfloat4_b: 4}
_MM_WORKSPACE_ZEROED, _MM_WEIGHTS_RESIDENT = 8, 64


def _local(t):
    return t.local if isinstance(t, MultiDeviceTensor) or type(t).__name__ == "FusedOutput" else t


def _check_linear_operands(op, x, weights):
    if x.dtype != T.bfloat16 or x.layout != T.TILE_LAYOUT or x.storage_type() != T.StorageType.DEVICE:
        raise RuntimeError(f"{op}: the activation must be a bfloat16 TILE_LAYOUT tensor on device")
    padded = list(x.shape.padded)
    rows = 1
    for d in padded[:-1]:
        rows *= d
    K = padded[-1]
    fmt = weights[0].dtype
    for w in weights:
        if w.dtype not in (T.bfloat8_b, T.bfloat4_b) or w.dtype != fmt or w.layout != T.TILE_LAYOUT:
            raise RuntimeError(f"{op}: weights must be TILE_LAYOUT tensors of one block-float dtype")
        if w.storage_type() != T.StorageType.DEVICE:
            raise RuntimeError(f"{op}: weights must be on device")
        wp = list(w.shape.padded)
        if wp[-2] != K or any(d != 1 for d in wp[:-2]):
            raise RuntimeError(f"{op}: The width of the first tensor must be equal to the height of the second tensor")
    return rows, K, fmt


_STATES = {}


def _mesh_state(holder):
    """Scratch of the fused ops per mesh (or per device): split-K workspace (zero between launches), the ring of gather
    points, and the gather point that no launch has waited for yet."""
    key = id(holder)
    if key not in _STATES:
        _STATES[key] = {"ws": None, "ring": None, "pending": None, "holder": holder}
    return _STATES[key]


def _workspace(st, nbytes, device_index):
    if nbytes and (st["ws"] is None or st["ws"].numel() < nbytes):
        st["ws"] = torch.zeros(nbytes, dtype=torch.uint8, device=torch.device("cuda", device_index))
    return st["ws"]


_PLANS = {}          # launch descriptions of _fused_linear, keyed by the identity of the weights (which they keep alive)
_PLANS_MAX = 8192


def _fused_plan(op, x, weights, biases):
    """Everything about a fused launch that depends only on the weights, the biases and the activation's shape: validated
    once, then reused (a decode step calls the same few hundred launches over and over; rebuilding the argument arrays
    costs more host time than the kernels take on several GPUs)."""
    import ctypes
    from ..peer import _rt
    padded = tuple(x.shape.padded)
    key = (tuple(id(w) for w in weights), tuple(id(b) for b in biases) if biases is not None else None, padded, tuple(x.shape))
    plan = _PLANS.get(key)
    if plan is not None:
        return plan
    ws_local = [_local(w) for w in weights]
    rows, K, fmt = _check_linear_operands(op, x, ws_local)
    n = len(ws_local)
    if not 1 <= n <= 4:
        raise RuntimeError(f"{op}: between one and four weights per launch")
    Ns = [list(w.shape.padded)[-1] for w in ws_local]
    arr_n = (ctypes.c_int64 * n)(*Ns)
    arr_b = None
    if biases is not None:
        arr_b = (ctypes.c_void_p * n)(*[(_local(b).buffer_address() if b is not None else None) for b in biases])
    lead, lead_padded = list(x.shape)[:-1], list(padded)[:-1]
    offsets = [0]
    for N in Ns:
        offsets.append(offsets[-1] + rows * N)
    plan = {
        "keep": (list(weights), list(biases) if biases is not None else None),
        "rows": rows, "K": K, "fmt": _DTYPE_CODE[fmt], "n": n, "Ns": Ns, "arr_n": arr_n, "arr_b": arr_b,
        "arr_w": (ctypes.c_void_p * n)(*[w.buffer_address() for w in ws_local]),
        "need": _rt.cdll.ttb_matmul_multi_workspace_bytes(_DTYPE_CODE[fmt], 1, rows, K, n, arr_n),
        "offsets": offsets, "lead": lead, "lead_padded": lead_padded, "logical_N": [list(w.shape)[-1] for w in ws_local],
    }
    if len(_PLANS) >= _PLANS_MAX:
        _PLANS.clear()
    _PLANS[key] = plan
    return plan


def _fused_linear(op, input_tensor, weights, biases, activation, gather_first, ring_slots=8):
    """One launch of ttb_matmul_multi: up to four weights on one activation; optionally the first result is gathered over
    the mesh by the kernel's epilogue. Returns the list of results (MultiDeviceTensor when the input is one)."""
    import ctypes
    from ..peer import GatherRing, _rt, _check
    multi = isinstance(input_tensor, MultiDeviceTensor)
    mesh = input_tensor.mesh if multi else None
    x = _local(input_tensor)
    plan = _fused_plan(op, x, weights, biases)
    rows, K, n, Ns = plan["rows"], plan["K"], plan["n"], plan["Ns"]
    dev = x.device()
    st = _mesh_state(mesh if multi else dev)
    G = mesh.get_num_devices() if multi else 1
    gather = None
    slot = None
    if gather_first and G > 1:
        nbytes = G * rows * Ns[0] * 2
        if st["ring"] is None or st["ring"].slot_bytes < nbytes:
            # (re)built collectively: every rank reaches this point with the same shapes
            st["ring"] = GatherRing(mesh.local_index, G, max(nbytes, 1 << 20), slots=ring_slots, group=mesh.process_group)
        slot = st["ring"].take(nbytes)
        gather = ctypes.byref(st["ring"].gather(slot))
    wait = None
    in_slot = getattr(input_tensor, "_gather_slot", None) if multi else None
    if in_slot is not None:
        wait = ctypes.byref(st["ring"].wait(in_slot))      # the kernel itself waits for its gathered activation
        if st["pending"] == in_slot:
            st["pending"] = None
    if slot is not None and st["pending"] is not None:
        st["ring"].stream_wait(st["pending"])              # keeps the ranks within one gather of each other
        st["pending"] = None
    # one allocation for all local outputs of the launch
    first_local = 1 if gather is not None else 0
    offsets = plan["offsets"]
    total = offsets[n] - offsets[first_local]
    block = torch.empty(max(total, 1), dtype=torch.bfloat16, device=torch.device("cuda", dev.id())) if total else None
    base = block.data_ptr() if block is not None else 0
    ptrs = [None if j < first_local else base + 2 * (offsets[j] - offsets[first_local]) for j in range(n)]
    arr_o = (ctypes.c_void_p * n)(*ptrs)
    need = plan["need"]
    ws = _workspace(st, need, dev.id()) if need else None
    _check(_rt.cdll.ttb_matmul_multi(x.buffer_address(), 0, n, plan["arr_w"], plan["fmt"], plan["arr_b"], arr_o, 0, 1, rows, K, plan["arr_n"],
                                     _ACT[activation], _MM_WORKSPACE_ZEROED | _MM_WEIGHTS_RESIDENT,
                                     ws.data_ptr() if ws is not None else None, need, gather, wait, None))
    if slot is not None:
        st["pending"] = slot
    results = []
    lead, lead_padded = plan["lead"], plan["lead_padded"]
    for j in range(n):
        N, Nl = Ns[j], plan["logical_N"][j]
        if ptrs[j] is None:
            t = _ttnn.wrap_device_memory(st["ring"].out_ptr(slot), T.Shape(lead + [G * Nl], lead_padded + [G * N]), T.bfloat16, T.TILE_LAYOUT, dev)
            t = MultiDeviceTensor(t, mesh)
            t._gather_slot = slot
        else:
            t = _ttnn.wrap_device_memory(ptrs[j], T.Shape(lead + [Nl], lead_padded + [N]), T.bfloat16, T.TILE_LAYOUT, dev)
            if multi:
                t = MultiDeviceTensor(t, mesh)
                t._keepalive = block
            else:
                t = FusedOutput(t, block)
        results.append(t)
    return results


class FusedOutput:
    """A single-device result of linear_multi: the ttnn tensor plus the allocation that owns its memory. Behaves like the
    tensor for the operations of this package (they unwrap `.local`)."""

    def __init__(self, tensor, owner):
        self.local = tensor
        self._owner = owner

    shape = property(lambda self: self.local.shape)
    dtype = property(lambda self: self.local.dtype)
    layout = property(lambda self: self.local.layout)

    def __getattr__(self, name):
        return getattr(self.local, name)


def linear_multi(input_tensor, weights, *, biases=None, activation=None, all_gather_first=False):
    """[ttnn.linear(x, w, bias=b, activation=activation) for w, b in zip(weights, biases)] as ONE launch: the weights share
    the activation (q / k / v projections; w1 / w3 of a gated MLP) and stay separate tensors. Decode shapes (at most 256
    rows, every N a multiple of 128, block-float weights). Results equal those of the separate calls. With
    all_gather_first the first result is gathered along its last dimension over the mesh by the kernel's own epilogue
    (see linear_all_gather)."""
    return _fused_linear("ttnn.linear_multi", input_tensor, weights, biases, activation, all_gather_first)


def linear_all_gather(input_tensor, weight, *, bias=None, activation=None, dim=-1, num_links=1, ring_slots=8):
    """ttnn.all_gather(ttnn.linear(x, w, bias=bias, activation=activation), dim=-1) as one kernel: every rank computes the
    columns of its weight shard and stores each finished tile into every rank's copy of the result over NVLink (plain
    peer stores, no separate collective). The result carries the gather point it came from; ttnn.linear_multi /
    linear_all_gather on it wait inside their own kernel, every other use (ttnn.to_torch, ttnn.linear, ...) first holds the
    stream until the result is complete. The result lives in a ring of `ring_slots` buffers: it stays valid until
    ring_slots - 1 further gathering launches on this mesh."""
    if not isinstance(input_tensor, MultiDeviceTensor) or not isinstance(weight, MultiDeviceTensor):
        raise RuntimeError("ttnn.linear_all_gather requires input tensors to be multi-device tensor")
    if dim not in (-1, len(list(input_tensor.shape)) - 1):
        raise RuntimeError("ttnn.linear_all_gather: only the last dimension can be gathered")
    return _fused_linear("ttnn.linear_all_gather", input_tensor, [weight], [bias] if bias is not None else None, activation, True,
                         ring_slots)[0]


def wait_for_gather(tensor):
    """Holds the stream until a linear_all_gather result is complete on this rank (no-op for other tensors); called by
    every consumer that is not itself a fused linear."""
    if isinstance(tensor, MultiDeviceTensor) and getattr(tensor, "_gather_slot", None) is not None:
        st = _mesh_state(tensor.mesh)
        st["ring"].stream_wait(tensor._gather_slot)
        if st["pending"] == tensor._gather_slot:
            st["pending"] = None
        tensor._gather_slot = None
    return tensor
