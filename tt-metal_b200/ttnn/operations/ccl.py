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
