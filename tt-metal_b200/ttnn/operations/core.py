"""from_torch / to_torch / to_layout / to_device / from_device / reshape / tensor cache.

Mirrors ttnn/ttnn/operations/core.py of the reference (from_torch :245-311, to_torch :336-394, to_device :409-445,
from_device :460-482, to_layout :609-803, as_tensor / dump_tensor / load_tensor :806-980). torch tensors exist
only here: the C++ host layer receives data pointers and shapes. All conversions run as CUDA kernels; without a
usable GPU they raise instead of falling back to the CPU.
"""
import json
import os
import pathlib
import struct
from typing import Optional

import torch

from .. import _ttnn
from .. import types as T
from ..multi_device import MultiDeviceTensor, TensorToMesh, MeshToTensor

_TORCH_TO_TTNN = {torch.bfloat16: T.bfloat16, torch.float32: T.float32, torch.int32: T.uint32, torch.int16: T.uint16}
_TTNN_TO_TORCH = {T.bfloat16: torch.bfloat16, T.float32: torch.float32, T.uint32: torch.int32, T.uint16: torch.int16}


def _is_block_float(dtype):
    return dtype in (T.bfloat8_b, T.bfloat4_b)


def _unwrap(tensor):
    if isinstance(tensor, MultiDeviceTensor):
        if getattr(tensor, "_gather_slot", None) is not None:
            from .ccl import wait_for_gather     # result of a fused linear + all-gather: hold the stream until it is complete
            wait_for_gather(tensor)
        return tensor.local
    if type(tensor).__name__ == "FusedOutput":     # single-device result of ttnn.linear_multi
        return tensor.local
    return tensor


def _rewrap(like, tensor):
    return MultiDeviceTensor(tensor, like.mesh) if isinstance(like, MultiDeviceTensor) else tensor


def from_torch(tensor: "torch.Tensor", dtype: Optional[T.DataType] = None, *, layout: Optional[T.Layout] = T.ROW_MAJOR_LAYOUT,
               device=None, memory_config: Optional[T.MemoryConfig] = None, mesh_mapper: Optional[TensorToMesh] = None):
    """Converts a torch.Tensor into a ttnn.Tensor of `dtype` and `layout`, on `device` when one is given.

    bfloat8_b / bfloat4_b need TILE_LAYOUT and at least two dimensions; the last two dimensions are zero-padded to
    multiples of 32 and the logical shape is remembered. With `mesh_mapper` each rank keeps its own shard."""
    if not isinstance(tensor, torch.Tensor):
        raise RuntimeError("ttnn.from_torch: expected a torch.Tensor")
    if _is_block_float(dtype):
        if len(tensor.shape) < 2:
            raise RuntimeError("ttnn.from_torch: bfloat8_b/bfloat4_b requires at least 2 dimensions!")
        if layout != T.TILE_LAYOUT:
            raise RuntimeError("ttnn.from_torch: bfloat8_b/bfloat4_b requires TILE_LAYOUT!")
    if memory_config is not None and device is None:
        raise RuntimeError("device must be specified when memory_config is specified")
    mesh = None
    if mesh_mapper is not None:
        mesh = mesh_mapper.device_mesh
        shards = mesh_mapper.map(tensor)
        tensor = shards[mesh.local_index]
        if device is None:
            device = None
    if layout is None:
        layout = T.ROW_MAJOR_LAYOUT
    if dtype is None:
        if tensor.dtype not in _TORCH_TO_TTNN:
            raise RuntimeError(f"ttnn.from_torch: unsupported torch dtype {tensor.dtype}")
        dtype = _TORCH_TO_TTNN[tensor.dtype]
    if _is_block_float(dtype):
        # block-float tensors are packed from fp32 (bf16 sources are widened exactly inside the kernel)
        if tensor.dtype not in (torch.float32, torch.bfloat16):
            tensor = tensor.to(torch.float32)
        src_dtype = _TORCH_TO_TTNN[tensor.dtype]
    else:
        want = _TTNN_TO_TORCH[dtype]
        if tensor.dtype != want:
            tensor = tensor.to(want)  # torch's own conversion (round-to-nearest-even for bfloat16), like the reference
        src_dtype = dtype
    tensor = tensor.detach().contiguous()
    if tensor.device.type != "cpu":
        tensor = tensor.cpu()
    if tensor.dim() == 0:
        raise RuntimeError("ttnn.from_torch: rank-0 tensors are not supported")
    out = _ttnn.from_host_pointer(tensor.data_ptr(), list(tensor.shape), src_dtype, dtype, layout, device)
    return MultiDeviceTensor(out, mesh) if mesh is not None else out


def to_torch(tensor, *, torch_rank: Optional[int] = None, mesh_composer: Optional[MeshToTensor] = None) -> "torch.Tensor":
    """Converts a ttnn.Tensor into a torch.Tensor of its logical shape: float32 for block-float tensors, the matching
    torch dtype otherwise."""
    if mesh_composer is not None:
        return mesh_composer.compose(tensor)
    t = _unwrap(tensor)
    host_dtype = t.host_dtype()
    out = torch.empty(tuple(t.shape), dtype=_TTNN_TO_TORCH[host_dtype])
    t.copy_to_host_pointer(out.data_ptr())
    if torch_rank is None:
        return out
    while out.dim() != torch_rank:
        if out.shape[0] != 1:
            raise RuntimeError("ttnn: Unable to squeeze to desired rank!")
        out = out.squeeze(0)
    return out


def to_layout(tensor, layout: T.Layout, dtype=None, memory_config=None, use_multicore=False):
    if layout not in (T.ROW_MAJOR_LAYOUT, T.TILE_LAYOUT):
        raise RuntimeError(f"Unsupported layout: {layout}")
    t = _unwrap(tensor)
    if dtype is not None and dtype != t.dtype:
        # the reference converts the data type only while tilizing a device tensor (ttl.tensor.tilize(output_dtype=dtype),
        # core.py:677-711); everything else is "Unsupported datatype conversion"
        if t.storage_type() != T.StorageType.DEVICE or layout != T.TILE_LAYOUT:
            raise RuntimeError(f"Unsupported datatype conversion to {dtype}")
        return _rewrap(tensor, _ttnn.to_tile_layout_as(t, dtype))
    return _rewrap(tensor, _ttnn.to_layout(t, layout))


def to_device(tensor, device, *, memory_config: T.MemoryConfig = T.DRAM_MEMORY_CONFIG):
    return _rewrap(tensor, _ttnn.to_device(_unwrap(tensor), device))


def from_device(tensor):
    return _rewrap(tensor, _ttnn.from_device(_unwrap(tensor)))


def deallocate(tensor, *, force=True):
    _unwrap(tensor).deallocate(force)


def reshape(tensor, shape):
    if not isinstance(shape, T.Shape):
        shape = T.Shape(list(shape))
    return _rewrap(tensor, _unwrap(tensor).reshape(shape))


def is_tensor_storage_on_device(tensor) -> bool:
    return _unwrap(tensor).storage_type() == T.StorageType.DEVICE


# ---- packed-tensor cache ---------------------------------------------------------------------------------
# A portable container for converted weights so that a 70B-parameter model is packed once:
#   8 bytes magic "TTNNB200", uint32 header length, JSON header {shape, padded_shape, dtype, layout, nbytes},
#   then the physical buffer bytes (packed tiles for block-float).
# The reference's dump_tensor writes an in-memory C++ struct (tt_eager/tensor/serialization.cpp:87-141), which is
# not portable; the file-naming convention of as_tensor is kept.
_MAGIC = b"TTNNB200"


def dump_tensor(file_name, tensor) -> None:
    t = _unwrap(tensor)
    raw = t.buffer()
    header = json.dumps({"shape": list(t.shape), "padded_shape": list(t.shape.padded), "dtype": t.dtype.name,
                         "layout": t.layout.name, "nbytes": len(raw)}).encode()
    with open(file_name, "wb") as f:
        f.write(_MAGIC)
        f.write(struct.pack("<I", len(header)))
        f.write(header)
        f.write(raw)


def load_tensor(file_name, *, device=None):
    with open(file_name, "rb") as f:
        if f.read(8) != _MAGIC:
            raise RuntimeError(f"ttnn.load_tensor: {file_name} is not a tensor cache file")
        (hlen,) = struct.unpack("<I", f.read(4))
        header = json.loads(f.read(hlen))
        raw = f.read(header["nbytes"])
    if len(raw) != header["nbytes"]:
        raise RuntimeError(f"ttnn.load_tensor: {file_name} is truncated")
    t = _ttnn.tensor_from_buffer(raw, T.Shape(header["shape"], header["padded_shape"]), getattr(T.DataType, header["dtype"]),
                                 getattr(T.Layout, header["layout"]))
    return _ttnn.to_device(t, device) if device is not None else t


def as_tensor(tensor, dtype=None, *, layout=T.ROW_MAJOR_LAYOUT, device=None, memory_config=None, cache_file_name=None,
              mesh_mapper=None):
    """from_torch with an optional on-disk cache of the converted tensor (file name convention of the reference:
    `<cache_file_name>_dtype_<DTYPE>_layout_<LAYOUT>.bin`)."""
    if cache_file_name is None or mesh_mapper is not None:
        return from_torch(tensor, dtype, layout=layout, device=device, memory_config=memory_config, mesh_mapper=mesh_mapper)
    dtype_name = (dtype or _TORCH_TO_TTNN[tensor.dtype]).name
    path = pathlib.Path(f"{cache_file_name}_dtype_{dtype_name}_layout_{layout.name}.bin")
    if path.exists():
        try:
            return load_tensor(str(path), device=device)
        except RuntimeError:
            pass
    out = from_torch(tensor, dtype, layout=layout, device=device, memory_config=memory_config)
    path.parent.mkdir(parents=True, exist_ok=True)
    dump_tensor(str(path), out)
    return out
