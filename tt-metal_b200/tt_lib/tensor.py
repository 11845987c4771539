"""tt_lib.tensor: the Tensor class, its enums and the tensor-level ops of the block-float weight path."""
from typing import List, Optional, Sequence, Union

import ttnn
from ttnn import _ttnn
from ttnn.multi_device import MultiDeviceTensor

Tensor = _ttnn.Tensor
DataType = _ttnn.DataType
Layout = _ttnn.Layout
StorageType = _ttnn.StorageType
BufferType = _ttnn.BufferType
TensorMemoryLayout = _ttnn.TensorMemoryLayout
MemoryConfig = _ttnn.MemoryConfig
MathFidelity = _ttnn.MathFidelity
Shape = _ttnn.Shape
WormholeComputeKernelConfig = ttnn.WormholeComputeKernelConfig
GrayskullComputeKernelConfig = ttnn.GrayskullComputeKernelConfig


def _one(x):
    return x[0] if isinstance(x, (list, tuple)) else x


def _like(x, y):
    return [y] if isinstance(x, (list, tuple)) else y


def matmul(input_a, input_b, output_mem_config=None, kernel_config=None, untilize_out=False):
    """tt::tt_metal::matmul (tt_eager/tt_dnn/op_library/bmm/bmm_op.hpp:388-456): weights broadcast over the batch."""
    return ttnn.matmul(input_a, input_b)


def bmm(input_a, input_b, output_mem_config=None, kernel_config=None, untilize_out=False):
    """tt::tt_metal::bmm: a batched second operand, one [K, N] matrix per batch entry."""
    return ttnn.matmul(input_a, input_b)


def mul(input_a, input_b, fused_activations=None, output_mem_config=None, output_dtype=None):
    """Elementwise product of two bfloat16 tensors of one shape: the gate multiply silu(x w1) * (x w3) of the gated MLP
    (models/demos/llama2_70b/tt/llama_mlp_optimized.py:191-197)."""
    return ttnn.mul(input_a, input_b)


def all_gather(input_tensors: Union[Sequence, "ttnn.MultiDeviceTensor"], dim: int, num_links: int = 1, output_mem_config=None):
    """ttl.tensor.all_gather on the per-device list (tt_eager/tt_dnn/op_library/all_gather/all_gather_op.cpp:67-104). With one
    process per GPU the list holds this rank's tensor; it must belong to a device mesh (ttnn.MultiDeviceTensor)."""
    t = _one(input_tensors)
    if not isinstance(t, MultiDeviceTensor):
        raise RuntimeError("tt_lib.tensor.all_gather: the tensor must be a shard of a device mesh (ttnn.from_torch(..., mesh_mapper=...))")
    return _like(input_tensors, ttnn.all_gather(t, dim if dim < len(t.shape) else -1, num_links))


def sharded_to_interleaved(input_tensor, output_mem_config=None, output_dtype=None):
    """L1-sharded and interleaved tensors are the same thing in HBM: returns the tensor."""
    return input_tensor


def interleaved_to_sharded(input_tensor, *args, **kwargs):
    return input_tensor


def load_tensor(file_name: str, device=None):
    return ttnn.load_tensor(file_name, device=device)


def dump_tensor(file_name: str, tensor):
    return ttnn.dump_tensor(file_name, tensor)


def tilize(input_tensor, output_mem_config=None, output_dtype=None, use_multicore=False):
    return ttnn.to_layout(input_tensor, ttnn.TILE_LAYOUT, dtype=output_dtype)


def untilize(input_tensor, output_mem_config=None, use_multicore=False):
    return ttnn.to_layout(input_tensor, ttnn.ROW_MAJOR_LAYOUT)
