"""ttnn.matmul / ttnn.linear (mirrors ttnn/ttnn/operations/matmul.py :295-516 of the reference).

Tensix tiling hints (`core_grid`, `program_config`, `use_1d_systolic_array`, `compute_kernel_config`,
`memory_config`) are accepted so call sites do not change; the only one that affects the result is a fused
activation carried by a program config. Kernel selection happens inside libttb from the shapes."""
from typing import Optional

from .. import _ttnn
from .. import types as T
from ..multi_device import MultiDeviceTensor

MatmulProgramConfig = _ttnn.MatmulProgramConfig


def _make_config(kind, **kw):
    cfg = _ttnn.MatmulProgramConfig()
    cfg.kind = kind
    grid = kw.pop("compute_with_storage_grid_size", None)
    if grid is not None:
        cfg.compute_grid_x, cfg.compute_grid_y = int(grid[0]), int(grid[1])
    act = kw.pop("fused_activation", None)
    if act is not None:
        cfg.fused_activation = act[0] if isinstance(act, tuple) else act
    for k, v in kw.items():
        if not hasattr(cfg, k):
            raise TypeError(f"unexpected program-config field {k}")
        setattr(cfg, k, v)
    return cfg


def MatmulDefaultProgramConfig():
    return _make_config("default")


def MatmulMultiCoreReuseProgramConfig(**kw):
    return _make_config("multi_core_reuse", **kw)


def MatmulMultiCoreReuseMultiCastProgramConfig(**kw):
    return _make_config("mcast_2d", **kw)


def MatmulMultiCoreReuseMultiCast1DProgramConfig(**kw):
    return _make_config("mcast_1d", **kw)


def _split(a, b, bias=None):
    mesh = None
    out = []
    for t in (a, b, bias):
        if isinstance(t, MultiDeviceTensor):
            mesh = t.mesh
            if getattr(t, "_gather_slot", None) is not None:
                from .ccl import wait_for_gather     # gathered by a fused linear: complete it before a plain matmul reads it
                wait_for_gather(t)
            t = t.local
        elif type(t).__name__ == "FusedOutput":
            t = t.local
        out.append(t)
    return mesh, out


def matmul(input_tensor_a, input_tensor_b, *, memory_config: T.MemoryConfig = T.DRAM_MEMORY_CONFIG, dtype: Optional[T.DataType] = None,
           core_grid=None, program_config=None, use_1d_systolic_array: Optional[bool] = None, compute_kernel_config=None):
    """Returns input_tensor_a @ input_tensor_b. Both must be TILE_LAYOUT tensors on the same device; the second operand
    ([.., K, N], bfloat8_b / bfloat4_b / bfloat16) is shared by every batch entry of the first (bfloat16)."""
    mesh, (a, b, _) = _split(input_tensor_a, input_tensor_b)
    out = _ttnn.matmul(a, b, dtype=dtype, program_config=program_config)
    return MultiDeviceTensor(out, mesh) if mesh is not None else out


def linear(input_tensor_a, input_tensor_b, *, bias=None, memory_config: T.MemoryConfig = T.DRAM_MEMORY_CONFIG,
           dtype: Optional[T.DataType] = None, core_grid=None, program_config=None, activation: Optional[str] = None,
           use_1d_systolic_array: Optional[bool] = None, compute_kernel_config=None):
    """Returns activation(input_tensor_a @ input_tensor_b + bias); `activation` is one of None, "relu", "gelu", "silu"."""
    if activation is not None and activation not in ("relu", "gelu", "silu"):
        raise RuntimeError(f"ttnn.linear: {activation} is not supported as activation function")
    mesh, (a, b, bias_t) = _split(input_tensor_a, input_tensor_b, bias)
    out = _ttnn.linear(a, b, bias=bias_t, dtype=dtype, activation=activation, program_config=program_config)
    return MultiDeviceTensor(out, mesh) if mesh is not None else out


def mul(input_tensor_a, input_tensor_b, *, memory_config: T.MemoryConfig = T.DRAM_MEMORY_CONFIG, dtype: Optional[T.DataType] = None):
    """Elementwise product of two bfloat16 device tensors of one shape: the gate multiply of the gated MLP when it is not
    fused into the matmul (ttnn.linear_gated does that in one launch)."""
    mesh, (a, b, _) = _split(input_tensor_a, input_tensor_b)
    out = _ttnn.mul(a, b)
    return MultiDeviceTensor(out, mesh) if mesh is not None else out
