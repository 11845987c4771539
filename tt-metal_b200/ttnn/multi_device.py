"""Device meshes and tensor-parallel mappers (mirrors ttnn/ttnn/multi_device.py of the reference).

The reference drives all devices of a mesh from one process and a multi-device tensor holds one shard per device.
Here a mesh is a set of processes, one per GPU, joined by a torch.distributed process group: every rank holds
its own shard and calls the same operations. A mesh of one device needs no process group."""
import contextlib
from typing import Dict, List

import torch

from . import _ttnn
from . import types as T


def get_num_devices() -> int:
    return _ttnn.get_num_devices()


def get_device_ids() -> List[int]:
    return list(range(get_num_devices()))


class DeviceMesh:
    """`device_ids[i]` is the CUDA device of rank i. The calling process owns device_ids[rank]."""

    def __init__(self, device_grid, device_ids: List[int], process_group=None):
        self.device_grid = tuple(device_grid)
        self.device_ids = list(device_ids)
        n = len(self.device_ids)
        if n == 0:
            raise RuntimeError("ttnn.open_device_mesh: device_ids must not be empty")
        self.process_group = process_group
        if n > 1:
            import torch.distributed as dist
            if not dist.is_initialized():
                raise RuntimeError("ttnn.open_device_mesh: a mesh of several devices needs torch.distributed to be initialised "
                                   "(one process per GPU)")
            if dist.get_world_size(process_group) != n:
                raise RuntimeError(f"ttnn.open_device_mesh: {n} device ids for a process group of {dist.get_world_size(process_group)} ranks")
            self.local_index = dist.get_rank(process_group)
        else:
            self.local_index = 0
        self.device = _ttnn.open_device(self.device_ids[self.local_index]) if torch.cuda.is_available() else None
        self._comm = None          # NCCL communicator behind the C ABI, made at first use
        self._ring = None          # ring of gather points of the fused linears
        self.pending = None        # (ring, point) of the last gathering launch no later launch has waited for yet

    def communicator(self, timeout_ms: int = 120000):
        """The mesh's communicator (ttb_comm_* behind _ttnn.Comm), created collectively at first use: rank 0 makes the id,
        the process group carries it to the others (bootstrap only), every rank joins within `timeout_ms`."""
        if self._comm is None:
            import torch.distributed as dist
            n = len(self.device_ids)
            box = [_ttnn.Comm.make_unique_id() if self.local_index == 0 else None]
            dist.broadcast_object_list(box, src=dist.get_global_rank(self.process_group, 0) if self.process_group is not None else 0,
                                       group=self.process_group)
            self._comm = _ttnn.Comm(n, self.local_index, box[0], timeout_ms)
        return self._comm

    def current_ring(self):
        return self._ring

    def gather_ring(self, nbytes: int, slots: int = 8):
        """The ring of gather points, large enough for a gathered tensor of `nbytes`. Growing it is collective: the point
        still pending in the old ring is settled on the stream, the ranks meet, and the old ring goes away once no tensor
        refers to it any more (tensors keep the ring they were gathered in)."""
        if self._ring is None or self._ring.slot_bytes < nbytes:
            from .peer import GatherRing
            import torch.distributed as dist
            if self._ring is not None:
                if self.pending is not None:
                    self.pending[0].stream_wait(self.pending[1])
                    self.pending = None
                self.device.synchronize()
                dist.barrier(group=self.process_group)
            self._ring = GatherRing(self.local_index, len(self.device_ids), max(nbytes, 1 << 20), slots=slots, group=self.process_group)
        return self._ring

    def get_num_devices(self) -> int:
        return len(self.device_ids)

    def get_device_ids(self) -> List[int]:
        return list(self.device_ids)

    def get_device(self, index: int):
        if index != self.local_index:
            raise RuntimeError("ttnn.DeviceMesh: only this rank's own device is reachable from this process")
        return self.device


class MultiDeviceTensor:
    """This rank's shard of a tensor that lives on a mesh."""

    def __init__(self, local, mesh):
        self.local = local
        self.mesh = mesh

    shape = property(lambda self: self.local.shape)
    dtype = property(lambda self: self.local.dtype)
    layout = property(lambda self: self.local.layout)

    def storage_type(self):
        on_device = self.local.storage_type() == T.StorageType.DEVICE
        return T.StorageType.MULTI_DEVICE if on_device else T.StorageType.MULTI_DEVICE_HOST

    def device(self):
        return self.local.device()

    def is_allocated(self):
        return self.local.is_allocated()

    def deallocate(self, force=False):
        self.local.deallocate(force)

    def __repr__(self):
        return f"ttnn.MultiDeviceTensor(rank {self.mesh.local_index} of {self.mesh.get_num_devices()}, {self.local!r})"


def open_device_mesh(device_grid: T.DeviceGrid, device_ids: List[int], process_group=None) -> DeviceMesh:
    grid = device_grid.as_tuple() if hasattr(device_grid, "as_tuple") else tuple(device_grid)
    return DeviceMesh(grid, device_ids, process_group)


def close_device_mesh(device_mesh: DeviceMesh) -> None:
    if device_mesh.device is not None:
        _ttnn.close_device(device_mesh.device)


@contextlib.contextmanager
def create_device_mesh(device_grid: T.DeviceGrid, device_ids: List[int], process_group=None):
    mesh = open_device_mesh(device_grid, device_ids, process_group)
    try:
        yield mesh
    finally:
        close_device_mesh(mesh)


def get_device_tensors(tensor) -> list:
    """The shards reachable from this process: the local one."""
    return [tensor.local] if isinstance(tensor, MultiDeviceTensor) else [tensor]


def aggregate_as_tensor(tensors, mesh=None):
    if len(tensors) != 1:
        raise RuntimeError("ttnn.aggregate_as_tensor: each process holds exactly one shard")
    return MultiDeviceTensor(tensors[0], mesh) if mesh is not None else tensors[0]


class TensorToMesh:
    def __init__(self, device_mesh):
        self.device_mesh = device_mesh
        self.device_id_to_tensor = {}

    def map(self, tensor: "torch.Tensor"):
        raise NotImplementedError("Subclasses must implement this method")


class MeshToTensor:
    def compose(self, tensor):
        raise NotImplementedError("Subclasses must implement this method")


class ShardTensorToMesh(TensorToMesh):
    def __init__(self, device_mesh, dim):
        super().__init__(device_mesh)
        self.shard_dim = dim

    def map(self, tensor: "torch.Tensor") -> Dict[int, "torch.Tensor"]:
        sliced = torch.chunk(tensor, self.device_mesh.get_num_devices(), dim=self.shard_dim)
        self.device_id_to_tensor = {i: t for i, t in enumerate(sliced)}
        return self.device_id_to_tensor


class ReplicateTensorToMesh(TensorToMesh):
    def map(self, tensor: "torch.Tensor"):
        self.device_id_to_tensor = {i: tensor for i in range(self.device_mesh.get_num_devices())}
        return self.device_id_to_tensor


def _gather_torch(device_mesh, local: "torch.Tensor") -> list:
    n = device_mesh.get_num_devices()
    if n == 1:
        return [local]
    import torch.distributed as dist
    backend = dist.get_backend(device_mesh.process_group)
    src = local.cuda() if backend == "nccl" else local
    outs = [torch.empty_like(src) for _ in range(n)]
    dist.all_gather(outs, src.contiguous(), group=device_mesh.process_group)
    return [o.cpu() for o in outs]


class ConcatMeshToTensor(MeshToTensor):
    def __init__(self, device_mesh, dim: int):
        self.concat_dim = dim
        self.device_mesh = device_mesh

    def compose(self, tensor) -> "torch.Tensor":
        from .operations.core import to_torch
        return torch.cat(_gather_torch(self.device_mesh, to_torch(get_device_tensors(tensor)[0])), dim=self.concat_dim)


class ListMeshToTensor(MeshToTensor):
    def __init__(self, device_mesh):
        self.device_mesh = device_mesh

    def compose(self, tensor) -> List["torch.Tensor"]:
        from .operations.core import to_torch
        return _gather_torch(self.device_mesh, to_torch(get_device_tensors(tensor)[0]))
