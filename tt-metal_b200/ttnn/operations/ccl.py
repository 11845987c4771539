"""ttnn.all_gather (mirrors ttnn/ttnn/operations/ccl.py:26-39 and the AllGather op,
tt_eager/tt_dnn/op_library/all_gather/all_gather_op.cpp:18-104): every rank ends up with the concatenation of all
ranks' shards along `dim`, dtype and layout preserved. The ethernet ring of the reference is replaced by NCCL over NVLink
behind the C ABI (one process per GPU); shapes, allocation and launches live in the C++ host layer, this module unwraps
and wraps the per-rank tensors.

Also the linears whose epilogue is the all-gather and the launch that serves several weights of one activation
(linear_all_gather, linear_multi, linear_gated)."""
from .. import _ttnn
from .. import types as T
from ..multi_device import MultiDeviceTensor


def gather_plan(dims, padded, dtype, layout, dim, n):
    """Pure shape logic of the all-gather: how the rank-major concatenation an NCCL all-gather leaves relates to the
    result tensor. Returns (interleave, rows, row_bytes, out_dims, out_padded): when `interleave` is set the result is
    rows x [n shards x row_bytes] and a device kernel re-orders the staged buffer; otherwise the staged buffer already
    is the result."""
    interleave, rows, row_bytes, out_shape = _ttnn.plan_all_gather(T.Shape(list(dims), list(padded)), dtype, layout, dim, n)
    return interleave, rows, row_bytes, list(out_shape), list(out_shape.padded)


def all_gather(multidevice_tensor, dim: int, num_links: int = 1, *, memory_config: T.MemoryConfig = T.DRAM_MEMORY_CONFIG):
    if not isinstance(multidevice_tensor, MultiDeviceTensor):
        raise RuntimeError("ttnn.all_gather requires input tensors to be multi-device tensor")
    mesh = multidevice_tensor.mesh
    if mesh.get_num_devices() == 1:
        return multidevice_tensor
    wait_for_gather(multidevice_tensor)
    return MultiDeviceTensor(_ttnn.all_gather(multidevice_tensor.local, dim, mesh.communicator()), mesh)


# ---- linear with the all-gather in its epilogue, and several linears of one activation in one launch ---------------------
def _local(t):
    return t.local if isinstance(t, MultiDeviceTensor) else t


def _fused_linear(input_tensor, weights, biases, activation, gather_first, ring_slots=8, gated=False):
    """One launch of ttb_matmul_multi through the host layer: up to four weights on one activation; optionally the first
    result is gathered over the mesh by the kernel's epilogue. Returns the list of results (MultiDeviceTensor when the
    input is one)."""
    multi = isinstance(input_tensor, MultiDeviceTensor)
    mesh = input_tensor.mesh if multi else None
    x = _local(input_tensor)
    G = mesh.get_num_devices() if multi else 1
    ring, wait_slot = None, -1
    if multi and G > 1:
        if gather_first:
            rows = 1
            for d in list(x.shape.padded)[:-1]:
                rows *= d
            # (re)built collectively when a larger gathered tensor arrives: every rank reaches this point with the same shapes
            ring = mesh.gather_ring(G * rows * list(_local(weights[0]).shape.padded)[-1] * 2, ring_slots)
        in_slot = getattr(input_tensor, "_gather_slot", None)
        if in_slot is not None:
            in_ring = input_tensor._gather_ring
            if ring is not None and in_ring is not ring:
                wait_for_gather(input_tensor)           # gathered in a ring that has been replaced since: settle it on the stream
            else:
                ring, wait_slot = in_ring, in_slot     # the kernel itself waits for its gathered activation
                if mesh.pending == (in_ring, in_slot):
                    mesh.pending = None
        if gather_first and mesh.pending is not None:
            # keeps the ranks within one gather of each other: the launch itself waits for the previous gather where it has
            # no gathered input of its own to wait for (its weights stream meanwhile), else the stream is held
            if wait_slot < 0 and mesh.pending[0] is ring:
                wait_slot = mesh.pending[1]
            else:
                mesh.pending[0].stream_wait(mesh.pending[1])
            mesh.pending = None
    native = ring.native if (ring is not None and (gather_first or wait_slot >= 0)) else None
    outs, slot = _ttnn.linear_multi(x, [_local(w) for w in weights],
                                    [(_local(b) if b is not None else None) for b in biases] if biases is not None else [],
                                    activation, native, bool(gather_first and G > 1), wait_slot, gated)
    results = []
    for j, t in enumerate(outs):
        if multi:
            t = MultiDeviceTensor(t, mesh)
            if gather_first and G > 1 and j == 0:
                t._gather_slot, t._gather_ring = slot, ring
                mesh.pending = (ring, slot)
        results.append(t)
    return results


def linear_multi(input_tensor, weights, *, biases=None, activation=None, all_gather_first=False):
    """[ttnn.linear(x, w, bias=b, activation=activation) for w, b in zip(weights, biases)] as ONE launch: the weights share
    the activation (q / k / v projections; w1 / w3 of a gated MLP) and stay separate tensors. Decode shapes (at most 256
    rows, block-float weights; a gathered first result needs an N that is a multiple of 128). Results equal those of the separate calls. With
    all_gather_first the first result is gathered along its last dimension over the mesh by the kernel's own epilogue
    (see linear_all_gather)."""
    return _fused_linear(input_tensor, weights, biases, activation, all_gather_first)


def linear_gated(input_tensor, gate_weight, up_weight, *, gate_bias=None, up_bias=None, activation="silu", all_gather=False):
    """activation(x @ gate_weight + gate_bias) * (x @ up_weight + up_bias) as ONE launch: both weights stream through one
    persistent kernel and the product is formed where the second of a column tile's two halves is finished - the gated MLP's
    silu(x w1) * (x w3) (models/demos/mistral7b/tt/mistral_mlp.py:51-73, models/demos/llama2_70b/tt/llama_mlp_optimized.py:165-197)
    without the two intermediate tensors and the separate multiply. With `all_gather` the product is gathered over the mesh
    by the same kernel (as linear_all_gather)."""
    biases = [gate_bias, up_bias] if (gate_bias is not None or up_bias is not None) else None
    return _fused_linear(input_tensor, [gate_weight, up_weight], biases, activation, all_gather, gated=True)[0]


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
    return _fused_linear(input_tensor, [weight], [bias] if bias is not None else None, activation, True, ring_slots)[0]


def wait_for_gather(tensor):
    """Holds the stream until a linear_all_gather result is complete on this rank (no-op for other tensors); called by
    every consumer that is not itself a fused linear."""
    if isinstance(tensor, MultiDeviceTensor) and getattr(tensor, "_gather_slot", None) is not None:
        ring, slot = tensor._gather_ring, tensor._gather_slot
        ring.stream_wait(slot)
        if tensor.mesh.pending == (ring, slot):
            tensor.mesh.pending = None
        tensor._gather_slot = None
    return tensor
