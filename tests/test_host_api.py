"""Host-side logic of the ttnn surface that needs no GPU: types, shapes, validation messages, the row-major host
path, the tensor cache format, the all-gather shape plan and the multi-process mappers over gloo."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import ttnn
from ttnn.operations.ccl import gather_plan


def test_enum_values_follow_the_reference():
    # tt_eager/tensor/types.hpp:24-34
    assert int(ttnn.DataType.BFLOAT16) == 0 and int(ttnn.DataType.FLOAT32) == 1 and int(ttnn.DataType.UINT32) == 2
    assert int(ttnn.DataType.BFLOAT8_B) == 3 and int(ttnn.DataType.BFLOAT4_B) == 4 and int(ttnn.DataType.UINT16) == 6
    assert int(ttnn.Layout.ROW_MAJOR) == 0 and int(ttnn.Layout.TILE) == 1
    assert ttnn.TILE_SIZE == 32


def test_shape_with_tile_padding():
    s = ttnn.Shape([1, 7, 3], [1, 32, 32])
    assert list(s) == [1, 7, 3] and len(s) == 3 and s[-1] == 3
    assert list(s.with_tile_padding()) == [1, 32, 32]
    assert s == ttnn.Shape([1, 7, 3], [1, 32, 32]) and not (s == ttnn.Shape([1, 7, 3]))
    with pytest.raises(RuntimeError):
        ttnn.Shape([4, 4], [2, 4])


def test_row_major_host_tensors_round_trip_without_a_gpu():
    for dt in (torch.float32, torch.bfloat16, torch.int32):
        x = (torch.arange(2 * 3 * 5, dtype=torch.float32).reshape(2, 3, 5) - 7).to(dt)
        t = ttnn.from_torch(x)
        assert list(t.shape) == [2, 3, 5] and t.layout == ttnn.ROW_MAJOR_LAYOUT
        assert t.storage_type() == ttnn.StorageType.OWNED
        assert torch.equal(ttnn.to_torch(t), x)
    t = ttnn.from_torch(torch.ones(1, 1, 2, 4))
    assert ttnn.to_torch(t, torch_rank=2).shape == (2, 4)
    with pytest.raises(RuntimeError, match="Unable to squeeze"):
        ttnn.to_torch(ttnn.from_torch(torch.ones(2, 2, 4)), torch_rank=2)
    # fp32 -> bfloat16 uses torch's round-to-nearest-even like the reference (pytensor.cpp:86-90)
    x = torch.tensor([[1.00390625, 1.01171875]])
    assert torch.equal(ttnn.to_torch(ttnn.from_torch(x, dtype=ttnn.bfloat16)), x.bfloat16())


def test_from_torch_validation_messages():
    with pytest.raises(RuntimeError, match="requires TILE_LAYOUT"):
        ttnn.from_torch(torch.zeros(32, 32), dtype=ttnn.bfloat8_b)
    with pytest.raises(RuntimeError, match="at least 2 dimensions"):
        ttnn.from_torch(torch.zeros(32), dtype=ttnn.bfloat4_b, layout=ttnn.TILE_LAYOUT)
    with pytest.raises(RuntimeError, match="device must be specified"):
        ttnn.from_torch(torch.zeros(32, 32), memory_config=ttnn.DRAM_MEMORY_CONFIG)


def test_matmul_validation_happens_before_any_device_work():
    a = ttnn.from_torch(torch.zeros(32, 64, dtype=torch.bfloat16))
    b = ttnn.from_torch(torch.zeros(64, 32, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="must be of layout Layout.TILE"):
        ttnn.matmul(a, b)
    with pytest.raises(RuntimeError, match="not supported as activation"):
        ttnn.linear(a, b, activation="tanh")
    with pytest.raises(RuntimeError, match="rank 2, 3 or 4"):
        ttnn.matmul(ttnn.from_torch(torch.zeros(64, dtype=torch.bfloat16)), b)


def test_program_and_kernel_configs_are_accepted():
    cfg = ttnn.MatmulMultiCoreReuseMultiCast1DProgramConfig(compute_with_storage_grid_size=(8, 4), in0_block_w=2, out_subblock_h=1,
                                                            out_subblock_w=4, per_core_M=1, per_core_N=8, fuse_batch=True,
                                                            fused_activation=("gelu", True), mcast_in0=True)
    assert cfg.kind == "mcast_1d" and cfg.fused_activation == "gelu" and cfg.per_core_N == 8
    ckc = ttnn.WormholeComputeKernelConfig(math_fidelity=ttnn.MathFidelity.HiFi2, fp32_dest_acc_en=True, packer_l1_acc=True)
    assert ckc.fp32_dest_acc_en and ckc.math_fidelity == ttnn.MathFidelity.HiFi2
    assert ttnn.CoreGrid(x=8, y=4).num_cores == 32


def test_tensor_cache_round_trip(tmp_path):
    x = torch.arange(6 * 10, dtype=torch.float32).reshape(6, 10)
    t = ttnn.from_torch(x)
    f = tmp_path / "w.bin"
    ttnn.dump_tensor(str(f), t)
    u = ttnn.load_tensor(str(f))
    assert list(u.shape) == [6, 10] and u.dtype == ttnn.float32 and torch.equal(ttnn.to_torch(u), x)
    (tmp_path / "bad.bin").write_bytes(b"nope")
    with pytest.raises(RuntimeError, match="not a tensor cache file"):
        ttnn.load_tensor(str(tmp_path / "bad.bin"))
    v = ttnn.as_tensor(x, cache_file_name=str(tmp_path / "cache" / "w"))
    assert (tmp_path / "cache" / "w_dtype_FLOAT32_layout_ROW_MAJOR.bin").exists()
    w = ttnn.as_tensor(torch.zeros_like(x), cache_file_name=str(tmp_path / "cache" / "w"))   # served from the cache
    assert torch.equal(ttnn.to_torch(w), x) and torch.equal(ttnn.to_torch(v), x)


def _emulate_gather(shards, plan):
    interleave, rows, row_bytes, _, _ = plan
    staged = np.concatenate(shards)
    if not interleave:
        return staged
    n = len(shards)
    return staged.reshape(n, rows, row_bytes).transpose(1, 0, 2).reshape(-1)


@pytest.mark.parametrize("shape,dim", [((1, 1, 32, 256), 3), ((1, 1, 64, 128), 3), ((2, 1, 32, 64), -1), ((1, 1, 64, 64), 2)])
def test_all_gather_plan_reproduces_concat_for_tiled_tensors(orc, shape, dim):
    """The rank-major concatenation (plus the tile-row interleave where the plan asks for it) of tiled shards equals the
    tiling of torch.cat of the shards: the reference's emulated all-gather (models/demos/llama2_70b/tt/llama_common.py:99-106)."""
    n = 4
    full_shape = list(shape)
    full_shape[dim] *= n
    x = torch.arange(int(np.prod(full_shape)), dtype=torch.float32).reshape(full_shape).to(torch.bfloat16)
    shards = torch.chunk(x, n, dim=dim)

    def tiled_bytes(t):
        o = int(np.prod(t.shape[:-2]))
        return orc.tilize(t.contiguous().view(torch.int16).numpy().view(np.uint16), o, t.shape[-2], t.shape[-1]).reshape(-1).view(np.uint8)

    plan = gather_plan(list(shape), list(shape), ttnn.bfloat16, ttnn.TILE_LAYOUT, dim, n)
    got = _emulate_gather([tiled_bytes(s) for s in shards], plan)
    assert plan[3] == full_shape
    assert np.array_equal(got, tiled_bytes(x))


def test_all_gather_plan_rejects_unsupported_dims():
    with pytest.raises(RuntimeError, match="not supported"):
        gather_plan([2, 2, 32, 32], [2, 2, 32, 32], ttnn.bfloat16, ttnn.TILE_LAYOUT, 1, 2)
    with pytest.raises(RuntimeError, match="requires input tensors to be multi-device"):
        ttnn.all_gather(ttnn.from_torch(torch.zeros(2, 2)), dim=1, num_links=1)


_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path[:0] = [os.environ["TTB_PKG"]]
import ttnn
dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
mesh = ttnn.open_device_mesh(ttnn.DeviceGrid(1, 2), [0, 1])
assert mesh.get_num_devices() == 2 and mesh.local_index == dist.get_rank()
w = torch.arange(8 * 12, dtype=torch.float32).reshape(8, 12)
shard = ttnn.from_torch(w, mesh_mapper=ttnn.ShardTensorToMesh(mesh, dim=-1))       # column-sharded like the TP weights
assert isinstance(shard, ttnn.MultiDeviceTensor) and list(shard.shape) == [8, 6]
assert shard.storage_type() == ttnn.StorageType.MULTI_DEVICE_HOST
assert torch.equal(ttnn.to_torch(shard.local), torch.chunk(w, 2, dim=-1)[dist.get_rank()])
back = ttnn.to_torch(shard, mesh_composer=ttnn.ConcatMeshToTensor(mesh, dim=-1))
assert torch.equal(back, w)
rep = ttnn.from_torch(w, mesh_mapper=ttnn.ReplicateTensorToMesh(mesh))
parts = ttnn.to_torch(rep, mesh_composer=ttnn.ListMeshToTensor(mesh))
assert len(parts) == 2 and all(torch.equal(p, w) for p in parts)
dist.barrier()
dist.destroy_process_group()
print("rank", os.environ["RANK"], "ok")
"""


def test_mesh_mappers_over_two_gloo_ranks(tmp_path):
    """world_size 2 on CPU: ShardTensorToMesh / ReplicateTensorToMesh / ConcatMeshToTensor / ListMeshToTensor with one
    process per device (tests/ttnn/unit_tests/test_multi_device.py:106-222 of the reference, restated for ranks)."""
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29731",
                   TTB_PKG=os.path.join(root, "tt-metal_b200"))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    for p in procs:
        out, _ = p.communicate(timeout=180)
        assert p.returncode == 0, out.decode()


def _walk_plan(plan, nkb):
    """Re-walks the decomposition of the persistent decode kernel on the CPU exactly as its blocks do (rounds of whole tiles
    or pieces, then the evenly dealt remainder) and returns {tile: [(kb0, kb1, block), ...]}."""
    nb, tiles, grid, pieces, kbps, waves, rem0, units, upt, slots = plan
    q, r = (units // grid, units % grid) if grid else (0, 0)
    begin = lambda b: b * q + min(b, r)
    cover = {}
    for b in range(grid):
        for w in range(waves):
            x = w * grid + b
            if x < rem0:
                if pieces > 1:
                    part, tile = divmod(x, tiles)
                    kb0 = part * kbps
                    cover.setdefault(tile, []).append((kb0, min(nkb, kb0 + kbps), b))
                else:
                    cover.setdefault(x, []).append((0, nkb, b))
        u, u_end = begin(b), begin(b + 1)
        while u < u_end:
            rt = u // upt
            t0 = rt * upt
            e = min(u_end, t0 + upt)
            cover.setdefault(rem0 + rt, []).append(((u - t0) * 8, min(nkb, (e - t0) * 8), b))
            u = e
    return cover


def test_decode_plan_covers_every_k_block_exactly_once():
    """Host logic of the persistent decode kernel, no GPU: for single weights and groups of weights, every K block of every
    128-column tile belongs to exactly one block, blocks never exceed the SM count, and the partial-sum slots suffice."""
    import ctypes
    import cabi
    lib = cabi.load()
    shapes = [(32, 4544, [18176]), (32, 8192, [8192]), (32, 8192, [8192, 1024, 1024]), (32, 8192, [28672, 28672]), (32, 28672, [8192]),
              (32, 8192, [1024, 128, 128]), (32, 8192, [128]), (32, 4096, [4096, 1024, 1024]), (64, 4096, [14336, 14336]),
              (128, 2048, [256]), (256, 16384, [7680]), (96, 1056, [384, 128]), (32, 32, [128]), (32, 8192, [3584, 3584]),
              (32, 4544, [4672]), (32, 18176, [4544]), (96, 512, [160, 96])]
    for M, K, Ns in shapes:
        arr = (ctypes.c_int64 * len(Ns))(*Ns)
        out = (ctypes.c_int32 * 10)()
        assert lib.cdll.ttb_matmul_decode_plan(cabi.BFLOAT8_B, 1, M, K, len(Ns), arr, out, 10) == 0
        plan = list(out)
        nb, tiles, grid, pieces, kbps, waves, rem0, units, upt, slots = plan
        nkb = K // 32
        assert nb in (32, 64, 128) and M % nb == 0 and tiles == sum((n + 127) // 128 for n in Ns) * (M // nb) and 1 <= grid <= 148
        cover = _walk_plan(plan, nkb)
        assert sorted(cover) == list(range(tiles)), (M, K, Ns, plan)
        shared = 0
        for tile, segs in cover.items():
            segs.sort()
            assert segs[0][0] == 0 and segs[-1][1] == nkb and all(a[1] == b[0] for a, b in zip(segs, segs[1:])), (M, K, Ns, tile, segs)
            assert all(s[1] > s[0] for s in segs)
            shared += len(segs) if len(segs) > 1 else 0
        assert shared <= slots or shared == 0, (M, K, Ns, plan, shared)
    ragged = (ctypes.c_int64 * 1)(96)
    out = (ctypes.c_int32 * 10)()
    assert lib.cdll.ttb_matmul_decode_plan(cabi.BFLOAT8_B, 1, 64, 64, 1, ragged, out, 10) == 0 and out[0] == 32   # a partial column tile: one tile row per block
    assert lib.cdll.ttb_matmul_decode_plan(cabi.BFLOAT8_B, 1, 32, 64, 1, ragged, out, 10) == 0 and out[0] == 32
    whole = (ctypes.c_int64 * 1)(128)
    assert lib.cdll.ttb_matmul_decode_plan(cabi.BFLOAT8_B, 1, 64, 64, 1, whole, out, 10) == 0 and out[0] == 64


def _check_plan(lib, fmt, M, K, Ns):
    import ctypes
    arr = (ctypes.c_int64 * len(Ns))(*Ns)
    out = (ctypes.c_int32 * 10)()
    assert lib.cdll.ttb_matmul_decode_plan(fmt, 1, M, K, len(Ns), arr, out, 10) == 0, (M, K, Ns)
    plan = list(out)
    nb, tiles, grid, pieces, kbps, waves, rem0, units, upt, slots = plan
    nkb = K // 32
    assert nb == (64 if M % 64 == 0 and all(n % 128 == 0 for n in Ns) else 32) and tiles == sum((n + 127) // 128 for n in Ns) * (M // nb) and 1 <= grid <= 148, (M, K, Ns, plan)
    cover = _walk_plan(plan, nkb)
    assert sorted(cover) == list(range(tiles)), (M, K, Ns, plan)
    shared = 0
    for tile, segs in cover.items():
        segs.sort()
        assert segs[0][0] == 0 and segs[-1][1] == nkb and all(a[1] == b[0] for a, b in zip(segs, segs[1:])), (M, K, Ns, plan, tile, segs)
        assert all(s[1] > s[0] for s in segs), (M, K, Ns, plan, tile, segs)
        shared += len(segs) if len(segs) > 1 else 0
    assert shared <= slots or shared == 0, (M, K, Ns, plan, shared)


def test_decode_plan_covers_every_k_block_for_seeded_random_shapes():
    """The same property over a seeded sweep of shapes in both formats: 1 to 4 weights, 32 to 256 rows, K from one K block to
    32768, column counts from one tile to 32768, with and without a partial last column tile."""
    import random
    import cabi
    lib = cabi.load()
    rng = random.Random(20240229)
    for _ in range(600):
        M = 32 * rng.randint(1, 8)
        K = 32 * rng.choice([1, 2, 3, 7, 8, 9, 33, 64, 100, 128, 142, 256, 257, 512, 896, 1024])
        count = rng.randint(1, 4)
        step = rng.choice([32, 128])
        Ns = [step * rng.randint(1, rng.choice([4, 36, 256]) * 128 // step) for _ in range(count)]
        _check_plan(lib, rng.choice([cabi.BFLOAT8_B, cabi.BFLOAT4_B]), M, K, Ns)


def test_matmul_plan_names_the_kernels_without_a_gpu():
    """ttb_matmul_plan: which tensor-core kernels a shape gets - decode up to 256 rows (any N % 32 == 0), prefill for multiples
    of 128 from 512 (N % 128 == 0), two row ranges in between and for ragged counts, ranges of 256 rows on the decode kernel
    where N has a partial last tile, else the CUDA-core kernel."""
    import ctypes
    import cabi
    lib = cabi.load()

    def plan(M, K, N, w_dtype=cabi.BFLOAT8_B, flags=0):
        out = (ctypes.c_int64 * 5)()
        assert lib.cdll.ttb_matmul_plan(w_dtype, 1, M, K, N, flags, out, 5) == 0
        return list(out)

    assert plan(32, 4544, 18176) == [1, 32, 0, 0, 0]
    assert plan(32, 4544, 4672) == [1, 32, 0, 0, 0]           # last column tile of 64 columns
    assert plan(64, 4544, 4672) == [1, 64, 0, 0, 0]           # ... also with several tile rows
    assert plan(256, 4096, 14336) == [1, 256, 0, 0, 0]
    assert plan(2048, 8192, 28672) == [1, 2048, 1, 0, 0]
    assert plan(320, 1024, 512) == [2, 256, 0, 64, 0]
    assert plan(608, 1024, 512) == [2, 512, 1, 96, 0]
    assert plan(384, 1024, 512) == [2, 256, 0, 128, 0]
    assert plan(512, 4544, 4672) == [2, 256, 0, 256, 0]       # a partial last column tile: decode launches over row ranges
    out = (ctypes.c_int64 * 33)()
    assert lib.cdll.ttb_matmul_plan(cabi.BFLOAT8_B, 1, 2080, 4544, 4544, 0, out, 33) == 0
    assert list(out)[:19] == [9] + [256, 0] * 8 + [32, 0] and not any(list(out)[19:])
    for M in range(32, 4097, 32):                              # every row count up to 4096 stays on the tensor cores
        for N in (512, 4672, 96):
            assert lib.cdll.ttb_matmul_plan(cabi.BFLOAT8_B, 1, M, 1024, N, 0, out, 33) == 0
            assert out[0] > 0 and sum(list(out)[1::2]) == M, (M, N, list(out))
    assert plan(4128, 1024, 96)[0] == 0                        # more than 16 ranges: the shape-generic kernel
    assert plan(32, 1024, 512, cabi.BFLOAT16)[0] == 0          # bf16 weights: the shape-generic kernel
    assert plan(32, 4544, 18176, flags=cabi.MM_FORCE_GENERIC)[0] == 0
    assert lib.cdll.ttb_matmul_plan(cabi.BFLOAT8_B, 1, 32, 64, 128, 0, None, 5) == -1
