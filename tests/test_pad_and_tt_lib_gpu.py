"""Tensor.pad / unpad / pad_to_tile / unpad_from_tile (tt_eager/tensor/tensor_impl.hpp:508-677, tensor_impl.cpp:200-283,
tensor.cpp:209-254) against numpy restatements of the reference's loops, block-float tensors against the oracle's
unpack -> pad -> pack sequence; and the `tt_lib` spellings the 70B decoder uses
(models/demos/llama2_70b/tt/llama_mlp_optimized.py:165-228)."""
import numpy as np
import pytest
import torch

import oracle
import ttnn
import vectors

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    dev = ttnn.open_device(0)
    yield dev
    ttnn.close_device(dev)


def np_pad(x, out_shape, start, value):
    out = np.full(out_shape, value, dtype=x.dtype)
    sl = tuple(slice(s, s + n) for s, n in zip(start, x.shape))
    out[sl] = x
    return out


@pytest.mark.parametrize("dtype,tdtype", [(ttnn.float32, torch.float32), (ttnn.bfloat16, torch.bfloat16), (ttnn.uint32, torch.int32)])
@pytest.mark.parametrize("on_device", [False, True])
def test_pad_then_unpad_row_major(device, dtype, tdtype, on_device):
    x = (vectors.randn(3, (2, 3, 5, 7), 4.0)).to(tdtype)
    t = ttnn.from_torch(x, dtype=dtype, layout=ttnn.ROW_MAJOR_LAYOUT, device=device if on_device else None)
    p = t.pad([3, 4, 9, 16], [1, 0, 2, 5], 1.5 if tdtype != torch.int32 else 7)
    assert list(p.shape) == [3, 4, 9, 16] and p.layout == ttnn.ROW_MAJOR_LAYOUT and p.storage_type() == t.storage_type()
    want = np_pad(x.float().numpy(), (3, 4, 9, 16), (1, 0, 2, 5), 1.5 if tdtype != torch.int32 else 7)
    assert np.array_equal(ttnn.to_torch(p).float().numpy(), want)
    u = p.unpad([1, 0, 2, 5], [2, 2, 6, 11])                       # inclusive ends: the original box
    assert list(u.shape) == [2, 3, 5, 7]
    assert torch.equal(ttnn.to_torch(u), x)
    with pytest.raises(RuntimeError):
        t.pad([2, 3, 5, 6], [0, 0, 0, 0], 0.0)                      # output smaller than the input
    with pytest.raises(RuntimeError):
        p.unpad([0, 0, 0, 0], [3, 0, 0, 0])                         # end outside the tensor
    with pytest.raises(RuntimeError):
        ttnn.to_layout(ttnn.from_torch(torch.zeros(32, 32), dtype=ttnn.float32, device=device), ttnn.TILE_LAYOUT).pad([64, 64], [0, 0], 0.0)


def test_pad_to_tile_and_back(device):
    x = vectors.randn(5, (1, 2, 45, 70), 1.0).bfloat16()
    t = ttnn.from_torch(x, dtype=ttnn.bfloat16, layout=ttnn.ROW_MAJOR_LAYOUT, device=device)
    p = t.pad_to_tile(0.0)
    assert list(p.shape) == [1, 2, 45, 70] and list(p.shape.with_tile_padding()) == [1, 2, 64, 96]
    tiled = ttnn.to_layout(p, ttnn.TILE_LAYOUT)                         # already padded: tilizes in place
    assert torch.equal(ttnn.to_torch(tiled), x)
    back = ttnn.to_layout(tiled, ttnn.ROW_MAJOR_LAYOUT).unpad_from_tile([1, 2, 45, 70])
    assert list(back.shape) == [1, 2, 45, 70] and torch.equal(ttnn.to_torch(back), x)
    with pytest.raises(RuntimeError):
        ttnn.to_layout(tiled, ttnn.ROW_MAJOR_LAYOUT).unpad_from_tile([1, 2, 20, 70])   # not within one tile of the padded extent


@pytest.mark.parametrize("dtype,ofmt", [(ttnn.bfloat8_b, oracle.BFP8_B), (ttnn.bfloat4_b, oracle.BFP4_B)])
def test_block_float_pad_and_unpad_follow_the_reference_sequence(device, orc, dtype, ofmt):
    """pad_bfloat8_b / unpad_bfloat8_b: unpack in stored order, pad the fp32 tensor, pack in stored order."""
    x = vectors.randn(9, (1, 1, 32, 64), 0.05)
    t = ttnn.to_layout(ttnn.from_torch(x, dtype=dtype, layout=ttnn.TILE_LAYOUT), ttnn.ROW_MAJOR_LAYOUT)     # block-float row-major form
    stored = np.frombuffer(t.buffer(), np.uint8)
    f = orc.unpack(stored, ofmt).reshape(1, 1, 32, 64)
    p = t.pad([1, 2, 64, 64], [0, 1, 16, 0], 0.25)
    want = orc.pack(np_pad(f, (1, 2, 64, 64), (0, 1, 16, 0), np.float32(0.25)), ofmt)
    assert np.array_equal(np.frombuffer(p.buffer(), np.uint8), want)
    u = p.unpad([0, 1, 16, 0], [0, 1, 47, 63])
    want_u = orc.pack(orc.unpack(want, ofmt).reshape(1, 2, 64, 64)[:, 1:2, 16:48, :].copy(), ofmt)
    assert np.array_equal(np.frombuffer(u.buffer(), np.uint8), want_u)


def test_tt_lib_spellings_of_the_gated_mlp(device, orc):
    """matmul_1d with a fused activation, matmul_1d, tt_lib.tensor.mul, matmul_1d: the single-device form of
    TtLlamaMLP_optimized.forward, against fp32 torch on the oracle-unpacked weights."""
    import tt_lib
    from test_matmul_gpu import check
    H, F = 512, 1024
    x = vectors.randn(11, (1, 1, 32, H), 1.0).bfloat16()
    ws, refs = [], []
    for seed, (K, N) in zip((12, 13, 14), ((H, F), (H, F), (F, H))):
        w = vectors.randn(seed, (K, N), 0.05)
        t = ttnn.from_torch(w, dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device)
        assert isinstance(t, tt_lib.tensor.Tensor)
        ws.append(t)
        refs.append(torch.from_numpy(orc.to_torch(np.frombuffer(t.buffer(), np.uint8), oracle.BFP8_B, 1, K, N).reshape(K, N).copy()))
    xt = ttnn.from_torch(x, dtype=ttnn.bfloat16, layout=ttnn.TILE_LAYOUT, device=device)
    cfg = tt_lib.operations.primary.MatmulMultiCoreReuseMultiCast1DProgramConfig(
        compute_with_storage_grid_size=(8, 4), in0_block_w=8, out_subblock_h=1, out_subblock_w=4, per_core_M=1, per_core_N=4,
        fuse_batch=True, fused_activation="silu", mcast_in0=True)
    w1_out = tt_lib.operations.primary.matmul_1d(xt, ws[0], program_config=cfg, output_dtype=tt_lib.tensor.DataType.BFLOAT16)
    w3_out = tt_lib.operations.primary.matmul_1d(xt, ws[1])
    hidden = tt_lib.tensor.mul(w1_out, w3_out)
    hidden = tt_lib.tensor.interleaved_to_sharded(tt_lib.tensor.sharded_to_interleaved(hidden))
    out = tt_lib.operations.primary.matmul_1d(hidden, ws[2])
    xf = x.float().reshape(32, H)
    a = torch.nn.functional.silu(xf @ refs[0]).bfloat16().float() * (xf @ refs[1]).bfloat16().float()
    check(ttnn.to_torch(hidden).reshape(32, F), a)
    check(ttnn.to_torch(out).reshape(32, H), a.bfloat16().float() @ refs[2])
    w1_out.deallocate(True)
