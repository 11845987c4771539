"""The ttnn Python surface on a GPU: the reference's own API tests for this path, restated
(tests/ttnn/unit_tests/test_to_and_from_torch.py:22-43, tests/tt_eager/.../misc/test_tensor.py:27-90,
tests/ttnn/unit_tests/operations/test_linear.py, test_matmul.py), plus bit-exact checks against the oracle."""
import numpy as np
import pytest
import torch

import oracle
import ttnn
import vectors
from golden_util import digests, sha

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    dev = ttnn.open_device(0)
    yield dev
    ttnn.close_device(dev)


@pytest.mark.parametrize("dtype,ofmt,name", [(ttnn.bfloat8_b, 0, "bfp8"), (ttnn.bfloat4_b, 1, "bfp4")])
@pytest.mark.parametrize("on_device", [False, True])
def test_from_torch_bytes_and_to_torch_values_match_golden(device, dtype, ofmt, name, on_device):
    d = digests()
    x = vectors.randn(0, (2, 3, 64, 96), 0.02)
    t = ttnn.from_torch(x, dtype=dtype, layout=ttnn.TILE_LAYOUT, device=device if on_device else None)
    assert list(t.shape) == [2, 3, 64, 96] and t.dtype == dtype and t.layout == ttnn.TILE_LAYOUT
    assert t.storage_type() == (ttnn.StorageType.DEVICE if on_device else ttnn.StorageType.OWNED)
    assert sha(np.frombuffer(t.buffer(), np.uint8)) == d[f"rand_2x3x64x96_seed0_{name}_from_torch"]
    y = ttnn.to_torch(t)
    assert y.dtype == torch.float32 and y.shape == x.shape
    assert sha(y.numpy().view(np.uint32)) == d[f"rand_2x3x64x96_seed0_{name}_to_torch"]


@pytest.mark.parametrize("dtype,atol", [(ttnn.bfloat8_b, 1e-2), (ttnn.bfloat4_b, 0.2)])
def test_rand_round_trip_tolerance(device, dtype, atol):
    torch.manual_seed(0)
    x = torch.rand(2, 3, 64, 96)
    t = ttnn.from_torch(x, dtype=dtype, layout=ttnn.TILE_LAYOUT, device=device)
    t = ttnn.from_device(t)
    assert torch.allclose(ttnn.to_torch(t), x, atol=atol, rtol=0)


@pytest.mark.parametrize("dtype,ofmt", [(ttnn.bfloat8_b, 0), (ttnn.bfloat4_b, 1)])
def test_shapes_that_need_tile_padding(device, orc, dtype, ofmt):
    """7x3 bf16, as tests/ttnn/unit_tests/test_to_and_from_torch.py: zero-padded to one tile, logical shape kept."""
    torch.manual_seed(0)
    x = torch.rand(7, 3, dtype=torch.bfloat16)
    t = ttnn.from_torch(x, dtype=dtype, layout=ttnn.TILE_LAYOUT)
    assert list(t.shape) == [7, 3] and list(t.shape.with_tile_padding()) == [32, 32]
    xp = np.zeros((32, 32), np.float32)
    xp[:7, :3] = x.float().numpy()
    assert np.array_equal(np.frombuffer(t.buffer(), np.uint8), orc.from_torch(xp, ofmt, 1, 32, 32))
    y = ttnn.to_torch(t)
    assert y.shape == (7, 3)
    want = orc.to_torch(orc.from_torch(xp, ofmt, 1, 32, 32), ofmt, 1, 32, 32).reshape(32, 32)[:7, :3]
    assert np.array_equal(y.numpy(), want)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(32, 32), (1, 1, 64, 96), (3, 50, 70)])
def test_to_layout_round_trip_plain_types(device, dt, shape):
    x = torch.randn(shape).to(dt)
    t = ttnn.from_torch(x, layout=ttnn.ROW_MAJOR_LAYOUT, device=device)
    tt = ttnn.to_layout(t, ttnn.TILE_LAYOUT)
    assert tt.layout == ttnn.TILE_LAYOUT and list(tt.shape) == list(shape)
    assert torch.equal(ttnn.to_torch(tt), x)
    direct = ttnn.from_torch(x, layout=ttnn.TILE_LAYOUT, device=device)
    assert direct.buffer() == tt.buffer()


def test_block_float_row_major_form_matches_the_reference_sequence(device, orc):
    """to(ROW_MAJOR) of a block-float tensor packs the row-major fp32 stream (tensor_impl.cpp:179-197)."""
    x = vectors.randn(5, (64, 96), 0.02)
    t = ttnn.from_torch(x, dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device)
    rm = ttnn.to_layout(t, ttnn.ROW_MAJOR_LAYOUT)
    packed = orc.from_torch(x.numpy(), 0, 1, 64, 96)
    want = orc.pack(orc.untilize(orc.unpack(packed, 0), 1, 64, 96), 0)
    assert np.array_equal(np.frombuffer(rm.buffer(), np.uint8), want)
    back = ttnn.to_layout(rm, ttnn.TILE_LAYOUT)
    assert back.buffer() == t.buffer()


@pytest.mark.parametrize("w_dtype", [ttnn.bfloat8_b, ttnn.bfloat4_b, ttnn.bfloat16])
@pytest.mark.parametrize("a_shape,w_shape", [((1, 1, 32, 256), (256, 384)), ((32, 128), (128, 128)), ((2, 64, 96), (96, 160)),
                                              ((1, 1, 7, 100), (100, 60))])
def test_matmul_against_torch(device, w_dtype, a_shape, w_shape):
    x = vectors.randn(11, a_shape, 1.0).bfloat16()
    w = vectors.randn(12, w_shape, 0.02)
    a = ttnn.from_torch(x, layout=ttnn.TILE_LAYOUT, device=device)
    b = ttnn.from_torch(w, dtype=w_dtype, layout=ttnn.TILE_LAYOUT, device=device)
    y = ttnn.matmul(a, b)
    assert list(y.shape) == list(a_shape[:-1]) + [w_shape[-1]] and y.dtype == ttnn.bfloat16
    w_ref = ttnn.to_torch(b).float()
    y_ref = x.float() @ w_ref
    got = ttnn.to_torch(y).float()
    assert oracle.comp_pcc(y_ref.numpy(), got.numpy()) >= 0.9999
    assert (got - y_ref).abs().max() / y_ref.abs().max() <= 1e-2
    assert torch.equal(ttnn.to_torch(a @ b), ttnn.to_torch(y))


@pytest.mark.parametrize("activation", [None, "relu", "gelu", "silu"])
def test_linear_with_bias_and_activation(device, activation):
    x = vectors.randn(21, (1, 1, 32, 4544 // 8 // 32 * 32), 1.0).bfloat16()
    K = x.shape[-1]
    w = vectors.randn(22, (K, 1024), 0.02)
    bias = vectors.randn(23, (1, 1024), 0.5).bfloat16()
    a = ttnn.from_torch(x, layout=ttnn.TILE_LAYOUT, device=device)
    b = ttnn.from_torch(w, dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device)
    bt = ttnn.from_torch(bias, layout=ttnn.TILE_LAYOUT, device=device)
    y = ttnn.to_torch(ttnn.linear(a, b, bias=bt, activation=activation, core_grid=ttnn.CoreGrid(y=4, x=8),
                                  use_1d_systolic_array=True)).float()
    ref = x.float() @ ttnn.to_torch(b) + bias.float()
    ref = {None: lambda v: v, "relu": torch.relu, "gelu": torch.nn.functional.gelu, "silu": torch.nn.functional.silu}[activation](ref)
    assert oracle.comp_pcc(ref.numpy(), y.numpy()) >= 0.9999
    assert (y - ref).abs().max() / ref.abs().max() <= 1e-2
    y32 = ttnn.linear(a, b, bias=bt, activation=activation, dtype=ttnn.float32)
    assert y32.dtype == ttnn.float32


def test_matmul_errors(device):
    a = ttnn.from_torch(torch.zeros(32, 64, dtype=torch.bfloat16), layout=ttnn.TILE_LAYOUT, device=device)
    b = ttnn.from_torch(torch.zeros(32, 64), dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device)
    with pytest.raises(RuntimeError, match="width of the first tensor must be equal to the height of the second"):
        ttnn.matmul(a, b)
    host = ttnn.from_torch(torch.zeros(64, 32), dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT)
    with pytest.raises(RuntimeError, match="must be on device"):
        ttnn.matmul(a, host)


def test_single_device_mesh_and_cache_on_device(device, tmp_path):
    mesh = ttnn.open_device_mesh(ttnn.DeviceGrid(1, 1), [0])
    w = vectors.randn(3, (64, 128), 0.02)
    t = ttnn.as_tensor(w, dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device, cache_file_name=str(tmp_path / "w"))
    u = ttnn.as_tensor(torch.zeros_like(w), dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device, cache_file_name=str(tmp_path / "w"))
    assert u.buffer() == t.buffer() and u.storage_type() == ttnn.StorageType.DEVICE
    s = ttnn.from_torch(w, dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device, mesh_mapper=ttnn.ShardTensorToMesh(mesh, dim=-1))
    g = ttnn.all_gather(s, dim=-1, num_links=1)
    assert torch.equal(ttnn.to_torch(g, mesh_composer=ttnn.ConcatMeshToTensor(mesh, dim=-1)), ttnn.to_torch(t))


def test_linear_multi_equals_separate_linears(device):
    """ttnn.linear_multi: q / k / v style projections of one activation in one launch, then a further linear on a result."""
    x = vectors.randn(31, (1, 1, 32, 2048), 1.0).bfloat16()
    a = ttnn.from_torch(x, layout=ttnn.TILE_LAYOUT, device=device)
    ws = [ttnn.from_torch(vectors.randn(32 + j, (2048, n), 0.02), dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device)
          for j, n in enumerate((1024, 128, 256))]
    bias = ttnn.from_torch(vectors.randn(40, (1, 1024), 0.5).bfloat16(), layout=ttnn.TILE_LAYOUT, device=device)
    outs = ttnn.linear_multi(a, ws, biases=[bias, None, None], activation="silu")
    assert len(outs) == 3
    for j, (w, y) in enumerate(zip(ws, outs)):
        want = ttnn.to_torch(ttnn.linear(a, w, bias=bias if j == 0 else None, activation="silu")).float()
        got = ttnn.to_torch(y).float()
        assert list(y.shape) == [1, 1, 32, [1024, 128, 256][j]]
        assert oracle.comp_pcc(want.numpy(), got.numpy()) >= 0.9999
        assert (got - want).abs().max() / want.abs().max() <= 1e-2
    # a result feeds the next op like any other tensor
    w2 = ttnn.from_torch(vectors.randn(45, (1024, 256), 0.02), dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device)
    z = ttnn.to_torch(ttnn.linear(outs[0], w2)).float()
    z_ref = ttnn.to_torch(outs[0]).float() @ ttnn.to_torch(w2)
    assert oracle.comp_pcc(z_ref.numpy(), z.numpy()) >= 0.9999
    with pytest.raises(RuntimeError):
        ttnn.linear_multi(a, ws + ws)                     # more than four weights
    with pytest.raises(RuntimeError):
        ttnn.linear_all_gather(a, ws[0])                  # needs multi-device tensors


@pytest.mark.parametrize("dtype,ofmt", [(ttnn.bfloat8_b, 0), (ttnn.bfloat4_b, 1)])
@pytest.mark.parametrize("shape", [(1, 1, 64, 96), (2, 3, 32, 32), (1, 1, 50, 70)])
def test_to_layout_with_dtype_packs_on_the_device(device, orc, dtype, ofmt, shape):
    """ttnn.to_layout(x, TILE_LAYOUT, dtype=bfloat8_b) on a device tensor (the reference's tilize with output_dtype,
    ttnn/ttnn/operations/core.py:677-711): the packed bytes equal the host packer's on the tile-padded tensor."""
    x = vectors.randn(51, shape, 0.05)
    for src in (x, x.bfloat16()):
        rm = ttnn.from_torch(src, layout=ttnn.ROW_MAJOR_LAYOUT, device=device)
        t = ttnn.to_layout(rm, ttnn.TILE_LAYOUT, dtype=dtype)
        assert t.dtype == dtype and t.layout == ttnn.TILE_LAYOUT and list(t.shape) == list(shape)
        H, W = shape[-2], shape[-1]
        Hp, Wp = (H + 31) // 32 * 32, (W + 31) // 32 * 32
        outer = int(np.prod(shape[:-2]))
        padded = np.zeros((outer, Hp, Wp), dtype=np.float32)
        padded[:, :H, :W] = src.float().numpy().reshape(outer, H, W)
        want = orc.pack(orc.tilize(padded, outer, Hp, Wp), ofmt)                   # host packer on the padded, tilized tensor
        got = ttnn.to_torch(t)                                    # values: unpacked on the device
        ref = torch.from_numpy(orc.untilize(orc.unpack(want, ofmt), outer, Hp, Wp).reshape(outer, Hp, Wp)[:, :H, :W].copy()).reshape(shape)
        assert torch.equal(got, ref)
        # and back: block-float tiles -> bfloat16 tiles on the device
        back = ttnn.to_layout(t, ttnn.TILE_LAYOUT, dtype=ttnn.bfloat16)
        assert back.dtype == ttnn.bfloat16 and torch.equal(ttnn.to_torch(back).float(), ref)
    with pytest.raises(RuntimeError, match="Unsupported datatype conversion"):
        ttnn.to_layout(ttnn.from_torch(x, layout=ttnn.ROW_MAJOR_LAYOUT), ttnn.TILE_LAYOUT, dtype=dtype)      # not on device
    with pytest.raises(RuntimeError, match="Unsupported datatype conversion"):
        ttnn.to_layout(rm, ttnn.ROW_MAJOR_LAYOUT, dtype=dtype)


def _unpacked(t, ofmt, orc):
    """fp32 values of a block-float ttnn tensor, by the ORACLE's unpacker on the tensor's own bytes."""
    shape = list(t.shape.with_tile_padding())
    outer = int(np.prod(shape[:-2])) if len(shape) > 2 else 1
    return torch.from_numpy(orc.to_torch(np.frombuffer(t.buffer(), np.uint8), ofmt, outer, shape[-2], shape[-1]).reshape(shape).copy())


def test_batched_matmul_with_block_float_operands_and_output(device, orc):
    """The attention-style bmm of tests/tt_eager/python_api_testing/unit_testing/misc/test_matmul.py:204-320: both operands
    bfloat8_b with the same batch dimensions, bfloat8_b output (dtype defaults to the first operand's). The output bytes are
    the host packer's applied to the fp32 product: checked against the oracle packing of an fp32 torch matmul of the
    oracle-unpacked operands."""
    B, H, M, K, N = 2, 4, 96, 64, 128
    a = vectors.randn(31, (B, H, M, K), 1.0)
    b = vectors.randn(32, (B, H, K, N), 1.0)
    at = ttnn.from_torch(a, dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device)
    bt = ttnn.from_torch(b, dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device)
    out = ttnn.matmul(at, bt)
    assert out.dtype == ttnn.bfloat8_b and list(out.shape) == [B, H, M, N]
    ref = _unpacked(at, oracle.BFP8_B, orc) @ _unpacked(bt, oracle.BFP8_B, orc)
    got = ttnn.to_torch(out)
    pcc = oracle.comp_pcc(ref.numpy(), got.numpy())
    assert pcc >= 0.9999, pcc
    # bit-level: pack-after-matmul. The fp32 product itself differs from torch's in summation order (a few ulps), which
    # moves a packed code by at most one step: compare the unpacked values within one code step of each row's exponent.
    want = orc.to_torch(orc.from_torch(ref.numpy(), oracle.BFP8_B, B * H, M, N), oracle.BFP8_B, B * H, M, N).reshape(B, H, M, N)
    step = np.abs(want).reshape(B, H, M, N // 16, 16).max(-1, keepdims=True) / 64.0
    assert np.all(np.abs(got.numpy() - want).reshape(B, H, M, N // 16, 16) <= step + 1e-12)
    # bfloat16 output on request, float32 too
    out16 = ttnn.matmul(at, bt, dtype=ttnn.bfloat16)
    assert out16.dtype == ttnn.bfloat16
    assert oracle.comp_pcc(ref.numpy(), ttnn.to_torch(out16).float().numpy()) >= 0.9999
    with pytest.raises(RuntimeError):
        ttnn.matmul(at, ttnn.from_torch(b[:1], dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device))   # batch mismatch


@pytest.mark.parametrize("out_dtype,ofmt", [(ttnn.bfloat8_b, 0), (ttnn.bfloat4_b, 1)])
def test_linear_with_block_float_activation_and_output(device, orc, out_dtype, ofmt):
    """bfloat8_b activations (the reference admits them, tt_eager/tt_dnn/op_library/bmm/bmm_op.cpp:839) are expanded exactly;
    a block-float output equals the device packer applied to the float32 result of the same matmul, bit for bit."""
    M, K, N = 32, 1024, 512
    x = vectors.randn(41, (1, 1, M, K), 1.0)
    w = vectors.randn(42, (K, N), 0.05)
    xt = ttnn.from_torch(x, dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device)
    wt = ttnn.from_torch(w, dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device)
    y32 = ttnn.linear(xt, wt, dtype=ttnn.float32, activation="relu")
    yq = ttnn.linear(xt, wt, dtype=out_dtype, activation="relu")
    assert yq.dtype == out_dtype and list(yq.shape) == [1, 1, M, N]
    want = orc.from_torch(ttnn.to_torch(y32).numpy(), ofmt, 1, M, N)          # host packer on the fp32 result
    assert np.array_equal(np.frombuffer(yq.buffer(), np.uint8), want)
    ref = torch.relu(_unpacked(xt, oracle.BFP8_B, orc).reshape(M, K) @ _unpacked(wt, oracle.BFP8_B, orc).reshape(K, N))
    assert oracle.comp_pcc(ref.numpy(), ttnn.to_torch(y32).reshape(M, N).numpy()) >= 0.9999
    # the packed result feeds the next linear directly
    w2 = ttnn.from_torch(vectors.randn(43, (N, 128), 0.05), dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device)
    z = ttnn.linear(yq, w2, dtype=ttnn.bfloat16)
    zref = _unpacked(yq, ofmt, orc).reshape(M, N) @ _unpacked(w2, oracle.BFP8_B, orc).reshape(N, 128)
    assert oracle.comp_pcc(zref.numpy(), ttnn.to_torch(z).float().reshape(M, 128).numpy()) >= 0.9999


@pytest.mark.parametrize("rows", [32, 64])
def test_linear_gated_equals_the_three_op_sequence(device, orc, rows):
    """ttnn.linear_gated against ttnn.linear(silu) x ttnn.linear -> ttnn.mul (mistral_mlp.py:51-73): one launch for 32 rows,
    the fallback sequence for 64; both within bf16 rounding of the unfused result (which rounds the two factors first)."""
    H, F = 1024, 2048
    x = vectors.randn(51, (1, 1, rows, H), 1.0).bfloat16()
    w1 = ttnn.from_torch(vectors.randn(52, (H, F), 0.05), dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device)
    w3 = ttnn.from_torch(vectors.randn(53, (H, F), 0.05), dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device)
    xt = ttnn.from_torch(x, layout=ttnn.TILE_LAYOUT, device=device)
    fused = ttnn.linear_gated(xt, w1, w3)
    assert list(fused.shape) == [1, 1, rows, F] and fused.dtype == ttnn.bfloat16
    unfused = ttnn.mul(ttnn.linear(xt, w1, activation="silu"), ttnn.linear(xt, w3))
    xf = x.float().reshape(rows, H)
    ref = torch.nn.functional.silu(xf @ _unpacked(w1, oracle.BFP8_B, orc).reshape(H, F)) * (xf @ _unpacked(w3, oracle.BFP8_B, orc).reshape(H, F))
    for got in (fused, unfused):
        y = ttnn.to_torch(got).float().reshape(rows, F)
        assert oracle.comp_pcc(ref.numpy(), y.numpy()) >= 0.9999
        assert float((y - ref).abs().max() / ref.abs().max()) <= 1e-2
