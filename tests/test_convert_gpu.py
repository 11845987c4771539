"""GPU parity of the layout-conversion and block-float kernels against the CPU oracle and the golden
vectors, through the C ABI. Bit-exact everywhere."""
import numpy as np
import pytest

import cabi
import vectors
from golden_util import arrays, digests, sha

pytestmark = pytest.mark.gpu
FMTS = [(0, cabi.BFLOAT8_B, "bfp8"), (1, cabi.BFLOAT4_B, "bfp4")]


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


@pytest.mark.parametrize("ofmt,fmt,name", FMTS)
def test_known_answer_and_adversarial_goldens(ttb, orc, ofmt, fmt, name):
    g, d = arrays(), digests()
    tile = vectors.arange_tile()
    # the reference's known-answer case: row-major in == tilized in
    p_rm = host(ttb.pack(dev(tile), fmt, 1, 32, 32, row_major=True))
    p_t = host(ttb.pack(dev(orc.tilize(tile, 1, 32, 32)), fmt, 1, 32, 32, row_major=False))
    assert np.array_equal(p_rm, g[f"arange_{name}_packed"])
    assert np.array_equal(p_t, g[f"arange_{name}_packed"])
    u_rm = host(ttb.unpack(dev(p_rm), fmt, 1, 32, 32, row_major=True)).view(np.uint32)
    assert np.array_equal(u_rm, g[f"arange_{name}_unpacked_rm"])
    # adversarial bit patterns, consumed as a sequential (already tiled) stream like the oracle does
    adv = vectors.adversarial_bits()
    x = dev(adv.view(np.float32))
    p = host(ttb.pack(x, fmt, 1, 16 * 32, 32, row_major=False))
    assert np.array_equal(p, g[f"adv_{name}_packed"])
    assert sha(host(ttb.unpack(dev(p), fmt, 1, 16 * 32, 32, row_major=False)).view(np.uint32)) == d[f"adv_{name}_unpacked"]
    # the literal host sequence of from_torch (pack, unpack, tilize, pack) on a [512, 32] tensor
    p2 = host(ttb.pack(x, fmt, 1, 16 * 32, 32, row_major=True, two_pass=True))
    assert sha(p2) == d[f"adv_{name}_from_torch_16x1024"]
    assert np.array_equal(p2, orc.from_torch(adv, ofmt, 1, 512, 32))


@pytest.mark.parametrize("ofmt,fmt,name", FMTS)
def test_exhaustive_unpack(ttb, orc, ofmt, fmt, name):
    d = digests()
    ex = vectors.exhaustive_packed(ofmt)
    u = host(ttb.unpack(dev(ex), fmt, 1, 256 * 32, 32, row_major=False)).view(np.uint32)
    assert sha(u) == d[f"exhaustive_{name}_unpacked"]
    u2 = host(ttb.unpack(dev(ex), fmt, 1, 256 * 32, 32, row_major=True, two_pass=True)).view(np.uint32)
    assert sha(u2) == d[f"exhaustive_{name}_to_torch"]
    # bf16 destination is the exact high half of the fp32 result
    import torch
    ub = host(ttb.unpack(dev(ex), fmt, 1, 256 * 32, 32, row_major=False, dtype=torch.bfloat16).view(torch.int16)).view(np.uint16)
    assert np.array_equal(ub, (u >> 16).astype(np.uint16))


@pytest.mark.parametrize("ofmt,fmt,name", FMTS)
@pytest.mark.parametrize("label,seed,shape", [("rand_2x3x64x96_seed0", 0, (6, 64, 96)), ("c2_slice_256x512_seed1", 1, (1, 256, 512)),
                                               ("c1_4096x4096_seed0", 0, (1, 4096, 4096))])
def test_seeded_tensors_match_golden_digests(ttb, ofmt, fmt, name, label, seed, shape):
    d = digests()
    x = vectors.randn(seed, shape, 0.02)
    for two_pass in (False, True):
        packed = ttb.pack(x.cuda(), fmt, *shape, row_major=True, two_pass=two_pass)
        assert sha(host(packed)) == d[f"{label}_{name}_from_torch"]
        back = ttb.unpack(packed, fmt, *shape, row_major=True, two_pass=two_pass)
        assert sha(host(back).view(np.uint32)) == d[f"{label}_{name}_to_torch"]


@pytest.mark.parametrize("ofmt,fmt,name", FMTS)
@pytest.mark.parametrize("shape", [(1, 32, 32), (1, 32, 64), (1, 64, 32), (3, 96, 160), (1, 7, 3), (2, 33, 100), (1, 1, 129), (5, 31, 31)])
def test_ragged_and_small_shapes_against_oracle(ttb, orc, ofmt, fmt, name, shape):
    """Shapes that are not multiples of 32 are zero-padded to tiles, like ttnn.from_torch's pad-to-tile detour."""
    o, H, W = shape
    Hp, Wp = (H + 31) // 32 * 32, (W + 31) // 32 * 32
    rng = np.random.default_rng(H * 1000 + W)
    x = (rng.standard_normal(shape) * 0.05).astype(np.float32)
    xp = np.zeros((o, Hp, Wp), np.float32)
    xp[:, :H, :W] = x
    want = orc.pack(orc.tilize(xp, o, Hp, Wp), ofmt)
    got = host(ttb.pack(dev(x), fmt, o, H, W, row_major=True))
    assert np.array_equal(got, want)
    # bf16 source: exact widening
    import torch
    xb = torch.from_numpy(x).bfloat16()
    xbp = np.zeros((o, Hp, Wp), np.float32)
    xbp[:, :H, :W] = xb.float().numpy()
    got_b = host(ttb.pack(xb.cuda(), fmt, o, H, W, row_major=True))
    assert np.array_equal(got_b, orc.pack(orc.tilize(xbp, o, Hp, Wp), ofmt))
    # unpack drops the padding again
    back = host(ttb.unpack(dev(want), fmt, o, H, W, row_major=True)).reshape(o, H, W)
    full = orc.untilize(orc.unpack(want, ofmt), o, Hp, Wp).reshape(o, Hp, Wp)
    assert np.array_equal(back.view(np.uint32), full[:, :H, :W].copy().view(np.uint32))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "int32", "int16"])
@pytest.mark.parametrize("shape", [(1, 32, 32), (2, 64, 96), (1, 7, 3), (3, 50, 130), (1, 32, 4544)])
def test_tilize_untilize(ttb, orc, dtype, shape):
    import torch
    o, H, W = shape
    Hp, Wp = (H + 31) // 32 * 32, (W + 31) // 32 * 32
    tdt = getattr(torch, dtype)
    x = (torch.arange(o * H * W, dtype=torch.float32) % 30011).to(tdt).reshape(shape)
    npdt = np.uint32 if x.element_size() == 4 else np.uint16
    raw = x.view(torch.int32 if x.element_size() == 4 else torch.int16).numpy().view(npdt)
    xp = np.zeros((o, Hp, Wp), npdt)
    xp[:, :H, :W] = raw
    want = orc.tilize(xp, o, Hp, Wp).reshape(-1)
    tiled = ttb.tilize(x.cuda(), o, H, W)
    got = host(tiled.view(torch.int32 if x.element_size() == 4 else torch.int16)).view(npdt)
    assert np.array_equal(got, want)
    back = ttb.untilize(tiled, o, H, W)
    assert torch.equal(back.cpu().reshape(shape), x)


@pytest.mark.parametrize("fmt", [cabi.BFLOAT8_B, cabi.BFLOAT4_B])
def test_full_size_round_trip_properties(ttb, fmt):
    """At the largest weight of the benchmark configurations (8192 x 28672) the oracle is too slow to run in
    a test, so check size-independent properties: packing the unpacked values reproduces the packed bytes
    (idempotence), and tiled-in / row-major-in packing agree after an explicit tilize."""
    import torch
    K, N = 8192, 28672
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(K, N, generator=g, device="cuda", dtype=torch.float32) * 0.02
    p1 = ttb.pack(x, fmt, 1, K, N, row_major=True)
    u = ttb.unpack(p1, fmt, 1, K, N, row_major=True)
    p2 = ttb.pack(u, fmt, 1, K, N, row_major=True)
    assert torch.equal(p1, p2)
    tiled = ttb.tilize(x, 1, K, N)
    p3 = ttb.pack(tiled, fmt, 1, K, N, row_major=False)
    assert torch.equal(p1, p3)
    err = (u.reshape(K, N) - x).abs().max().item()
    assert err < (2e-3 if fmt == cabi.BFLOAT8_B else 2e-2)
