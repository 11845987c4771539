"""Pins the CPU oracle (the plain-C restatement) against (1) the golden vectors generated from the
reference's own host code, (2) the reference's known-answer tests, restated, and (3) the compiled reference
itself wherever its shared object is available. No GPU needed."""
import numpy as np
import pytest

import oracle
import vectors
from golden_util import arrays, digests, sha

FMTS = [(0, "bfp8"), (1, "bfp4")]


@pytest.mark.parametrize("fmt,name", FMTS)
def test_port_matches_golden_vectors(orc, fmt, name):
    g, d = arrays(), digests()
    tile, adv = vectors.arange_tile(), vectors.adversarial_bits()
    assert np.array_equal(orc.pack(tile, fmt, in_tile_row_major=True), g[f"arange_{name}_packed"])
    assert np.array_equal(orc.unpack(g[f"arange_{name}_packed"], fmt, in_tile_row_major=True).view(np.uint32),
                          g[f"arange_{name}_unpacked_rm"])
    p = orc.pack(adv, fmt)
    assert np.array_equal(p, g[f"adv_{name}_packed"])
    assert sha(orc.unpack(p, fmt).view(np.uint32)) == d[f"adv_{name}_unpacked"]
    assert sha(orc.from_torch(adv, fmt, 1, 512, 32)) == d[f"adv_{name}_from_torch_16x1024"]
    ex = vectors.exhaustive_packed(fmt)
    assert sha(orc.unpack(ex, fmt).view(np.uint32)) == d[f"exhaustive_{name}_unpacked"]
    assert sha(orc.to_torch(ex, fmt, 1, 256 * 32, 32).view(np.uint32)) == d[f"exhaustive_{name}_to_torch"]


@pytest.mark.parametrize("fmt,name", FMTS)
@pytest.mark.parametrize("label,seed,shape", [("rand_2x3x64x96_seed0", 0, (6, 64, 96)), ("c2_slice_256x512_seed1", 1, (1, 256, 512)),
                                               ("c1_4096x4096_seed0", 0, (1, 4096, 4096))])
def test_port_matches_golden_digests_on_seeded_tensors(orc, fmt, name, label, seed, shape):
    d = digests()
    x = vectors.randn(seed, shape, 0.02).numpy()
    packed = orc.from_torch(x, fmt, *shape)
    assert sha(packed) == d[f"{label}_{name}_from_torch"]
    assert sha(orc.to_torch(packed, fmt, *shape).view(np.uint32)) == d[f"{label}_{name}_to_torch"]
    # the four-step host sequence collapses to one tilize + pack (and unpack + untilize) for finite inputs
    assert np.array_equal(packed, orc.pack(orc.tilize(x, *shape), fmt))
    assert np.array_equal(orc.to_torch(packed, fmt, *shape).view(np.uint32),
                          orc.untilize(orc.unpack(packed, fmt), *shape).view(np.uint32))


def test_tilize_golden(orc):
    t = np.arange(3 * 64 * 96, dtype=np.float32)
    tiled = orc.tilize(t, 3, 64, 96)
    assert sha(tiled) == digests()["tilize_3x64x96_arange"]
    assert np.array_equal(orc.untilize(tiled, 3, 64, 96), t)
    h = np.arange(2 * 32 * 64, dtype=np.uint16)
    assert np.array_equal(orc.untilize(orc.tilize(h, 2, 32, 64), 2, 32, 64), h)


@pytest.mark.parametrize("fmt,rtol", [(0, 0.01), (1, 0.15)])
def test_reference_known_answer_test_restated(orc, fmt, rtol):
    """tests/tt_metal/tt_metal/test_bfp8_conversion.cpp:30-75 and test_bfp4_conversion.cpp: row-major-in pack equals
    tilize-then-pack, unpacked values are close to the source (rtol 0.01 / 0.15, atol 8), and the two unpack
    orders are layout conversions of each other."""
    x = vectors.arange_tile()
    tiled = orc.tilize(x, 1, 32, 32)
    p_rm = orc.pack(x, fmt, in_tile_row_major=True)
    p_t = orc.pack(tiled, fmt, in_tile_row_major=False)
    assert np.array_equal(p_rm, p_t)
    u_rm = orc.unpack(p_rm, fmt, in_tile_row_major=True)
    u_t = orc.unpack(p_t, fmt, in_tile_row_major=False)
    assert np.all(np.abs(u_rm - x) <= 8.0 + rtol * np.abs(u_rm))
    assert np.all(np.abs(u_t - tiled) <= 8.0 + rtol * np.abs(u_t))
    assert np.array_equal(u_rm, orc.untilize(u_t, 1, 32, 32))
    assert np.array_equal(u_t, orc.tilize(u_rm, 1, 32, 32))


@pytest.mark.parametrize("fmt,atol", [(0, 1e-2), (1, 0.2)])
def test_round_trip_tolerance_of_reference_tensor_test(orc, fmt, atol):
    """tests/tt_eager/python_api_testing/unit_testing/misc/test_tensor.py:27-90: torch.rand(2,3,64,96) survives
    the block-float round trip within atol 1e-2 (bfloat8_b) / 0.2 (bfloat4_b)."""
    import torch
    torch.manual_seed(0)
    x = torch.rand(2, 3, 64, 96).numpy()
    y = orc.to_torch(orc.from_torch(x, fmt, 6, 64, 96), fmt, 6, 64, 96).reshape(x.shape)
    assert np.allclose(x, y, atol=atol, rtol=0)


@pytest.mark.parametrize("fmt", [0, 1])
def test_port_matches_compiled_reference(orc, fmt):
    ref = oracle.ref()
    if ref is None:
        pytest.skip("compiled reference not available here")
    rng = np.random.default_rng(11)
    for case in range(4):
        u = vectors.adversarial_bits(seed=100 + case) if case < 2 else \
            rng.integers(0, 2 ** 32, 8 * 1024, dtype=np.uint64).astype(np.uint32)
        for rm in (False, True):
            p = orc.pack(u, fmt, in_tile_row_major=rm)
            assert np.array_equal(p, ref.pack(u, fmt, in_tile_row_major=rm))
            assert np.array_equal(orc.unpack(p, fmt, in_tile_row_major=rm).view(np.uint32),
                                  ref.unpack(p, fmt, in_tile_row_major=rm).view(np.uint32))
        nt = u.size // 1024
        assert np.array_equal(orc.from_torch(u, fmt, 1, nt * 32, 32), ref.from_torch(u, fmt, 1, nt * 32, 32))
    ex = vectors.exhaustive_packed(fmt)
    assert np.array_equal(orc.unpack(ex, fmt).view(np.uint32), ref.unpack(ex, fmt).view(np.uint32))
    assert np.array_equal(orc.to_torch(ex, fmt, 2, 128 * 32, 32).view(np.uint32), ref.to_torch(ex, fmt, 2, 128 * 32, 32).view(np.uint32))
    x = (rng.standard_normal((3, 64, 96)) * 0.02).astype(np.float32)
    assert np.array_equal(orc.tilize(x, 3, 64, 96), ref.tilize(x, 3, 64, 96))
    assert np.array_equal(orc.untilize(x, 3, 64, 96), ref.untilize(x, 3, 64, 96))


def test_comp_pcc_definition():
    a = np.linspace(-1, 1, 1000)
    assert oracle.comp_pcc(a, a) == 1.0
    assert oracle.comp_pcc(a, -a) < -0.99
    assert oracle.comp_pcc(a, np.zeros_like(a)) == 0.0
    assert oracle.comp_pcc(a, a + 1e-3 * np.sin(37 * a)) > 0.9999
