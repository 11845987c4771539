"""Deterministic test inputs shared by the oracle tests, the GPU parity tests and the golden generator."""
import numpy as np


def arange_tile():
    """The reference's own known-answer input: one 32x32 tile holding 0..1023
    (tests/tt_metal/tt_metal/test_bfp8_conversion.cpp:25-33, test_bfp4_conversion.cpp)."""
    return np.arange(1024, dtype=np.float32)


def adversarial_bits(ntiles=16, seed=7):
    """fp32 bit patterns (row-major stream, 16 values per shared-exponent group) that exercise every branch
    of the packers: zeros of both signs, a huge value beside tiny ones (alignment shifts past 24 and past
    32), denormals, Inf/NaN, all-ones mantissas (saturation), exact rounding ties and their neighbours,
    negative maxima, groups with very small exponents (the unpacker's unclamped exponent arithmetic) and
    arbitrary 32-bit patterns."""
    rng = np.random.default_rng(seed)
    n = ntiles * 1024
    u = (rng.standard_normal(n) * 0.02).astype(np.float32).view(np.uint32).copy()
    f = lambda v: np.float32(v).view(np.uint32)
    u[0:16] = 0
    u[16:32] = 0x80000000
    u[32:48] = [0, 0x80000000] * 8
    u[48] = f(1e30); u[49:64] = f(1e-30)
    u[64] = f(-3.0e4); u[65:80] = f(1.0e-3) ; u[66] = f(2.0e-3)
    u[80:96] = np.arange(16, dtype=np.uint32) + 1                      # denormals
    u[96] = 0x7F800000; u[97] = 0xFF800000; u[98] = 0x7FC01234; u[99:112] = f(1.5)
    u[112:128] = 0x3F7FFFFF                                             # all-ones mantissa -> saturates
    u[128:144] = 0x3F800000 | (np.arange(16, dtype=np.uint32) << 16); u[128] = 0x40000000   # ties at bit 16, d = 1
    u[144:160] = 0x3F800000 | (np.arange(16, dtype=np.uint32) << 20); u[144] = 0x40000000   # ties at bit 20 (bfp4)
    u[160:176] = 0x3F808000 + np.arange(16, dtype=np.uint32) - 8        # one ulp either side of a tie
    u[176:192] = 0x00800000 | rng.integers(0, 1 << 23, 16).astype(np.uint32); u[177] = 1; u[178] = 0x80400000
    u[192:208] = 0x01000000 | rng.integers(0, 1 << 23, 16).astype(np.uint32)   # E = 2
    u[208:224] = 0x03000000 | rng.integers(0, 1 << 23, 16).astype(np.uint32); u[209] = 0x00812345   # E = 6 with a small one
    u[224:240] = 0xBF800000 | rng.integers(0, 1 << 23, 16).astype(np.uint32)   # all negative
    u[240:256] = f(1.0); u[241] = f(1.0 / 64); u[242] = f(1.0 / 128); u[243] = f(1.0 / 256); u[244] = f(-1.0 / 128)
    k = 2048
    u[k:k + 4096] = rng.integers(0, 2 ** 32, 4096, dtype=np.uint64).astype(np.uint32)   # arbitrary patterns
    u[k + 4096:k + 6144] = (rng.integers(0, 2 ** 32, 2048, dtype=np.uint64).astype(np.uint32) & 0x807FFFFF) | \
        (rng.integers(100, 140, 2048).astype(np.uint32) << 23)                            # wide exponent spread
    return u


def exhaustive_packed(fmt):
    """Packed tiles covering every code under many shared exponents: tile t uses exponent t for all rows.
    bfloat8_b: 256 tiles x all 256 byte values; bfloat4_b: 256 tiles x all 256 nibble pairs."""
    tb = 1088 if fmt == 0 else 576
    raw = np.zeros((256, tb), np.uint8)
    for t in range(256):
        raw[t, :64] = t
        raw[t, 64:] = np.tile(np.arange(256, dtype=np.uint8), (tb - 64) // 256)
    return raw.reshape(-1)


def randn(seed, shape, std=1.0):
    """torch CPU generator: the seeded inputs of the benchmark configurations."""
    import torch
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std)
