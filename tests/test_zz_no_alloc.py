"""The allocation-free decode entry point (ttb_matmul_decode_static) against the regular one.

Some callers cannot call cudaMalloc at the point where they need a matmul: an inference server that gave all device
memory to its own pool at start-up, or code running inside another runtime's callback where an allocation would
synchronise the device. For them the library carries its split-K scratch as a fixed device array. This file checks, through
the C ABI, that the variant produces what ttb_matmul produces - on two calls in a row, because the scratch is shared
between calls and keeps the previous call's contents - and that it refuses what it cannot serve. It is collected last so
that a run stopping at the first failure has already run every other test; it also passes when run alone."""
import pytest

import cabi
import vectors

pytestmark = pytest.mark.gpu


def _operands(ttb, M, K, N, w_dtype, seed):
    import torch
    x = vectors.randn(seed, (M, K), 1.0).bfloat16().cuda()
    w = (vectors.randn(seed + 1, (K, N), 0.02)).cuda()
    packed = ttb.pack(w, w_dtype, 1, K, N)
    return ttb.tilize(x, 1, M, K), packed


def _static(ttb, a, w, w_dtype, M, K, N, out_fp32=True):
    import torch
    out = torch.empty(M * N, dtype=torch.float32 if out_fp32 else torch.bfloat16, device="cuda")
    ttb.check(ttb.cdll.ttb_matmul_decode_static(a.data_ptr(), cabi.BFLOAT16, w.data_ptr(), w_dtype, None, out.data_ptr(),
                                                cabi.FLOAT32 if out_fp32 else cabi.BFLOAT16, 1, M, K, N, 0, 0, None))
    ttb.check(ttb.check_status(None))
    return out


@pytest.mark.parametrize("M,K,N,w_dtype", [(32, 4096, 1024, cabi.BFLOAT8_B),     # K split over many blocks: uses the scratch
                                           (32, 4096, 4096, cabi.BFLOAT8_B),
                                           (64, 4096, 512, cabi.BFLOAT4_B),
                                           (32, 256, 18176, cabi.BFLOAT8_B)])    # one block per tile: no scratch needed
def test_static_scratch_variant_matches_regular_entry_point_twice_in_a_row(ttb, M, K, N, w_dtype):
    import torch
    assert (ttb.matmul_workspace_bytes(w_dtype, 1, M, K, N, 0) > 0) == (N < 18176)
    a, w = _operands(ttb, M, K, N, w_dtype, 51)
    want = ttb.matmul(a, w, w_dtype, 1, M, K, N, out_fp32=True)
    first = _static(ttb, a, w, w_dtype, M, K, N)
    # a different problem in between leaves its own partial sums in the shared scratch
    a2, w2 = _operands(ttb, 32, 2048, 256, cabi.BFLOAT8_B, 61)
    _static(ttb, a2, w2, cabi.BFLOAT8_B, 32, 2048, 256)
    second = _static(ttb, a, w, w_dtype, M, K, N)
    scale = want.abs().max().item()
    for got in (first, second):
        # Same kernel and operands; the static entry always adds the split-K partial sums in block order, ttb_matmul may
        # add them in arrival order, so the two can differ in the last bits: the tolerance of the kernel-agreement tests.
        assert torch.allclose(got, want, rtol=1e-4, atol=1e-4 * scale)
    assert torch.equal(first, second)      # the static entry itself is bit-reproducible
    # What the name promises: a further call neither takes nor returns device memory (cudaMemGetInfo before and after,
    # with the output buffer allocated beforehand).
    import ctypes
    out = torch.empty(M * N, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    before, after = ctypes.c_int64(), ctypes.c_int64()
    ttb.check(ttb.mem_info(ctypes.byref(before), None))
    ttb.check(ttb.cdll.ttb_matmul_decode_static(a.data_ptr(), cabi.BFLOAT16, w.data_ptr(), w_dtype, None, out.data_ptr(), cabi.FLOAT32,
                                                1, M, K, N, 0, 0, None))
    ttb.check(ttb.check_status(None))
    ttb.check(ttb.mem_info(ctypes.byref(after), None))
    assert before.value == after.value
    assert torch.equal(out, first)


def test_static_scratch_variant_takes_the_layout_flags(ttb, orc):
    """Row-major activations in, row-major result out, through the allocation-free entry point."""
    import torch
    from test_matmul_gpu import check, make_case
    M, K, N = 32, 4096, 1024
    x, w_dev, w_ref = make_case(ttb, orc, 81, M, K, N, cabi.BFLOAT8_B)
    out = torch.empty(M * N, dtype=torch.float32, device="cuda")
    xd = x.cuda().contiguous()
    ttb.check(ttb.cdll.ttb_matmul_decode_static(xd.data_ptr(), cabi.BFLOAT16, w_dev.data_ptr(), cabi.BFLOAT8_B, None, out.data_ptr(),
                                                cabi.FLOAT32, 1, M, K, N, 0, cabi.MM_A_ROW_MAJOR | cabi.MM_OUT_ROW_MAJOR, None))
    ttb.check(ttb.check_status(None))
    check(out.reshape(M, N), x.float() @ w_ref)


def test_static_scratch_variant_refuses_what_it_cannot_serve(ttb):
    import torch
    a, w = _operands(ttb, 32, 256, 128, cabi.BFLOAT8_B, 71)
    out = torch.empty(32 * 128, dtype=torch.bfloat16, device="cuda")
    # prefill-sized row count: not a decode shape
    rc = ttb.cdll.ttb_matmul_decode_static(a.data_ptr(), cabi.BFLOAT16, w.data_ptr(), cabi.BFLOAT8_B, None, out.data_ptr(), cabi.BFLOAT16,
                                           1, 512, 256, 128, 0, 0, None)
    assert rc == -3 and b"ttb_matmul" in ttb.cdll.ttb_last_error()
    # A reduction that needs more scratch than the built-in array is refused before anything is launched. The library's own
    # figure is checked first, and the operands are full-sized for the shape, so that a planner change can neither turn
    # this into a launch that the test did not expect nor into one that leaves its buffers.
    M2, K2, N2 = 256, 65536, 4096
    assert ttb.matmul_decode_static_scratch_bytes(cabi.BFLOAT8_B, 1, M2, K2, N2) > (16 << 20) + 65536
    a2, w2 = _operands(ttb, M2, K2, N2, cabi.BFLOAT8_B, 72)
    out2 = torch.empty(M2 * N2, dtype=torch.bfloat16, device="cuda")
    rc = ttb.cdll.ttb_matmul_decode_static(a2.data_ptr(), cabi.BFLOAT16, w2.data_ptr(), cabi.BFLOAT8_B, None, out2.data_ptr(), cabi.BFLOAT16,
                                           1, M2, K2, N2, 0, 0, None)
    assert rc == -4 and b"ttb_matmul" in ttb.cdll.ttb_last_error()
    # a large shape that fits runs through the entry point
    M3, K3, N3 = 256, 16384, 7680
    assert 0 < ttb.matmul_decode_static_scratch_bytes(cabi.BFLOAT8_B, 1, M3, K3, N3) <= (16 << 20) + 65536
    a3, w3 = _operands(ttb, M3, K3, N3, cabi.BFLOAT8_B, 73)
    out3 = torch.empty(M3 * N3, dtype=torch.bfloat16, device="cuda")
    ttb.check(ttb.cdll.ttb_matmul_decode_static(a3.data_ptr(), cabi.BFLOAT16, w3.data_ptr(), cabi.BFLOAT8_B, None, out3.data_ptr(), cabi.BFLOAT16,
                                                1, M3, K3, N3, 0, 0, None))
    ttb.check(ttb.check_status(None))
    ref3 = ttb.matmul(a3, w3, cabi.BFLOAT8_B, 1, M3, K3, N3)
    assert torch.allclose(out3.float(), ref3.float(), rtol=2 ** -6, atol=1e-3 * float(ref3.float().abs().max()))
    rc = ttb.cdll.ttb_matmul_decode_static(None, cabi.BFLOAT16, w.data_ptr(), cabi.BFLOAT8_B, None, out.data_ptr(), cabi.BFLOAT16,
                                           1, 32, 256, 128, 0, 0, None)
    assert rc == -1
