"""GPU parity of ttb_matmul_sequence: several ttb_matmul_multi-shaped stages in one launch agree with the separate launches
to the last bf16 digit (the first stage to the byte; later stages may add their fp32 partial sums in another order, because
a block's two accumulators take alternate pairs of K groups counted over everything the block has done), repeat their own
bytes from launch to launch, match the fp32 reference within the matmul tolerances, and leave the scratch clean."""
import ctypes

import pytest

import cabi
import vectors
from test_matmul_gpu import check, make_big_case, make_case

pytestmark = pytest.mark.gpu


def _weight(ttb, orc, seed, M, K, N, w_dtype):
    if K * N > 8 << 20:
        return make_big_case(ttb, orc, seed, K, N, w_dtype)
    _, w, r = make_case(ttb, orc, seed, M, K, N, w_dtype, w_std=0.05)
    return w, r


def same_to_the_last_digit(a, b):
    """|a - b| <= one bf16 unit of the element (2^-7 relative) plus 1e-5 of the largest magnitude (cancellation)."""
    a, b = a.float(), b.float()
    return bool(((a - b).abs() <= b.abs() * 2.0 ** -7 + 1e-5 * b.abs().max()).all())


def _stages(stage_list):
    arr = (cabi.MatmulStage * len(stage_list))(*stage_list)
    return arr


@pytest.mark.parametrize("w_dtype", [cabi.BFLOAT8_B, cabi.BFLOAT4_B])
@pytest.mark.parametrize("M,H,F", [(32, 512, 256), (32, 1024, 3584), (96, 1024, 384), (32, 4096, 14336)])
def test_gated_mlp_as_two_stages(ttb, orc, w_dtype, M, H, F):
    """down(silu(x w1) * (x w3)) as one launch: stage 0 the gated pair, stage 1 the down projection reading stage 0's
    output. Agrees with ttb_matmul_multi(MM_GATED) followed by ttb_matmul under a fixed reduction order."""
    import torch
    x = vectors.randn(81, (M, H), 1.0).bfloat16()
    a = ttb.tilize(x.cuda(), 1, M, H)
    (w1, r1), (w3, r3) = (_weight(ttb, orc, 82 + j, M, H, F, w_dtype) for j in range(2))
    w2, r2 = _weight(ttb, orc, 85, M, F, H, w_dtype)
    hidden = torch.zeros(M * F, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(M * H, dtype=torch.bfloat16, device="cuda")
    det = cabi.MM_DETERMINISTIC
    st = _stages([
        cabi.matmul_stage(a.data_ptr(), [w1.data_ptr(), w3.data_ptr()], [hidden.data_ptr(), None], H, [F, F], act=cabi.ACT_SILU,
                          flags=cabi.MM_GATED | det),
        cabi.matmul_stage(hidden.data_ptr(), [w2.data_ptr()], [out.data_ptr()], F, [H], flags=det, input_from=0),
    ])
    nbytes = ttb.matmul_sequence_workspace_bytes(w_dtype, 1, M, st, 2)
    assert nbytes >= 65536
    ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    results = []
    for rep in range(3):
        hidden.zero_()
        out.zero_()
        ttb.check(ttb.cdll.ttb_matmul_sequence(st, 2, cabi.BFLOAT16, w_dtype, 1, M, cabi.MM_WORKSPACE_ZEROED | (cabi.MM_WEIGHTS_RESIDENT if rep else 0),
                                               ws.data_ptr(), nbytes, None))
        ttb.check(ttb.check_status(None))
        results.append((hidden.clone(), out.clone()))
        assert int(ws[: 2 * 65536 + (16 << 20)].count_nonzero().item()) == 0
    for h, o in results[1:]:
        assert torch.equal(h, results[0][0]) and torch.equal(o, results[0][1])
    # the separate launches
    hidden2 = torch.zeros_like(hidden)
    arr_w = (ctypes.c_void_p * 2)(w1.data_ptr(), w3.data_ptr())
    arr_o = (ctypes.c_void_p * 2)(hidden2.data_ptr(), None)
    arr_n = (ctypes.c_int64 * 2)(F, F)
    gbytes = ttb.matmul_gated_workspace_bytes(w_dtype, 1, M, H, F)
    gws = torch.zeros(gbytes, dtype=torch.uint8, device="cuda")
    ttb.check(ttb.cdll.ttb_matmul_multi(a.data_ptr(), cabi.BFLOAT16, 2, arr_w, w_dtype, None, arr_o, cabi.BFLOAT16, 1, M, H, arr_n, cabi.ACT_SILU,
                                        cabi.MM_GATED | cabi.MM_WORKSPACE_ZEROED | det, gws.data_ptr(), gbytes, None, None, None))
    out2 = ttb.matmul(hidden2, w2, w_dtype, 1, M, F, H, flags=det)
    assert torch.equal(hidden2, results[0][0])
    assert same_to_the_last_digit(out2, results[0][1])
    # and the fp32 reference (the hidden tensor rounded to bf16 as the kernels store it)
    xf = x.float().cuda()
    h_ref = torch.nn.functional.silu(xf @ r1.cuda()) * (xf @ r3.cuda())
    check(ttb.untilize(results[0][0], 1, M, F).reshape(M, F), h_ref)
    check(ttb.untilize(results[0][1], 1, M, H).reshape(M, H), h_ref.bfloat16().float() @ r2.cuda())


@pytest.mark.parametrize("M", [32, 96])
def test_four_stages_chained_and_grouped(ttb, orc, M):
    """A chain of four stages (three weights on one activation, then one stage per link of a chain), row-major in and out at
    the ends: every output agrees with the result of the separate launches."""
    import torch
    w_dtype = cabi.BFLOAT8_B
    K0, Ns0, N1, N2, N3 = 1024, [512, 128, 128], 2048, 256, 1152
    x = vectors.randn(91, (M, K0), 1.0).bfloat16().cuda()
    ws0 = [_weight(ttb, orc, 92 + j, M, K0, n, w_dtype) for j, n in enumerate(Ns0)]
    w1, r1 = _weight(ttb, orc, 96, M, Ns0[0], N1, w_dtype)
    w2, r2 = _weight(ttb, orc, 97, M, N1, N2, w_dtype)
    w3, r3 = _weight(ttb, orc, 98, M, N2, N3, w_dtype)
    o0 = [torch.zeros(M * n, dtype=torch.bfloat16, device="cuda") for n in Ns0]
    o1 = torch.zeros(M * N1, dtype=torch.bfloat16, device="cuda")
    o2 = torch.zeros(M * N2, dtype=torch.bfloat16, device="cuda")
    o3 = torch.zeros(M * N3, dtype=torch.float32, device="cuda")
    det = cabi.MM_DETERMINISTIC
    st = _stages([
        cabi.matmul_stage(x.data_ptr(), [w.data_ptr() for w, _ in ws0], [o.data_ptr() for o in o0], K0, Ns0, act=cabi.ACT_GELU,
                          flags=det | cabi.MM_A_ROW_MAJOR),
        cabi.matmul_stage(o0[0].data_ptr(), [w1.data_ptr()], [o1.data_ptr()], Ns0[0], [N1], flags=det, input_from=0),
        cabi.matmul_stage(o1.data_ptr(), [w2.data_ptr()], [o2.data_ptr()], N1, [N2], act=cabi.ACT_RELU, flags=det | cabi.MM_OUT_ROW_MAJOR, input_from=1),
        cabi.matmul_stage(o2.data_ptr(), [w3.data_ptr()], [o3.data_ptr()], N2, [N3], out_dtype=cabi.FLOAT32,
                          flags=det | cabi.MM_A_ROW_MAJOR | cabi.MM_OUT_ROW_MAJOR, input_from=2),
    ])
    nbytes = ttb.matmul_sequence_workspace_bytes(w_dtype, 1, M, st, 4)
    ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    for rep in range(2):
        ttb.check(ttb.cdll.ttb_matmul_sequence(st, 4, cabi.BFLOAT16, w_dtype, 1, M, cabi.MM_WORKSPACE_ZEROED, ws.data_ptr(), nbytes, None))
        ttb.check(ttb.check_status(None))
        assert int(ws[:65536].count_nonzero().item()) == 0
    # separate launches
    s0 = [ttb.matmul(x.reshape(-1), w, w_dtype, 1, M, K0, n, act=cabi.ACT_GELU, flags=det | cabi.MM_A_ROW_MAJOR) for (w, _), n in zip(ws0, Ns0)]
    for a, b in zip(o0, s0):
        assert torch.equal(a, b)
    # (each later stage is compared on the sequence's own input to it, so that differences do not compound)
    assert same_to_the_last_digit(o1, ttb.matmul(o0[0], w1, w_dtype, 1, M, Ns0[0], N1, flags=det))
    assert same_to_the_last_digit(o2, ttb.matmul(o1, w2, w_dtype, 1, M, N1, N2, act=cabi.ACT_RELU, flags=det | cabi.MM_OUT_ROW_MAJOR))
    assert same_to_the_last_digit(o3, ttb.matmul(o2, w3, w_dtype, 1, M, N2, N3, flags=det | cabi.MM_A_ROW_MAJOR | cabi.MM_OUT_ROW_MAJOR, out_fp32=True))
    y0 = torch.nn.functional.gelu(x.float() @ ws0[0][1].cuda())
    check(ttb.untilize(o0[0], 1, M, Ns0[0]).reshape(M, Ns0[0]), y0)


def test_sequence_arguments_are_validated(ttb):
    import torch
    buf = torch.zeros(4 << 20, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    ok = cabi.matmul_stage(p, [p], [p], 64, [128])
    later = cabi.matmul_stage(p, [p], [p], 128, [128], input_from=1)            # names itself
    st = _stages([ok, later])
    assert ttb.cdll.ttb_matmul_sequence(st, 2, cabi.BFLOAT16, cabi.BFLOAT8_B, 1, 32, 0, p, 4 << 20, None) == -1
    assert b"input_from" in ttb.cdll.ttb_last_error()
    st = _stages([ok])
    assert ttb.cdll.ttb_matmul_sequence(st, 1, cabi.BFLOAT16, cabi.BFLOAT8_B, 1, 64, 0, p, 4 << 20, None) == -3     # 64 rows: two tile rows per block
    assert ttb.cdll.ttb_matmul_sequence(st, 1, cabi.BFLOAT16, cabi.BFLOAT8_B, 1, 32, 0, p, 1024, None) == -4        # workspace too small
    assert ttb.cdll.ttb_matmul_sequence(st, 5, cabi.BFLOAT16, cabi.BFLOAT8_B, 1, 32, 0, p, 4 << 20, None) == -1
    fp32_out = cabi.matmul_stage(p, [p], [p], 64, [128], out_dtype=cabi.FLOAT32)
    reads_fp32 = cabi.matmul_stage(p, [p], [p], 128, [128], input_from=0)
    st = _stages([fp32_out, reads_fp32])
    assert ttb.cdll.ttb_matmul_sequence(st, 2, cabi.BFLOAT16, cabi.BFLOAT8_B, 1, 32, 0, p, 4 << 20, None) == -1
    torch.cuda.synchronize()
    assert int(buf.count_nonzero().item()) == 0
