"""The gather epilogue of ttb_matmul_peer, exercised on ONE GPU: the "ranks" are launches on one stream whose peer pointers
are other buffers of the same device, so every address computation, counter and wait runs exactly as between GPUs
while no kernel ever waits for a kernel that has not finished (all waits are already satisfied when they start)."""
import ctypes

import numpy as np
import pytest

import cabi
import oracle
import vectors
from test_matmul_gpu import check, make_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("G,M,K,N", [(2, 32, 512, 256), (2, 32, 4096, 256), (4, 64, 1024, 128), (2, 128, 2048, 256), (8, 32, 8192, 128)])
def test_gather_epilogue_fills_every_rank(ttb, orc, G, M, K, N):
    import torch
    x = vectors.randn(5, (M, K), 1.0).bfloat16()
    a = ttb.tilize(x.cuda(), 1, M, K)
    w_dev, w_ref = [], []
    for r in range(G):
        _, wd, wr = make_case(ttb, orc, 100 + r, M, K, N, cabi.BFLOAT8_B)
        w_dev.append(wd)
        w_ref.append(wr)
    y_ref = torch.cat([x.float() @ wr for wr in w_ref], dim=1)                      # [M, G*N]
    outs = [torch.zeros(M * G * N, dtype=torch.bfloat16, device="cuda") for _ in range(G)]
    counters = torch.zeros(G, 64, dtype=torch.int32, device="cuda")                  # [rank]: arrived at [0], expected at [32]
    nbytes = ttb.matmul_peer_workspace_bytes(cabi.BFLOAT8_B, 1, M, K, N)
    ws = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(G)]
    arrived = [counters[r, 0:].data_ptr() for r in range(G)]
    uses = [counters[r, 32:].data_ptr() for r in range(G)]
    K2, N2 = G * N, 128
    _, w2_dev, w2_ref = make_case(ttb, orc, 300, M, K2, N2, cabi.BFLOAT8_B)
    for use in (1, 2, 3):
        for o in outs:
            o.zero_()
        for r in range(G):
            g = cabi.peer_gather(r, [o.data_ptr() for o in outs], arrived, uses[r])
            ttb.check(ttb.cdll.ttb_matmul_peer(a.data_ptr(), cabi.BFLOAT16, w_dev[r].data_ptr(), cabi.BFLOAT8_B, None, None, cabi.BFLOAT16,
                                               1, M, K, N, 0, cabi.MM_WORKSPACE_ZEROED | cabi.MM_WEIGHTS_RESIDENT, ws[r].data_ptr(), nbytes,
                                               ctypes.byref(g), None, None))
        # a consumer on "rank" 0 that waits for the gather point, then a plain stream wait on rank 1
        wt = cabi.peer_wait(arrived[0], uses[0])
        y2 = torch.empty(M * N2, dtype=torch.bfloat16, device="cuda")
        nb2 = ttb.matmul_peer_workspace_bytes(cabi.BFLOAT8_B, 1, M, K2, N2)
        ws2 = torch.zeros(nb2, dtype=torch.uint8, device="cuda")
        ttb.check(ttb.cdll.ttb_matmul_peer(outs[0].data_ptr(), cabi.BFLOAT16, w2_dev.data_ptr(), cabi.BFLOAT8_B, None, y2.data_ptr(),
                                           cabi.BFLOAT16, 1, M, K2, N2, 0, cabi.MM_WORKSPACE_ZEROED, ws2.data_ptr(), nb2, None,
                                           ctypes.byref(wt), None))
        wt1 = cabi.peer_wait(arrived[1], uses[1])
        ttb.check(ttb.cdll.ttb_peer_wait(ctypes.byref(wt1), None))
        ttb.check(ttb.check_status(None))
        c = counters.cpu()
        tiles = (N // 128) * (M // (64 if M % 64 == 0 else 32))      # blocks of one or two tile rows
        assert c[:, 0].tolist() == [use * G * tiles] * G and c[:, 32].tolist() == [use * G * tiles] * G
        for r in range(G):
            y = ttb.untilize(outs[r], 1, M, G * N).reshape(M, G * N)
            check(y, y_ref)
            assert torch.equal(outs[r], outs[0])
        y_gathered = ttb.untilize(outs[0], 1, M, G * N).reshape(M, G * N).float().cpu()
        check(ttb.untilize(y2, 1, M, N2).reshape(M, N2), y_gathered @ w2_ref)
        for r in range(G):
            assert int(ws[r][:65536].count_nonzero().item()) == 0           # arrival counters of the split-K tiles are back to zero


def test_peer_arguments_are_validated(ttb):
    """Refusals happen before any launch. The buffers are nevertheless large enough for every shape used here, so that a
    call that was not refused would still stay inside them."""
    import torch
    buf = torch.zeros(4 << 20, dtype=torch.uint8, device="cuda")
    M, K, N = 32, 4096, 128
    args = (buf.data_ptr(), cabi.BFLOAT16, buf.data_ptr(), cabi.BFLOAT8_B, None, None)
    g1 = cabi.peer_gather(0, [buf.data_ptr()], [buf.data_ptr()], buf.data_ptr())      # one rank only
    rc = ttb.cdll.ttb_matmul_peer(*args, cabi.BFLOAT16, 1, M, K, N, 0, 0, buf.data_ptr(), 4 << 20, ctypes.byref(g1), None, None)
    assert rc == -1 and b"ranks" in ttb.cdll.ttb_last_error()
    g = cabi.peer_gather(0, [buf.data_ptr(), buf.data_ptr()], [buf.data_ptr(), buf.data_ptr()], buf.data_ptr())
    rc = ttb.cdll.ttb_matmul_peer(*args, cabi.FLOAT32, 1, M, K, N, 0, 0, buf.data_ptr(), 4 << 20, ctypes.byref(g), None, None)
    assert rc == -3 and b"bfloat16" in ttb.cdll.ttb_last_error()
    assert ttb.matmul_peer_workspace_bytes(cabi.BFLOAT8_B, 1, M, K, N) > 16              # this shape splits K
    rc = ttb.cdll.ttb_matmul_peer(*args, cabi.BFLOAT16, 1, M, K, N, 0, 0, buf.data_ptr(), 16, ctypes.byref(g), None, None)
    assert rc == -4                                                                       # workspace too small
    rc = ttb.cdll.ttb_matmul_peer(*args, cabi.BFLOAT16, 1, 512, 64, 128, 0, 0, buf.data_ptr(), 4 << 20, ctypes.byref(g), None, None)
    assert rc == -3                                                                       # not a decode shape
    torch.cuda.synchronize()
    assert int(buf.count_nonzero().item()) == 0                                          # nothing ran
