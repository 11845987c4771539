"""Bounded device-side waits that run out: the kernel returns by itself, ttb_check_status reports TTB_E_TIMEOUT once with the
wait site, the status word is clear afterwards, and the next matmul on the stream is correct.

The failure is made without faulting anything: a gather point whose `expected` counter says one arrival and whose
`arrived` counter nothing ever increments, together with a wait limit of about a millisecond (ttb_set_wait_limit_cycles).
Nothing spins without a bound, nothing traps; the context stays usable."""
import ctypes

import pytest

import cabi
import vectors
from test_matmul_gpu import check, make_case

pytestmark = pytest.mark.gpu
TTB_E_TIMEOUT = -5
LIMIT_CYCLES = 2_000_000      # ~1 ms at the B200's clocks


@pytest.fixture
def short_waits(ttb):
    ttb.check(ttb.set_wait_limit_cycles(LIMIT_CYCLES))
    yield
    ttb.check(ttb.set_wait_limit_cycles(0))


def _dead_gather_point():
    """arrived = 0 at +0, expected = 1 at +128 bytes: a wait on it can never be satisfied."""
    import torch
    counters = torch.zeros(64, dtype=torch.int32, device="cuda")
    counters[32] = 1
    torch.cuda.synchronize()
    return counters, cabi.peer_wait(counters.data_ptr(), counters.data_ptr() + 128)


def test_stream_wait_gives_up_and_reports_once(ttb, short_waits):
    counters, wt = _dead_gather_point()
    ttb.check(ttb.cdll.ttb_peer_wait(ctypes.byref(wt), None))
    assert ttb.check_status(None) == TTB_E_TIMEOUT
    assert b"wait site 7" in ttb.cdll.ttb_last_error()
    assert ttb.check_status(None) == 0                      # reading the status clears it
    assert counters.cpu().tolist()[0] == 0


def test_negative_limit_is_refused(ttb):
    assert ttb.set_wait_limit_cycles(-1) == -1
    assert ttb.set_wait_limit_cycles(0) == 0


@pytest.mark.parametrize("w_dtype", [cabi.BFLOAT8_B, cabi.BFLOAT4_B])
@pytest.mark.parametrize("M,K,N", [(32, 4096, 512), (64, 4096, 256), (32, 256, 18176)])
def test_matmul_waiting_for_peers_gives_up_and_the_next_one_is_right(ttb, orc, short_waits, w_dtype, M, K, N):
    """A decode matmul whose activations "come from other GPUs" that never deliver: every role of every block leaves through
    the kernel's teardown, the status says so, and after clearing the workspace head (the header's rule after a timeout)
    the same workspace serves a correct matmul."""
    import torch
    x, w_dev, w_ref = make_case(ttb, orc, 91, M, K, N, w_dtype)
    a = ttb.tilize(x.cuda(), 1, M, K)
    counters, wt = _dead_gather_point()
    nbytes = ttb.matmul_peer_workspace_bytes(w_dtype, 1, M, K, N)
    assert (nbytes > 0) == (N < 18176)                     # K split over blocks (scratch in play), and one block per tile
    ws = torch.zeros(max(nbytes, 65536 + (16 << 20)), dtype=torch.uint8, device="cuda")
    out = torch.zeros(M * N, dtype=torch.bfloat16, device="cuda")
    ttb.check(ttb.cdll.ttb_matmul_peer(a.data_ptr(), cabi.BFLOAT16, w_dev.data_ptr(), w_dtype, None, out.data_ptr(), cabi.BFLOAT16,
                                       1, M, K, N, 0, cabi.MM_WORKSPACE_ZEROED, ws.data_ptr(), nbytes, None, ctypes.byref(wt), None))
    assert ttb.check_status(None) == TTB_E_TIMEOUT
    assert b"wait site" in ttb.cdll.ttb_last_error()
    assert ttb.check_status(None) == 0
    # the rule after a timeout: the workspace head is cleared before it is trusted again
    ws[: 65536 + (16 << 20)].zero_()
    out2 = torch.empty(M * N, dtype=torch.bfloat16, device="cuda")
    ttb.check(ttb.cdll.ttb_matmul_peer(a.data_ptr(), cabi.BFLOAT16, w_dev.data_ptr(), w_dtype, None, out2.data_ptr(), cabi.BFLOAT16,
                                       1, M, K, N, 0, cabi.MM_WORKSPACE_ZEROED, ws.data_ptr(), nbytes, None, None, None))
    assert ttb.check_status(None) == 0
    check(ttb.untilize(out2, 1, M, N).reshape(M, N), x.float() @ w_ref)
    assert int(ws[: 65536 + (16 << 20)].count_nonzero().item()) == 0


def test_host_layer_raises_on_a_timeout_and_clears_its_scratch(ttb, short_waits):
    """ttnn.synchronize_device / ttnn.to_torch read the status word: after a wait that ran out they raise (once), the device's
    matmul scratch is zero again, and the next ttnn.linear is right. (libttb is loaded once per process: the status word the
    C-ABI call below raises is the one the host layer reads.)"""
    import torch
    import ttnn
    device = ttnn.open_device(device_id=0)
    torch.manual_seed(3)
    x = torch.randn(1, 1, 32, 4096).bfloat16()
    w = torch.randn(4096, 512) * 0.03
    tx = ttnn.from_torch(x, layout=ttnn.TILE_LAYOUT, device=device)
    tw = ttnn.from_torch(w, dtype=ttnn.bfloat8_b, layout=ttnn.TILE_LAYOUT, device=device)
    want = ttnn.to_torch(ttnn.linear(tx, tw)).float()          # (split over K: uses the device's scratch)
    counters, wt = _dead_gather_point()
    ttb.check(ttb.cdll.ttb_peer_wait(ctypes.byref(wt), None))
    with pytest.raises(RuntimeError, match="ran out"):
        ttnn.synchronize_device(device)
    ttnn.synchronize_device(device)                              # reported once
    got = ttnn.to_torch(ttnn.linear(tx, tw)).float()
    # (sums over K may be added in another order from launch to launch: equal to the last bf16 digit, not to the bit)
    assert torch.allclose(got, want, rtol=2 ** -6, atol=1e-3 * float(want.abs().max()))
