"""The C-ABI library loads and exports every function include/ttb.h declares (no GPU needed)."""
import cabi


def test_library_exports_every_declared_symbol():
    lib = cabi.load()
    names = cabi.declared_symbols()
    assert len(names) >= 20
    missing = [n for n in names if not hasattr(lib.cdll, n)]
    assert not missing, missing
    undeclared = [n for n in cabi._SIGS if n not in names]
    assert not undeclared, undeclared


def test_host_only_entry_points():
    lib = cabi.load()
    assert lib.version() >= 100
    assert lib.buffer_bytes(cabi.BFLOAT8_B, 1, 4096, 4096) == 17825792
    assert lib.buffer_bytes(cabi.BFLOAT4_B, 1, 64, 64) == 4 * 576
    assert lib.buffer_bytes(cabi.BFLOAT16, 2, 32, 64) == 2 * 32 * 64 * 2
    # argument validation happens before any CUDA call
    rc = lib.cdll.ttb_pack_bfp(None, cabi.FLOAT32, None, cabi.BFLOAT8_B, 1, 32, 32, 1, 0, None)
    assert rc == -1 and b"null" in lib.cdll.ttb_last_error()
    rc = lib.cdll.ttb_matmul(1 << 12, cabi.BFLOAT16, 1 << 12, cabi.BFLOAT8_B, None, 1 << 12, cabi.BFLOAT16, 1, 32, 48, 64, 0, 0,
                             None, 0, None)
    assert rc == -1 and b"multiples of 32" in lib.cdll.ttb_last_error()
    # split-K shapes report their scratch need; single-block-per-tile shapes need none
    assert lib.matmul_workspace_bytes(cabi.BFLOAT8_B, 1, 32, 4096, 4096, 0) > 0
    assert lib.matmul_workspace_bytes(cabi.BFLOAT8_B, 1, 32, 4096, 4096, cabi.MM_FORCE_GENERIC) == 0


def test_peer_structs_match_the_header(tmp_path):
    """The ctypes mirrors of ttb_peer_gather / ttb_peer_wait_t (tests/cabi.py and ttnn/peer.py) have the layout a C compiler
    gives the header's structs."""
    import ctypes
    import os
    import subprocess
    import sys
    src = tmp_path / "sizes.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "ttb.h"\n'
                   'int main(void) { printf("%zu %zu %zu %zu %zu %zu %d %d\\n", sizeof(ttb_peer_gather), offsetof(ttb_peer_gather, out), '
                   'offsetof(ttb_peer_gather, arrived), offsetof(ttb_peer_gather, expected), sizeof(ttb_peer_wait_t), '
                   'offsetof(ttb_peer_wait_t, expected), TTB_MAX_RANKS, TTB_MAX_GROUP); return 0; }\n')
    exe = tmp_path / "sizes"
    inc = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")
    subprocess.run(["gcc", "-I", inc, str(src), "-o", str(exe)], check=True)
    got = [int(v) for v in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    sys.path.insert(0, os.path.join(os.path.dirname(inc), "tt-metal_b200"))
    from ttnn import peer
    for G, W, max_ranks in ((cabi.PeerGather, cabi.PeerWait, cabi.MAX_RANKS), (peer.PeerGather, peer.PeerWait, peer.MAX_RANKS)):
        assert [ctypes.sizeof(G), G.out.offset, G.arrived.offset, G.expected.offset, ctypes.sizeof(W), W.expected.offset, max_ranks] == got[:7]
    assert got[7] == 4


def test_gather_ring_layout():
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tt-metal_b200"))
    from ttnn import peer
    counters, slot, arena = peer.ring_layout(4, 32 * 8192 * 2)
    assert counters % 4096 == 0 and counters >= 4 * 256 and slot == 524288 and arena == counters + 4 * slot
    assert peer.ring_layout(8, 1000)[1] == 4096
    import pytest
    with pytest.raises(RuntimeError):
        peer.ring_layout(1, 4096)          # consecutive gathers must not share a buffer
