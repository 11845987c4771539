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
