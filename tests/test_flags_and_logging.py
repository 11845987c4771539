"""The ttnn package's environment flags, logger and per-operation record (ttnn/ttnn/__init__.py:13-33 and
ttnn/ttnn/decorators.py:312-366 of the reference), without a GPU."""
import io
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "tt-metal_b200")


def _run(code, **env):
    e = dict(os.environ)
    e.update(env)
    return subprocess.run([sys.executable, "-c", f"import sys; sys.path.insert(0, {PKG!r}); " + code], capture_output=True, text=True, env=e)


def test_flags_take_only_true_or_false():
    r = _run("import ttnn; print(ttnn.TTNN_ENABLE_LOGGING, ttnn.TTNN_ENABLE_FAST_RUNTIME_MODE, ttnn.TTNN_ENABLE_MODEL_CACHE)")
    assert r.returncode == 0 and r.stdout.split() == ["False", "False", "False"], r.stderr
    r = _run("import ttnn; print(ttnn.TTNN_ENABLE_LOGGING)", TTNN_ENABLE_LOGGING="True")
    assert r.returncode == 0 and r.stdout.strip() == "True" and "enabled logging" in r.stderr
    r = _run("import ttnn", TTNN_ENABLE_LOGGING="yes")
    assert r.returncode != 0 and 'either "True" or "False"' in r.stderr


def test_fast_runtime_mode_leaves_operations_unwrapped():
    r = _run("import ttnn; print(ttnn.matmul is ttnn.decorators.REGISTERED_OPERATIONS['ttnn.matmul'])", TTNN_ENABLE_FAST_RUNTIME_MODE="True")
    assert r.returncode == 0 and r.stdout.strip() == "True", r.stderr
    r = _run("import ttnn; print(ttnn.matmul is ttnn.decorators.REGISTERED_OPERATIONS['ttnn.matmul'])")
    assert r.returncode == 0 and r.stdout.strip() == "False", r.stderr


def test_logger_level_comes_from_the_environment():
    r = _run("from ttnn.logger import logger; logger.debug('quiet'); logger.warning('loud')", TT_METAL_LOGGER_LEVEL="WARNING")
    assert r.returncode == 0 and "loud" in r.stderr and "quiet" not in r.stderr
    r = _run("from ttnn.logger import logger; logger.debug('now visible')", TT_METAL_LOGGER_LEVEL="DEBUG")
    assert "now visible" in r.stderr
    r = _run("import ttnn.logger", TT_METAL_LOGGER_LEVEL="CHATTY")
    assert r.returncode != 0


def test_operation_record_of_a_matmul():
    sys.path.insert(0, PKG)
    import ttnn
    from ttnn import decorators

    class FakeShape(list):
        padded = property(lambda self: list(self))

    class FakeTensor:
        def __init__(self, shape, dtype, nbytes):
            self.shape, self.dtype, self.layout, self._n = FakeShape(shape), dtype, ttnn.TILE_LAYOUT, nbytes

        def buffer_bytes(self): return self._n
        def is_allocated(self): return True

    a = FakeTensor([1, 1, 32, 4544], ttnn.bfloat16, 32 * 4544 * 2)
    w = FakeTensor([4544, 18176], ttnn.bfloat8_b, 87753728)
    y = FakeTensor([1, 1, 32, 18176], ttnn.bfloat16, 32 * 18176 * 2)
    rec = decorators.operation_record("ttnn.linear", [a, w], [y], 25e-6)
    assert rec["bytes"] == 89207808 and rec["flops"] == 2 * 32 * 4544 * 18176
    assert abs(rec["GB/s"] - 89207808 / 25e-6 / 1e9) < 1e-6 and rec["inputs"][1]["dtype"] == "BFLOAT8_B"
    json.dumps(rec)


def test_hooks_run_around_top_level_operations():
    sys.path.insert(0, PKG)
    import ttnn
    seen = []
    pre = ttnn.register_pre_operation_hook(lambda name, args, kwargs: seen.append(("pre", name)))
    post = ttnn.register_post_operation_hook(lambda name, args, kwargs, out: seen.append(("post", name)))
    try:
        with pytest.raises(RuntimeError):
            ttnn.from_torch("not a tensor")          # validation error inside the wrapped function
        assert seen == [("pre", "ttnn.from_torch")]
    finally:
        ttnn.decorators.PRE_OPERATION_HOOKS.remove(pre)
        ttnn.decorators.POST_OPERATION_HOOKS.remove(post)
