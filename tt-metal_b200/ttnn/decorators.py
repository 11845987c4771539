"""Per-operation wrapper of the public ttnn functions (mirrors ttnn/ttnn/decorators.py:312-366 of the reference): with
TTNN_ENABLE_LOGGING=True every top-level operation is timed with the device synchronised on both sides and one JSON line per
operation goes to the log - name, operand shapes / dtypes / layouts, bytes of the operands and result as stored, wall time,
and for matmuls GB/s of operand bytes and TFLOP/s; NVTX ranges mark the same calls for timeline tools. Pre- and
post-operation hooks run for top-level operations. TTNN_ENABLE_FAST_RUNTIME_MODE=True leaves the functions unwrapped."""
import functools
import json
import time

from . import _flags
from .logger import logger

OPERATION_CALL_STACK = []
PRE_OPERATION_HOOKS = []
POST_OPERATION_HOOKS = []
REGISTERED_OPERATIONS = {}


def register_pre_operation_hook(hook):
    PRE_OPERATION_HOOKS.append(hook)
    return hook


def register_post_operation_hook(hook):
    POST_OPERATION_HOOKS.append(hook)
    return hook


def _tensors_in(obj, out):
    local = getattr(obj, "local", None)
    if local is not None and hasattr(local, "buffer_bytes"):
        out.append(local)
    elif hasattr(obj, "buffer_bytes") and hasattr(obj, "shape"):
        out.append(obj)
    elif isinstance(obj, (list, tuple)):
        for o in obj:
            _tensors_in(o, out)
    elif isinstance(obj, dict):
        for o in obj.values():
            _tensors_in(o, out)
    return out


def describe(t):
    try:
        return {"shape": list(t.shape), "dtype": str(t.dtype).split(".")[-1], "layout": str(t.layout).split(".")[-1],
                "bytes": int(t.buffer_bytes()) if t.is_allocated() else 0}
    except Exception:       # torch tensors and the like
        return {"shape": list(getattr(t, "shape", [])), "dtype": str(getattr(t, "dtype", "?"))}


def _synchronize(tensors):
    seen = set()
    for t in tensors:
        dev = t.device() if hasattr(t, "device") and callable(t.device) else None
        if dev is not None and id(dev) not in seen:
            seen.add(id(dev))
            dev.synchronize()


def operation_record(name, inputs, outputs, seconds):
    """The JSON-serialisable record of one finished operation."""
    rec = {"op": name, "inputs": [describe(t) for t in inputs], "outputs": [describe(t) for t in outputs], "ms": seconds * 1e3}
    moved = sum(d.get("bytes", 0) for d in rec["inputs"] + rec["outputs"])
    rec["bytes"] = moved
    if seconds > 0:
        rec["GB/s"] = moved / seconds / 1e9
    if name in ("ttnn.matmul", "ttnn.linear") and len(inputs) >= 2:
        a, b = list(inputs[0].shape.padded), list(inputs[1].shape.padded)
        rows = 1
        for d in a[:-1]:
            rows *= d
        flops = 2 * rows * a[-1] * b[-1]
        rec["flops"] = flops
        if seconds > 0:
            rec["TFLOP/s"] = flops / seconds / 1e12
    return rec


def register_operation(name):
    """Decorator for a public ttnn function."""
    def wrap(function):
        REGISTERED_OPERATIONS[name] = function
        if _flags.TTNN_ENABLE_FAST_RUNTIME_MODE:
            return function

        @functools.wraps(function)
        def call(*args, **kwargs):
            OPERATION_CALL_STACK.append(name)
            top = len(OPERATION_CALL_STACK) == 1
            try:
                if top:
                    for hook in PRE_OPERATION_HOOKS:
                        if hook(name, args, kwargs) is not None:
                            raise RuntimeError(f"Pre-operation hook {hook} must return None")
                if not (top and _flags.TTNN_ENABLE_LOGGING):
                    output = function(*args, **kwargs)
                else:
                    from . import _ttnn
                    inputs = _tensors_in((args, kwargs), [])
                    _synchronize(inputs)
                    _ttnn.nvtx_push(name)
                    start = time.perf_counter()
                    try:
                        output = function(*args, **kwargs)
                        outputs = _tensors_in(output, [])
                        _synchronize(inputs + outputs)
                    finally:
                        _ttnn.nvtx_pop()
                    logger.info(json.dumps(operation_record(name, inputs, outputs, time.perf_counter() - start)))
                if top:
                    for hook in POST_OPERATION_HOOKS:
                        if hook(name, args, kwargs, output) is not None:
                            raise RuntimeError(f"Post-operation hook {hook} must return None")
                return output
            finally:
                OPERATION_CALL_STACK.pop()
        return call
    return wrap
