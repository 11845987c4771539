"""The three environment flags of the ttnn package (ttnn/ttnn/__init__.py:13-33 of the reference); values must be the
strings "True" or "False"."""
import os


def get_bool_env_var(name, default):
    variable = os.environ.get(name, f"{default}")
    if variable == "True":
        return True
    if variable == "False":
        return False
    raise RuntimeError('The value has to be either "True" or "False"')


TTNN_ENABLE_MODEL_CACHE = get_bool_env_var("TTNN_ENABLE_MODEL_CACHE", "False")
TTNN_ENABLE_FAST_RUNTIME_MODE = get_bool_env_var("TTNN_ENABLE_FAST_RUNTIME_MODE", "False")
TTNN_ENABLE_LOGGING = get_bool_env_var("TTNN_ENABLE_LOGGING", "False")
