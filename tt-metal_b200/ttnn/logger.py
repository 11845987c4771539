"""stderr logger of the ttnn package, level from the environment (the reference's tt::log_* with TT_METAL_LOGGER_LEVEL,
tt_metal/common/logger.hpp, and loguru on the Python side). Levels: TRACE, DEBUG, INFO, WARNING, ERROR, FATAL; default INFO."""
import os
import sys
import time

_LEVELS = {"TRACE": 0, "DEBUG": 1, "INFO": 2, "WARNING": 3, "ERROR": 4, "FATAL": 5}


def _level_from_env():
    name = os.environ.get("TT_METAL_LOGGER_LEVEL", os.environ.get("TTNN_LOGGER_LEVEL", "INFO")).upper()
    if name not in _LEVELS:
        raise RuntimeError(f"TT_METAL_LOGGER_LEVEL must be one of {', '.join(_LEVELS)}, got {name}")
    return _LEVELS[name]


class Logger:
    def __init__(self, stream=None):
        self.level = _level_from_env()
        self.stream = stream

    def log(self, level, message):
        if _LEVELS[level] >= self.level:
            out = self.stream or sys.stderr
            out.write(f"{time.strftime('%Y-%m-%d %H:%M:%S')} | {level:<7} | ttnn | {message}\n")
            out.flush()

    def trace(self, m): self.log("TRACE", m)
    def debug(self, m): self.log("DEBUG", m)
    def info(self, m): self.log("INFO", m)
    def warning(self, m): self.log("WARNING", m)
    def error(self, m): self.log("ERROR", m)


logger = Logger()
