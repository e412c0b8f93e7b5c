"""Log lines with a level and a module tag, written to standard error.

    from ..utils.log import log
    log.info("build", "compiling gemm_tcgen05.cu for sm_100a ...")
        -> 14:03:27 [INFO] [build] compiling gemm_tcgen05.cu for sm_100a ...

The line format is the reference's (bug/logger.hpp:27-38, 50-57: time, level, module,
message); the reference writes to standard output, beside the generated text, which this
library keeps clean by logging to standard error.  The threshold comes from the
environment variable ORACLE_LOG (debug, info, warn, error, off; default info) or
`log.set_level(...)`.
"""
from __future__ import annotations

import os
import sys
import threading
import time

LEVELS = {"debug": 10, "info": 20, "warn": 30, "error": 40, "off": 100}
_NAMES = {10: "DEBUG", 20: "INFO", 30: "WARN", 40: "ERR"}


class Logger:
    def __init__(self, stream=None):
        self._stream = stream
        self._lock = threading.Lock()
        self._level = LEVELS.get(os.environ.get("ORACLE_LOG", "info").lower(), 20)

    def set_level(self, name: str) -> None:
        try:
            self._level = LEVELS[name.lower()]
        except KeyError:
            raise ValueError(f"log level must be one of {', '.join(LEVELS)}; got {name!r}") from None

    def set_stream(self, stream) -> None:
        self._stream = stream

    def enabled(self, level: int) -> bool:
        return level >= self._level

    def write(self, level: int, module: str, message: str) -> None:
        if level < self._level:
            return
        line = f"{time.strftime('%H:%M:%S')} [{_NAMES[level]}] [{module}] {message}\n"
        with self._lock:
            stream = self._stream or sys.stderr
            stream.write(line)
            stream.flush()

    def debug(self, module: str, message: str) -> None:
        self.write(10, module, message)

    def info(self, module: str, message: str) -> None:
        self.write(20, module, message)

    def warn(self, module: str, message: str) -> None:
        self.write(30, module, message)

    def error(self, module: str, message: str) -> None:
        self.write(40, module, message)


log = Logger()
