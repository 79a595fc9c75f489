"""Levelled, pid-prefixed print logger with the reference's five levels
(`tspipe/logger.py:26-59`): ``Log.d/v/i/w/e``; default threshold is WARN and can be
set with ``TSPIPE_LOG=debug|verbose|info|warn|error`` or :func:`Log.set_level`."""
from __future__ import annotations

import os
import sys
import time
from enum import IntEnum


class LogLevel(IntEnum):
    DEBUG = 0
    VERBOSE = 1
    INFO = 2
    WARN = 3
    ERROR = 4


_NAMES = {"debug": LogLevel.DEBUG, "verbose": LogLevel.VERBOSE, "info": LogLevel.INFO,
          "warn": LogLevel.WARN, "warning": LogLevel.WARN, "error": LogLevel.ERROR}


class Log:
    level: LogLevel = _NAMES.get(os.environ.get("TSPIPE_LOG", "warn").lower(), LogLevel.WARN)
    tag: str = ""

    @classmethod
    def set_level(cls, level) -> None:
        cls.level = _NAMES[level.lower()] if isinstance(level, str) else LogLevel(level)

    @classmethod
    def set_tag(cls, tag: str) -> None:
        cls.tag = tag

    @classmethod
    def _emit(cls, lvl: LogLevel, *args) -> None:
        if lvl < cls.level:
            return
        stamp = time.strftime("%H:%M:%S")
        print(f"[{stamp} {lvl.name[0]} pid={os.getpid()}{' ' + cls.tag if cls.tag else ''}]", *args,
              file=sys.stderr if lvl >= LogLevel.WARN else sys.stdout, flush=True)

    @classmethod
    def d(cls, *a): cls._emit(LogLevel.DEBUG, *a)

    @classmethod
    def v(cls, *a): cls._emit(LogLevel.VERBOSE, *a)

    @classmethod
    def i(cls, *a): cls._emit(LogLevel.INFO, *a)

    @classmethod
    def w(cls, *a): cls._emit(LogLevel.WARN, *a)

    @classmethod
    def e(cls, *a): cls._emit(LogLevel.ERROR, *a)
