"""Leveled logging to stderr in the reference's line format:

    HH:MM:SS.mmm LEVEL file:line] message

(reference src/log.c:42-76, include/sgl/log.h:7-28: levels DEBUG < INFO < WARN < ERROR, a lock
around each line, the level set once for the process).  The level comes from `set_level` (the
command line's --verbose sets DEBUG) and defaults to WARN, so a library user sees nothing unless
something is wrong; the build's progress lines are INFO lines that are always shown while nvcc
runs (a first call that compiles must not look hung).
"""
import os
import sys
import threading
import time

DEBUG, INFO, WARN, ERROR = 10, 20, 30, 40
_NAMES = {DEBUG: "DEBUG", INFO: "INFO", WARN: "WARN", ERROR: "ERROR"}
_level = WARN
_lock = threading.Lock()
_sink = None            # a callable(line) set by tests; default: stderr


def set_level(level):
    """DEBUG, INFO, WARN or ERROR (or their names)."""
    global _level
    if isinstance(level, str):
        level = {v: k for k, v in _NAMES.items()}[level.upper()]
    _level = int(level)


def get_level():
    return _level


def set_sink(fn):
    global _sink
    _sink = fn


def log(level, msg, always=False, depth=1):
    if level < _level and not always:
        return
    f = sys._getframe(depth)
    t = time.time()
    lt = time.localtime(t)
    line = (f"{lt.tm_hour:02d}:{lt.tm_min:02d}:{lt.tm_sec:02d}.{int((t % 1) * 1000):03d} "
            f"{_NAMES.get(level, str(level))} {os.path.basename(f.f_code.co_filename)}:{f.f_lineno}] {msg}")
    with _lock:
        if _sink is not None:
            _sink(line)
        else:
            print(line, file=sys.stderr, flush=True)


def debug(msg):
    log(DEBUG, msg, depth=2)


def info(msg, always=False):
    log(INFO, msg, always=always, depth=2)


def warn(msg):
    log(WARN, msg, depth=2)


def error(msg):
    log(ERROR, msg, depth=2)
