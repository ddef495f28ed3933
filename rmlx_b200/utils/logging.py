"""Structured logging: global level filter, entries with key/value fields, JSON or text output.
Mirrors crates/rmlx-core/src/logging.rs:9-170 (``LogLevel``, ``LogEntry``, ``log`` /
``log_with_fields``, ``set_level`` / ``set_format``)."""
from __future__ import annotations

import json
import sys
import threading
import time
from dataclasses import dataclass, field
from enum import IntEnum
from typing import Any, Callable, Dict, List, Optional


class LogLevel(IntEnum):
    TRACE = 0
    DEBUG = 1
    INFO = 2
    WARN = 3
    ERROR = 4
    OFF = 5


@dataclass
class LogEntry:
    level: LogLevel
    target: str
    message: str
    fields: Dict[str, Any] = field(default_factory=dict)
    ts: float = field(default_factory=time.time)

    def to_json(self) -> str:
        return json.dumps({"ts": round(self.ts, 6), "level": self.level.name, "target": self.target,
                           "msg": self.message, **self.fields}, default=str)

    def to_text(self) -> str:
        kv = " ".join(f"{k}={v}" for k, v in self.fields.items())
        return f"{time.strftime('%H:%M:%S', time.localtime(self.ts))} {self.level.name:5s} " \
               f"{self.target}: {self.message}" + (f" [{kv}]" if kv else "")


_lock = threading.Lock()
_level = LogLevel.INFO
_json = False
_sink: Callable[[str], None] = lambda s: print(s, file=sys.stderr)
_capture: Optional[List[LogEntry]] = None


def set_level(level: LogLevel) -> None:
    global _level
    _level = LogLevel(level)


def get_level() -> LogLevel:
    return _level


def set_format(json_format: bool) -> None:
    global _json
    _json = bool(json_format)


def set_sink(fn: Callable[[str], None]) -> None:
    global _sink
    _sink = fn


def capture(entries: Optional[List[LogEntry]]) -> None:
    """Route entries to a list (tests) instead of the sink; None restores the sink."""
    global _capture
    _capture = entries


def enabled(level: LogLevel) -> bool:
    return level >= _level and _level != LogLevel.OFF


def log_with_fields(level: LogLevel, target: str, message: str, **fields) -> None:
    if not enabled(level):
        return
    e = LogEntry(LogLevel(level), target, message, fields)
    with _lock:
        if _capture is not None:
            _capture.append(e)
        else:
            _sink(e.to_json() if _json else e.to_text())


def log(level: LogLevel, target: str, message: str) -> None:
    log_with_fields(level, target, message)


def info(target, msg, **f): log_with_fields(LogLevel.INFO, target, msg, **f)
def warn(target, msg, **f): log_with_fields(LogLevel.WARN, target, msg, **f)
def error(target, msg, **f): log_with_fields(LogLevel.ERROR, target, msg, **f)
def debug(target, msg, **f): log_with_fields(LogLevel.DEBUG, target, msg, **f)
