"""Logging for hivemind_b200: one coloured stream handler, configured by environment variables.

Environment (same names as the reference, hivemind/utils/logging.py:20-31):
``HIVEMIND_LOGLEVEL`` (default INFO), ``HIVEMIND_COLORS`` (true/false; default: only on a tty),
``HIVEMIND_ALWAYS_LOG_CALLER`` (print file:line for every level, not only warnings and errors).
``use_hivemind_log_handler`` chooses where the handler is attached (reference :153-189).
"""
from __future__ import annotations

import logging
import os
import sys
import threading
from enum import Enum
from typing import Optional, Union

_PACKAGE_ROOT = "hivemind_b200"
_lock = threading.RLock()
_handler: Optional[logging.Handler] = None
_mode = None


class HandlerMode(Enum):
    NOWHERE = 0
    IN_HIVEMIND = 1
    IN_ROOT_LOGGER = 2


def _env_flag(name: str, default: Optional[bool]) -> Optional[bool]:
    raw = os.getenv(name)
    if raw is None:
        return default
    return raw.strip().lower() in ("1", "true", "yes", "on")


class TextStyle:
    """ANSI escapes; every attribute is an empty string when colours are off."""

    _codes = dict(RESET="\033[0m", BOLD="\033[1m", RED="\033[31m", BLUE="\033[34m", PURPLE="\033[35m",
                  ORANGE="\033[38;5;208m")
    enabled = False

    @classmethod
    def get(cls, name: str) -> str:
        return cls._codes[name] if cls.enabled else ""


class CustomFormatter(logging.Formatter):
    _level_colors = {logging.DEBUG: "PURPLE", logging.INFO: "BLUE", logging.WARNING: "ORANGE", logging.ERROR: "RED",
                     logging.CRITICAL: "RED"}

    def __init__(self, always_caller: bool):
        super().__init__(fmt="%(asctime)s.%(msecs)03d [%(levelname)s]%(caller)s %(message)s", datefmt="%b %d %H:%M:%S")
        self.always_caller = always_caller

    def format(self, record: logging.LogRecord) -> str:
        if hasattr(record, "origin_created"):  # records forwarded from the transport daemon keep their own time
            record.created = record.origin_created
            record.msecs = (record.created - int(record.created)) * 1000
        caller = getattr(record, "caller", None)
        if caller is None:
            if self.always_caller or record.levelno >= logging.WARNING:
                caller = f" [{record.name}.{record.funcName}:{record.lineno}]"
            else:
                caller = ""
        record.caller = caller
        color = TextStyle.get(self._level_colors.get(record.levelno, "RESET"))
        record.levelname = f"{TextStyle.get('BOLD')}{color}{record.levelname}{TextStyle.get('RESET')}"
        return super().format(record)


def _init() -> None:
    global _handler, _mode
    with _lock:
        if _handler is not None:
            return
        colors = _env_flag("HIVEMIND_COLORS", None)
        TextStyle.enabled = colors if colors is not None else (hasattr(sys.stderr, "isatty") and sys.stderr.isatty())
        _handler = logging.StreamHandler()
        _handler.setFormatter(CustomFormatter(bool(_env_flag("HIVEMIND_ALWAYS_LOG_CALLER", False))))
        _attach(HandlerMode.IN_HIVEMIND)


def _attach(mode: HandlerMode) -> None:
    global _mode
    pkg, root = logging.getLogger(_PACKAGE_ROOT), logging.getLogger()
    for lg in (pkg, root):
        if _handler in lg.handlers:
            lg.removeHandler(_handler)
    pkg.propagate = True
    level = os.getenv("HIVEMIND_LOGLEVEL", "INFO").upper()
    if mode == HandlerMode.IN_HIVEMIND:
        pkg.addHandler(_handler)
        pkg.setLevel(level)
        pkg.propagate = False
    elif mode == HandlerMode.IN_ROOT_LOGGER:
        root.addHandler(_handler)
        root.setLevel(level)
    _mode = mode


def get_logger(name: Optional[str] = None) -> logging.Logger:
    """Logger for module ``name`` (pass ``__name__``); names outside the package are nested under it."""
    _init()
    if name is None or name == "__main__":
        name = _PACKAGE_ROOT
    elif not name.startswith(_PACKAGE_ROOT):
        name = f"{_PACKAGE_ROOT}.{name}"
    return logging.getLogger(name)


def use_hivemind_log_handler(where: Union[HandlerMode, str]) -> None:
    """Attach the package handler ``"in_hivemind"`` (default), ``"in_root_logger"`` or ``"nowhere"``."""
    _init()
    if isinstance(where, str):
        where = HandlerMode[where.upper()]
    with _lock:
        _attach(where)


_DAEMON_LEVELS = {"DEBUG": logging.DEBUG, "INFO": logging.INFO, "WARN": logging.WARNING, "WARNING": logging.WARNING,
                  "ERROR": logging.ERROR, "FATAL": logging.CRITICAL, "PANIC": logging.CRITICAL}


def daemon_level_to_python(level: str) -> int:
    """Map a log level name printed by the transport daemon to a ``logging`` level."""
    return _DAEMON_LEVELS.get(level.upper(), logging.INFO)


def python_level_to_daemon(level: str) -> str:
    level = level.upper()
    return {"WARNING": "WARN", "CRITICAL": "FATAL"}.get(level, level)


TRUE_CONSTANTS = ("1", "true", "yes", "on")  # accepted spellings of a set boolean environment variable

_GOLOG_TO_PYTHON = {"DPANIC": logging.CRITICAL, "PANIC": logging.CRITICAL, "FATAL": logging.CRITICAL,
                    "WARN": logging.WARNING}


def golog_level_to_python(level: str) -> int:
    """Map a level name of the Go logging convention (used by libp2p daemons) to a ``logging`` level
    (reference: hivemind/utils/logging.py:192-201)."""
    level = level.upper()
    if level in _GOLOG_TO_PYTHON:
        return _GOLOG_TO_PYTHON[level]
    value = logging.getLevelName(level)
    if not isinstance(value, int):
        raise ValueError(f"unknown log level: {level}")
    return value


def python_level_to_golog(level: Union[str, int]) -> str:
    """The inverse mapping (reference: hivemind/utils/logging.py:204-212); ``level`` is a name or a number."""
    if isinstance(level, int):
        level = logging.getLevelName(level)
    if not isinstance(level, str):
        raise ValueError(f"unknown log level: {level}")
    level = level.upper()
    return {"WARNING": "WARN", "CRITICAL": "FATAL"}.get(level, level)


def in_ipython() -> bool:
    """True inside IPython / Jupyter, where the coloured handler should keep to the notebook's own stream."""
    try:
        get_ipython  # noqa: F821  (defined by IPython in its namespaces)
        return True
    except NameError:
        return False
