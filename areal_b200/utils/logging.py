"""Per-component loggers with coloured console output and optional file logging
(counterpart of areal/utils/logging.py:159-407)."""

from __future__ import annotations

import logging
import os
import sys

_COLORS = {"DEBUG": "\033[36m", "INFO": "\033[32m", "WARNING": "\033[33m", "ERROR": "\033[31m",
           "CRITICAL": "\033[41m"}
_RESET = "\033[0m"
_FILE_HANDLER: logging.Handler | None = None
_CONFIGURED: set[str] = set()


class _ColorFormatter(logging.Formatter):
    def __init__(self, use_color: bool):
        super().__init__("%(asctime)s.%(msecs)03d %(name)s %(levelname)s: %(message)s", "%Y%m%d-%H:%M:%S")
        self.use_color = use_color

    def format(self, record):
        msg = super().format(record)
        if self.use_color and record.levelname in _COLORS:
            return f"{_COLORS[record.levelname]}{msg}{_RESET}"
        return msg


def getLogger(name: str | None = None, level: str | None = None) -> logging.Logger:
    name = name or "areal_b200"
    logger = logging.getLogger(name)
    if name not in _CONFIGURED:
        h = logging.StreamHandler(sys.stdout)
        h.setFormatter(_ColorFormatter(sys.stdout.isatty()))
        logger.addHandler(h)
        if _FILE_HANDLER is not None:
            logger.addHandler(_FILE_HANDLER)
        logger.propagate = False
        logger.setLevel(os.environ.get("AREAL_LOG_LEVEL", "INFO").upper())
        _CONFIGURED.add(name)
    if level:
        logger.setLevel(level.upper())
    return logger


def setup_file_logging(log_dir: str, filename: str = "main.log") -> str:
    """Mirrors every logger created through :func:`getLogger` into ``log_dir/filename``."""
    global _FILE_HANDLER
    os.makedirs(log_dir, exist_ok=True)
    path = os.path.join(log_dir, filename)
    _FILE_HANDLER = logging.FileHandler(path)
    _FILE_HANDLER.setFormatter(_ColorFormatter(False))
    for name in _CONFIGURED:
        logging.getLogger(name).addHandler(_FILE_HANDLER)
    return path


def suppress_http_loggers(level: int = logging.WARNING) -> None:
    for n in ("httpx", "httpcore", "aiohttp.access", "uvicorn.access", "urllib3", "werkzeug"):
        logging.getLogger(n).setLevel(level)
