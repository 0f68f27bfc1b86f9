"""Structured logger: ``[time] [LEVEL] [name] message``, colours on a TTY, optional file sink
(same format as the reference, src/utils/logger.py:17-100)."""
from __future__ import annotations

import logging
import sys
from typing import Optional

_COLORS = {"DEBUG": "\033[36m", "INFO": "\033[32m", "WARNING": "\033[33m", "ERROR": "\033[31m", "CRITICAL": "\033[35m"}
_RESET = "\033[0m"
_ROOT = "b200fw"


class _Formatter(logging.Formatter):
    def __init__(self, color: bool):
        super().__init__("[%(asctime)s] [%(levelname)s] [%(name)s] %(message)s", "%Y-%m-%d %H:%M:%S")
        self.color = color

    def format(self, record):
        s = super().format(record)
        if self.color and record.levelname in _COLORS:
            s = s.replace(f"[{record.levelname}]", f"[{_COLORS[record.levelname]}{record.levelname}{_RESET}]", 1)
        return s


def setup_logger(name: str = _ROOT, level: str = "INFO", log_file: Optional[str] = None,
                 rank: Optional[int] = None, use_color: Optional[bool] = None) -> logging.Logger:
    """``use_color`` (the reference's fourth argument, src/utils/logger.py:44-100; a bool given in its place is taken
    as that): force colours on or off; by default the stream handler colours only when stderr is a terminal."""
    if isinstance(rank, bool):
        rank, use_color = None, rank
    logger = logging.getLogger(name)
    logger.setLevel(getattr(logging, level.upper(), logging.INFO))
    logger.propagate = False
    for h in list(logger.handlers):
        logger.removeHandler(h)
    sh = logging.StreamHandler(sys.stderr)
    sh.setFormatter(_Formatter(color=sys.stderr.isatty() if use_color is None else bool(use_color)))
    logger.addHandler(sh)
    if log_file:
        path = log_file if rank is None else f"{log_file}.rank{rank}"
        fh = logging.FileHandler(path)
        fh.setFormatter(_Formatter(color=False))
        logger.addHandler(fh)
    return logger


def get_logger(name: str = "") -> logging.Logger:
    root = logging.getLogger(_ROOT)
    if not root.handlers:
        setup_logger()
    return logging.getLogger(f"{_ROOT}.{name}" if name else _ROOT)
