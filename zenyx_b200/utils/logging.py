"""Logging helpers with the reference's names (zenyx/utils/logging.py:10,46,62)."""
from __future__ import annotations

import logging
from typing import Union

_FORMAT = "%(asctime)s - %(name)s - %(levelname)s - %(message)s"


def _level(level: Union[int, str]) -> int:
    if isinstance(level, str):
        value = logging.getLevelName(level.upper())
        if not isinstance(value, int):
            raise ValueError(f"unknown log level {level!r}")
        return value
    return int(level)


def setup_logging(level: Union[int, str] = logging.INFO, name: str = "zenyx_b200") -> logging.Logger:
    """Attaches one stream handler to the named logger (idempotent) and sets its level."""
    logger = logging.getLogger(name)
    logger.setLevel(_level(level))
    if not logger.handlers:
        handler = logging.StreamHandler()
        handler.setFormatter(logging.Formatter(_FORMAT))
        logger.addHandler(handler)
        logger.propagate = False
    return logger


def get_logger(name: str = "zenyx_b200") -> logging.Logger:
    return logging.getLogger(name)


def set_log_level(name: str, level: Union[int, str]) -> None:
    logging.getLogger(name).setLevel(_level(level))
