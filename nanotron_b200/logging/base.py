"""Rank-aware logging (parity: reference src/nanotron/logging/base.py)."""
from __future__ import annotations

import logging
import os
import sys
from dataclasses import dataclass
from functools import lru_cache
from logging import CRITICAL, DEBUG, ERROR, FATAL, INFO, NOTSET, WARNING, Formatter, Logger  # noqa: F401
from typing import List, Optional, Union

import torch

log_levels = {
    "debug": DEBUG,
    "info": INFO,
    "warning": WARNING,
    "error": ERROR,
    "critical": CRITICAL,
    "fatal": FATAL,
    "notset": NOTSET,
    "passive": ERROR,
}
_default_log_level = INFO
LIBRARY_NAME = __name__.split(".")[0]


def _get_default_logging_level() -> int:
    env = os.getenv("NANOTRON_LOGGING_LEVEL")
    if env is not None:
        if env.lower() in log_levels:
            return log_levels[env.lower()]
        logging.getLogger().warning(f"Unknown NANOTRON_LOGGING_LEVEL={env}; options: {', '.join(log_levels)}")
    return _default_log_level


def get_library_root_logger() -> Logger:
    return logging.getLogger(LIBRARY_NAME)


def get_logger(name: Optional[str] = None, log_level: Optional[str] = None) -> Logger:
    logger = logging.getLogger(name or LIBRARY_NAME)
    if log_level is not None:
        logger.setLevel(log_levels[log_level.lower()])
    return logger


def set_verbosity(verbosity: int) -> None:
    get_library_root_logger().setLevel(verbosity)


def human_format(num: float, billions: bool = False, divide_by_1024: bool = False) -> str:
    """1234567 -> '1.23M'."""
    if abs(num) < 1:
        return f"{num:.3g}"
    SIZES = ["", "K", "M", "G", "T", "P", "E"]
    num = float(f"{num:.3g}")
    i = 0
    base = 1024.0 if divide_by_1024 else 1000.0
    while abs(num) >= base and i < len(SIZES) - 1:
        i += 1
        num /= base
    value = f"{num:.3g}"
    return f"{value}{SIZES[i] if not (billions and SIZES[i] == 'G') else 'B'}"


def log_rank(msg: str, logger: Logger, level: int, group=None, rank: Optional[int] = None, is_separator: bool = False, main_rank_only: bool = False, **kwargs):
    """Log only on ``rank`` of ``group`` (every rank when ``rank`` is None)."""
    import nanotron_b200.distributed as dist

    if main_rank_only:
        rank = 0
    if rank is not None and dist.is_initialized():
        if dist.get_rank(group) != rank:
            return
    if is_separator:
        msg = "=" * 10 + " " + msg + " " + "=" * 10
    logger.log(level, msg, **kwargs)


@lru_cache(maxsize=None)
def warn_once(msg: str, logger: Logger, group=None, rank: Optional[int] = None):
    log_rank(msg, logger=logger, level=logging.WARNING, group=group, rank=rank)


def log_memory(logger: Logger, msg: str = ""):
    if not torch.cuda.is_available():
        return
    log_rank(
        f" Memory usage: {torch.cuda.memory_allocated() / 1024**2:.2f}MiB."
        f" Peak allocated {torch.cuda.max_memory_allocated() / 1024**2:.2f}MiB."
        f" Peak reserved: {torch.cuda.max_memory_reserved() / 1024**2:.2f}MiB {msg}",
        logger=logger,
        level=logging.INFO,
        rank=0,
    )
    torch.cuda.reset_peak_memory_stats()


@dataclass
class LogItem:
    tag: str
    scalar_value: Union[float, int, str]
    log_format: Optional[str] = None


class LoggerWriter:
    """Console writer for the per-iteration metric line."""

    def __init__(self, global_step: int):
        self.global_step = global_step
        self._logger = get_logger(__name__)

    def add_scalars_from_list(self, log_entries: List[LogItem], iteration_step: int):
        parts = [f"iteration: {iteration_step} / {self.global_step}"]
        for e in log_entries:
            if e.log_format is not None and not isinstance(e.scalar_value, str):
                if e.log_format == "human_format":
                    parts.append(f"{e.tag}: {human_format(e.scalar_value)}")
                else:
                    parts.append(f"{e.tag}: {e.scalar_value:{e.log_format}}")
            else:
                parts.append(f"{e.tag}: {e.scalar_value}")
        log_rank(" | ".join(parts), logger=self._logger, level=logging.INFO)


class _RankFormatter(Formatter):
    COLORS = {DEBUG: "\x1b[36m", INFO: "\x1b[32m", WARNING: "\x1b[33m", ERROR: "\x1b[31m", CRITICAL: "\x1b[31;1m"}

    def __init__(self, prefix: str, colour: bool):
        super().__init__(fmt=f"%(asctime)s [%(levelname)s|{prefix}]: %(message)s", datefmt="%m/%d/%Y %H:%M:%S")
        self.colour = colour

    def format(self, record):
        s = super().format(record)
        if self.colour:
            s = self.COLORS.get(record.levelno, "") + s + "\x1b[0m"
        return s


def set_logger_verbosity_format(logging_level: str, parallel_context) -> None:
    import nanotron_b200.distributed as dist

    node = os.environ.get("SLURMD_NODENAME", os.uname().nodename)
    ep = dist.get_rank(parallel_context.ep_pg) if parallel_context.expert_parallel_size > 1 else 0
    prefix = (
        f"%(name)s|EP={ep}|CP={dist.get_rank(parallel_context.cp_pg)}|DP={dist.get_rank(parallel_context.dp_pg)}"
        f"|PP={dist.get_rank(parallel_context.pp_pg)}|TP={dist.get_rank(parallel_context.tp_pg)}|{node}"
    )
    handler = logging.StreamHandler(sys.stdout)
    handler.setLevel(log_levels[logging_level])
    handler.setFormatter(_RankFormatter(prefix, colour=sys.stdout.isatty()))
    root = get_library_root_logger()
    root.handlers.clear()
    root.addHandler(handler)
    root.setLevel(log_levels[logging_level])
    root.propagate = False


def show_metric_lines(logging_level: str) -> None:
    """Print the per-iteration metric line of THIS rank at ``logging_level`` whatever the rank's general verbosity: the line is
    written by the rank that holds the loss (the last pipeline stage), which is a "replica" for every other message."""
    root = get_library_root_logger()
    own = get_logger(__name__)  # the logger of ``LoggerWriter``
    handler = logging.StreamHandler(sys.stdout)
    handler.setLevel(log_levels[logging_level])
    if root.handlers:
        handler.setFormatter(root.handlers[0].formatter)
    own.handlers.clear()
    own.addHandler(handler)
    own.setLevel(log_levels[logging_level])
    own.propagate = False


def set_ranks_logging_level(parallel_context, logging_config) -> None:
    """World rank 0 uses ``log_level``; every other rank ``log_level_replica``."""
    import nanotron_b200.distributed as dist

    if dist.get_rank(parallel_context.world_pg) == 0:
        set_logger_verbosity_format(logging_config.log_level or "info", parallel_context)
    else:
        set_logger_verbosity_format(logging_config.log_level_replica or "info", parallel_context)


def log_libraries_versions(logger: Logger):
    import numpy

    log_rank("Libraries versions:", logger=logger, level=logging.INFO, rank=0)
    log_rank(f"torch: {torch.__version__}  numpy: {numpy.__version__}  python: {sys.version.split()[0]}", logger=logger, level=logging.INFO, rank=0)
    if torch.cuda.is_available():
        log_rank(f"cuda: {torch.version.cuda}  nccl: {torch.cuda.nccl.version()}  device: {torch.cuda.get_device_name()}", logger=logger, level=logging.INFO, rank=0)


def _configure_library_root_logger():
    root = get_library_root_logger()
    if not root.handlers:
        h = logging.StreamHandler(sys.stdout)
        h.setFormatter(Formatter("%(asctime)s [%(levelname)s|%(name)s]: %(message)s", datefmt="%m/%d/%Y %H:%M:%S"))
        root.addHandler(h)
        root.setLevel(_get_default_logging_level())
        root.propagate = False


_configure_library_root_logger()
