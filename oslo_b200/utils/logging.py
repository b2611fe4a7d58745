"""Rank-aware logging: by default only global rank 0 emits records below WARNING."""
from __future__ import annotations

import logging
import os


class _RankFilter(logging.Filter):
    def filter(self, record: logging.LogRecord) -> bool:
        rank = int(os.environ.get("RANK", "0"))
        record.rank = rank
        return rank == 0 or record.levelno >= logging.WARNING or os.environ.get("OSLO_B200_LOG_ALL_RANKS") == "1"


def get_logger(name: str = "oslo_b200") -> logging.Logger:
    logger = logging.getLogger(name)
    if not any(isinstance(f, _RankFilter) for f in logger.filters):
        logger.addFilter(_RankFilter())
        if not logger.handlers:
            h = logging.StreamHandler()
            h.setFormatter(logging.Formatter("%(asctime)s [rank %(rank)s] %(levelname)s %(name)s: %(message)s"))
            # records of child loggers (`oslo_b200.parallelism_utils`, ...) reach this handler without passing the
            # logger's own filters, so the handler carries the filter too
            h.addFilter(_RankFilter())
            logger.addHandler(h)
        logger.setLevel(os.environ.get("OSLO_B200_LOG_LEVEL", "INFO").upper())
        logger.propagate = False
    return logger
