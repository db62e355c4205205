"""Root logger ``[titan] <time> - <logger> - <level> - msg`` and ``warn_once``.

Parity: torchtitan/tools/logging.py:15-45.
"""

import logging
import os

logger = logging.getLogger()
_seen: set[str] = set()


def init_logger() -> None:
    logger.setLevel(logging.INFO)
    if not any(getattr(h, "_titan", False) for h in logger.handlers):
        h = logging.StreamHandler()
        h.setLevel(logging.INFO)
        h.setFormatter(
            logging.Formatter("[titan] %(asctime)s - %(name)s - %(levelname)s - %(message)s")
        )
        h._titan = True
        logger.addHandler(h)
    # keep Kineto's chatter out of training logs
    os.environ.setdefault("KINETO_LOG_LEVEL", "5")


def warn_once(log: logging.Logger, msg: str) -> None:
    if msg not in _seen:
        _seen.add(msg)
        log.warning(msg)
