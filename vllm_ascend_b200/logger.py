"""Package logger.  With ``VLLM_B200_LOG_PATH`` set, every process additionally writes to
``<path>/vllm_b200_<pid>.log`` (rotating, 10 MB x 5), the file-logging behaviour of
vllm_ascend/logger.py:35-103."""
from __future__ import annotations

import logging
import os
from logging.handlers import RotatingFileHandler

_FORMAT = "%(levelname)s %(asctime)s [%(filename)s:%(lineno)d] %(message)s"

logger = logging.getLogger("vllm_ascend_b200")
_configured = False


def configure_logging(force: bool = False) -> logging.Logger:
    global _configured
    if _configured and not force:
        return logger
    _configured = True
    level = os.getenv("VLLM_B200_LOG_LEVEL", os.getenv("VLLM_LOGGING_LEVEL", "INFO")).upper()
    logger.setLevel(getattr(logging, level, logging.INFO))
    if not any(isinstance(h, logging.StreamHandler) and not isinstance(h, RotatingFileHandler)
               for h in logger.handlers):
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter(_FORMAT, datefmt="%m-%d %H:%M:%S"))
        logger.addHandler(h)
    path = os.getenv("VLLM_B200_LOG_PATH")
    if path:
        for h in list(logger.handlers):
            if isinstance(h, RotatingFileHandler):
                logger.removeHandler(h)
                h.close()
        os.makedirs(path, exist_ok=True)
        fh = RotatingFileHandler(os.path.join(path, f"vllm_b200_{os.getpid()}.log"),
                                 maxBytes=10 << 20, backupCount=5)
        fh.setFormatter(logging.Formatter(_FORMAT, datefmt="%m-%d %H:%M:%S"))
        logger.addHandler(fh)
    logger.propagate = False
    return logger


configure_logging()
