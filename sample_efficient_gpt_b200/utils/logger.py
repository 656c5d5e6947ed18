"""Package logger (INFO by default, ``LOGLEVEL`` env overrides). Parity: utils/logger.py:1-4."""

import logging
import os

logging.basicConfig(level=os.environ.get("LOGLEVEL", "INFO").upper(), format="%(asctime)s %(levelname)s %(message)s")
logger = logging.getLogger("sample_efficient_gpt_b200")
