"""Process logging: INFO on the main process, WARNING elsewhere."""

from __future__ import annotations

import logging


def setup_process_logging(is_main_process: bool) -> None:
    level = logging.INFO if is_main_process else logging.WARNING
    logging.basicConfig(level=level, format="%(asctime)s | %(levelname)s | %(name)s | %(message)s", force=True)
