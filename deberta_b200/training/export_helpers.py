"""Final export hook: run ``deberta export`` on the last checkpoint in a subprocess (``training/export_helpers.py``)."""

from __future__ import annotations

import logging
import subprocess
import sys
from pathlib import Path

logger = logging.getLogger(__name__)


def export_discriminator_hf_subprocess(*, checkpoint_dir: Path, output_dir: Path, timeout_s: float | None = None) -> bool:
    """Export the discriminator of ``checkpoint_dir`` to ``output_dir`` as Hugging Face artifacts.

    A separate interpreter keeps the export's full-precision copy of the model out of the
    training process. ``--allow-partial-export`` is passed because HF's DeBERTa-v2 drops
    ``position_embeddings`` when ``position_biased_input`` is false.
    """
    cmd = [sys.executable, "-m", "deberta_b200", "export", str(checkpoint_dir), "--what", "discriminator",
           "--output-dir", str(output_dir), "--allow-partial-export"]
    try:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s)
    except Exception as e:
        logger.warning("Final HF export failed to launch: %s", e)
        return False
    if res.returncode != 0:
        logger.warning("Final HF export failed (rc=%d): %s", res.returncode, (res.stderr or "")[-2000:])
        return False
    logger.info("Exported final discriminator to %s", output_dir)
    return True
