"""Host-side liveness checks: a per-step deadline for this process and a heartbeat table across ranks.

The reference has neither (its failure handling is the non-finite guard, crash rows and transactional
checkpoints, ``training/entrypoint.py:1886-2005``). Both helpers live entirely on the host: they never touch a
kernel in flight, they only observe that the Python loop stopped making progress and say where.

``StepWatchdog`` — a daemon thread; the training loop calls ``beat(step)`` once per optimizer step. When no beat
arrives within ``deadline_s`` it writes a report (step, age, Python stacks of all threads, the device status word
if a reader was given) and calls ``on_timeout``; by default that only logs. It fires once per stall.

``RankHeartbeat`` — every rank publishes ``(step, wall time)`` under its key in a ``torch.distributed`` store
(the rendezvous store works; so does a ``FileStore`` or ``HashStore`` in tests); ``stale_ranks`` lists the ranks
whose last beat is older than a limit, so that a rank can stop before entering a collective that a dead peer will
never join.
"""

from __future__ import annotations

import json
import logging
import sys
import threading
import time
import traceback
from pathlib import Path
from typing import Any, Callable

logger = logging.getLogger(__name__)

__all__ = ["StepWatchdog", "RankHeartbeat"]


def _all_stacks() -> dict[str, list[str]]:
    frames = sys._current_frames()
    names = {t.ident: t.name for t in threading.enumerate()}
    return {f"{names.get(tid, '?')}:{tid}": traceback.format_stack(fr) for tid, fr in frames.items()}


class StepWatchdog:
    def __init__(self, deadline_s: float, *, report_dir: str | Path | None = None,
                 on_timeout: Callable[[dict[str, Any]], None] | None = None,
                 status_reader: Callable[[], Any] | None = None, poll_s: float | None = None) -> None:
        if deadline_s <= 0:
            raise ValueError("deadline_s must be positive")
        self.deadline_s = float(deadline_s)
        self.report_dir = Path(report_dir) if report_dir is not None else None
        self.on_timeout = on_timeout
        self.status_reader = status_reader
        self.poll_s = poll_s if poll_s is not None else min(1.0, self.deadline_s / 4)
        self._last = time.monotonic()
        self._step = -1
        self._fired_for = None
        self._stop = threading.Event()
        self._lock = threading.Lock()
        self.reports: list[dict[str, Any]] = []
        self._thread = threading.Thread(target=self._run, name="step-watchdog", daemon=True)

    def start(self) -> "StepWatchdog":
        self._last = time.monotonic()
        self._thread.start()
        return self

    def beat(self, step: int) -> None:
        with self._lock:
            self._last = time.monotonic()
            self._step = int(step)

    def stop(self) -> None:
        self._stop.set()
        if self._thread.is_alive():
            self._thread.join(timeout=2 * self.poll_s + 1.0)

    def __enter__(self) -> "StepWatchdog":
        return self.start()

    def __exit__(self, *exc) -> None:
        self.stop()

    def _run(self) -> None:
        while not self._stop.wait(self.poll_s):
            with self._lock:
                age, step = time.monotonic() - self._last, self._step
            if age <= self.deadline_s or self._fired_for == step:
                continue
            self._fired_for = step
            report: dict[str, Any] = {"event": "step_deadline_exceeded", "last_step": step, "age_s": round(age, 3),
                                      "deadline_s": self.deadline_s, "stacks": _all_stacks()}
            if self.status_reader is not None:
                try:
                    report["device_status"] = self.status_reader()
                except Exception as e:  # noqa: BLE001
                    report["device_status_error"] = repr(e)
            self.reports.append(report)
            logger.error("No optimizer step finished for %.1f s (deadline %.1f s, last step %d).", age, self.deadline_s, step)
            if self.report_dir is not None:
                try:
                    self.report_dir.mkdir(parents=True, exist_ok=True)
                    (self.report_dir / f"watchdog_step{step}.json").write_text(json.dumps(report, indent=1))
                except OSError as e:
                    logger.error("Could not write the watchdog report: %s", e)
            if self.on_timeout is not None:
                try:
                    self.on_timeout(report)
                except Exception:  # noqa: BLE001
                    logger.exception("watchdog on_timeout callback failed")


class RankHeartbeat:
    def __init__(self, store: Any, rank: int, world_size: int, *, prefix: str = "deberta_hb") -> None:
        self.store, self.rank, self.world_size, self.prefix = store, int(rank), int(world_size), prefix

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), json.dumps({"step": int(step), "t": time.time()}))

    def read(self, rank: int) -> dict[str, float] | None:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(rank)]):
                return None
            return json.loads(bytes(self.store.get(self._key(rank))).decode())
        except Exception:  # noqa: BLE001
            return None

    def stale_ranks(self, max_age_s: float, *, now: float | None = None) -> list[int]:
        """Ranks that never reported or whose last report is older than ``max_age_s`` seconds."""
        now = time.time() if now is None else now
        out = []
        for r in range(self.world_size):
            rec = self.read(r)
            if rec is None or now - float(rec["t"]) > max_age_s:
                out.append(r)
        return out

    def lagging_ranks(self, behind_steps: int) -> list[int]:
        """Ranks whose reported step is at least ``behind_steps`` behind this rank's."""
        mine = self.read(self.rank)
        if mine is None:
            return []
        out = []
        for r in range(self.world_size):
            rec = self.read(r)
            if rec is not None and mine["step"] - rec["step"] >= behind_steps:
                out.append(r)
        return out
