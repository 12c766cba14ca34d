"""
Profiler callback (``olmax/train/callbacks/profiler.py:11-50``): skip the first steps, trace a few, write a Chrome /
Perfetto trace under ``work_dir/profiler`` and persist that directory to the save folder.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Optional

import torch

from .callback import Callback

log = logging.getLogger(__name__)

__all__ = ["ProfilerCallback"]


@Callback.register("profiler")
@dataclass
class ProfilerCallback(Callback):
    skip_first: int = 3
    active: int = 3
    ranks: Optional[list] = None
    """Ranks that record a trace (default: rank 0 only)."""

    def __post_init__(self):
        super().__post_init__()
        self._prof = None
        self._first_step: Optional[int] = None

    def _selected(self) -> bool:
        from ...parallel import dist_utils

        return dist_utils.get_rank() in (self.ranks if self.ranks is not None else [0])

    def pre_step(self) -> None:
        if not self._selected():
            return
        if self._first_step is None:
            self._first_step = self.step
        rel = self.step - self._first_step
        if rel == self.skip_first and self._prof is None:
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self._prof = torch.profiler.profile(activities=acts, record_shapes=False)
            self._prof.__enter__()
            log.info("Profiler started at step %d", self.step)

    def post_step(self) -> None:
        if self._prof is None or self._first_step is None:
            return
        rel = self.step - self._first_step
        if rel >= self.skip_first + self.active - 1:
            self._stop()

    def _stop(self) -> None:
        prof, self._prof = self._prof, None
        if prof is None:
            return
        prof.__exit__(None, None, None)
        out_dir = self.trainer.work_dir / "profiler"
        out_dir.mkdir(parents=True, exist_ok=True)
        from ...parallel import dist_utils

        path = out_dir / f"trace_rank{dist_utils.get_rank()}.json"
        prof.export_chrome_trace(str(path))
        log.info("Profiler trace written to %s", path)
        self.trainer.persist_working_subdir("profiler")

    def close(self) -> None:
        self._stop()
