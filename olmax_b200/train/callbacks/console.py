"""Metric sinks: a JSON-lines file writer (the hook where W&B / Comet style loggers attach in the reference)."""

from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Dict, Optional

from .callback import Callback

__all__ = ["JSONLMetricsCallback"]


@Callback.register("jsonl_metrics")
@dataclass
class JSONLMetricsCallback(Callback):
    file_name: str = "metrics.jsonl"

    def __post_init__(self):
        super().__post_init__()
        self._fh = None

    def log_metrics(self, step: int, metrics: Dict[str, float]) -> None:
        from ...parallel import dist_utils

        if dist_utils.get_rank() != 0:
            return
        if self._fh is None:
            self._fh = open(self.trainer.work_dir / self.file_name, "a")
        self._fh.write(json.dumps({"step": step, **metrics}) + "\n")
        self._fh.flush()

    def close(self) -> None:
        if self._fh is not None:
            self._fh.close()
            self._fh = None
            self.trainer.persist_working_file(self.file_name)
