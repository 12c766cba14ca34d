"""
Trainer callback API (``olmax/train/callbacks/callback.py:13-161``): a registrable base class with a priority, an
enabled flag, resumable state and the trainer's hook points.  Unlike the reference there is a host-side process group,
so a ``post_checkpoint_saved`` hook exists as well.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import TYPE_CHECKING, Any, Dict, Optional, Sequence

from ...utils.dataclass_codec import Registrable

if TYPE_CHECKING:
    from ..trainer import Trainer

__all__ = ["Callback"]


@dataclass
class Callback(Registrable):
    priority: int = 0
    """Callbacks run in order of decreasing priority; ties keep insertion order (identical on every rank)."""
    enabled: bool = True

    def __post_init__(self):
        self._trainer: Optional["Trainer"] = None

    @property
    def trainer(self) -> "Trainer":
        if getattr(self, "_trainer", None) is None:
            raise RuntimeError("callback is not attached to a trainer")
        return self._trainer  # type: ignore[return-value]

    @trainer.setter
    def trainer(self, trainer: "Trainer") -> None:
        self._trainer = trainer

    @property
    def step(self) -> int:
        return self.trainer.step

    # ---- state ---------------------------------------------------------------------------------------------------
    def get_state(self) -> Dict[str, Any]:
        return {}

    def load_state(self, state: Dict[str, Any]) -> None:
        del state

    # ---- hooks ---------------------------------------------------------------------------------------------------
    def post_attach(self) -> None: ...
    def pre_train(self) -> None: ...
    def pre_epoch(self) -> None: ...
    def pre_step(self) -> None: ...
    def pre_load_batch(self) -> None: ...
    def post_load_batch(self, batch: Sequence[Any]) -> None: ...
    def post_train_batch(self) -> None: ...
    def post_step(self) -> None: ...
    def post_checkpoint_saved(self, path: str) -> None: ...
    def post_checkpoint_loaded(self, path: str) -> None: ...
    def log_metrics(self, step: int, metrics: Dict[str, float]) -> None: ...
    def post_epoch(self) -> None: ...
    def post_train(self) -> None: ...
    def on_error(self, exc: BaseException) -> None: ...
    def close(self) -> None: ...
