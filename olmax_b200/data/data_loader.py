"""Data-loader interface (``olmax/data/data_loader.py:11-36``): an iterable of batches, each a sequence of
micro-batches, with resumable state."""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Dict, Generic, Iterator, Sequence, TypeVar

B = TypeVar("B")

__all__ = ["DataLoader"]


class DataLoader(ABC, Generic[B]):
    @abstractmethod
    def __iter__(self) -> Iterator[Sequence[B]]:
        """Yield batches; a batch is a sequence of micro-batches processed by one optimizer step."""
        raise NotImplementedError

    @abstractmethod
    def get_state(self) -> Dict[str, Any]:
        raise NotImplementedError

    @abstractmethod
    def load_state(self, state: Dict[str, Any]) -> None:
        raise NotImplementedError

    def __len__(self) -> int:
        raise TypeError(f"{type(self).__name__} has no length")
