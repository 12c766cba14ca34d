"""
Shared enums, the :class:`Duration` type and type aliases (public surface of ``olmax/types.py:28-124``).
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from enum import Enum
from typing import Any, Optional, Union

__all__ = [
    "StrEnum",
    "PyTree",
    "Specs",
    "Scalar",
    "PathOrStr",
    "GPUArchitecture",
    "DeviceType",
    "Duration",
    "DurationUnit",
]


class StrEnum(str, Enum):
    """String-valued enum whose ``str()`` is the value."""

    def __str__(self) -> str:
        return str(self.value)

    def __repr__(self) -> str:
        return f"'{self.value}'"


PyTree = Any
Specs = Any
Scalar = Union[float, int, Any]
PathOrStr = Union[os.PathLike, str]


class GPUArchitecture(StrEnum):
    blackwell = "blackwell"
    hopper = "hopper"
    ampere = "ampere"


class DeviceType(StrEnum):
    NVIDIA_H100 = "NVIDIA_H100"
    NVIDIA_A100_80GB = "NVIDIA_A100_80GB"
    NVIDIA_A100_40GB = "NVIDIA_A100_40GB"
    NVIDIA_L4 = "NVIDIA_L4"
    NVIDIA_RTX_A5000 = "NVIDIA_RTX_A5000"
    NVIDIA_RTX_A6000 = "NVIDIA_RTX_A6000"
    NVIDIA_RTX_8000 = "NVIDIA_RTX_8000"
    NVIDIA_T4 = "NVIDIA_T4"
    NVIDIA_P100 = "NVIDIA_P100"
    NVIDIA_P4 = "NVIDIA_P4"
    NVIDIA_V100 = "NVIDIA_V100"
    NVIDIA_L40 = "NVIDIA_L40"
    NVIDIA_L40S = "NVIDIA_L40S"
    NVIDIA_B200 = "NVIDIA_B200"

    @property
    def architecture(self) -> Optional[GPUArchitecture]:
        if self == DeviceType.NVIDIA_B200:
            return GPUArchitecture.blackwell
        if self == DeviceType.NVIDIA_H100:
            return GPUArchitecture.hopper
        if self in (DeviceType.NVIDIA_A100_80GB, DeviceType.NVIDIA_A100_40GB):
            return GPUArchitecture.ampere
        return None


class DurationUnit(StrEnum):
    """Units a :class:`Duration` can be expressed in."""

    steps = "steps"
    epochs = "epochs"
    tokens = "tokens"


@dataclass
class Duration:
    """A training length: ``value`` steps, epochs or tokens."""

    value: int
    unit: DurationUnit

    @classmethod
    def steps(cls, steps: int) -> "Duration":
        return cls(value=steps, unit=DurationUnit.steps)

    @classmethod
    def epochs(cls, epochs: int) -> "Duration":
        return cls(value=epochs, unit=DurationUnit.epochs)

    @classmethod
    def tokens(cls, tokens: int) -> "Duration":
        return cls(value=tokens, unit=DurationUnit.tokens)

    def due(self, *, step: Optional[int] = None, tokens: Optional[int] = None, epoch: Optional[int] = None) -> bool:
        """True once the duration has elapsed: steps and tokens compare with ``>=``, epochs with ``>``."""
        if self.unit == DurationUnit.steps:
            if step is None:
                raise ValueError("step is required for a duration in steps")
            return step >= self.value
        if self.unit == DurationUnit.tokens:
            if tokens is None:
                raise ValueError("tokens is required for a duration in tokens")
            return tokens >= self.value
        if self.unit == DurationUnit.epochs:
            if epoch is None:
                raise ValueError("epoch is required for a duration in epochs")
            return epoch > self.value
        raise NotImplementedError(self.unit)
