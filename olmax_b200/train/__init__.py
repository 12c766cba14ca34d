"""
Training runtime: :class:`Trainer`, callbacks, checkpointer and the environment preparation step
(``olmax/train/__init__.py:24-85``).
"""

from __future__ import annotations

import logging
import os
from typing import Optional, Union

from ..env import CUDAConfig, EnvConfig, JAXConfig, NCCLConfig, RuntimeConfig, XLAConfig
from ..types import GPUArchitecture
from ..utils.tree import get_cudnn_version
from .callbacks import Callback, JSONLMetricsCallback, ProfilerCallback
from .checkpointer import Checkpointer, SimpleCheckpointer, TrainState
from .trainer import Trainer, TrainMetrics

__all__ = [
    "Trainer", "TrainMetrics", "TrainState", "Checkpointer", "SimpleCheckpointer", "Callback", "ProfilerCallback",
    "JSONLMetricsCallback", "prepare_training_environment",
]

log = logging.getLogger(__name__)

_Choice = Union[str, None]


def _resolve(value, cls, gpu_architecture):
    """``"recommended"`` -> cls.recommended(arch); ``"system_default"`` / None -> leave the environment alone."""
    if isinstance(value, cls):
        return value
    if value == "recommended":
        return cls.recommended(gpu_architecture)
    if value in (None, "system_default"):
        return None
    raise ValueError(f"expected a {cls.__name__}, 'recommended' or 'system_default', got {value!r}")


def prepare_training_environment(
    xla_config: Union[XLAConfig, _Choice] = "recommended",
    nccl_config: Union[NCCLConfig, _Choice] = "recommended",
    cuda_config: Union[CUDAConfig, _Choice] = "recommended",
    jax_config: Union[JAXConfig, _Choice] = "recommended",
    runtime_config: Union[RuntimeConfig, _Choice] = "recommended",
    gpu_architecture: Optional[GPUArchitecture] = None,
) -> None:
    """Apply the environment settings (must run before the first CUDA / NCCL use) and log the resulting variables."""
    for value, cls in ((xla_config, XLAConfig), (nccl_config, NCCLConfig), (cuda_config, CUDAConfig),
                       (jax_config, JAXConfig), (runtime_config, RuntimeConfig)):
        cfg = _resolve(value, cls, gpu_architecture)
        if cfg is not None:
            cfg.apply()
    for key in sorted(os.environ):
        if key.startswith(("XLA_", "CUDA_", "NCCL_", "OLMAX_B200_")):
            log.info("Env: %s=%s", key, os.environ[key])
    log.info("cuDNN version: %s (not used by the compute path)", get_cudnn_version())
