"""
olmax_b200: a Blackwell-native LLM pre-training framework with the capabilities of OLMax.

PyTorch is the framework layer; every hot op is a hand-written sm_100a CUDA kernel (tcgen05 / TMEM GEMMs fed by TMA,
flash attention, fused norms, RoPE, gated-MLP epilogues, fused cross-entropy, fused AdamW) loaded from the in-tree
library ``olmax_b200/lib/libolmax_b200.so``; ranks are one process per GPU over ``torch.distributed``.
"""

from .version import VERSION as __version__
from . import types, utils
from .activation_checkpointing import (
    ActivationCheckpointingPolicy,
    DotsSaveable,
    DotsWithNoBatchDimsSaveable,
    EverythingSaveable,
    NoPolicy,
    NothingSaveable,
    SaveAnyNamesButThese,
    SaveAnythingExceptTheseNames,
    SaveOnlyTheseNames,
)
from .config import parse_config_from_args
from .env import CUDAConfig, EnvConfig, JAXConfig, NCCLConfig, RuntimeConfig, XLAConfig
from .exceptions import *  # noqa: F401,F403
from .utils import prepare_cli_environment


def prepare_training_environment(*args, **kwargs):
    from .train import prepare_training_environment as _impl

    return _impl(*args, **kwargs)
