"""
Activation-checkpointing policies (registry names of ``olmax/activation_checkpointing.py:19-182``).

A policy decides, for a named region of the model (a transformer layer ``layers.{i}`` or one of its sub-blocks
``layers.{i}.attention`` / ``layers.{i}.mlp``), whether the activations inside it are kept for the backward pass or
recomputed from the region's input.  Recomputation re-invokes the same kernels; there is no compiler pass involved.
Whole layers are recomputed through a checkpoint; the two sub-blocks recompute inside their own autograd nodes, so
that only what is cheap runs twice: the MLP block keeps its input and repeats the gate / up GEMM (not the down
projection), the attention block keeps its input, its output and the softmax statistics and repeats the q / k / v
projections with their norm and rotation (neither the attention forward nor the output projection).

Mapping of the reference's policy names:

* ``default`` / ``everything_saveable``: keep everything the ops save (the ops already avoid keeping cheap
  elementwise results, e.g. ``act(gate) * up`` is recomputed inside the MLP backward).
* ``nothing_saveable``: full recomputation of every layer from its input (what the 32B / 70B recipes use).
* ``dots_saveable`` / ``dots_with_no_batch_dims_saveable``: matmul outputs kept, everything else recomputed.  The
  fused ops implement exactly this split internally, so at region granularity nothing more is recomputed.
* ``save_only_these_names`` / ``save_anything_except_these_names`` / ``save_any_names_but_these``: glob patterns over
  region names choose which regions are kept.
"""

from __future__ import annotations

import fnmatch
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch
from torch.utils.checkpoint import checkpoint as _torch_checkpoint

from .utils.dataclass_codec import Registrable

__all__ = [
    "ActivationCheckpointingPolicy",
    "NoPolicy",
    "EverythingSaveable",
    "NothingSaveable",
    "DotsSaveable",
    "DotsWithNoBatchDimsSaveable",
    "NamedCheckpointPolicy",
    "SaveAnythingExceptTheseNames",
    "SaveAnyNamesButThese",
    "SaveOnlyTheseNames",
]


@dataclass
class ActivationCheckpointingPolicy(Registrable):
    prevent_cse: bool = True
    """Kept for config compatibility (an XLA concept); has no effect here."""

    def should_recompute(self, region_name: str) -> bool:
        """True when the activations inside ``region_name`` are to be recomputed in the backward pass."""
        raise NotImplementedError

    def resolve_names(self, all_names: Sequence[str]) -> None:
        """Hook for name-based policies: validate patterns against the model's region names."""

    def wrap(self, fun: Callable, region_name: str) -> Callable:
        if not self.should_recompute(region_name):
            return fun

        def wrapped(*args, **kwargs):
            if not torch.is_grad_enabled():
                return fun(*args, **kwargs)
            return _torch_checkpoint(fun, *args, use_reentrant=False, **kwargs)

        return wrapped


@ActivationCheckpointingPolicy.register("default", default=True)
@dataclass
class NoPolicy(ActivationCheckpointingPolicy):
    def should_recompute(self, region_name: str) -> bool:
        return False


@ActivationCheckpointingPolicy.register("everything_saveable")
@dataclass
class EverythingSaveable(ActivationCheckpointingPolicy):
    def should_recompute(self, region_name: str) -> bool:
        return False


@ActivationCheckpointingPolicy.register("nothing_saveable")
@dataclass
class NothingSaveable(ActivationCheckpointingPolicy):
    def should_recompute(self, region_name: str) -> bool:
        # whole layers are the recomputation unit; sub-blocks inside a recomputed layer are not wrapped again
        return region_name.count(".") == 1


@ActivationCheckpointingPolicy.register("dots_saveable")
@dataclass
class DotsSaveable(ActivationCheckpointingPolicy):
    """
    In the reference this policy keeps matrix-product results and recomputes every element-wise result between them.
    Here no region is wrapped for recomputation under it, and the autograd nodes decide what they keep:

    * recomputed in backward, never stored: the gated activation ``act(gate) * up`` (the gated-MLP node keeps the two
      projections and forms the product again), attention probabilities (flash attention keeps the log-sum-exp only),
      logits and their gradients beyond one chunk of rows;
    * still stored although element-wise: the outputs of the normalisation layers (block-output norms of OLMo2 / Gemma,
      pre-norm outputs, QK-norm outputs) and the rotated q / k.  For OLMo2-7B at 2 x 4096 tokens per micro-batch that is
      6 x [tokens, 4096] bf16 per layer = 12.9 GB of the 154 GB peak over 32 layers; a run that needs that memory
      back uses ``save_anything_except_these_names`` with ``layers.*.attention`` / ``layers.*.mlp`` (sub-block
      recomputation) or ``nothing_saveable``.
    """

    def should_recompute(self, region_name: str) -> bool:
        return False


@ActivationCheckpointingPolicy.register("dots_with_no_batch_dims_saveable")
@dataclass
class DotsWithNoBatchDimsSaveable(DotsSaveable):
    pass


@dataclass
class NamedCheckpointPolicy(ActivationCheckpointingPolicy):
    names: List[str] = field(default_factory=list)
    """Region names or glob patterns (``layers.*.mlp``)."""

    def _matches(self, region_name: str) -> bool:
        return any(region_name == p or fnmatch.fnmatch(region_name, p) for p in self.names)

    def resolve_names(self, all_names: Sequence[str]) -> None:
        for p in self.names:
            if not any(n == p or fnmatch.fnmatch(n, p) for n in all_names):
                raise ValueError(f"activation checkpointing pattern '{p}' matches no region; regions: {list(all_names)[:8]}...")


@ActivationCheckpointingPolicy.register("save_anything_except_these_names")
@dataclass
class SaveAnythingExceptTheseNames(NamedCheckpointPolicy):
    def should_recompute(self, region_name: str) -> bool:
        return self._matches(region_name)


@ActivationCheckpointingPolicy.register("save_any_names_but_these")
@dataclass
class SaveAnyNamesButThese(SaveAnythingExceptTheseNames):
    pass


@ActivationCheckpointingPolicy.register("save_only_these_names")
@dataclass
class SaveOnlyTheseNames(NamedCheckpointPolicy):
    def should_recompute(self, region_name: str) -> bool:
        # regions are layers and their attention / mlp sub-blocks; a layer is recomputed as a whole only when none of
        # its sub-blocks is to be saved, otherwise the decision is taken per sub-block
        if self._matches(region_name):
            return False
        if region_name.count(".") == 1:
            subs = [f"{region_name}.attention", f"{region_name}.mlp"]
            return not any(self._matches(s) for s in subs)
        return True
