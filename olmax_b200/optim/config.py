"""
Optimizer configuration (``olmax/optim/config.py:19-156``): learning-rate schedules, the AdamW config, and the
weight-decay mask by glob over dotted parameter names.

A schedule is a callable ``step -> value`` evaluated with the number of optimizer steps already taken (0 for the first
update), the same convention optax uses.
"""

from __future__ import annotations

import fnmatch
import logging
import math
import warnings
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional

from ..utils.dataclass_codec import Registrable

__all__ = [
    "Schedule",
    "ConstantSchedule",
    "WarmupCosineDecaySchedule",
    "WarmupStableDecaySchedule",
    "OptimConfig",
    "AdamWConfig",
]

log = logging.getLogger(__name__)


@dataclass
class Schedule(Registrable):
    def build(self) -> Callable[[int], float]:
        raise NotImplementedError

    def __call__(self, step: int) -> float:
        return self.build()(step)


@Schedule.register("constant")
@dataclass
class ConstantSchedule(Schedule):
    value: float = 0.0

    def build(self) -> Callable[[int], float]:
        v = self.value
        return lambda step: v


def _linear(init: float, end: float, steps: int, t: int) -> float:
    if steps <= 0:
        return end
    frac = min(max(t, 0), steps) / steps
    return init + (end - init) * frac


@Schedule.register("warmup_cosine_decay")
@dataclass
class WarmupCosineDecaySchedule(Schedule):
    """Linear warm-up from ``init_value`` to ``peak_value`` over ``warmup_steps``, then a cosine decay to ``end_value``
    over ``decay_steps`` (which does not include the warm-up)."""

    warmup_steps: int = 0
    decay_steps: int = 0
    peak_value: float = 0.0
    init_value: float = 0.0
    end_value: float = 0.0

    def build(self) -> Callable[[int], float]:
        w, d, peak, init, end = self.warmup_steps, self.decay_steps, self.peak_value, self.init_value, self.end_value

        def fn(step: int) -> float:
            if step < w:
                return _linear(init, peak, w, step)
            t = min(step - w, d)
            cos = 0.5 * (1.0 + math.cos(math.pi * (t / d if d > 0 else 1.0)))
            return end + (peak - end) * cos

        return fn


@Schedule.register("warmup_stable_decay")
@dataclass
class WarmupStableDecaySchedule(Schedule):
    """Linear warm-up, hold at ``peak_value`` for ``stable_steps``, then a linear decay to ``end_value``."""

    warmup_steps: int = 0
    stable_steps: int = 0
    decay_steps: int = 0
    peak_value: float = 0.0
    init_value: float = 0.0
    end_value: float = 0.0

    def build(self) -> Callable[[int], float]:
        w, s, d = self.warmup_steps, self.stable_steps, self.decay_steps
        peak, init, end = self.peak_value, self.init_value, self.end_value

        def fn(step: int) -> float:
            if step < w:
                return _linear(init, peak, w, step)
            if step < w + s:
                return peak
            return _linear(peak, end, d, step - w - s)

        return fn


@dataclass
class OptimConfig(Registrable):
    @classmethod
    def AdamW(cls, *args, **kwargs) -> "AdamWConfig":
        return AdamWConfig(*args, **kwargs)

    def build(self, model, num_grad_accumulation_steps: int = 1):
        raise NotImplementedError

    @classmethod
    def build_weight_decay_mask(cls, param_names: Iterable[str], no_decay_modules: Optional[List[str]]) -> Dict[str, bool]:
        """name -> True when weight decay applies.  Patterns are fnmatch globs over dotted parameter names
        (``embedding.weight``, ``layers.*.attention_norm.weight``); a pattern that matches nothing warns."""
        patterns = list(no_decay_modules or [])
        hit = {p: False for p in patterns}
        mask: Dict[str, bool] = {}
        for name in param_names:
            decay = True
            for p in patterns:
                if fnmatch.fnmatch(name, p):
                    hit[p] = True
                    decay = False
                    log.info("Weight decay will not be applied to parameter '%s'", name)
                    break
            mask[name] = decay
        for p, matched in hit.items():
            if not matched:
                warnings.warn(f"no decay pattern '{p}' did not match any parameters")
        return mask


@OptimConfig.register("adamw", default=True)
@dataclass
class AdamWConfig(OptimConfig):
    lr: Schedule = None  # type: ignore[assignment]
    b1: float = 0.9
    b2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 1e-4
    no_decay_modules: Optional[List[str]] = None
    max_grad_norm: Optional[float] = None
    track_grad_norm: Optional[bool] = None
    """Compute the global gradient norm every step (one pass over the gradient + a scalar all-reduce) for the
    ``optim/g_norm`` metric.  None: only when ``max_grad_norm`` is set, which is when the reference has that metric
    (it reads it from the clipping state, ``olmax/optim/utils.py:22-38``)."""

    def __post_init__(self):
        if self.lr is None:
            self.lr = ConstantSchedule(1e-3)
        elif isinstance(self.lr, (int, float)):
            self.lr = ConstantSchedule(float(self.lr))

    def build(self, model, num_grad_accumulation_steps: int = 1):
        """``model`` is a :class:`Transformer` (or anything with a ``store``); returns the optimizer (its state lives
        inside it, sharded like the parameters)."""
        from .adamw import AdamW

        store = getattr(model, "store", model)
        mask = self.build_weight_decay_mask([m.name for m in store.metas], self.no_decay_modules)
        for m in store.metas:
            m.decay = mask[m.name]
        return AdamW(store, self, num_grad_accumulation_steps)
