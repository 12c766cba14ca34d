"""
AdamW over the flat sharded buffers of a :class:`ParamStore`.

Semantics are those of the reference's optax chain (``olmax/optim/config.py:125-156``): optional clipping of the
*accumulated* gradient by its global norm, Adam moments with bias correction, decoupled weight decay on the masked-in
parameters, learning rate from the schedule evaluated at the number of completed optimizer steps; with k micro-batches
the gradient is the running mean and the inner optimizer (and the schedule) advance once per k micro-batches.

Differences in mechanism: the mean over micro-batches and data-parallel ranks is applied as a scale at accumulation
time; the cross-replica all-reduce (HSDP / DDP) and the optimizer run once per step rather than once per micro-batch;
on the GPU one fused kernel per weight-decay group updates master weights and moments, writes the bf16 compute copy,
and clears the gradient, reading the clip coefficient from device memory so the step never synchronises with the host.
"""

from __future__ import annotations

import math
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..parallel.param_store import ParamStore

__all__ = ["AdamW"]


class AdamW:
    def __init__(self, store: ParamStore, config, num_microbatches: int = 1):
        self.store = store
        self.config = config
        self.num_microbatches = max(1, int(num_microbatches))
        self.schedule = config.lr.build()
        self.count = 0        # optimizer steps taken ("gradient_step" / Adam "count")
        self.mini_step = 0    # micro-batches accumulated towards the next step
        n = store.numel_local
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=store.device)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=store.device)
        dev = store.device
        self._sumsq = torch.zeros(1, dtype=torch.float64, device=dev)
        self._coef = torch.ones(2, dtype=torch.float32, device=dev)  # [clip coefficient, grad norm]
        self.last_lr = float(self.schedule(0))
        self.update_grad_scale()

    # ------------------------------------------------------------------ protocol with the trainer
    def update_grad_scale(self) -> None:
        """Every gradient contribution is scaled by 1 / (ranks whose losses are averaged x micro-batches)."""
        mesh = self.store.mesh
        # every rank (data, tensor and context parallel alike) reports the mean loss of its own tokens and the
        # gradient contributions of all ranks are summed, so the divisor is the whole job
        self.store.set_grad_scale(1.0 / (mesh.world_size * self.num_microbatches))

    def accumulate(self) -> bool:
        """Call after each micro-batch's backward.  Returns True when the optimizer step is due."""
        self.store.finish_backward()
        self.mini_step += 1
        return self.mini_step >= self.num_microbatches

    @property
    def learning_rate(self) -> float:
        return float(self.schedule(self.count))

    @property
    def tracks_grad_norm(self) -> bool:
        cfg = self.config
        return cfg.max_grad_norm is not None if cfg.track_grad_norm is None else bool(cfg.track_grad_norm)

    @property
    def grad_norm(self) -> Optional[torch.Tensor]:
        """Global gradient norm of the last step (device scalar; reading it synchronises); None when it is not
        computed (no clipping configured and ``track_grad_norm`` off)."""
        return self._coef[1] if self.tracks_grad_norm else None

    def step(self) -> None:
        cfg, st = self.config, self.store
        st.reduce_replicated_grads()
        lr = self.learning_rate
        self.last_lr = lr
        t = self.count + 1
        bc1 = 1.0 - cfg.b1 ** t
        bc2 = 1.0 - cfg.b2 ** t
        max_norm = float(cfg.max_grad_norm) if cfg.max_grad_norm is not None else 0.0
        decay_runs, nodecay_runs = st.decay_runs()
        if st.grad.is_cuda:
            gscale = None
            if self.tracks_grad_norm:
                self._sumsq.zero_()
                if st.mesh.tp.size > 1:
                    self._sumsq.copy_(st.global_grad_sumsq().double().view(1))
                else:
                    K.sumsq(st.grad, self._sumsq)
                    if st.mesh.shard.size > 1:
                        dist.all_reduce(self._sumsq, group=st.mesh.shard.pg)
                K.clip_coef(self._sumsq, max_norm, 1.0, self._coef)
                gscale = self._coef
            for runs, wd in ((decay_runs, cfg.weight_decay), (nodecay_runs, 0.0)):
                for s, e in runs:
                    K.adamw(st.master[s:e], self.exp_avg[s:e], self.exp_avg_sq[s:e], st.grad[s:e],
                            st.shadow[s:e] if st.shadow is not st.master else None, lr=lr, b1=cfg.b1, b2=cfg.b2,
                            eps=cfg.eps, wd=wd, bias_corr1=bc1, bias_corr2=bc2, gscale=gscale, zero_grad=True)
            st.invalidate_gathered()
            st.sync_peers()  # peers may read the new weights / add into the cleared accumulator only after this
        else:
            coef = 1.0
            if self.tracks_grad_norm:
                norm = st.global_grad_sumsq().sqrt()
                if max_norm > 0.0:
                    coef = max_norm / max(max_norm, float(norm))
                self._coef[0] = coef
                self._coef[1] = norm
            g = st.grad * coef if coef != 1.0 else st.grad
            self.exp_avg.mul_(cfg.b1).add_(g, alpha=1.0 - cfg.b1)
            self.exp_avg_sq.mul_(cfg.b2).addcmul_(g, g, value=1.0 - cfg.b2)
            update = (self.exp_avg / bc1) / ((self.exp_avg_sq / bc2).sqrt() + cfg.eps)
            for s, e in decay_runs:
                update[s:e].add_(st.master[s:e].float(), alpha=cfg.weight_decay)
            st.master.add_(update.to(st.master.dtype), alpha=-lr)
            st.zero_grad()
            st.sync_shadow()
        self.count += 1
        self.mini_step = 0

    # ------------------------------------------------------------------ state
    def state_dict(self) -> Dict[str, Any]:
        """Scalars plus the LOCAL shards of the moments (use ``ParamStore.full_tensor_like`` for logical tensors)."""
        return {
            "count": self.count,
            "mini_step": self.mini_step,
            "exp_avg": self.exp_avg,
            "exp_avg_sq": self.exp_avg_sq,
        }

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        self.count = int(state["count"])
        self.mini_step = int(state.get("mini_step", 0))
        self.exp_avg.copy_(state["exp_avg"])
        self.exp_avg_sq.copy_(state["exp_avg_sq"])

    def hyperparameters(self) -> Dict[str, float]:
        cfg = self.config
        return {"learning_rate": self.learning_rate, "b1": cfg.b1, "b2": cfg.b2, "eps": cfg.eps,
                "weight_decay": cfg.weight_decay}
