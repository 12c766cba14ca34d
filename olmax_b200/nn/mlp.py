"""Gated MLP (``olmax/nn/mlp.py:1-73``): ``down(act(gate(x)) * up(x))``; gate/up colwise and down rowwise under TP."""

from __future__ import annotations

import torch

from ..ops import functional as F
from ..parallel import collectives as coll
from ..parallel.mesh import TPStyle
from .linear import Linear
from .module import Module, current_build_context

__all__ = ["GatedMLP"]


class GatedMLP(Module):
    def __init__(self, d_model: int, hidden_size: int, bias: bool = False, activation: str = "silu", init_std: float = 0.02):
        super().__init__()
        if bias:
            raise ValueError("GatedMLP has no bias (the fused kernels and tensor parallelism do not support one)")
        ctx = current_build_context()
        self.activation = activation
        self.recompute = False
        """Set by the layer when the activation-checkpointing policy recomputes this block: only the block input is
        kept for backward and the gate/up GEMM runs again there."""
        with ctx.scope("gate_proj"):
            self.gate_proj = Linear(d_model, hidden_size, tp_style=TPStyle.colwise, init_std=init_std)
        with ctx.scope("up_proj"):
            self.up_proj = Linear(d_model, hidden_size, tp_style=TPStyle.colwise, init_std=init_std)
        with ctx.scope("down_proj"):
            self.down_proj = Linear(hidden_size, d_model, tp_style=TPStyle.rowwise, init_std=init_std)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        tp = self.mesh.tp
        tpc = self.store.tp_symm if x.is_cuda else None
        if tpc is not None:   # both tensor-parallel collectives are fused into the GEMMs of the block
            return F.gated_mlp(x, self.gate_proj.weight, self.up_proj.weight, self.down_proj.weight, self.activation, tpc,
                               recompute=self.recompute)
        x = coll.seq_all_gather(x, tp)
        y = F.gated_mlp(x, self.gate_proj.weight, self.up_proj.weight, self.down_proj.weight, self.activation,
                        recompute=self.recompute)
        return coll.seq_reduce_scatter(y, tp)
