"""
Differentiable ops of the transformer, as ``torch.autograd.Function``s over *activations*.  Weights are not autograd
leaves: an op receives a :class:`~olmax_b200.parallel.param_store.ParamHandle`, reads the gathered weight through
it and writes the weight gradient straight into the sharded fp32 accumulator (through the weight-gradient GEMM's
epilogue on the GPU).  This is what lets the FSDP all-gather / reduce-scatter be fused with, or overlapped around,
the GEMMs instead of being inferred by a compiler.

On CUDA tensors (bf16) every op launches the hand-written sm_100a kernels from :mod:`olmax_b200.ops.kernels`; on CPU
tensors it evaluates the PyTorch restatement in :mod:`olmax_b200.ops.reference` (backward through autograd of that
restatement), which is the path the gloo multi-process tests use.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import kernels as K
from ..parallel import collectives as coll
from . import reference as ref

__all__ = [
    "linear", "gated_mlp", "rms_norm", "layer_norm", "rope", "attention", "attention_block_fwd", "attention_block_bwd",
    "embedding", "linear_cross_entropy", "glu", "tp_column_linears", "tp_row_linear",
]


def _on_gpu(x: torch.Tensor) -> bool:
    if x.is_cuda:
        if x.dtype != torch.bfloat16:
            raise K.KernelError(f"the CUDA path computes in bf16; got {x.dtype}")
        return True
    return False


def _b_operand(handle):
    """(first piece, kwargs for an N-sharded K-major B) of a gathered weight."""
    first, stride = handle.pieces()
    R = handle.shard_count
    if R == 1:
        return first, {}
    return first, {"N_s": handle.rows_local, "b_shard_stride": stride}


def _ag_kwargs(handle, second=None, extra: Optional[dict] = None) -> dict:
    """GEMM arguments that fuse the FSDP all-gather of ``handle`` (and ``second``, the up-projection of a gated
    MLP) into the launch, when the peer-memory backend still has to fetch their remote shards.  A launch fuses one
    all-gather: when ``extra`` already carries the tensor-parallel gather of the activation rows, the weight's remote
    shards are fetched by the stand-alone plain-load kernel first (``ParamHandle.full``)."""
    if extra and "ag_src" in extra:
        handle.full()
        if second is not None:
            second.full()
        return {}
    ag = handle.take_ag()
    if ag is None:
        return {}
    table, flags, rank = ag
    out = {"ag_src": table, "ag_flags": flags, "ag_rank": rank}
    if second is not None:
        ag2 = second.take_ag()
        if ag2 is not None:
            out["ag_src2"] = ag2[0]
    return out


def _gemm_fwd(x2: torch.Tensor, handle, out: Optional[torch.Tensor] = None, epi: int = K.EPI_BF16,
              extra: Optional[dict] = None) -> torch.Tensor:
    """y[M, N] = x2[M, K] @ W[N, K]^T with W read from the gathered unit buffer.  ``extra``: more GEMM arguments
    (tensor-parallel all-gather of x2's rows, or reduce-scatter of the output rows; then ``out`` is only a placeholder)."""
    M, Kd = x2.shape
    N = handle.tp_shape[0]
    first, kw = _b_operand(handle)
    kw.update(_ag_kwargs(handle, extra=extra))
    kw["prefetch"] = handle.store.prefetch_slice(N * Kd)
    if extra:
        kw.update(extra)
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32 if epi == K.EPI_F32 else torch.bfloat16, device=x2.device)
    K.gemm(x2, first, out, M, N, Kd, epi=epi, ldb=Kd, ldc=N, **kw)
    return out


def _gemm_dgrad(dy2: torch.Tensor, handle, out: Optional[torch.Tensor] = None, accumulate: bool = False,
                extra: Optional[dict] = None) -> torch.Tensor:
    """dx[M, K] (+)= dy2[M, N] @ W[N, K], the contraction running over the weight's row shards.  With a reduce-scatter
    in ``extra`` (``c_shards``) the result leaves through the peers' staging slots: ``out`` is then the local partial
    sum that is folded in when ``accumulate`` is set (it is not written), or a placeholder."""
    M, N = dy2.shape
    Kd = handle.tp_shape[1]
    first, stride = handle.pieces()
    R = handle.shard_count
    kw = {} if R == 1 else {"Kc_s": handle.rows_local, "b_shard_stride": stride}
    kw.update(_ag_kwargs(handle, extra=extra))
    kw["prefetch"] = handle.store.prefetch_slice(N * Kd)
    if extra:
        kw.update(extra)
    if out is None:
        out = torch.empty((M, Kd), dtype=torch.bfloat16, device=dy2.device)
    K.gemm(dy2, first, out, M, Kd, N, b_mn=True, ldb=Kd, ldc=Kd, epi=K.EPI_BF16_ACC if accumulate else K.EPI_BF16, **kw)
    return out


def _gemm_wgrad(dy2: torch.Tensor, x2: torch.Tensor, handle) -> None:
    """dW[N, K] += scale * dy2[M, N]^T @ x2[M, K], written into the handle's gradient destination."""
    M, N = dy2.shape
    Kd = x2.shape[1]
    R = handle.shard_count
    symm = getattr(handle.store, "symm_rs", None)
    peer = symm.stage_pointer_table(handle) if (symm is not None and R > 1) else None
    pf = handle.store.prefetch_slice(N * Kd)
    if peer is not None:
        # reduce-scatter fused into the epilogue: row block r is STORED into this rank's slot of GPU r's staging buffer
        # (plain stores over NVLink, rank-staggered tile order); the owner folds the slots after the unit's barrier
        epi = K.EPI_BF16 if symm.wire_dtype == torch.bfloat16 else K.EPI_F32
        K.gemm(dy2, x2, handle.local_grad, N, Kd, M, a_mn=True, b_mn=True, epi=epi, alpha=1.0, ldc=Kd,
               M_s=handle.rows_local, c_shards=peer, prefetch=pf, m_shard_rot=handle.store.mesh.shard.rank)
        handle.unit._staged.add(handle.name)
    else:
        dst, gstride, scale = handle.grad_pieces()
        kw = {} if R == 1 else {"M_s": handle.rows_local, "c_shard_stride": gstride}
        K.gemm(dy2, x2, dst, N, Kd, M, a_mn=True, b_mn=True, epi=K.EPI_F32_ACC, alpha=scale, ldc=Kd, prefetch=pf, **kw)


# ----------------------------------------------------------------------------------------------------------------------
# Linear
# ----------------------------------------------------------------------------------------------------------------------
class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, handle, bias_handle):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        ctx.handle, ctx.bias_handle, ctx.shape = handle, bias_handle, shp
        if _on_gpu(x):
            x2 = x2.contiguous()
            y = _gemm_fwd(x2, handle)
            if bias_handle is not None:
                y = y + bias_handle.full()
        else:
            y = x2 @ handle.full().t()
            if bias_handle is not None:
                y = y + bias_handle.full()
        ctx.save_for_backward(x2)
        return y.view(*shp[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        handle = ctx.handle
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = None
        if _on_gpu(dy2):
            dy2 = dy2.contiguous()
            if ctx.needs_input_grad[0]:
                dx = _gemm_dgrad(dy2, handle)
            _gemm_wgrad(dy2, x2, handle)
        else:
            if ctx.needs_input_grad[0]:
                dx = dy2 @ handle.full()
            handle.add_grad(dy2.t() @ x2)
        if ctx.bias_handle is not None:
            ctx.bias_handle.add_grad(dy2.float().sum(0))
        return (dx.view(ctx.shape) if dx is not None else None), None, None


def linear(x: torch.Tensor, handle, bias_handle=None) -> torch.Tensor:
    """``x @ W^T (+ b)`` with W ``(out, in)`` (``olmax/nn/functional.py:14-27``)."""
    return _LinearFn.apply(x, handle, bias_handle)


# ----------------------------------------------------------------------------------------------------------------------
# Gated MLP: down(act(gate(x)) * up(x)) in one autograd node so that act(g)*u is never kept for backward
# ----------------------------------------------------------------------------------------------------------------------
class _GatedMLPFn(torch.autograd.Function):
    """``tpc`` (a ``TPSymmContext``; GPU only): x holds this rank's rows of the sequence-parallel activation; their
    all-gather is fused into the gate/up GEMM and the reduce-scatter of the output into the down GEMM's epilogue
    (forward), and symmetrically in backward (gather of dy into the down dgrad, reduce-scatter of dx out of the
    up dgrad, which folds in the gate dgrad's partial sum).

    ``recompute``: keep only the block's input for backward and run the gate/up GEMM again there (activation
    checkpointing of the block at the price of that one GEMM: the gate / up pre-activations, 2 x [tokens, hidden],
    are neither written in forward nor held until backward)."""

    @staticmethod
    def _gate_up(x2, gate, up, act, a, g, u, ag_kw):
        """a = act(x2 Wg^T) * (x2 Wu^T); g / u receive the two pre-activations when given."""
        M, d = x2.shape
        h = gate.tp_shape[0]
        gfirst, kw = _b_operand(gate)
        ufirst, _ = up.pieces()
        kw.update(_ag_kwargs(gate, up, extra=ag_kw))
        kw["prefetch"] = gate.store.prefetch_slice(2 * h * d)
        if ag_kw:
            kw.update(ag_kw)
        K.gemm(x2, gfirst, a, M, h, d, epi=K.EPI_GEGLU if act != "silu" else K.EPI_SWIGLU, b2=ufirst, c2=g, c3=u,
               ldb=d, **kw)

    @staticmethod
    def forward(ctx, x, gate, up, down, act, tpc=None, recompute=False):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        ctx.handles, ctx.act, ctx.shape, ctx.tpc, ctx.recompute = (gate, up, down), act, shp, tpc, recompute
        if _on_gpu(x):
            x2 = x2.contiguous()
            ag_kw = {}
            if tpc is not None:
                x2, ag_kw = tpc.gather_begin(x2)
            M, d = x2.shape
            h = gate.tp_shape[0]
            a = torch.empty((M, h), dtype=torch.bfloat16, device=x.device)
            g = u = None
            if not recompute:
                g = torch.empty_like(a)
                u = torch.empty_like(a)
            _GatedMLPFn._gate_up(x2, gate, up, act, a, g, u, ag_kw)
            # act(g) * u is never kept: backward gets it back from glu_bwd
            ctx.save_for_backward(*((x2,) if recompute else (x2, g, u)))
            if tpc is not None:
                M_s = M // tpc.n
                stage, rs_kw = tpc.rs_begin(M_s, d)
                _gemm_fwd(a, down, out=stage, extra=rs_kw)
                del a
                y = tpc.rs_finish(stage, M_s, d)
                return y.view(*shp[:-1], d)
            y = _gemm_fwd(a, down)
            del a
            return y.view(*shp[:-1], y.shape[-1])
        g = x2 @ gate.full().t()
        u = x2 @ up.full().t()
        a = ref.glu(g, u, act)
        ctx.save_for_backward(*((x2,) if recompute else (x2, g, u)))
        y = a @ down.full().t()
        return y.view(*shp[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        gate, up, down = ctx.handles
        dy2 = dy.reshape(-1, dy.shape[-1])
        tpc = ctx.tpc
        if ctx.recompute:
            (x2,) = ctx.saved_tensors
            g = u = None
        else:
            x2, g, u = ctx.saved_tensors
        if _on_gpu(dy2):
            dy2 = dy2.contiguous()
            ag_kw = None
            if tpc is not None:
                dy2, ag_kw = tpc.gather_begin(dy2)
            da = _gemm_dgrad(dy2, down, extra=ag_kw)
            a = torch.empty((x2.shape[0], gate.tp_shape[0]), dtype=torch.bfloat16, device=dy2.device)
            if ctx.recompute:   # the gate / up pre-activations again (x2 is already the gathered activation under TP)
                g = torch.empty_like(a)
                u = torch.empty_like(a)
                _GatedMLPFn._gate_up(x2, gate, up, ctx.act, a, g, u, None)
            dg = torch.empty_like(g)
            du = torch.empty_like(u)
            K.glu_bwd(g, u, da, dg, du, a, gelu=ctx.act != "silu")
            del da
            _gemm_wgrad(dy2, a, down)
            del a
            _gemm_wgrad(dg, x2, gate)
            _gemm_wgrad(du, x2, up)
            dx = None
            if ctx.needs_input_grad[0]:
                dx = _gemm_dgrad(dg, gate)
                if tpc is not None:
                    M_s, d = dx.shape[0] // tpc.n, dx.shape[1]
                    stage, rs_kw = tpc.rs_begin(M_s, d)
                    _gemm_dgrad(du, up, out=dx, accumulate=True, extra=rs_kw)   # stores dx + du.Wu to the row owners
                    dx = tpc.rs_finish(stage if rs_kw else dx, M_s, d)
                else:
                    _gemm_dgrad(du, up, out=dx, accumulate=True)
        else:
            if ctx.recompute:
                g = x2 @ gate.full().t()
                u = x2 @ up.full().t()
            with torch.enable_grad():
                gg = g.detach().requires_grad_(True)
                uu = u.detach().requires_grad_(True)
                a = ref.glu(gg, uu, ctx.act)
            da = dy2 @ down.full()
            dg, du = torch.autograd.grad(a, (gg, uu), da)
            down.add_grad(dy2.t() @ a.detach())
            gate.add_grad(dg.t() @ x2)
            up.add_grad(du.t() @ x2)
            dx = dg @ gate.full() + du @ up.full() if ctx.needs_input_grad[0] else None
        return (dx.view(ctx.shape) if dx is not None else None), None, None, None, None, None, None


def gated_mlp(x: torch.Tensor, gate, up, down, act: str = "silu", tpc=None, recompute: bool = False) -> torch.Tensor:
    """``down(act(gate(x)) * up(x))``.  With ``tpc`` x is this rank's row shard of a sequence-parallel activation and
    so is the result (the tensor-parallel collectives are fused into the GEMMs).  ``recompute``: hold only x for the
    backward pass and run the gate/up GEMM again there."""
    return _GatedMLPFn.apply(x, gate, up, down, act, tpc if x.is_cuda else None, bool(recompute) and torch.is_grad_enabled())


# ----------------------------------------------------------------------------------------------------------------------
# Tensor parallelism with sequence parallelism, collectives fused into the GEMMs (GPU, peer-memory context)
# ----------------------------------------------------------------------------------------------------------------------
class _TPColumnLinearsFn(torch.autograd.Function):
    """x_local [M/tp, d] -> (x_full @ W_i^T for every column-parallel weight i): the all-gather of x is fused into the
    first GEMM, the others read the gathered buffer.  Backward: the weight gradients use the gathered x; the input
    gradient sum_i dy_i W_i is accumulated locally and reduce-scattered out of the LAST dgrad GEMM's epilogue."""

    @staticmethod
    def forward(ctx, x_local, tpc, *handles):
        x_full, ag_kw = tpc.gather_begin(x_local.contiguous())
        ys = []
        for i, h in enumerate(handles):
            ys.append(_gemm_fwd(x_full, h, extra=ag_kw if i == 0 else None))
        ctx.tpc, ctx.handles = tpc, handles
        ctx.save_for_backward(x_full)
        return tuple(ys)

    @staticmethod
    def backward(ctx, *dys):
        (x_full,) = ctx.saved_tensors
        tpc, handles = ctx.tpc, ctx.handles
        dys = [dy.contiguous() for dy in dys]
        for dy, h in zip(dys, handles):
            _gemm_wgrad(dy, x_full, h)
        if not ctx.needs_input_grad[0]:
            return (None, None) + (None,) * len(handles)
        M, d = x_full.shape
        M_s = M // tpc.n
        partial = None
        for dy, h in zip(dys[:-1], handles[:-1]):
            partial = _gemm_dgrad(dy, h, out=partial, accumulate=partial is not None)
        stage, rs_kw = tpc.rs_begin(M_s, d)
        _gemm_dgrad(dys[-1], handles[-1], out=partial if partial is not None else stage,
                    accumulate=partial is not None, extra=rs_kw)
        # without the fused epilogue the sum sits in the local partial buffer and is reduce-scattered from there
        dx_local = tpc.rs_finish(stage if (rs_kw or partial is None) else partial, M_s, d)
        return (dx_local, None) + (None,) * len(handles)


class _TPRowLinearFn(torch.autograd.Function):
    """x [M, K/tp] -> this rank's rows [M/tp, N] of sum over the group of x W^T: the reduce-scatter is the GEMM's
    epilogue.  Backward: the all-gather of dy is fused into the dgrad GEMM; the weight gradient uses the gathered dy."""

    @staticmethod
    def forward(ctx, x, tpc, handle):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        M = x2.shape[0]
        N = handle.tp_shape[0]
        M_s = M // tpc.n
        stage, rs_kw = tpc.rs_begin(M_s, N)
        _gemm_fwd(x2, handle, out=stage, extra=rs_kw)
        y = tpc.rs_finish(stage, M_s, N)
        ctx.tpc, ctx.handle, ctx.shape = tpc, handle, x.shape
        ctx.save_for_backward(x2)
        return y

    @staticmethod
    def backward(ctx, dy_local):
        (x2,) = ctx.saved_tensors
        tpc, handle = ctx.tpc, ctx.handle
        dy_full, ag_kw = tpc.gather_begin(dy_local.contiguous())
        dx = _gemm_dgrad(dy_full, handle, extra=ag_kw) if ctx.needs_input_grad[0] else None
        if dx is None:   # nobody pulled the peers' rows: complete the gather with the copy kernel
            tpc.finish_gather(dy_full, ag_kw)
        _gemm_wgrad(dy_full, x2, handle)
        return (dx.view(ctx.shape) if dx is not None else None), None, None


def tp_column_linears(x_local: torch.Tensor, tpc, handles):
    """Column-parallel projections of a sequence-parallel activation with the all-gather fused into the first GEMM."""
    return _TPColumnLinearsFn.apply(x_local, tpc, *handles)


def tp_row_linear(x: torch.Tensor, tpc, handle) -> torch.Tensor:
    """Row-parallel projection whose partial sums are reduce-scattered over the TP group by the GEMM epilogue."""
    return _TPRowLinearFn.apply(x, tpc, handle)


def glu(g: torch.Tensor, u: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """Stand-alone ``act(g) * u`` (not differentiable through the kernels; use :func:`gated_mlp` in models)."""
    if _on_gpu(g):
        a = torch.empty_like(g)
        K.glu_fwd(g.contiguous(), u.contiguous(), a, gelu=act != "silu")
        return a
    return ref.glu(g, u, act)


# ----------------------------------------------------------------------------------------------------------------------
# RMSNorm (+ residual variants, + per-head mode)
# ----------------------------------------------------------------------------------------------------------------------
class _RMSNormFn(torch.autograd.Function):
    """
    mode None : y = norm(x) * w
    mode post : y = residual + norm(x) * w                      (OLMo2 / Gemma post-norms)
    mode pre  : h = x + residual ; y = norm(h) * w ; returns (h, y)   (pre-norm residual stream)
    """

    @staticmethod
    def forward(ctx, x, residual, handle, eps, mode, heads):
        shp = x.shape
        w = handle.full()
        d = w.numel()
        ctx.handle, ctx.mode, ctx.heads, ctx.eps, ctx.shape = handle, mode, heads, eps, shp
        if _on_gpu(x):
            xc = x.contiguous()
            rows = xc.numel() // d
            y = torch.empty_like(xc)
            rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
            ld = d * heads if heads > 1 else d
            if mode == "pre":
                h = torch.empty_like(xc)
                K.rmsnorm_fwd(xc, w, y, rows=rows, d=d, eps=eps, res=residual.contiguous(), sum_out=h, rstd=rstd,
                              heads=heads, ld_x=ld, ld_res=ld, ld_y=ld, add_before=True)
                ctx.save_for_backward(h, w, rstd)
                return h, y
            res = residual.contiguous() if mode == "post" else None
            K.rmsnorm_fwd(xc, w, y, rows=rows, d=d, eps=eps, res=res, rstd=rstd, heads=heads, ld_x=ld, ld_res=ld, ld_y=ld)
            ctx.save_for_backward(xc, w, rstd)
            return y
        # CPU
        xin = x + residual if mode == "pre" else x
        xv = xin.reshape(-1, d) if heads == 1 else xin.reshape(-1, heads, d)
        y = ref.rms_norm(xv, w, eps).reshape(shp)
        ctx.save_for_backward(xin, w)
        if mode == "pre":
            return xin, y
        if mode == "post":
            return residual + y
        return y

    @staticmethod
    def backward(ctx, *grads):
        handle, mode, heads, eps, shp = ctx.handle, ctx.mode, ctx.heads, ctx.eps, ctx.shape
        if mode == "pre":
            dh, dy = grads
        else:
            (dy,) = grads
            dh = None
        saved = ctx.saved_tensors
        w = saved[1]
        d = w.numel()
        if _on_gpu(dy):
            xin, _, rstd = saved
            dyc = dy.contiguous()
            rows = dyc.numel() // d
            dx = torch.empty_like(dyc)
            ld = d * heads if heads > 1 else d
            R = handle.shard_count
            direct = R == 1 and getattr(handle.store, "symm_rs", None) is None
            if direct:
                dw, dw_scale = handle.local_grad, handle.store.grad_scale
            else:
                dw, dw_scale = torch.zeros(d, dtype=torch.float32, device=dy.device), 1.0
            K.rmsnorm_bwd(dyc, xin, w, rstd, dx, rows=rows, d=d, dw=dw, dsum=dh.contiguous() if dh is not None else None,
                          heads=heads, ld_dy=ld, ld_x=ld, ld_dx=ld, dw_scale=dw_scale)
            if not direct:
                handle.add_grad(dw)
        else:
            xin = saved[0]
            with torch.enable_grad():
                xx = xin.detach().requires_grad_(True)
                ww = w.detach().requires_grad_(True)
                xv = xx.reshape(-1, d) if heads == 1 else xx.reshape(-1, heads, d)
                y = ref.rms_norm(xv, ww, eps).reshape(shp)
            dx, dw = torch.autograd.grad(y, (xx, ww), dy)
            handle.add_grad(dw)
            if dh is not None:
                dx = dx + dh
        dx = dx.view(shp)
        if mode == "pre":
            return dx, dx, None, None, None, None
        if mode == "post":
            return dx, dy, None, None, None, None
        return dx, None, None, None, None, None


def rms_norm(x: torch.Tensor, handle, eps: float = 1e-5, residual: Optional[torch.Tensor] = None,
             mode: Optional[str] = None, heads: int = 1):
    """See :class:`_RMSNormFn`.  ``heads > 1`` normalises every ``d``-wide head of the last dimension separately."""
    if mode is None:
        residual = None
    return _RMSNormFn.apply(x, residual, handle, eps, mode, heads)


class _LayerNormFn(torch.autograd.Function):
    """y = (x - mean) * rstd * w (+ b) over the last dimension (``olmax/nn/functional.py:30-49``)."""

    @staticmethod
    def forward(ctx, x, w_handle, b_handle, eps):
        shp = x.shape
        d = shp[-1]
        w = w_handle.full() if w_handle is not None else None
        b = b_handle.full() if b_handle is not None else None
        ctx.handles, ctx.eps, ctx.shape = (w_handle, b_handle), eps, shp
        if _on_gpu(x):
            xc = x.contiguous()
            rows = xc.numel() // d
            y = torch.empty_like(xc)
            mean = torch.empty(rows, dtype=torch.float32, device=x.device)
            rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
            K.layernorm_fwd(xc, w, b, y, mean, rstd, rows=rows, d=d, eps=eps)
            ctx.save_for_backward(xc, mean, rstd, *([w] if w is not None else []))
            return y
        ctx.save_for_backward(x, *([w] if w is not None else []), *([b] if b is not None else []))
        return ref.layer_norm(x, w, b, eps)

    @staticmethod
    def backward(ctx, dy):
        w_handle, b_handle = ctx.handles
        d = ctx.shape[-1]
        if _on_gpu(dy):
            x, mean, rstd = ctx.saved_tensors[:3]
            w = ctx.saved_tensors[3] if w_handle is not None else None
            dyc = dy.contiguous()
            rows = dyc.numel() // d
            dx = torch.empty_like(dyc)
            dw = torch.zeros(d, dtype=torch.float32, device=dy.device) if w_handle is not None else None
            db = torch.zeros(d, dtype=torch.float32, device=dy.device) if b_handle is not None else None
            K.layernorm_bwd(dyc, x, w, mean, rstd, dx, rows=rows, d=d, dw=dw, db=db)
            if dw is not None:
                w_handle.add_grad(dw)
            if db is not None:
                b_handle.add_grad(db)
            return dx.view(ctx.shape), None, None, None
        saved = list(ctx.saved_tensors)
        x = saved.pop(0)
        with torch.enable_grad():
            xx = x.detach().requires_grad_(True)
            ww = saved.pop(0).detach().requires_grad_(True) if w_handle is not None else None
            bb = saved.pop(0).detach().requires_grad_(True) if b_handle is not None else None
            y = ref.layer_norm(xx, ww, bb, ctx.eps)
        leaves = [t for t in (xx, ww, bb) if t is not None]
        grads = list(torch.autograd.grad(y, leaves, dy))
        dx = grads.pop(0)
        if ww is not None:
            w_handle.add_grad(grads.pop(0))
        if bb is not None:
            b_handle.add_grad(grads.pop(0))
        return dx, None, None, None


def layer_norm(x: torch.Tensor, weight, bias, eps: float = 1e-5, residual: Optional[torch.Tensor] = None,
               mode: Optional[str] = None, heads: int = 1):
    """LayerNorm with the calling convention of :func:`rms_norm`: ``mode`` None: norm(x); ``post``: residual + norm(x);
    ``pre``: returns (x + residual, norm(x + residual)).  ``heads > 1`` normalises every head separately.  The residual
    adds are ordinary tensor ops (no recipe uses LayerNorm on the residual stream)."""
    if mode == "pre":
        x = x + residual
    shp = x.shape
    xv = x.reshape(-1, shp[-1] // heads) if heads > 1 else x
    y = _LayerNormFn.apply(xv, weight, bias, eps).reshape(shp)
    if mode == "pre":
        return x, y
    if mode == "post":
        return residual + y
    return y


# ----------------------------------------------------------------------------------------------------------------------
# RoPE
# ----------------------------------------------------------------------------------------------------------------------
class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        ctx.save_for_backward(cos, sin)
        if _on_gpu(x):
            y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
            K.rope(x, y, cos, sin, sign=1.0)
            return y
        return ref.apply_rope(x, cos, sin, 1.0)

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        if _on_gpu(dy):
            dyc = dy if dy.stride(-1) == 1 else dy.contiguous()
            dx = torch.empty(dy.shape, dtype=dy.dtype, device=dy.device)
            K.rope(dyc, dx, cos, sin, sign=-1.0)
            return dx, None, None
        return ref.apply_rope(dy, cos, sin, -1.0), None, None


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [B, S, H, D]; cos/sin fp32 [>= S, D/2]."""
    return _RopeFn.apply(x, cos, sin)


class _RMSNormRopeFn(torch.autograd.Function):
    """``rope(rms_norm(x) * w)`` for the q / k projections in one kernel per direction: x ``[B * S, n * hd]`` ->
    ``[B, S, n, hd]``.  ``heads`` = 1 normalises the whole projection, ``heads`` = n every head separately."""

    @staticmethod
    def forward(ctx, x, handle, eps, heads, cos, sin, batch, hd):
        w = handle.full()
        d = w.numel()
        T, width = x.shape
        S = T // batch
        ctx.handle, ctx.cfg = handle, (eps, heads, batch, hd, d, S)
        if _on_gpu(x):
            xc = x.contiguous()
            rows = T * heads
            y = torch.empty_like(xc)
            rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
            K.rmsnorm_rope_fwd(xc, w, y, rstd, cos, sin, rows=rows, d=d, hd=hd, heads=heads, seq_len=S, eps=eps,
                               ld_x=width, ld_y=width)
            ctx.save_for_backward(xc, w, rstd, cos, sin)
            return y.view(batch, S, width // hd, hd)
        xv = x.reshape(-1, d) if heads == 1 else x.reshape(-1, heads, d)
        y = ref.rms_norm(xv, w, eps).reshape(batch, S, width // hd, hd)
        ctx.save_for_backward(x, w, cos, sin)
        return ref.apply_rope(y, cos, sin, 1.0)

    @staticmethod
    def backward(ctx, dy):
        handle = ctx.handle
        eps, heads, batch, hd, d, S = ctx.cfg
        if _on_gpu(dy):
            xc, w, rstd, cos, sin = ctx.saved_tensors
            T, width = xc.shape
            dyc = dy.contiguous().view(T, width)
            dx = torch.empty_like(xc)
            direct = handle.shard_count == 1 and getattr(handle.store, "symm_rs", None) is None
            if direct:
                dw, dw_scale = handle.local_grad, handle.store.grad_scale
            else:
                dw, dw_scale = torch.zeros(d, dtype=torch.float32, device=dy.device), 1.0
            K.rmsnorm_rope_bwd(dyc, xc, w, rstd, dx, cos, sin, rows=T * heads, d=d, hd=hd, heads=heads, seq_len=S, dw=dw,
                               dw_scale=dw_scale, ld_dy=width, ld_x=width, ld_dx=width)
            if not direct:
                handle.add_grad(dw)
            return dx, None, None, None, None, None, None, None
        x, w, cos, sin = ctx.saved_tensors
        with torch.enable_grad():
            xx = x.detach().requires_grad_(True)
            ww = w.detach().requires_grad_(True)
            xv = xx.reshape(-1, d) if heads == 1 else xx.reshape(-1, heads, d)
            y = ref.apply_rope(ref.rms_norm(xv, ww, eps).reshape(dy.shape), cos, sin, 1.0)
        dx, dw = torch.autograd.grad(y, (xx, ww), dy)
        handle.add_grad(dw)
        return dx, None, None, None, None, None, None, None


def rms_norm_rope(x: torch.Tensor, handle, eps: float, heads: int, cos: torch.Tensor, sin: torch.Tensor, batch: int,
                  head_dim: int) -> torch.Tensor:
    """See :class:`_RMSNormRopeFn` (the q_norm / k_norm + rotary sequence of ``olmax/nn/attention.py:270-300``)."""
    return _RMSNormRopeFn.apply(x, handle, eps, heads, cos, sin, batch, head_dim)


# ----------------------------------------------------------------------------------------------------------------------
# Attention
# ----------------------------------------------------------------------------------------------------------------------
class _AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, window, softcap, scale):
        ctx.cfg = (causal, window, softcap, scale)
        if _on_gpu(q):
            o, lse = K.flash_attn_fwd(q, k, v, causal=causal, window=window, softcap=softcap, scale=scale)
            ctx.save_for_backward(q, k, v, o, lse)
            return o
        o, _ = ref.attention(q, k, v, causal, window, softcap, scale)
        ctx.save_for_backward(q, k, v)
        return o

    @staticmethod
    def backward(ctx, d_o):
        causal, window, softcap, scale = ctx.cfg
        if _on_gpu(d_o):
            q, k, v, o, lse = ctx.saved_tensors
            d_o = d_o if d_o.stride(-1) == 1 else d_o.contiguous()
            dq, dk, dv = K.flash_attn_bwd(q, k, v, o, lse, d_o, causal=causal, window=window, softcap=softcap, scale=scale)
            return dq, dk, dv, None, None, None, None
        q, k, v = ctx.saved_tensors
        with torch.enable_grad():
            qq, kk, vv = (t.detach().requires_grad_(True) for t in (q, k, v))
            o, _ = ref.attention(qq, kk, vv, causal, window, softcap, scale)
        dq, dk, dv = torch.autograd.grad(o, (qq, kk, vv), d_o)
        return dq, dk, dv, None, None, None, None


def attention(q, k, v, causal: bool = True, window: int = -1, softcap: float = 0.0, scale: Optional[float] = None):
    """q [B,S,H,D], k/v [B,S,Hkv,D] -> [B,S,H,D]."""
    return _AttentionFn.apply(q, k, v, causal, window if window is not None else -1, softcap or 0.0, scale)


class _RecomputedAttentionFn(torch.autograd.Function):
    """The q / k / v projections (with their norm and rotation) and the attention as ONE autograd node that keeps only
    the block input, the attention output and its row statistics.  Backward runs the projections again to get q, k, v
    (their own nodes then take the weight gradients as usual), but neither the attention forward nor anything after
    it.  This is what the activation-checkpointing policies that name ``layers.*.attention`` select
    (``olmax/activation_checkpointing.py:19-182``); a plain checkpoint of the block would also repeat the attention
    forward and the output projection."""

    @staticmethod
    def forward(ctx, x, qkv_fn, window, softcap, scale):
        with torch.no_grad():
            q, k, v = qkv_fn(x)
            o, lse = attention_block_fwd(q, k, v, window=window, softcap=softcap, scale=scale)
        ctx.qkv_fn, ctx.cfg = qkv_fn, (window, softcap, scale)
        ctx.save_for_backward(x, o, lse)
        return o

    @staticmethod
    def backward(ctx, d_o):
        x, o, lse = ctx.saved_tensors
        window, softcap, scale = ctx.cfg
        with torch.enable_grad():
            xd = x.detach().requires_grad_(True)
            q, k, v = ctx.qkv_fn(xd)
        dq, dk, dv = attention_block_bwd(q.detach(), k.detach(), v.detach(), o, lse, d_o, window=window, softcap=softcap,
                                         scale=scale)
        torch.autograd.backward([q, k, v], [dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)])
        return xd.grad, None, None, None, None


def recomputed_attention(x: torch.Tensor, qkv_fn, window: int = -1, softcap: float = 0.0,
                         scale: Optional[float] = None) -> torch.Tensor:
    """``attention(*qkv_fn(x))`` (causal) keeping only x, the output and the row statistics for the backward pass; see
    :class:`_RecomputedAttentionFn`.  ``qkv_fn`` maps the block input to (q [B,S,H,D], k, v [B,S,Hkv,D])."""
    return _RecomputedAttentionFn.apply(x, qkv_fn, window if window is not None else -1, softcap or 0.0, scale)


def attention_block_fwd(q, k, v, *, q_off: int = 0, causal: bool = True, window: int = -1, softcap: float = 0.0,
                        scale: Optional[float] = None):
    """One (query block, key block) pair without autograd: q [B,S,H,D], k/v [B,Sk,Hkv,D], query row i at key-axis
    position ``q_off + i`` -> (o [B,S,H,D], lse [B,H,S] fp32).  Building block of context-parallel attention."""
    if _on_gpu(q):
        return K.flash_attn_fwd(q, k, v, causal=causal, window=window, softcap=softcap, scale=scale, q_off=q_off)
    return ref.attention(q, k, v, causal, window, softcap, scale, q_off=q_off)


def attention_block_bwd(q, k, v, o, lse, d_o, *, q_off: int = 0, causal: bool = True, window: int = -1,
                        softcap: float = 0.0, scale: Optional[float] = None):
    """Gradients (dq, dk, dv) of one block pair given the row statistics ``lse`` and the output ``o`` of the WHOLE
    softmax row (so the blocks of a ring add up to the full gradient)."""
    if _on_gpu(q):
        d_o = d_o if d_o.stride(-1) == 1 else d_o.contiguous()
        return K.flash_attn_bwd(q, k, v, o, lse, d_o, causal=causal, window=window, softcap=softcap, scale=scale,
                                q_off=q_off)
    return ref.attention_bwd(q, k, v, o, lse, d_o, causal, window, softcap, scale, q_off=q_off)


# ----------------------------------------------------------------------------------------------------------------------
# Embedding
# ----------------------------------------------------------------------------------------------------------------------
_PTR_CACHE: dict = {}


def _piece_pointer_table(first: torch.Tensor, stride: int, R: int) -> torch.Tensor:
    key = (first.data_ptr(), stride, R, first.device.index)
    t = _PTR_CACHE.get(key)
    if t is None:
        es = first.element_size()
        t = K.pointer_table([first.data_ptr() + r * stride * es for r in range(R)], first.device)
        if len(_PTR_CACHE) > 256:
            _PTR_CACHE.clear()
        _PTR_CACHE[key] = t
    return t


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, handle, scale, anchor):
        ctx.handle, ctx.scale = handle, scale
        ctx.save_for_backward(ids)
        d = handle.tp_shape[1]
        if ids.is_cuda:
            R = handle.shard_count
            symm = getattr(handle.store, "symm_ag", None)
            if symm is not None and R > 1:
                table = symm.shadow_pointer_table(handle)   # rows are read from the GPU that owns them
            else:
                first, stride = handle.pieces()
                table = _piece_pointer_table(first, stride, R)
            out = torch.empty(ids.shape + (d,), dtype=torch.bfloat16, device=ids.device)
            K.embed_gather(ids.contiguous(), table, handle.rows_local, R, out, d, scale)
            return out
        w = handle.full()
        out = w[ids]
        return out * scale if scale != 1.0 else out

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        handle = ctx.handle
        d = handle.tp_shape[1]
        if dout.is_cuda:
            R = handle.shard_count
            symm = getattr(handle.store, "symm_rs", None)
            if symm is not None and R > 1:
                table, gscale = symm.grad_pointer_table(handle), handle.store.grad_scale
            else:
                dst, gstride, gscale = handle.grad_pieces()
                table = _piece_pointer_table(dst, gstride, R)
            K.embed_scatter(ids.contiguous(), table, handle.rows_local, R, dout.contiguous(), d, ctx.scale * gscale)
        else:
            g = torch.zeros(handle.tp_shape, dtype=torch.float32, device=dout.device)
            g.index_add_(0, ids.reshape(-1), dout.reshape(-1, d).float() * ctx.scale)
            handle.add_grad(g)
        return None, None, None, None


def embedding(ids: torch.Tensor, handle, scale: float = 1.0, anchor: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row gather ``W[ids] * scale`` (``olmax/nn/embedding.py:30-32``).  ``anchor`` is any tensor that requires grad;
    passing it makes the output part of the autograd graph although ids and weights are not autograd leaves."""
    return _EmbeddingFn.apply(ids, handle, float(scale), anchor)


# ----------------------------------------------------------------------------------------------------------------------
# LM head + cross entropy, never materialising [tokens, vocab] logits for the whole micro-batch
# ----------------------------------------------------------------------------------------------------------------------
class _LinearCrossEntropyFn(torch.autograd.Function):
    """
    loss = mean over counted tokens of CE(x @ W^T, labels) (+ z-loss).  The gradient w.r.t. x and W is computed during
    the forward pass, one chunk of rows at a time (logits chunk -> soft-max statistics -> d logits -> two GEMMs), so
    only ``chunk_rows x vocab`` logits exist at any time.  The weight gradient is accumulated immediately, therefore
    the returned loss must be back-propagated with a unit gradient (what ``loss.backward()`` does).
    """

    @staticmethod
    def forward(ctx, x, handle, labels, ignore_index, softcap, z_loss, chunk_rows):
        shp = x.shape
        d = shp[-1]
        x2 = x.reshape(-1, d)
        lab = labels.reshape(-1)
        V = handle.tp_shape[0]
        need_grad = bool(ctx.needs_input_grad[0])
        if _on_gpu(x):
            x2 = x2.contiguous()
            lab = lab.contiguous()
            M = x2.shape[0]
            dev = x.device
            stats = torch.zeros(2, dtype=torch.float32, device=dev)
            inv = torch.empty(2, dtype=torch.float32, device=dev)
            counter = torch.zeros(2, dtype=torch.int32, device=dev)
            K.count_valid(lab, ignore_index, V, inv, counter)
            dx = torch.empty_like(x2) if need_grad else None
            rc = min(chunk_rows, M)
            logits = torch.empty((rc, V), dtype=torch.float32, device=dev)
            # The store-based reduce-scatter of the peer-memory backend cannot accumulate several partial weight
            # gradients into a staging slot, so there d(logits) is kept for all rows and ONE weight-gradient GEMM runs at
            # the end; otherwise each chunk's weight gradient is accumulated right away and its d(logits) dropped.
            single_wgrad = need_grad and getattr(handle.store, "symm_rs", None) is not None and handle.shard_count > 1
            drows = M if single_wgrad else rc
            dlogits = torch.empty((drows, V), dtype=torch.bfloat16, device=dev) if need_grad else None
            for r0 in range(0, M, rc):
                r1 = min(M, r0 + rc)
                n = r1 - r0
                xc = x2[r0:r1]
                dl = (dlogits[r0:r1] if single_wgrad else dlogits[:n]) if need_grad else None
                _gemm_fwd(xc, handle, out=logits[:n], epi=K.EPI_F32)
                K.ce_fwd_bwd(logits[:n], lab[r0:r1], dl, stats, inv, V=V, ignore_index=ignore_index, softcap=softcap,
                             z_loss=z_loss)
                if need_grad:
                    _gemm_dgrad(dl, handle, out=dx[r0:r1])
                    if not single_wgrad:
                        _gemm_wgrad(dl, xc, handle)
            if single_wgrad:
                _gemm_wgrad(dlogits, x2, handle)
                # This weight gradient is staged during the FORWARD pass.  Its unit (the head, or the embedding for a
                # tied head) is folded now rather than in backward order, so that no layer's weight gradients can land
                # in the same staging buffer before it has been folded.
                handle.store.reduce_unit_now(handle.unit)
            loss = stats[0] * inv[0]
            zl = stats[1] * inv[0] * z_loss
            ctx.save_for_backward(dx if need_grad else torch.empty(0))
            ctx.shape = shp
            ctx.mark_non_differentiable(zl)
            return loss + zl if z_loss else loss, zl
        # CPU: autograd through the restatement
        w = handle.full()
        with torch.enable_grad():
            xx = x2.detach().requires_grad_(need_grad)
            ww = w.detach().requires_grad_(need_grad)
            logits = (xx @ ww.t()).float()
            loss, zl = ref.fused_cross_entropy(logits, lab, ignore_index=ignore_index, z_loss_multiplier=z_loss,
                                               logit_softcap=softcap)
            total = loss + zl if z_loss else loss
        if need_grad:
            dx, dw = torch.autograd.grad(total, (xx, ww))
            handle.add_grad(dw)
            ctx.save_for_backward(dx)
        else:
            ctx.save_for_backward(torch.empty(0))
        ctx.shape = shp
        zl = zl.detach()
        ctx.mark_non_differentiable(zl)
        return total.detach(), zl

    @staticmethod
    def backward(ctx, dloss, _dz):
        (dx,) = ctx.saved_tensors
        # dloss is 1 for loss.backward(); the weight gradient was already accumulated under that assumption
        return dx.view(ctx.shape) * dloss.to(dx.dtype), None, None, None, None, None, None


class _VocabParallelLinearCrossEntropyFn(torch.autograd.Function):
    """
    LM head + cross entropy with the VOCABULARY split over a tensor-parallel group (north-star "fused vocab-parallel
    cross-entropy"; replaces ``olmax/nn/lm_head.py:59-61`` + ``olmax/nn/functional.py:94-121``).  Every member owns
    ``V / n`` rows of the head weight.  ``x`` holds this member's rows of the sequence-parallel activation; the rows
    of all members are gathered, each member computes the logits of ITS vocabulary slice for all of them (a chunk of
    rows at a time), the per-row softmax statistics of the slices (max, sum-exp, target logit) are exchanged and
    combined (on the GPU: written to peer-mapped buffers, one bounded flag barrier, then every member's gradient
    kernel reads all members' statistics with plain loads), and the input gradient leaves through a reduce-scatter
    over the group.  No member ever holds logits or logit gradients for more than ``chunk_rows x V / n`` entries and
    the head's weight gradient needs no reduction over the group.  A row is normalised by the number of counted labels
    of the member it came from, so every member reports the mean loss of its own tokens, as without vocabulary
    parallelism.  Like :class:`_LinearCrossEntropyFn` the weight gradient is accumulated in forward (unit upstream
    gradient assumed).
    """

    @staticmethod
    def forward(ctx, x, handle, labels, ignore_index, softcap, z_loss, chunk_rows, group, tpc):
        shp = x.shape
        d = shp[-1]
        x2 = x.reshape(-1, d).contiguous()
        lab = labels.reshape(-1).contiguous()
        n, me = group.size, group.rank
        M_l = x2.shape[0]
        M = n * M_l
        V_l = handle.tp_shape[0]
        V, voff = V_l * n, me * V_l
        need_grad = bool(ctx.needs_input_grad[0])
        dev = x.device
        counts = (lab != ignore_index).sum().to(torch.float32).clamp(min=1).view(1)
        inv_counts = 1.0 / coll.all_gather(counts, group, dim=0)              # [n]
        x_full = coll.all_gather(x2, group, dim=0)                            # [M, d]
        lab_full = coll.all_gather(lab, group, dim=0)                         # [M]
        rc = min(chunk_rows, M)
        dx_full = torch.empty((M, d), dtype=x2.dtype, device=dev) if need_grad else None
        if _on_gpu(x):
            loss_sums = torch.zeros(2, dtype=torch.float32, device=dev)
            logits = torch.empty((rc, V_l), dtype=torch.float32, device=dev)
            single_wgrad = need_grad and getattr(handle.store, "symm_rs", None) is not None and handle.shard_count > 1
            dlogits = torch.empty((M if single_wgrad else rc, V_l), dtype=torch.bfloat16, device=dev) if need_grad else None
            for ci, r0 in enumerate(range(0, M, rc)):
                r1 = min(M, r0 + rc)
                rows = r1 - r0
                xc = x_full[r0:r1]
                _gemm_fwd(xc, handle, out=logits[:rows], epi=K.EPI_F32)
                if tpc is not None:
                    stats, table = tpc.stats_buffer(rc * 4, ci)
                    K.ce_vp_stats(logits[:rows], lab_full[r0:r1], stats, V=V_l, vocab_offset=voff, softcap=softcap)
                    tpc.barrier()    # every member's statistics of this chunk are in its buffer
                else:
                    mine = torch.empty(rc * 4, dtype=torch.float32, device=dev)
                    K.ce_vp_stats(logits[:rows], lab_full[r0:r1], mine, V=V_l, vocab_offset=voff, softcap=softcap)
                    gathered = coll.all_gather(mine.view(1, -1), group, dim=0)          # [n, rc * 4]
                    table = K.pointer_table([gathered[r].data_ptr() for r in range(n)], dev)
                dl = (dlogits[r0:r1] if single_wgrad else dlogits[:rows]) if need_grad else None
                K.ce_vp_grad(logits[:rows], lab_full[r0:r1], dl, table, n, inv_counts, loss_sums, V=V_l, vocab_offset=voff,
                             V_total=V, rows_per_src=M_l, row0=r0, my_src=me, ignore_index=ignore_index, softcap=softcap,
                             z_loss=z_loss)
                if need_grad:
                    _gemm_dgrad(dl, handle, out=dx_full[r0:r1])
                    if not single_wgrad:
                        _gemm_wgrad(dl, xc, handle)
            if single_wgrad:
                _gemm_wgrad(dlogits, x_full, handle)
                handle.store.reduce_unit_now(handle.unit)
            loss = loss_sums[0] * inv_counts[me]
            zl = loss_sums[1] * inv_counts[me] * z_loss
        else:
            w = handle.full().float()                                          # [V_l, d]
            z = ref.softcap(x_full.float() @ w.t(), softcap)                    # [M, V_l]
            m = z.max(dim=-1).values
            mg = m.clone()
            dist.all_reduce(mg, op=dist.ReduceOp.MAX, group=group.pg)
            ssum = (z - mg[:, None]).exp().sum(-1)
            local = lab_full - voff
            here = (local >= 0) & (local < V_l)
            t = torch.where(here, z.gather(1, local.clamp(0, V_l - 1)[:, None])[:, 0], torch.zeros_like(m))
            packed = torch.stack([ssum, t])
            dist.all_reduce(packed, group=group.pg)
            lse = mg + packed[0].log()
            counted = lab_full != ignore_index
            in_range = counted & (lab_full >= 0) & (lab_full < V)
            src = torch.arange(M, device=dev) // M_l
            w_row = inv_counts[src]
            mine = src == me
            loss = (torch.where(in_range & mine, lse - packed[1], torch.zeros_like(lse))).sum() * inv_counts[me]
            zl = torch.where(counted & mine, lse.pow(2), torch.zeros_like(lse)).sum() * inv_counts[me] * z_loss
            if need_grad:
                gs = torch.where(in_range, w_row, torch.zeros_like(w_row))
                gz = torch.where(counted, w_row * 2.0 * z_loss * lse, torch.zeros_like(w_row))
                g = (z - lse[:, None]).exp() * (gs + gz)[:, None]
                onehot_rows = here & in_range
                g[onehot_rows, local[onehot_rows]] -= gs[onehot_rows]
                if softcap:
                    raw = x_full.float() @ w.t()
                    g = g * (1.0 - torch.tanh(raw / softcap).pow(2))
                dx_full = (g @ w).to(x2.dtype)
                handle.add_grad(g.t() @ x_full.float())
        if need_grad:
            dx_local = coll.reduce_scatter(dx_full.contiguous(), group, dim=0)
            ctx.save_for_backward(dx_local)
        else:
            ctx.save_for_backward(torch.empty(0))
        ctx.shape = shp
        zl = zl.detach()
        ctx.mark_non_differentiable(zl)
        return (loss + zl if z_loss else loss).detach(), zl

    @staticmethod
    def backward(ctx, dloss, _dz):
        (dx,) = ctx.saved_tensors
        return dx.view(ctx.shape) * dloss.to(dx.dtype), None, None, None, None, None, None, None, None


def vocab_parallel_linear_cross_entropy(x: torch.Tensor, handle, labels: torch.Tensor, group, tpc=None,
                                        ignore_index: int = -100, logit_softcap: float = 0.0,
                                        z_loss_multiplier: float = 0.0, chunk_rows: int = 2048):
    """(loss, z_loss) with the head weight ``handle`` split over ``group`` along the vocabulary (``tp_dim = 0``); ``x`` and
    ``labels`` are this member's rows of the sequence-parallel batch.  ``tpc``: the group's ``TPSymmContext`` (GPU)."""
    return _VocabParallelLinearCrossEntropyFn.apply(x, handle, labels, ignore_index, float(logit_softcap or 0.0),
                                                    float(z_loss_multiplier or 0.0), int(chunk_rows), group, tpc)


def linear_cross_entropy(x: torch.Tensor, handle, labels: torch.Tensor, ignore_index: int = -100,
                         logit_softcap: float = 0.0, z_loss_multiplier: float = 0.0, chunk_rows: int = 2048):
    """(loss, z_loss) of the LM head fused with the cross entropy; ``handle`` is the ``(vocab, d)`` head weight."""
    return _LinearCrossEntropyFn.apply(x, handle, labels, ignore_index, float(logit_softcap or 0.0),
                                       float(z_loss_multiplier or 0.0), int(chunk_rows))
