"""
Library arm of the benchmark (``bench.py --impl torchlib``): the same architecture and the same training step as the
benchmarked recipe, built only from library code, for a same-box comparison of this repository's kernels against what
PyTorch ships:

* GEMMs: ``torch.nn.functional.linear`` (cuBLAS / cuBLASLt),
* attention: ``torch.nn.functional.scaled_dot_product_attention`` (its flash / cuDNN back-ends); a model with an
  attention soft-cap or a sliding window uses ``flash_attn.flash_attn_func`` instead, when that package works on the
  device,
* parameter sharding, all-gather and reduce-scatter: ``torch.distributed.fsdp.fully_shard`` over NCCL with bf16
  parameters for compute and fp32 gradient reduction, the fp32 master weights and AdamW state sharded the same way,
* optimizer: ``torch.optim.AdamW(fused=True)``.

None of this repository's kernels, models or engine is on this path and no kernel here is ever given another GPU's
memory.  It is NOT the reference (which is JAX): ``bench.py --impl reference`` stays a separate arm.  The JSON line has
the format of the main arm with ``"impl": "torchlib"``.
"""

from __future__ import annotations

import json
import math
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _unavailable(why: str) -> int:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "torchlib", "unavailable": why}), flush=True)
    return 0


def build_model(cfg, device, checkpoint_blocks: bool):
    """A plain ``torch.nn`` decoder with the structure of ``cfg`` (a ``TransformerConfig`` of this repository, used
    only as a description of the architecture)."""
    import torch
    import torch.nn as nn
    import torch.nn.functional as F
    from torch.utils.checkpoint import checkpoint

    att = cfg.layer.attention
    d, hd = cfg.d_model, att.head_dim or cfg.d_model // att.n_heads
    H, Hkv = att.n_heads, att.n_kv_heads or att.n_heads
    layer_kind = type(cfg.layer).__name__
    softcap = float(att.logit_softcap or 0.0)
    eps = cfg.layer.norm.eps
    gelu = layer_kind.startswith("Gemma")
    flash_attn_func = None
    if softcap or cfg.sliding_window is not None:
        from flash_attn import flash_attn_func  # noqa: F811  (ImportError is reported by the caller)

    def rope_tables(S):
        inv = 1.0 / (att.rope.theta ** (torch.arange(0, hd, 2, device=device, dtype=torch.float32) / hd))
        ang = torch.arange(S, device=device, dtype=torch.float32)[:, None] * inv[None, :]
        return ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]

    def rope(x, cos, sin):   # x [B, S, h, hd]; rotate-half convention
        x1, x2 = x[..., : hd // 2].float(), x[..., hd // 2 :].float()
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)

    class Block(nn.Module):
        def __init__(self, window):
            super().__init__()
            self.window = window
            self.q = nn.Linear(d, H * hd, bias=False)
            self.k = nn.Linear(d, Hkv * hd, bias=False)
            self.v = nn.Linear(d, Hkv * hd, bias=False)
            self.o = nn.Linear(H * hd, d, bias=False)
            self.gate = nn.Linear(d, cfg.hidden_size, bias=False)
            self.up = nn.Linear(d, cfg.hidden_size, bias=False)
            self.down = nn.Linear(cfg.hidden_size, d, bias=False)
            self.n1, self.n2 = nn.RMSNorm(d, eps=eps), nn.RMSNorm(d, eps=eps)
            if gelu:
                self.n1_in, self.n2_in = nn.RMSNorm(d, eps=eps), nn.RMSNorm(d, eps=eps)
            self.qn = self.kn = None
            if att.qk_norm is not None:
                per_head = att.use_head_qk_norm
                self.per_head = per_head
                self.qn = nn.RMSNorm(hd if per_head else H * hd, eps=att.qk_norm.eps)
                self.kn = nn.RMSNorm(hd if per_head else Hkv * hd, eps=att.qk_norm.eps)

        def attn(self, x, cos, sin):
            B, S, _ = x.shape
            q, k, v = self.q(x), self.k(x), self.v(x)
            if self.qn is not None and not self.per_head:
                q, k = self.qn(q), self.kn(k)
            q, k, v = q.view(B, S, H, hd), k.view(B, S, Hkv, hd), v.view(B, S, Hkv, hd)
            if self.qn is not None and self.per_head:
                q, k = self.qn(q), self.kn(k)
            q, k = rope(q, cos, sin), rope(k, cos, sin)
            if flash_attn_func is not None:
                w = (self.window, 0) if self.window is not None else (-1, -1)
                a = flash_attn_func(q, k, v, causal=True, window_size=w, softcap=softcap)
            else:
                a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                                   enable_gqa=Hkv != H).transpose(1, 2)
            return self.o(a.reshape(B, S, H * hd))

        def mlp(self, x):
            g = self.gate(x)
            return self.down((F.gelu(g, approximate="tanh") if gelu else F.silu(g)) * self.up(x))

        def forward(self, x, cos, sin):
            if layer_kind.startswith("ReorderedNorm"):      # OLMo2: norm on the block outputs
                h = x + self.n1(self.attn(x, cos, sin))
                return h + self.n2(self.mlp(h))
            if gelu:                                        # Gemma: norm before and after each block
                h = x + self.n1(self.attn(self.n1_in(x), cos, sin))
                return h + self.n2(self.mlp(self.n2_in(h)))
            h = x + self.attn(self.n1(x), cos, sin)         # pre-norm
            return h + self.mlp(self.n2(h))

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(cfg.vocab_size, d)
            self.blocks = nn.ModuleList([Block(cfg.window_size_for_layer(i)) for i in range(cfg.num_layers)])
            self.norm = nn.RMSNorm(d, eps=cfg.norm.eps)
            self.head = None if cfg.tie_embeddings else nn.Linear(d, cfg.vocab_size, bias=False)
            self.final_cap = float(cfg.lm_head.logit_softcap or 0.0)
            self.tables = None

        def forward(self, ids, labels):
            B, S = ids.shape
            if self.tables is None or self.tables[0].shape[1] != S:
                self.tables = rope_tables(S)
            cos, sin = self.tables
            x = self.emb(ids)
            if cfg.scale_embeddings:
                x = x * math.sqrt(d)
            for blk in self.blocks:
                x = checkpoint(blk, x, cos, sin, use_reentrant=False) if checkpoint_blocks else blk(x, cos, sin)
            x = self.norm(x)
            logits = F.linear(x, self.emb.weight) if self.head is None else self.head(x)
            logits = logits.float()
            if self.final_cap:
                logits = self.final_cap * torch.tanh(logits / self.final_cap)
            return F.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1))

    with torch.device(device):
        model = Model()
    for p in model.parameters():
        if p.dim() == 2:
            torch.nn.init.trunc_normal_(p, std=cfg.init_std, a=-3 * cfg.init_std, b=3 * cfg.init_std)
    return model


def run(args, clock_sampler_cls, published) -> int:
    import dataclasses

    import torch
    import torch.distributed as dist

    from olmax_b200.data import generate_batches_of_uniform_tokens
    from olmax_b200.models import TransformerRecipeType

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but the job has {world} ranks")
    if args.mesh not in ("FSDP", "HSDP"):
        return _unavailable(f"the library arm shards with fully_shard only (FSDP / HSDP), not {args.mesh}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    recipe = TransformerRecipeType(args.recipe).build_recipe()
    cfg = recipe.model
    if args.layers is not None:
        cfg = dataclasses.replace(cfg, num_layers=args.layers)
    ac = args.ac if args.ac != "recipe" else ("full" if cfg.layer_ac_policy is not None else "none")
    try:
        model = build_model(cfg, dev, checkpoint_blocks=(ac == "full"))
    except ImportError as e:
        return _unavailable(f"soft-capped / windowed attention needs flash_attn, which did not import ({e})")

    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    if args.mesh == "HSDP":
        shard = args.shard_degree or max(1, world // 2)
        mesh = init_device_mesh("cuda", (world // shard, shard), mesh_dim_names=("replicate", "shard"))
    else:
        mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("shard",))
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    for blk in model.blocks:
        fully_shard(blk, mesh=mesh, mp_policy=mp)
    fully_shard(model, mesh=mesh, mp_policy=mp)
    decay = [p for n, p in model.named_parameters() if p.dim() == 2 and not n.startswith("emb.")]
    no_decay = [p for n, p in model.named_parameters() if not (p.dim() == 2 and not n.startswith("emb."))]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": no_decay, "weight_decay": 0.0}],
                            lr=1e-4, betas=(0.9, 0.95), eps=1e-8, fused=True)

    seq = recipe.sequence_length
    inst = recipe.local_microbatch_size // seq
    k = args.microbatches
    tokens_per_step = inst * world * k * seq
    total_steps = args.warmup + 2 * args.steps + 1
    batches = list(generate_batches_of_uniform_tokens(
        7, vocab_size=cfg.vocab_size, sequence_length=seq, global_microbatch_instances=inst * world, num_microbatches=k,
        dp_rank=rank, dp_size=world, num_batches=min(total_steps, 8), pin_memory=True))
    dev_batches = [[(i.to(dev), l.to(dev)) for i, l in b] for b in batches]

    def step(batch):
        total = None
        for ids, labels in batch:
            ids, labels = ids.to(dev, non_blocking=True), labels.to(dev, non_blocking=True)
            loss = model(ids, labels) / k
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return total

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    try:
        for w in range(args.warmup):
            step(dev_batches[w % len(dev_batches)])
    except torch.OutOfMemoryError as e:
        return _unavailable(f"does not fit on {world} GPU(s) without this repository's memory savings ({str(e)[:80]})")
    sync_all()
    sampler = clock_sampler_cls(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for s in range(args.steps):
        loss = step(dev_batches[(args.warmup + s) % len(dev_batches)])
    e1.record()
    sync_all()
    ms = e0.elapsed_time(e1) / args.steps
    h2d = sum(i.numel() * i.element_size() + l.numel() * l.element_size() for i, l in batches[0])
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    t0.record()
    for s in range(args.steps):
        loss = step(batches[(args.warmup + s) % len(batches)])
        loss.item()
    t1.record()
    sync_all()
    ms_e2e = t0.elapsed_time(t1) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])
    if rank == 0:
        per_gpu = tokens_per_step / (ms / 1e3) / world
        print(json.dumps({
            "impl": "torchlib", "metric": "tokens_per_sec", "value": round(tokens_per_step / (ms / 1e3), 1),
            "unit": "tokens/s (whole job)", "per_gpu": round(per_gpu, 1), "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": round(per_gpu / published, 4) if published else None, "dtype": "bf16",
            "data": "synthetic uniform token ids, random-init weights",
            "config": {"model": args.recipe, "global_batch": inst * world * k, "seq_len": seq, "microbatches": k,
                       "parallelism": f"{args.mesh.lower()}{world} (torch fully_shard over NCCL)", "layers": cfg.num_layers,
                       "kernels": "cuBLAS linear, torch SDPA" + (" / flash_attn" if (cfg.sliding_window or cfg.layer.attention.logit_softcap) else "")
                                  + ", torch fused AdamW", "activation_checkpointing": ac},
            "loss": float(loss.item()),
            "e2e": {"value": round(tokens_per_step / (ms_e2e / 1e3), 1), "unit": "tokens/s (whole job)",
                    "ms_per_step": round(ms_e2e, 3), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "gpu_launches_note": "library kernels only: none of this repository's kernels run in this arm",
            "clocks": clocks, "peak_mem_gib": round(torch.cuda.max_memory_allocated(dev) / 2**30, 2),
        }), flush=True)
    if world > 1:
        dist.barrier()
    dist.destroy_process_group()
    return 0
