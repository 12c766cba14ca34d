"""
Benchmark of the flagship training step: OLMo2-7B (benchmark variant), sequence length 4096, bf16 compute with fp32
master weights / AdamW state, full FSDP over N GPUs of one node, synthetic uniform token ids, random-init weights.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Rank 0 prints ONE JSON line.  ``value`` is whole-job tokens per second over exactly K optimizer steps, timed on the
device with CUDA events (max over ranks) with the step's inputs already resident on the device.  ``e2e`` is the same
metric through the public ``Trainer.train_batch`` call, where every step copies its token ids and labels from pinned
host memory and reads the loss back to the host.  ``--impl reference`` would run the reference's own code from
``baseline/_ref``; it needs JAX, which this image does not have, so it prints the ``unavailable`` line.
``--impl torchlib`` runs the same model and step built from PyTorch's library kernels and NCCL (``baseline/torchlib.py``),
a same-box comparison that is not the reference.
"""

from __future__ import annotations

import os

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

import argparse
import json
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PUBLISHED_TPS_PER_GPU = {  # the reference's published tokens/s/GPU for the same model (its README; H100 unless noted)
    "olmo2_7B_bench": 12006.0,
    "llama_like_7B_bench": 12597.0,
    "gemma2_like_27B_bench": 5358.0,  # 2 x 8 B200
    "olmo2_32B_bench": 2155.0,
}


def reference_arm(args) -> int:
    line = {"impl": "reference"}
    try:
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
        import jax  # noqa: F401  (the reference imports jax at package import)
        import olmax  # noqa: F401

        line["unavailable"] = "reference imported but no runner is wired up in this build"
    except Exception as e:  # noqa: BLE001
        line["unavailable"] = (f"reference needs jax/jaxlib/equinox/optax/orbax which are not installed and cannot be "
                               f"installed offline ({type(e).__name__}: {e})")
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(line), flush=True)
    return 0


def comm_selfcheck(args, model_cfg, mesh, mesh_res, dev, seq, inst_local, k):
    """Outside the timed region, on the job's own mesh: a 2-layer copy of the benchmarked architecture is built twice from
    the same seed, once on the peer-memory ("fused") backend and once on NCCL, and trained for 2 optimizer steps of k
    micro-batches on identical data.  Returns the largest relative differences over all ranks of the losses, the
    accumulated gradient of step 1 and the fp32 master weights after step 2: evidence, in every benchmark record, that
    the all-gather / reduce-scatter / all-reduce fused into our kernels give the numbers of the library collectives
    (the sharded-vs-reference invariant of the reference's ``src/test/nn/transformer/model_test.py:79-134``)."""
    import dataclasses

    import torch
    import torch.distributed as dist

    from olmax_b200.ops import _lib
    from olmax_b200.optim import AdamWConfig, ConstantSchedule
    from olmax_b200.testing import rel_err

    small = dataclasses.replace(model_cfg, num_layers=2)
    inst = inst_local * mesh.tp.size * mesh.cp.size
    results = {}
    for backend in ("fused", "nccl"):
        model = small.build(seed=3, mesh=mesh, device=dev, comm_backend=backend)
        if backend == "fused" and model.store.symm is None and model.store.tp_symm is None:
            return {"skipped": "peer-memory backend not active on this mesh"}
        cache = model.get_buffer_cache(seq, dev)
        optim = AdamWConfig(lr=ConstantSchedule(1e-3), no_decay_modules=["embedding.weight"]).build(model, k)
        gen = torch.Generator().manual_seed(1234 + mesh.data_parallel_rank)
        losses, first_grad = [], None
        for step in range(2):
            for _ in range(k):
                ids = torch.randint(0, small.vocab_size, (inst, seq), generator=gen)
                labels = torch.roll(ids, -1, 1)
                if mesh.cp.size > 1:
                    from olmax_b200.parallel.context import shard_sequence_for_cp
                    ids = shard_sequence_for_cp(ids, mesh.cp.size, mesh.cp.rank)
                    labels = shard_sequence_for_cp(labels, mesh.cp.size, mesh.cp.rank)
                loss, _ = model(ids.to(dev), labels.to(dev), cache)
                loss.backward()
                optim.accumulate()
                losses.append(loss.detach().float())
            if step == 0:
                # peers add their embedding / norm-weight contributions straight into this rank's accumulator: they
                # have all landed only after the barrier that the optimizer step would begin with
                model.store.sync_peers()
                first_grad = model.store.grad.detach().clone()
            optim.step()
        torch.cuda.synchronize()
        _lib.check_status(dev)
        results[backend] = (torch.stack(losses).cpu(), first_grad.cpu(), model.store.master.detach().clone().cpu())
        del model, optim, cache
        torch.cuda.empty_cache()
    lf, gf, pf = results["fused"]
    ln, gn, pn = results["nccl"]
    t = torch.tensor([float(((lf - ln).abs() / ln.abs().clamp_min(1e-12)).max()), rel_err(gf, gn), rel_err(pf, pn)],
                     dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"loss_rel": float(t[0]), "grad_rel": float(t[1]), "param_rel_after_2_steps": float(t[2]),
            "layers": 2, "optimizer_steps": 2, "microbatches": k, "tolerance": 1e-2}


def selfcheck_verdict(selfcheck: dict, comm: str, tolerance: float = 1e-2):
    """What a multi-GPU run does with the result of :func:`comm_selfcheck`: ``("ok", [])`` when every difference is
    within the tolerance (a NaN is not), else ``("fail", names)`` when the fused backend was asked for explicitly and
    ``("fallback", names)`` with ``--comm auto`` (the NCCL backend is measured instead)."""
    if "skipped" in selfcheck:
        return "ok", []
    bad = [n for n in ("loss_rel", "grad_rel", "param_rel_after_2_steps") if not (selfcheck.get(n, 0.0) <= tolerance)]
    if not bad:
        return "ok", []
    return ("fail" if comm == "fused" else "fallback"), bad


class ClockSampler:
    """Samples SM clocks and throttle reasons of this rank's GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); pw.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torchlib"],
                    help="ours: this repository; reference: the unmodified reference from baseline/_ref; torchlib: the same "
                         "model and step from PyTorch's own library kernels and NCCL (baseline/torchlib.py)")
    ap.add_argument("--recipe", default="olmo2_7B_bench")
    ap.add_argument("--mesh", default="FSDP", choices=["FSDP", "HSDP", "DDP", "FSDP_with_TP", "FSDP_with_CP", "HSDP_with_CP"])
    ap.add_argument("--shard-degree", type=int, default=None)
    ap.add_argument("--tp-degree", type=int, default=2)
    ap.add_argument("--kernel-timing", action="store_true",
                    help="after the measurement run 2 more steps with per-kernel CUDA-event timing and print the table (stderr)")
    ap.add_argument("--cp-degree", type=int, default=None, help="context-parallel degree of the *_with_CP meshes")
    ap.add_argument("--cp-strategy", default=None, choices=["all_gather", "ring"])
    ap.add_argument("--microbatches", type=int, default=2)
    ap.add_argument("--layers", type=int, default=None, help="debug only: truncate the model (makes the run INVALID as a benchmark)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-selfcheck", action="store_true",
                    help="multi-GPU runs: do not compare the fused backend against NCCL on a 2-layer model first")
    ap.add_argument("--comm", default="auto", choices=["auto", "fused", "nccl"],
                    help="fused: collectives inside our kernels over peer memory (a failed self-check against NCCL "
                         "ends the run with exit code 2); nccl: the NCCL baseline path; auto: fused, but if the "
                         "self-check fails the NCCL backend is measured and the JSON line says so")
    ap.add_argument("--ac", default="recipe", choices=["recipe", "none", "mlp", "full"],
                    help="activation checkpointing: the recipe's policy, none, recompute the MLP blocks, or whole layers")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.impl == "torchlib":
        import importlib.util

        spec = importlib.util.spec_from_file_location("olmax_b200_torchlib_arm", ROOT / "baseline" / "torchlib.py")
        arm = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(arm)
        return arm.run(args, ClockSampler, PUBLISHED_TPS_PER_GPU.get(args.recipe))

    import torch
    import torch.distributed as dist

    from olmax_b200.data import generate_batches_of_uniform_tokens
    from olmax_b200.launch.train_transformer import build_mesh
    from olmax_b200.models import TransformerRecipeType
    from olmax_b200.ops import _lib, kernels as K
    from olmax_b200.optim import AdamWConfig, WarmupCosineDecaySchedule
    from olmax_b200.parallel import dist_utils, set_mesh
    from olmax_b200.train import Trainer

    if not torch.cuda.is_available():
        print(json.dumps({"error": "bench.py needs a CUDA device"}))
        return 1
    dist_utils.init_distributed()
    rank, world = dist_utils.get_rank(), dist_utils.get_world_size()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but the job has {world} ranks (launch with torchrun --nproc-per-node {args.gpus})")
    local_rank = dist_utils.get_local_rank()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    _lib.lib()  # fail now if the kernel library is missing

    recipe = TransformerRecipeType(args.recipe).build_recipe()
    model_cfg = recipe.model
    if args.layers is not None:
        import dataclasses
        model_cfg = dataclasses.replace(model_cfg, num_layers=args.layers)
    if args.cp_strategy is not None:
        import dataclasses
        layer = model_cfg.layer
        model_cfg = dataclasses.replace(model_cfg, layer=dataclasses.replace(
            layer, attention=dataclasses.replace(layer.attention, cp_strategy=args.cp_strategy)))
    if args.ac != "recipe":
        import dataclasses
        from olmax_b200.activation_checkpointing import NothingSaveable, SaveAnythingExceptTheseNames
        policy = {"none": None, "mlp": SaveAnythingExceptTheseNames(names=["layers.*.mlp"]), "full": NothingSaveable()}[args.ac]
        model_cfg = dataclasses.replace(model_cfg, layer_ac_policy=policy)
    mesh_res = build_mesh(args.mesh, world, world, args.shard_degree, args.cp_degree, args.tp_degree)
    mesh = mesh_res.build(device=dev)
    set_mesh(mesh)
    seq = recipe.sequence_length
    inst_local = recipe.local_microbatch_size // seq
    k = args.microbatches
    dp = mesh.data_parallel_size
    inst_per_dp = inst_local * mesh.tp.size * mesh.cp.size
    global_batch = inst_per_dp * dp * k
    tokens_per_step = global_batch * seq

    selfcheck = None
    if world > 1 and args.comm in ("auto", "fused") and not args.skip_selfcheck:
        selfcheck = comm_selfcheck(args, model_cfg, mesh, mesh_res, dev, seq, inst_local, k)
        action, bad = selfcheck_verdict(selfcheck, args.comm)
        if action == "fail":
            if rank == 0:
                print(json.dumps({"error": "fused and NCCL backends disagree", "selfcheck": selfcheck}), flush=True)
            return 2
        if action == "fallback":
            # Never time a backend that failed its check, and never report nothing: with --comm auto the measurement
            # falls back to the NCCL backend (the values are the all-reduced maxima, so every rank decides alike) and
            # the JSON line says so in "selfcheck" and "config".
            selfcheck["fused_backend_rejected"] = bad
            args.comm = "nccl"
            if rank == 0:
                print(f"bench: fused and NCCL backends disagree on {bad}: {selfcheck}; measuring the NCCL backend",
                      file=sys.stderr, flush=True)

    model = model_cfg.build(seed=1, mesh=mesh, device=dev, comm_backend=args.comm)
    cache = model.get_buffer_cache(seq, dev)
    lr = 1e-4
    optim_cfg = AdamWConfig(lr=WarmupCosineDecaySchedule(warmup_steps=20, decay_steps=80, peak_value=lr, init_value=0.01 * lr,
                                                         end_value=0.01 * lr), no_decay_modules=["embedding.weight"])
    tmp = tempfile.mkdtemp(prefix="olmax_b200_bench_")
    trainer = Trainer(work_dir=tmp, save_folder=tmp, optim=optim_cfg, mesh=mesh_res).setup(model, k, cache)

    total_steps = args.warmup + args.steps * (1 if args.skip_e2e else 2) + 1
    batches = list(generate_batches_of_uniform_tokens(
        7, vocab_size=model_cfg.vocab_size, sequence_length=seq, global_microbatch_instances=inst_per_dp * dp,
        num_microbatches=k, dp_rank=mesh.data_parallel_rank, dp_size=dp, cp_rank=mesh.cp.rank, cp_size=mesh.cp.size,
        num_batches=min(total_steps, 8), pin_memory=True))
    dev_batches = [[(i.to(dev), l.to(dev)) for i, l in b] for b in batches]

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    loss_first_step = None
    for w in range(args.warmup):
        first = trainer.train_batch(dev_batches[w % len(dev_batches)])
        if w == 0:
            loss_first_step = float(first.item())
    sync_all()
    _lib.check_status(dev)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # ---- device-timed region: exactly K optimizer steps -----------------------------------------------------------
    K.reset_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for s in range(args.steps):
        loss = trainer.train_batch(dev_batches[(args.warmup + s) % len(dev_batches)])
    e1.record()
    sync_all()
    ms = e0.elapsed_time(e1) / args.steps
    launches = K.launch_count()
    final_loss = float(loss.item())
    # ---- end-to-end region: pinned host inputs -> H2D every step, loss read back every step ----------------------
    e2e = None
    if not args.skip_e2e:
        h2d = sum(i.numel() * i.element_size() + l.numel() * l.element_size() for i, l in batches[0])
        sync_all()
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        for s in range(args.steps):
            loss = trainer.train_batch(batches[(args.warmup + s) % len(batches)])
            host_loss = loss.item()  # device -> host read of the step result (synchronises the step)
        t1.record()
        sync_all()
        ms_e2e = t0.elapsed_time(t1) / args.steps
        e2e = (ms_e2e, h2d, 4)
    clocks = sampler.stop() if rank == 0 else None
    _lib.check_status(dev)

    # max over ranks
    t = torch.tensor([ms, e2e[0] if e2e else 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])
    value = tokens_per_step / (ms / 1e3)
    per_gpu = value / world
    flops_tok = model.num_flops_per_token(seq)
    if rank == 0:
        peaks = {}
        try:
            peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        except Exception:
            pass
        sustained = peaks.get("bf16_tflops_sustained", 1400.0)
        published = PUBLISHED_TPS_PER_GPU.get(args.recipe)
        line = {
            "metric": "tokens_per_sec",
            "value": round(value, 1),
            "unit": "tokens/s (whole job)",
            "per_gpu": round(per_gpu, 1),
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": round(ms, 3),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": round(per_gpu / published, 4) if published else None,
            "vs_baseline_note": "per-GPU value / the reference's published tokens/s/GPU for this model",
            "dtype": "bf16",
            "data": "synthetic uniform token ids, random-init weights",
            "config": {
                "model": args.recipe, "global_batch": global_batch, "seq_len": seq, "microbatches": k,
                "parallelism": f"{args.mesh.lower()}{world}", "optimizer": "AdamW fp32 master/moments, no gradient clipping (as in the reference's benchmark runs)",
                "comm": ("fused peer-memory kernels" if (model.store.symm is not None or model.store.tp_symm is not None)
                         else ("nccl" if world > 1 else "none")),
                "layers": model_cfg.num_layers, "params": model.num_params(), "activation_checkpointing": args.ac,
                "l2": "working set (>14 GB of weights per step) exceeds L2, no explicit flush",
            },
            "mfu_of_measured_sustained": round(per_gpu * flops_tok / (sustained * 1e12), 4),
            "tflops_per_gpu": round(per_gpu * flops_tok / 1e12, 1),
            "loss": final_loss,
            "loss_first_step": loss_first_step,
            "selfcheck": selfcheck,
            "gpu_launches": launches,
            "clocks": clocks,
            "peak_mem_gib": round(torch.cuda.max_memory_allocated(dev) / 2**30, 2),
        }
        if e2e:
            line["e2e"] = {"value": round(tokens_per_step / (ms_e2e / 1e3), 1), "unit": "tokens/s (whole job)",
                           "ms_per_step": round(ms_e2e, 3), "h2d_bytes_per_step": e2e[1], "d2h_bytes_per_step": e2e[2] * 1}
        print(json.dumps(line), flush=True)
    if args.kernel_timing:
        # profiling pass, after (and outside) the measurement: device time per kernel label from CUDA events
        K.set_timing(True)
        for s in range(2):
            trainer.train_batch(dev_batches[s % len(dev_batches)])
        report = K.timing_report()
        K.set_timing(False)
        if rank == 0:
            print(f"per-kernel device time over 2 steps (rank 0):\n{K.format_timing(report)}", file=sys.stderr, flush=True)
    if world > 1:
        dist.barrier()
    dist_utils.teardown_distributed()
    return 0


if __name__ == "__main__":
    sys.exit(main())
