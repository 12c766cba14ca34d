"""
Recipe-driven training entry point with the command-line surface of the reference's
``src/integration_tests/train_transformer.py``:

    python -m olmax_b200.launch.train_transformer --recipe=olmo2_7B_bench --device-type=NVIDIA_B200 \
        [--mesh-type FSDP|HSDP|DDP|FSDP_with_TP|FSDP_with_CP|HSDP_with_CP] [--shard-degree N] [--tp-degree N] \
        [--steps N] [--dry-run] [--show-model] [dot.path.overrides=VALUE ...]

Launch one process per GPU with ``torchrun`` (or :mod:`olmax_b200.launch.local`); a single process runs on one device.
Any field of :class:`IntegrationTestConfig` can be overridden with ``--a.b.c=value`` (values parsed as YAML), e.g.
``--num_microbatches=2 --model.layer_ac_policy='{type: nothing_saveable}'``.
"""

from __future__ import annotations

import argparse
import dataclasses
import logging
import sys
import tempfile
import textwrap
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, Iterator, List, Optional, Sequence, Tuple

import torch

from .. import prepare_cli_environment
from ..config import config_to_yaml, parse_config_from_args
from ..data import DataLoader, generate_batches_of_sequential_tokens, generate_batches_of_uniform_tokens
from ..env import EnvConfig
from ..models import TransformerConfig, TransformerRecipeType
from ..optim import AdamWConfig, OptimConfig, WarmupCosineDecaySchedule
from ..parallel import DistConfig, MeshResource, dist_utils, set_mesh
from ..train import ProfilerCallback, Trainer, prepare_training_environment
from ..types import DeviceType, Duration
from ..utils import format_scalar
from ..utils.tree import fold_in

log = logging.getLogger(__name__)


@dataclass
class IntegrationTestConfig:
    model: TransformerConfig
    optim: OptimConfig
    sequence_length: int
    local_microbatch_size: int
    """Tokens per device per micro-batch."""
    mesh: MeshResource
    env: EnvConfig = field(default_factory=EnvConfig)
    distributed: Optional[DistConfig] = None
    num_microbatches: int = 1
    steps: int = 100
    param_dtype: torch.dtype = torch.float32
    compute_dtype: torch.dtype = torch.bfloat16
    save_folder: Optional[str] = None
    load_path: Optional[str] = None
    checkpoint_interval: Optional[int] = None
    data: str = "sequential"
    """``sequential``: the reference's synthetic stream; ``uniform``: uniform ids with shifted labels."""
    seed: int = 0
    profile: bool = True


class SyntheticDataLoader(DataLoader[Tuple[torch.Tensor, torch.Tensor]]):
    """Endless synthetic token stream with resumable state (``train_transformer.py:50-99`` of the reference)."""

    def __init__(self, seed: int, *, kind: str, vocab_size: int, sequence_length: int, global_microbatch_instances: int,
                 num_microbatches: int, dp_rank: int, dp_size: int, cp_rank: int = 0, cp_size: int = 1,
                 num_batches: Optional[int] = None):
        self.seed, self.kind = seed, kind
        self.kw = dict(vocab_size=vocab_size, sequence_length=sequence_length,
                       global_microbatch_instances=global_microbatch_instances, num_microbatches=num_microbatches,
                       dp_rank=dp_rank, dp_size=dp_size, cp_rank=cp_rank, cp_size=cp_size)
        self.num_batches = num_batches
        self.batches_processed = 0
        self.epoch = 0

    def __iter__(self) -> Iterator[List[Tuple[torch.Tensor, torch.Tensor]]]:
        gen = generate_batches_of_uniform_tokens if self.kind == "uniform" else generate_batches_of_sequential_tokens
        remaining = None if self.num_batches is None else max(0, self.num_batches - self.batches_processed)
        for batch in gen(fold_in(self.seed, self.epoch), start_batch=self.batches_processed, num_batches=remaining, **self.kw):
            self.batches_processed += 1
            yield batch
        self.epoch += 1
        self.batches_processed = 0

    def get_state(self) -> Dict[str, Any]:
        return {"seed": self.seed, "batches_processed": self.batches_processed, "epoch": self.epoch}

    def load_state(self, state: Dict[str, Any]) -> None:
        self.seed = int(state["seed"])
        self.batches_processed = int(state["batches_processed"])
        self.epoch = int(state["epoch"])


def build_mesh(mesh_type: str, world: int, local: int, shard_degree: Optional[int], cp_degree: Optional[int],
               tp_degree: Optional[int]) -> MeshResource:
    if mesh_type == "FSDP":
        return MeshResource.FSDP(world)
    if mesh_type == "HSDP":
        return MeshResource.HSDP(shard_degree, world, local)
    if mesh_type == "DDP":
        return MeshResource.DDP(world)
    if mesh_type == "FSDP_with_TP":
        return MeshResource.FSDP_with_TP(tp_degree or 2, world)
    if mesh_type == "FSDP_with_CP":
        return MeshResource.FSDP_with_CP(world, cp_degree if cp_degree is not None else -1)
    if mesh_type == "HSDP_with_CP":
        return MeshResource.HSDP_with_CP(shard_degree, world, local)
    raise ValueError(mesh_type)


def train(config: IntegrationTestConfig, callbacks: Optional[Dict[str, Any]] = None) -> Trainer:
    """Build mesh, model, trainer and synthetic data from ``config`` and run ``Trainer.fit``; ``callbacks`` (name ->
    Callback) are attached in addition to the profiler."""
    mesh = config.mesh.build()
    set_mesh(mesh)
    seq = config.sequence_length
    if config.local_microbatch_size % seq != 0:
        raise ValueError("local_microbatch_size (tokens) must be a multiple of sequence_length")
    instances_local = config.local_microbatch_size // seq
    dp = mesh.data_parallel_size
    # the ranks of a TP or CP group consume the same instances; their instances are pooled so that every device still
    # processes local_microbatch_size tokens
    instances_per_dp_rank = instances_local * mesh.tp.size * mesh.cp.size
    global_tokens = instances_per_dp_rank * dp * seq * config.num_microbatches
    dist_utils.barrier("pre-model-init")
    model = config.model.build(seed=fold_in(config.seed, 1), mesh=mesh, param_dtype=config.param_dtype,
                               compute_dtype=config.compute_dtype if mesh.device.type == "cuda" else config.param_dtype,
                               reshard_after_forward=config.env.runtime.reshard_after_forward,
                               comm_backend=config.env.runtime.comm_backend)
    n = model.num_params()
    log.info("Model has %s parameters (%s per device)", format_scalar(n), format_scalar(model.store.numel_local))
    cache = model.get_buffer_cache(seq)
    save_folder = config.save_folder or tempfile.mkdtemp(prefix="olmax_b200_")
    trainer = Trainer(
        work_dir=Path(save_folder) if not str(save_folder).startswith(("gs://", "s3://")) else Path(tempfile.mkdtemp()),
        save_folder=save_folder,
        optim=config.optim,
        mesh=config.mesh,
        max_duration=Duration.steps(config.steps),
        global_tokens_per_batch=global_tokens,
        checkpoint_interval=config.checkpoint_interval,
    )
    if config.profile:
        trainer.add_callback("profiler", ProfilerCallback())
    for name, cb in (callbacks or {}).items():
        trainer.add_callback(name, cb)
    loader = SyntheticDataLoader(
        fold_in(config.seed, 2), kind=config.data, vocab_size=config.model.vocab_size, sequence_length=seq,
        global_microbatch_instances=instances_per_dp_rank * dp, num_microbatches=config.num_microbatches,
        dp_rank=mesh.data_parallel_rank, dp_size=dp, cp_rank=mesh.cp.rank, cp_size=mesh.cp.size,
    )
    trainer.fit(model, loader, load_path=config.load_path, buffer_cache=cache)
    return trainer


def _parse_args(argv: Optional[Sequence[str]] = None):
    prog = "python -m olmax_b200.launch.train_transformer"
    parser = argparse.ArgumentParser(
        prog=prog,
        usage=f"{prog} --recipe=RECIPE [OPTIONS...] [CONFIG_OVERRIDES...]",
        description=textwrap.dedent("""
            Run a short transformer training job from a recipe.  Besides the options below, any config field can be
            overridden with dot notation (values parsed as YAML), e.g. --model.num_layers=4 --num_microbatches=2.
        """),
        formatter_class=argparse.ArgumentDefaultsHelpFormatter,
    )
    parser.add_argument("--recipe", choices=[r.value for r in TransformerRecipeType], required=True)
    parser.add_argument("--device-type", choices=[d.value for d in DeviceType], default=DeviceType.NVIDIA_B200.value)
    parser.add_argument("--dry-run", action="store_true", help="print the resolved config and exit")
    parser.add_argument("--show-model", action="store_true", help="print the model structure after initialisation")
    parser.add_argument("--local-device-count", type=int, default=None)
    parser.add_argument("--global-device-count", type=int, default=None)
    parser.add_argument("--mesh-type", default="FSDP",
                        choices=["FSDP", "HSDP", "DDP", "FSDP_with_TP", "FSDP_with_CP", "HSDP_with_CP"])
    parser.add_argument("--shard-degree", type=int, default=None)
    parser.add_argument("--cp-degree", type=int, default=None)
    parser.add_argument("--tp-degree", type=int, default=None)
    parser.add_argument("--steps", type=int, default=100)
    return parser.parse_known_args(argv)


def build_config(opts, overrides: Sequence[str]) -> IntegrationTestConfig:
    device_type = DeviceType(opts.device_type)
    env = EnvConfig.recommended(device_type.architecture)
    recipe = TransformerRecipeType(opts.recipe).build_recipe(env, device_type)
    name = opts.recipe
    if any(s in name for s in ("27B", "32B", "70B")):
        lr = 1e-5
    elif any(s in name for s in ("7B", "8B")):
        lr = 1e-4
    else:
        lr = 1e-3
    dist_cfg = DistConfig.from_env()
    world = opts.global_device_count or (dist_cfg.num_processes if dist_cfg else 1)
    local = opts.local_device_count or dist_utils.get_local_device_count()
    mesh = build_mesh(opts.mesh_type, world, min(local, world), opts.shard_degree, opts.cp_degree, opts.tp_degree)
    config = IntegrationTestConfig(
        model=recipe.model,
        optim=AdamWConfig(
            lr=WarmupCosineDecaySchedule(warmup_steps=20, decay_steps=max(1, opts.steps - 20), peak_value=lr,
                                         init_value=0.01 * lr, end_value=0.01 * lr),
            no_decay_modules=["embedding.weight"],
        ),
        sequence_length=recipe.sequence_length,
        local_microbatch_size=recipe.local_microbatch_size,
        mesh=mesh,
        env=recipe.env,
        distributed=dist_cfg,
        steps=opts.steps,
    )
    return parse_config_from_args(config, args=list(overrides))


def main(argv: Optional[Sequence[str]] = None) -> None:
    opts, overrides = _parse_args(argv)
    config = build_config(opts, overrides)
    if opts.dry_run:
        print(config_to_yaml(config))
        return
    prepare_training_environment(config.env.xla, config.env.nccl, config.env.cuda, config.env.jax, config.env.runtime,
                                 gpu_architecture=DeviceType(opts.device_type).architecture)
    dist_utils.init_distributed(config.distributed)
    try:
        trainer = train(config)
        if opts.show_model and dist_utils.get_rank() == 0:
            print(trainer.model)
    finally:
        dist_utils.teardown_distributed()


if __name__ == "__main__":
    prepare_cli_environment()
    main()
