"""
The recipe-driven entrypoint end to end on CPU ranks (gloo): the tiny Llama configuration (2 layers, d_model 256,
4 heads x 64, SwiGLU 688, RMSNorm eps 1e-6, RoPE theta 10000, vocabulary 1024, sequence 256, fp32; uniform ids with
labels shifted by one; AdamW lr 1e-3, betas (0.9, 0.95), weight decay 0.1; global batch 4 in 2 micro-batches) trained for
10 steps under FSDP over 2 ranks gives the loss curve of the single-process run of the same global batch, and so do the
other meshes (HSDP, DDP, FSDP x TP, FSDP with context parallelism).
"""

from dataclasses import dataclass

import pytest
import torch

from olmax_b200.testing import run_distributed_test
from olmax_b200.train import Callback


@dataclass
class _LossRecorder(Callback):
    def __post_init__(self):
        super().__post_init__()
        self.losses = {}

    def log_metrics(self, step, metrics):
        if "train/loss" in metrics:
            self.losses[step] = float(metrics["train/loss"])


def _entry_worker(mesh_type, extra_args, instances_per_device, tmp):
    from olmax_b200.launch.train_transformer import _parse_args, build_config, train
    from olmax_b200.parallel import dist_utils

    world = dist_utils.get_world_size()
    argv = ["--recipe=tiny_llama", f"--mesh-type={mesh_type}", f"--global-device-count={world}",
            f"--local-device-count={world}", "--steps=10", *extra_args,
            "--num_microbatches=2", "--data=uniform", "--profile=false", f"--save_folder={tmp}/run{dist_utils.get_rank()}",
            f"--local_microbatch_size={256 * instances_per_device}",
            "--optim.lr={type: constant, value: 1e-3}", "--optim.b1=0.9", "--optim.b2=0.95", "--optim.weight_decay=0.1",
            "--param_dtype=float32", "--compute_dtype=float32"]
    opts, overrides = _parse_args(argv)
    config = build_config(opts, overrides)
    rec = _LossRecorder()
    trainer = train(config, callbacks={"losses": rec})
    assert trainer.step == 10
    return [rec.losses[s] for s in sorted(rec.losses)]


@pytest.fixture(scope="module")
def single_process_curve(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("single")
    # one process holding the whole global micro-batch (2 instances x 2 micro-batches = global batch 4)
    (curve,) = run_distributed_test(_entry_worker, world_size=1, func_args=("FSDP", [], 2, str(tmp)))
    # uniform random ids carry nothing to learn: the loss stays near ln(1024), its trajectory is the fingerprint
    assert len(curve) == 10 and all(c == pytest.approx(6.93, abs=0.2) for c in curve) and len(set(curve)) == 10
    return curve


@pytest.mark.parametrize("mesh_type,world,extra,instances", [
    ("FSDP", 2, [], 1),
    ("HSDP", 2, ["--shard-degree=1"], 1),            # 2 replicas of 1 shard
    ("DDP", 2, [], 1),
    ("FSDP_with_TP", 2, ["--tp-degree=2"], 1),
    ("FSDP_with_CP", 2, ["--cp-degree=2"], 1),
])
def test_tiny_llama_loss_curve_matches_single_process(tmp_path, single_process_curve, mesh_type, world, extra, instances):
    curves = run_distributed_test(_entry_worker, world_size=world, func_args=(mesh_type, extra, instances, str(tmp_path)))
    for curve in curves:
        assert len(curve) == 10
        for got, want in zip(curve, single_process_curve):
            assert got == pytest.approx(want, rel=2e-4), (curve, single_process_curve)


def test_eight_ranks_fsdp_and_hsdp_2x4_train_alike(tmp_path):
    """The host side of the 8-GPU configurations (FSDP over 8, HSDP as 2 replicas of 4 shards) on 8 CPU ranks: same
    global batch, so the same loss curve on every rank of both meshes."""
    fsdp = run_distributed_test(_entry_worker, world_size=8, func_args=("FSDP", [], 1, str(tmp_path / "a")), timeout=600)
    hsdp = run_distributed_test(_entry_worker, world_size=8, func_args=("HSDP", ["--shard-degree=4"], 1, str(tmp_path / "b")),
                                timeout=600)
    for curve in fsdp + hsdp:
        assert len(curve) == 10
        for got, want in zip(curve, fsdp[0]):
            assert got == pytest.approx(want, rel=2e-4)

