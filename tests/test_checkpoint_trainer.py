"""
Checkpointing (tensor trees, sharded state, resharding on restore, async saves, corrupt files) and the Trainer
(callbacks, metrics, cancellation, auto-resume with identical continuation, failure paths).  All on CPU; multi-rank
parts run as gloo processes.  Failures are injected on the host: a callback that raises, a signal, a truncated file.
"""

import json
import os
import signal
from collections import OrderedDict
from dataclasses import dataclass
from pathlib import Path

import pytest
import torch

from olmax_b200 import checkpoint as ckpt
from olmax_b200.exceptions import CallbackExistsError
from olmax_b200.testing import run_distributed_test
from olmax_b200.train import Callback, Trainer
from olmax_b200.types import Duration


def test_tree_save_restore_sync_and_async(tmp_path):
    tree = {"a": torch.arange(6.0).view(2, 3), "b": {"c": torch.ones(4, dtype=torch.bfloat16), "n": 3}, "l": [torch.zeros(2)]}
    ckpt.save(tmp_path / "sync", tree)
    out = ckpt.restore(tmp_path / "sync", {"a": torch.empty(2, 3), "b": {"c": torch.empty(4, dtype=torch.bfloat16), "n": 0},
                                           "l": [torch.empty(2)]})
    assert torch.equal(out["a"], tree["a"]) and torch.equal(out["b"]["c"], tree["b"]["c"]) and out["b"]["n"] == 3
    handle = ckpt.save(tmp_path / "async", tree, block=False)
    handle.wait()
    meta = ckpt.get_metadata(tmp_path / "async")
    assert meta["arrays"]["a"]["shape"] == [2, 3] and meta["arrays"]["b.c"]["dtype"] == "bfloat16"
    free = ckpt.restore_from_metadata(tmp_path / "async")
    assert torch.equal(free["a"], tree["a"]) and free["b"]["n"] == 3
    with pytest.raises(FileExistsError):
        ckpt.save(tmp_path / "sync", tree)
    ckpt.save(tmp_path / "sync", tree, force=True)
    with pytest.raises(ValueError):
        ckpt.restore(tmp_path / "sync", {"a": torch.empty(3, 2)})


def test_truncated_chunk_is_detected(tmp_path):
    ckpt.save(tmp_path / "c", {"w": torch.randn(64, 8)})
    chunk = tmp_path / "c" / "w" / "c" / "0" / "0"
    data = chunk.read_bytes()
    chunk.write_bytes(data[: len(data) // 2])
    with pytest.raises(ValueError, match="truncated or corrupt"):
        ckpt.restore_from_metadata(tmp_path / "c")


def _tiny_model(mesh_resource, seed=0):
    from olmax_b200.models import TransformerRecipeType

    return TransformerRecipeType.tiny_llama.build_recipe().model.build(seed=seed, mesh_resource=mesh_resource, num_layers=1)


def _save_worker(path, kind):
    from olmax_b200.checkpoint.utils import save_sharded
    from olmax_b200.parallel import MeshResource, dist_utils

    world = dist_utils.get_world_size()
    res = {"fsdp": lambda: MeshResource.FSDP(world), "hsdp": lambda: MeshResource.HSDP(2, world, 2),
           "tp": lambda: MeshResource.FSDP_with_TP(2, world)}[kind]()
    model = _tiny_model(res, seed=4)
    moments = torch.arange(model.store.numel_local, dtype=torch.float32) + 1000 * dist_utils.get_rank()
    save_sharded(Path(path) / "params", model.store, {"": model.store.master}).wait()
    save_sharded(Path(path) / "opt", model.store, {"mu": model.store.master * 2}, scalars={"count": 7}).wait()
    dist_utils.barrier()
    return {n: model.store.full_parameter(n) for n, _ in model.store.named_parameters()}


def _load_worker(path, kind):
    from olmax_b200.checkpoint.utils import restore_sharded
    from olmax_b200.parallel import MeshResource, dist_utils

    world = dist_utils.get_world_size()
    res = {"fsdp": lambda: MeshResource.FSDP(world), "hsdp": lambda: MeshResource.HSDP(2, world, 2),
           "tp": lambda: MeshResource.FSDP_with_TP(2, world), "ddp": lambda: MeshResource.DDP(world)}[kind]()
    model = _tiny_model(res, seed=99)   # different init: everything must come from the checkpoint
    restore_sharded(Path(path) / "params", model.store, {"": model.store.master})
    mu = torch.zeros_like(model.store.master)
    scalars = restore_sharded(Path(path) / "opt", model.store, {"mu": mu})
    assert scalars["count"] == 7
    assert torch.equal(mu, model.store.master * 2)
    return {n: model.store.full_parameter(n) for n, _ in model.store.named_parameters()}


@pytest.mark.parametrize("save_kind,save_world,load_kind,load_world", [
    ("fsdp", 2, "hsdp", 4), ("fsdp", 4, "fsdp", 1), ("tp", 4, "fsdp", 2), ("hsdp", 4, "tp", 2), ("fsdp", 2, "ddp", 2),
])
def test_sharded_checkpoint_restores_under_another_mesh(tmp_path, save_kind, save_world, load_kind, load_world):
    saved = run_distributed_test(_save_worker, world_size=save_world, func_args=(str(tmp_path), save_kind))
    loaded = run_distributed_test(_load_worker, world_size=load_world, func_args=(str(tmp_path), load_kind))
    for rank_params in loaded:
        for name, want in saved[0].items():
            assert torch.equal(rank_params[name], want), name
    meta = json.loads((tmp_path / "params" / "embedding.weight" / "zarr.json").read_text())
    assert meta["zarr_format"] == 3 and meta["shape"] == [1024, 256] and meta["data_type"] == "float32"


# ----------------------------------------------------------------------------------------------------------------------
# Trainer
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class Recorder(Callback):
    def __post_init__(self):
        super().__post_init__()
        self.events = []
        self.metrics = {}

    def pre_train(self): self.events.append("pre_train")
    def pre_step(self): self.events.append(f"pre_step{self.step}")
    def post_step(self): self.events.append(f"post_step{self.step}")
    def post_train(self): self.events.append("post_train")
    def on_error(self, exc): self.events.append(f"error:{type(exc).__name__}")
    def close(self): self.events.append("close")
    def log_metrics(self, step, metrics): self.metrics[step] = dict(metrics)
    def get_state(self): return {"n": len(self.metrics)}
    def load_state(self, state): self.loaded = state


def _loader(seed=0, k=2, num_batches=None):
    from olmax_b200.launch.train_transformer import SyntheticDataLoader

    return SyntheticDataLoader(seed, kind="uniform", vocab_size=1024, sequence_length=32, global_microbatch_instances=2,
                               num_microbatches=k, dp_rank=0, dp_size=1, num_batches=num_batches)


def _trainer(tmp_path, steps, **kw):
    from olmax_b200.optim import AdamWConfig, ConstantSchedule

    return Trainer(work_dir=tmp_path, save_folder=tmp_path, optim=AdamWConfig(lr=ConstantSchedule(3e-3), track_grad_norm=True),
                   max_duration=Duration.steps(steps), global_tokens_per_batch=2 * 32 * 2, **kw)


def _model():
    from olmax_b200.parallel import MeshResource

    return _tiny_model(MeshResource.FSDP(1), seed=1)


def test_fit_runs_callbacks_metrics_and_learns(tmp_path):
    rec, late = Recorder(), Recorder(priority=-5)
    trainer = _trainer(tmp_path, 6, callbacks=OrderedDict(late=late, rec=rec))
    assert list(trainer.callbacks) == ["rec", "late"]          # sorted by priority, ties keep insertion order
    with pytest.raises(CallbackExistsError):
        trainer.add_callback("rec", Recorder())
    trainer.fit(_model(), _loader())
    assert rec.events[0] == "pre_train" and rec.events[-2:] == ["post_train", "close"]
    assert [e for e in rec.events if e.startswith("pre_step")] == [f"pre_step{i}" for i in range(1, 7)]
    assert sorted(rec.metrics) == [1, 2, 3, 4, 5, 6]
    assert {"train/loss", "optim/lr", "optim/g_norm"} <= set(rec.metrics[3])
    assert "throughput/TPS device" in rec.metrics[3]
    assert rec.metrics[6]["train/loss"] < rec.metrics[1]["train/loss"]
    assert trainer.global_train_tokens_seen == 6 * 128


def test_epochs_duration_and_disabled_callback(tmp_path):
    rec, off = Recorder(), Recorder(enabled=False)
    trainer = _trainer(tmp_path, 0, callbacks=OrderedDict(rec=rec, off=off))
    trainer.max_duration = Duration.epochs(2)
    trainer.fit(_model(), _loader(num_batches=3))
    assert trainer.step == 6 and trainer.epoch >= 2 and off.events == []


def test_error_in_callback_runs_on_error_and_reraises(tmp_path):
    @dataclass
    class Boom(Callback):
        def post_step(self):
            if self.step == 2:
                raise ValueError("injected failure")

    rec = Recorder()
    trainer = _trainer(tmp_path, 5, callbacks=OrderedDict(rec=rec, boom=Boom()))
    with pytest.raises(ValueError, match="injected failure"):
        trainer.fit(_model(), _loader())
    assert "error:ValueError" in rec.events and rec.events[-1] == "close"
    with pytest.raises(RuntimeError):
        trainer.training_complete


def test_nan_loss_is_reported(tmp_path):
    model = _model()
    model.store.master.fill_(float("nan"))
    model.store.sync_shadow()
    with pytest.raises(RuntimeError, match="train/loss"):
        _trainer(tmp_path, 3).fit(model, _loader())


def test_kernel_status_word_stops_training_before_a_checkpoint_is_written(tmp_path):
    """A kernel whose bounded wait ran out only leaves its status words behind.  Injected on the host: the words are
    set after step 2; fit() must raise at the next step and must not write the checkpoint due at step 3."""
    from olmax_b200.ops import _lib

    @dataclass
    class GiveUp(Callback):
        def pre_step(self):
            if self.step == 2:
                _lib.status_buffer(torch.device("cpu")).copy_(torch.tensor([2, 110, 7, 3005], dtype=torch.int32))

    trainer = _trainer(tmp_path, 6, callbacks=OrderedDict(g=GiveUp()), checkpoint_interval=3)
    try:
        with pytest.raises(_lib.KernelError, match="step 2: kernel reported 'peer flag wait timed out' at site 110"):
            trainer.fit(_model(), _loader())
    finally:
        _lib.status_buffer(torch.device("cpu")).zero_()
    assert trainer.step == 3
    saved = sorted(p.parent.name for p in tmp_path.rglob("_CHECKPOINT_METADATA"))
    assert saved == ["step0"], saved   # the initial checkpoint only: nothing from a step at or after the failure


def test_sigterm_cancels_gracefully_and_checkpoints(tmp_path):
    @dataclass
    class Killer(Callback):
        def post_step(self):
            if self.step == 2:
                os.kill(os.getpid(), signal.SIGTERM)

    trainer = _trainer(tmp_path, 50, callbacks=OrderedDict(k=Killer()), checkpoint_interval=100, cancel_check_interval=1)
    trainer.fit(_model(), _loader())
    assert trainer.is_canceled and 2 <= trainer.step <= 4
    assert (tmp_path / f"step{trainer.step}" / "_CHECKPOINT_METADATA").exists()   # final checkpoint on the way out


def test_resume_continues_identically(tmp_path):
    full = Recorder()
    _trainer(tmp_path / "full", 6, callbacks=OrderedDict(r=full)).fit(_model(), _loader())
    first = Recorder()
    _trainer(tmp_path / "resumed", 3, callbacks=OrderedDict(r=first), checkpoint_interval=3,
             async_checkpointing=True).fit(_model(), _loader())
    assert (tmp_path / "resumed" / "step3" / "params" / "_METADATA").exists()
    second = Recorder()
    t2 = _trainer(tmp_path / "resumed", 6, callbacks=OrderedDict(r=second), checkpoint_interval=3)
    from olmax_b200.parallel import MeshResource

    t2.fit(_tiny_model(MeshResource.FSDP(1), seed=77), _loader())      # different init: state must come from step3
    assert t2.step == 6 and second.loaded == {"n": 2}   # metrics are flushed one step late
    for step in (4, 5, 6):
        assert second.metrics[step]["train/loss"] == pytest.approx(full.metrics[step]["train/loss"], rel=1e-5)
    # an incomplete newer checkpoint directory is ignored by auto-resume
    (tmp_path / "resumed" / "step99").mkdir()
    assert Path(str(_trainer(tmp_path / "resumed", 6)._find_latest_checkpoint())).name == "step6"


def test_persist_and_write_files(tmp_path):
    trainer = Trainer(work_dir=tmp_path / "work", save_folder=tmp_path / "save", optim=None)
    trainer.write_file("config.yaml", "a: 1\n")
    assert (tmp_path / "save" / "config.yaml").read_text() == "a: 1\n"
    with pytest.raises(FileExistsError):
        trainer.write_file("config.yaml", "a: 2\n")
    (tmp_path / "work" / "sub").mkdir()
    (tmp_path / "work" / "sub" / "f").write_text("x")
    trainer.persist_working_subdir("sub")
    assert (tmp_path / "save" / "sub" / "f").read_text() == "x"


def test_native_chunk_io_checksums(tmp_path, monkeypatch):
    """The native chunk writer / reader: known CRC-32C vector, same bytes as the Python fallback, a flipped byte of
    equal length is detected on read, many chunks are written by the thread pool in one call."""
    from olmax_b200.checkpoint import zarr3

    assert zarr3._native() is not None, "the host checkpoint library should build wherever g++ exists"
    assert zarr3.crc32c(b"123456789") == 0xE3069283
    assert zarr3.crc32c(b"") == 0
    data = torch.arange(4 * 6, dtype=torch.float32).view(4, 6)
    a = tmp_path / "a"
    zarr3.write_metadata(a, (8, 6), (4, 6), torch.float32)
    zarr3.write_chunks([(a, (0, 0), data), (a, (1, 0), data + 100)])
    raw = (a / "c" / "0" / "0").read_bytes()
    assert len(raw) == 4 * 6 * 4 + 4
    assert int.from_bytes(raw[-4:], "little") == zarr3.crc32c(raw[:-4])
    assert torch.equal(zarr3.read_full(a), torch.cat([data, data + 100]))
    assert torch.equal(zarr3.read_region(a, (2, 1), (4, 3)), torch.cat([data, data + 100])[2:6, 1:4])
    # the Python fallback writes the same bytes and reads what the native writer wrote
    monkeypatch.setattr(zarr3, "_NATIVE", None)
    monkeypatch.setattr(zarr3, "_NATIVE_TRIED", True)
    b = tmp_path / "b"
    zarr3.write_metadata(b, (8, 6), (4, 6), torch.float32)
    zarr3.write_chunks([(b, (0, 0), data)])
    assert (b / "c" / "0" / "0").read_bytes() == raw
    assert zarr3.crc32c(b"123456789") == 0xE3069283
    assert torch.equal(zarr3.read_region(a, (0, 0), (4, 6)), data)
    monkeypatch.undo()
    # silent corruption: same length, one bit flipped
    damaged = bytearray(raw)
    damaged[10] ^= 0x01
    (a / "c" / "0" / "0").write_bytes(bytes(damaged))
    with pytest.raises(ValueError, match="checksum mismatch"):
        zarr3.read_full(a)
    # a bf16 scalar and a 0-d array survive the byte view
    s = tmp_path / "s"
    zarr3.write_metadata(s, (), (), torch.bfloat16)
    zarr3.write_chunk(s, (), torch.tensor(1.5, dtype=torch.bfloat16))
    assert zarr3.read_full(s).item() == 1.5


# ----------------------------------------------------------------------------------------------------------------------
# Failures injected on the host, among CPU (gloo) ranks
# ----------------------------------------------------------------------------------------------------------------------
def _two_rank_fit(tmp, mode):
    import time

    from olmax_b200.launch.train_transformer import SyntheticDataLoader
    from olmax_b200.parallel import MeshResource, dist_utils

    rank = dist_utils.get_rank()

    @dataclass
    class Saboteur(Callback):
        def post_step(self):
            if rank == 1 and self.step == 2:
                if mode == "cancel":
                    self.trainer.cancel_run("rank 1 wants out")
                elif mode == "die":
                    os._exit(17)          # the process disappears between two steps, nothing in flight

    model = _tiny_model(MeshResource.FSDP(2), seed=1)
    loader = SyntheticDataLoader(0, kind="uniform", vocab_size=1024, sequence_length=32, global_microbatch_instances=2,
                                 num_microbatches=1, dp_rank=rank, dp_size=2)
    trainer = _trainer(Path(tmp) / f"rank{rank}", 40, callbacks=OrderedDict(s=Saboteur()), cancel_check_interval=1)
    t0 = time.monotonic()
    try:
        trainer.fit(model, loader)
        outcome = ("finished", trainer.step, trainer.is_canceled)
    except BaseException as e:  # noqa: BLE001
        outcome = ("raised", type(e).__name__, round(time.monotonic() - t0, 1))
        (Path(tmp) / f"outcome{rank}.txt").write_text(repr(outcome))
        if mode == "die":
            os._exit(0)   # the process group is broken: do not try to barrier on the way out
        raise
    return outcome


def test_cancellation_requested_on_one_rank_stops_every_rank(tmp_path):
    r0, r1 = run_distributed_test(_two_rank_fit, world_size=2, func_args=(str(tmp_path), "cancel"))
    assert r0[0] == r1[0] == "finished"
    assert r0[1] == r1[1] and 2 <= r0[1] <= 4          # both stopped at the same step, right after the request
    assert r0[2] and r1[2]


def test_surviving_rank_notices_a_dead_peer(tmp_path):
    """Rank 1 exits between two steps.  Rank 0's next collective fails (gloo reports the closed connection), the
    trainer runs its error path and re-raises instead of waiting forever."""
    with pytest.raises(Exception):
        run_distributed_test(_two_rank_fit, world_size=2, func_args=(str(tmp_path), "die"), timeout=90)
    outcome = eval((tmp_path / "outcome0.txt").read_text())   # noqa: S307  (written by this test)
    assert outcome[0] == "raised" and outcome[2] < 60, outcome
    assert not (tmp_path / "outcome1.txt").exists()
