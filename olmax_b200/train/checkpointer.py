"""
Trainer-level checkpointing (``olmax/train/checkpointer.py:26-283``): a checkpoint is a directory
``save_folder/step{N}`` with the items ``trainer`` (JSON: step, epoch, tokens seen), ``params``, ``static``,
``opt_state``, ``data_loader_state`` and ``callbacks_state``, by default in the reference's Orbax / OCDBT layout
(``checkpoint/orbax_layout.py``); it is written locally first and then copied to the save folder by
file-system rank 0 when that is a different (e.g. remote) location; saves can be asynchronous with a finalizer that
uploads and signals completion; loads from a URL are staged through a hashed work directory.
"""

from __future__ import annotations

import hashlib
import logging
import shutil
import threading
import time
from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, Optional

import torch

from .. import fs
from ..checkpoint import utils as ckpt
from ..checkpoint.utils import AsyncSaveHandle
from ..parallel import dist_utils
from ..types import PathOrStr
from ..utils.dataclass_codec import Registrable

__all__ = ["TrainState", "Checkpointer", "SimpleCheckpointer"]

log = logging.getLogger(__name__)


@dataclass
class TrainState:
    step: int
    epoch: int
    global_train_tokens_seen: Optional[int]
    model: Any
    optim: Any
    data_loader_state: Dict[str, Any] = field(default_factory=dict)
    callbacks_state: Dict[str, Dict[str, Any]] = field(default_factory=dict)


@dataclass
class Checkpointer(Registrable, ABC):
    work_dir: Optional[Path] = None

    @abstractmethod
    def save(self, dir: PathOrStr, state: TrainState, overwrite: bool = False) -> None: ...

    @abstractmethod
    def save_async(self, dir: PathOrStr, state: TrainState, overwrite: bool = False) -> AsyncSaveHandle: ...

    @abstractmethod
    def load(self, dir: PathOrStr, state: TrainState) -> TrainState: ...


@Checkpointer.register("simple", default=True)
@dataclass
class SimpleCheckpointer(Checkpointer):
    format: str = "ocdbt"
    """``ocdbt``: the reference's Orbax layout (``checkpoint/orbax_layout.py``: composite items, zarr v3 arrays packed in
    OCDBT databases, the optimizer state named like the optax tree, a ``static`` item).  ``zarr3``: plain zarr v3
    directory stores, one file per chunk, written by the native threaded chunk writer.  Loading detects the format."""

    def _local_dir(self, dir: PathOrStr) -> Path:
        if fs.is_url(dir) and not str(dir).startswith("file://"):
            assert self.work_dir is not None, "work_dir is required to stage remote checkpoints"
            return Path(self.work_dir) / Path(str(dir).rstrip("/")).name
        return Path(fs.normalize_path(dir))

    # ------------------------------------------------------------------ writing
    @staticmethod
    def _optax_layout(opt) -> tuple:
        """(prefix of the MultiSteps level, prefix of the inject-hyperparams level) for this optimizer."""
        from ..checkpoint.orbax_layout import optax_prefixes

        clipped = getattr(getattr(opt, "config", None), "max_grad_norm", None) is not None
        return optax_prefixes(int(getattr(opt, "num_microbatches", 1)), clipped)

    def _write(self, local: Path, state: TrainState, block: bool) -> list:
        store = state.model.store
        if dist_utils.get_rank() == 0:
            ckpt.write_json(local / "trainer" / "metadata", {
                "step": state.step, "epoch": state.epoch, "global_train_tokens_seen": state.global_train_tokens_seen})
            ckpt.write_json(local / "data_loader_state" / "metadata", state.data_loader_state)
            ckpt.write_json(local / "callbacks_state" / "metadata", state.callbacks_state)
        if self.format == "zarr3":
            handles = [ckpt.save_sharded(local / "params", store, {"": store.master}, block=block)]
            if state.optim is not None:
                sd = state.optim.state_dict()
                handles.append(ckpt.save_sharded(local / "opt_state", store, {"mu": sd["exp_avg"], "nu": sd["exp_avg_sq"]},
                                                 scalars={"count": sd["count"], "mini_step": sd["mini_step"]}, block=block))
            return handles
        if self.format != "ocdbt":
            raise ValueError(f"unknown checkpoint format '{self.format}' (expected 'ocdbt' or 'zarr3')")
        from ..checkpoint import orbax_layout as ol

        # snapshot on this thread (device -> host copies), write on a worker thread
        jobs = [("params", {"": store.master.detach().to("cpu", copy=True)}, {}, ())]
        opt = state.optim
        if opt is not None:
            sd = opt.state_dict()
            outer, inj = self._optax_layout(opt)
            adam = f"{inj}inner_state.0."
            scalars = {f"{inj}count": sd["count"], f"{adam}count": sd["count"],
                       f"{inj}hyperparams.learning_rate": float(getattr(opt, "last_lr", 0.0)),
                       f"{inj}hyperparams_states.learning_rate.count": sd["count"]}
            cfg = getattr(opt, "config", None)
            for hp in ("b1", "b2", "eps", "weight_decay"):
                if cfg is not None and hasattr(cfg, hp):
                    scalars[f"{inj}hyperparams.{hp}"] = float(getattr(cfg, hp))
            zero = ()
            if outer:
                scalars.update({"mini_step": sd["mini_step"], "gradient_step": sd["count"]})
                zero = ("acc_grads",)   # between optimizer steps the accumulator is zero: metadata only, no chunks
            jobs.append(("opt_state", {f"{adam}mu": sd["exp_avg"].detach().to("cpu", copy=True),
                                       f"{adam}nu": sd["exp_avg_sq"].detach().to("cpu", copy=True)}, scalars, zero))
        jobs.append(("static", {}, {}, ()))   # the model's non-array leaves: none here (configuration lives in code)
        self._pending_items = {}

        def write() -> None:
            for name, buffers, scalars, zero in jobs:
                self._pending_items[name] = ol.save_store_item(local / name, store, buffers, scalars, zero)

        if block:
            write()
            return [AsyncSaveHandle()]
        handle = AsyncSaveHandle(None)
        th = threading.Thread(target=lambda: handle._run(write), name="checkpoint-writer", daemon=True)
        handle._thread, handle._finished = th, False
        th.start()
        return [handle]

    def _prepare(self, dir: PathOrStr, overwrite: bool) -> Path:
        local = self._local_dir(dir)
        self._started_ns = time.time_ns()
        exists = False
        if dist_utils.get_process_filesystem_rank() == 0:
            exists = local.exists() and any(local.iterdir())
        # every rank learns the answer of file-system rank 0, so that all of them raise (or none)
        exists = bool(dist_utils.synchronize_value(exists))
        if exists and not overwrite:
            raise FileExistsError(f"checkpoint directory {local} already exists (save_overwrite=False)")
        if dist_utils.get_process_filesystem_rank() == 0:
            if exists:
                shutil.rmtree(local)
            local.mkdir(parents=True, exist_ok=True)
        dist_utils.barrier("checkpoint-dir")
        return local

    def _finalize(self, local: Path, dir: PathOrStr) -> None:
        if self.format == "ocdbt" and dist_utils.get_rank() == 0:
            from ..checkpoint import orbax_layout as ol

            for name, (leaves, sharding) in getattr(self, "_pending_items", {}).items():
                ol.finalize_item(local / name, dist_utils.get_world_size(), leaves, sharding)
        if str(local) != fs.normalize_path(dir) and dist_utils.get_process_filesystem_rank() == 0:
            fs.copy_dir(local, dir, save_overwrite=True)
        if dist_utils.get_rank() == 0:
            if self.format == "ocdbt":
                from ..checkpoint import orbax_layout as ol

                ol.write_checkpoint_metadata(local, ["params", "static", "opt_state"], ["trainer"],
                                             getattr(self, "_started_ns", time.time_ns()))
            else:
                ckpt.write_json(local / "_CHECKPOINT_METADATA", {"complete": True})
            if str(local) != fs.normalize_path(dir):
                fs.copy_file(local / "_CHECKPOINT_METADATA", fs.join_path(dir, "_CHECKPOINT_METADATA"), save_overwrite=True)

    def save(self, dir: PathOrStr, state: TrainState, overwrite: bool = False) -> None:
        local = self._prepare(dir, overwrite)
        for h in self._write(local, state, block=True):
            h.wait()
        dist_utils.barrier("checkpoint-written")
        self._finalize(local, dir)
        dist_utils.barrier("checkpoint-finalized")

    def save_async(self, dir: PathOrStr, state: TrainState, overwrite: bool = False) -> AsyncSaveHandle:
        local = self._prepare(dir, overwrite)
        handles = self._write(local, state, block=False)

        def finish() -> None:
            # runs on the caller's thread inside AsyncSaveHandle.wait(): barriers stay on the main thread
            dist_utils.barrier("checkpoint-written")
            self._finalize(local, dir)
            dist_utils.barrier("checkpoint-finalized")

        def join_all() -> None:
            for h in handles:
                h.wait()

        handle = AsyncSaveHandle(None, on_done=finish)
        th = threading.Thread(target=lambda: handle._run(join_all), name="checkpoint-finalizer", daemon=True)
        handle._thread, handle._finished = th, False
        th.start()
        return handle

    # ------------------------------------------------------------------ reading
    def load(self, dir: PathOrStr, state: TrainState) -> TrainState:
        local = Path(fs.normalize_path(dir))
        if fs.is_url(dir) and not str(dir).startswith("file://"):
            assert self.work_dir is not None
            digest = hashlib.sha256(str(dir).encode()).hexdigest()[:16]
            local = Path(self.work_dir) / "checkpointer" / digest
            with fs.get_temp_dir_for_target_dir(local) as tmp:
                if dist_utils.get_process_filesystem_rank() == 0:
                    for f in fs.list_directory(dir, recurse=True, include_dirs=False):
                        rel = fs.normalize_path(f)[len(fs.normalize_path(dir)) + 1:]
                        fs.copy_file(f, tmp / rel, save_overwrite=True)
        if not (local / "_CHECKPOINT_METADATA").exists():
            raise FileNotFoundError(f"{local} is not a complete checkpoint (no _CHECKPOINT_METADATA)")
        store = state.model.store
        if (local / "params" / "manifest.ocdbt").exists():
            self._load_ocdbt(local, state)
        else:
            ckpt.restore_sharded(local / "params", store, {"": store.master})
            store.sync_shadow()
            if state.optim is not None and (local / "opt_state").exists():
                sd = state.optim.state_dict()
                scalars = ckpt.restore_sharded(local / "opt_state", store, {"mu": sd["exp_avg"], "nu": sd["exp_avg_sq"]})
                state.optim.count = int(scalars.get("count", 0))
                state.optim.mini_step = int(scalars.get("mini_step", 0))
        tmeta = ckpt.read_json(local / "trainer" / "metadata")
        state.step = int(tmeta["step"])
        state.epoch = int(tmeta["epoch"])
        state.global_train_tokens_seen = tmeta.get("global_train_tokens_seen")
        for item in ("data_loader_state", "callbacks_state"):
            if (local / item / "metadata").exists():
                setattr(state, item, ckpt.read_json(local / item / "metadata"))
        dist_utils.barrier("checkpoint-loaded")
        return state

    def _load_ocdbt(self, local: Path, state: TrainState) -> None:
        from ..checkpoint import orbax_layout as ol

        store = state.model.store
        ol.restore_store_item(local / "params", store, {"": store.master})
        store.sync_shadow()
        opt = state.optim
        if opt is None or not (local / "opt_state" / "manifest.ocdbt").exists():
            return
        sd = opt.state_dict()
        # the optax nesting depends on how the run that wrote the checkpoint was configured (micro-batches, clipping):
        # find the level that holds the Adam moments instead of assuming this run's
        reader = ol.ItemReader(local / "opt_state")
        try:
            names = reader.array_names()
        finally:
            reader.close()
        first = store.metas[0].name
        marker = f"inner_state.0.mu.{first}"
        hits = [n for n in names if n.endswith(marker)]
        if not hits:
            raise KeyError(f"{local / 'opt_state'}: no Adam moments found (looked for '*{marker}')")
        inj = hits[0][: -len(marker)]
        adam = f"{inj}inner_state.0."
        scalars = ol.restore_store_item(local / "opt_state", store, {f"{adam}mu": sd["exp_avg"], f"{adam}nu": sd["exp_avg_sq"]},
                                        scalar_names=[f"{adam}count", "mini_step", "gradient_step"])
        opt.count = int(scalars.get(f"{adam}count", scalars.get("gradient_step", 0)))
        opt.mini_step = int(scalars.get("mini_step", 0))
