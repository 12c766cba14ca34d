"""
Trainer-level checkpointing (``olmax/train/checkpointer.py:26-283``): a checkpoint is a directory
``save_folder/step{N}`` with the items ``trainer`` (JSON: step, epoch, tokens seen), ``params``, ``opt_state``,
``data_loader_state`` and ``callbacks_state``; it is written locally first and then copied to the save folder by
file-system rank 0 when that is a different (e.g. remote) location; saves can be asynchronous with a finalizer that
uploads and signals completion; loads from a URL are staged through a hashed work directory.
"""

from __future__ import annotations

import hashlib
import logging
import shutil
import threading
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
    def _local_dir(self, dir: PathOrStr) -> Path:
        if fs.is_url(dir) and not str(dir).startswith("file://"):
            assert self.work_dir is not None, "work_dir is required to stage remote checkpoints"
            return Path(self.work_dir) / Path(str(dir).rstrip("/")).name
        return Path(fs.normalize_path(dir))

    def _write(self, local: Path, state: TrainState, block: bool) -> list:
        store = state.model.store
        handles = []
        if dist_utils.get_rank() == 0:
            ckpt.write_json(local / "trainer" / "metadata", {
                "step": state.step, "epoch": state.epoch, "global_train_tokens_seen": state.global_train_tokens_seen})
            ckpt.write_json(local / "data_loader_state" / "metadata", state.data_loader_state)
            ckpt.write_json(local / "callbacks_state" / "metadata", state.callbacks_state)
        handles.append(ckpt.save_sharded(local / "params", store, {"": store.master}, block=block))
        opt = state.optim
        if opt is not None:
            sd = opt.state_dict()
            handles.append(ckpt.save_sharded(local / "opt_state", store, {"mu": sd["exp_avg"], "nu": sd["exp_avg_sq"]},
                                             scalars={"count": sd["count"], "mini_step": sd["mini_step"]}, block=block))
        return handles

    def _prepare(self, dir: PathOrStr, overwrite: bool) -> Path:
        local = self._local_dir(dir)
        if dist_utils.get_process_filesystem_rank() == 0:
            if local.exists() and any(local.iterdir()):
                if not overwrite:
                    raise FileExistsError(f"checkpoint directory {local} already exists (save_overwrite=False)")
                shutil.rmtree(local)
            local.mkdir(parents=True, exist_ok=True)
        dist_utils.barrier("checkpoint-dir")
        return local

    def _finalize(self, local: Path, dir: PathOrStr) -> None:
        if str(local) != fs.normalize_path(dir) and dist_utils.get_process_filesystem_rank() == 0:
            fs.copy_dir(local, dir, save_overwrite=True)
        if dist_utils.get_rank() == 0:
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
        state.data_loader_state = ckpt.read_json(local / "data_loader_state" / "metadata")
        state.callbacks_state = ckpt.read_json(local / "callbacks_state" / "metadata")
        dist_utils.barrier("checkpoint-loaded")
        return state
