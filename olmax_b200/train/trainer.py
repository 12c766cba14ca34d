"""
The training loop (``olmax/train/trainer.py:72-939``).

``Trainer.fit(model, data_loader)`` runs epochs of batches; a batch is a sequence of micro-batches and one optimizer
step.  Per micro-batch the inputs are copied host-to-device from pinned memory, the model's fused forward / loss /
backward runs on the hand-written kernels, and weight gradients accumulate into the sharded fp32 buffer; after the last
micro-batch the cross-replica all-reduce (HSDP / DDP) and the fused AdamW run once.  Everything else mirrors the
reference: callbacks sorted by priority, metrics recorded as device scalars and flushed one step late so the loop never
waits for the step in flight, throughput metrics, a NaN check, SIGTERM / SIGINT graceful cancellation propagated over the
host-side process group, garbage-collection control, periodic (optionally asynchronous) checkpoints with automatic
resume from the newest ``step{N}`` directory, and persistence of working files to the save folder.
"""

from __future__ import annotations

import dataclasses
import fnmatch
import gc
import logging
import math
import os
import re
import signal
import time
from collections import OrderedDict
from dataclasses import dataclass, field
from datetime import timedelta
from pathlib import Path
from typing import Any, Callable, Dict, Iterator, List, Optional, Sequence, Tuple, Type, Union

import torch
import torch.distributed as dist

from .. import fs, utils
from ..checkpoint.utils import AsyncSaveHandle
from ..data.data_loader import DataLoader
from ..exceptions import CallbackExistsError
from ..optim.config import OptimConfig
from ..parallel import dist_utils
from ..parallel.mesh import MeshResource
from ..types import Duration, PathOrStr
from ..utils.tree import get_peak_local_device_memory_usage
from .callbacks.callback import Callback
from .checkpointer import Checkpointer, SimpleCheckpointer, TrainState

__all__ = ["Trainer", "TrainMetrics", "TrainState"]

log = logging.getLogger(__name__)


class TrainMetrics:
    loss = "train/loss"
    z_loss = "train/z_loss"
    lr = "optim/lr"
    g_norm = "optim/g_norm"


def _nvtx(name: str):
    """NVTX range around a trainer phase (names as in the reference's profiler scopes); ``OLMAX_B200_NVTX=0`` disables."""
    if torch.cuda.is_available() and os.environ.get("OLMAX_B200_NVTX", "1") == "1":
        return torch.cuda.nvtx.range(name)
    import contextlib

    return contextlib.nullcontext()


@dataclass
class Trainer:
    work_dir: PathOrStr
    save_folder: PathOrStr
    optim: OptimConfig
    loss_fun: Optional[Callable[[Any, Any, Any], torch.Tensor]] = None
    """``loss_fun(model, micro_batch, buffer_cache) -> scalar``; default: ``model(ids, labels, cache)[0]``."""
    mesh: Optional[MeshResource] = None
    grad_dtype: str = "float32"
    compute_dtype: str = "bfloat16"
    callbacks: "OrderedDict[str, Callback]" = field(default_factory=OrderedDict)
    checkpointer: Checkpointer = field(default_factory=SimpleCheckpointer)
    async_checkpointing: bool = True
    checkpoint_interval: Optional[int] = None
    cancel_check_interval: int = 5
    gc_interval: int = 1000
    max_duration: Duration = field(default_factory=lambda: Duration.epochs(1))
    global_tokens_per_batch: Union[int, Callable[[Sequence[Any]], int], None] = None
    log_to_console: Sequence[str] = (
        "train/loss", "optim/lr", "optim/g_norm", "system/*", "throughput/data loading*", "throughput/TPS device*",
    )
    save_overwrite: bool = False
    z_loss_multiplier: float = 0.0

    def __post_init__(self):
        self.work_dir = Path(self.work_dir)
        self.work_dir.mkdir(parents=True, exist_ok=True)
        if not fs.is_url(self.save_folder):
            self.save_folder = Path(fs.normalize_path(self.save_folder))
            self.save_folder.mkdir(parents=True, exist_ok=True)
        self.checkpointer.work_dir = self.work_dir
        self._step = 0
        self._step_this_run = 0
        self._epoch = 1
        self._metrics: "OrderedDict[int, Dict[str, Any]]" = OrderedDict()
        self._kernel_status: Dict[int, Any] = {}   # step -> pending copy of the kernels' status words
        self._canceled = False
        self._canceled_synced = False
        self._cancel_reason: Optional[str] = None
        self._error: Optional[BaseException] = None
        self._tokens_seen: Optional[int] = None
        self._bps = utils.RunningAverage()
        self._last_checkpoint = -1
        self._save_handle: Optional[AsyncSaveHandle] = None
        self._model = None
        self._optimizer = None
        self._cache = None
        self._data_loader: Optional[DataLoader] = None
        self._old_handlers: Dict[int, Any] = {}
        for cb in self.callbacks.values():
            cb.trainer = self
        self._sort_callbacks()
        for cb in self._iter_callbacks():
            cb.post_attach()

    # ------------------------------------------------------------------ callbacks
    def _sort_callbacks(self) -> None:
        items = list(self.callbacks.items())
        order = sorted(range(len(items)), key=lambda i: (-items[i][1].priority, i))
        self.callbacks = OrderedDict(items[i] for i in order)

    def _iter_callbacks(self) -> Iterator[Callback]:
        for cb in self.callbacks.values():
            if cb.enabled:
                yield cb

    def add_callback(self, name: str, callback: Callback) -> "Trainer":
        if name in self.callbacks:
            raise CallbackExistsError(f"A callback with name '{name}' already exists!")
        callback.trainer = self
        self.callbacks[name] = callback
        self._sort_callbacks()
        if callback.enabled:
            callback.post_attach()
        return self

    def has_callback(self, cb_class: Type[Callback]) -> bool:
        return any(isinstance(cb, cb_class) for cb in self.callbacks.values())

    # ------------------------------------------------------------------ properties
    @property
    def step(self) -> int:
        return self._step

    @property
    def epoch(self) -> int:
        return self._epoch

    @property
    def global_train_tokens_seen(self) -> Optional[int]:
        return self._tokens_seen

    @property
    def model(self):
        return self._model

    @property
    def optimizer(self):
        return self._optimizer

    @property
    def is_canceled(self) -> bool:
        if self._error is not None:
            raise RuntimeError("An error occurred") from self._error
        return self._canceled

    @property
    def training_complete(self) -> bool:
        if self._error is not None:
            raise RuntimeError("An error occurred") from self._error
        if self._canceled_synced:
            return True
        return self.max_duration.due(step=self._step, tokens=self._tokens_seen, epoch=self._epoch)

    def cancel_run(self, reason: str) -> None:
        """Ask for a graceful stop: the loop ends after the current step on every rank (at the next cancel check)."""
        if not self._canceled:
            log.warning("Canceling run: %s", reason)
        self._canceled = True
        self._cancel_reason = reason

    # ------------------------------------------------------------------ metrics
    def record_metric(self, name: str, value: Any, step: Optional[int] = None) -> None:
        """Store a metric for ``step`` (default: current).  Device scalars are copied to the host asynchronously and
        only read when the step is flushed, one step later."""
        step = self._step if step is None else step
        if isinstance(value, torch.Tensor):
            value = value.detach()
            if value.is_cuda:
                host = torch.empty((), dtype=value.dtype, pin_memory=True)
                host.copy_(value.reshape(()), non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
                value = (host, ev)
        self._metrics.setdefault(step, OrderedDict())[name] = value

    @staticmethod
    def _resolve(value: Any) -> float:
        if isinstance(value, tuple):
            host, ev = value
            ev.synchronize()
            return float(host.item())
        if isinstance(value, torch.Tensor):
            return float(value.item())
        return float(value)

    def _record_kernel_status(self) -> None:
        """Queue a copy of the kernel library's status words behind this step's work.  A kernel whose bounded wait ran
        out (operands that never arrived from a peer, a barrier a peer never reached) tears down and returns, so the
        step itself completes; the words are the only trace, and a step that produced them has computed garbage."""
        from ..ops import _lib

        self._kernel_status[self._step] = _lib.snapshot_status(self._model.store.device)

    def _check_kernel_status(self, exclude_current: bool = True) -> None:
        """Raise :class:`~olmax_b200.ops._lib.KernelError` for the oldest recorded step whose status words show a
        failure: one step late (no synchronisation), and always before a checkpoint of a later step is written."""
        from ..ops import _lib

        for step in sorted(self._kernel_status):
            if exclude_current and step == self._step:
                continue
            snap = self._kernel_status.pop(step)
            try:
                _lib.resolve_status(snap)
            except _lib.KernelError as e:
                raise _lib.KernelError(f"step {step}: {e}") from None

    def _log_metrics(self, exclude_current: bool = True) -> None:
        self._check_kernel_status(exclude_current)
        for step in list(self._metrics):
            if exclude_current and step == self._step:
                continue
            raw = self._metrics.pop(step)
            metrics = {k: self._resolve(v) for k, v in raw.items()}
            loss = metrics.get(TrainMetrics.loss)
            if loss is not None and not math.isfinite(loss):
                raise RuntimeError(f"{TrainMetrics.loss} is {loss} at step {step}")
            shown = [f"{k}={utils.format_float(v)}" for k, v in metrics.items()
                     if any(k == p or fnmatch.fnmatch(k, p) for p in self.log_to_console)]
            if dist_utils.get_rank() == 0:
                log.info("[step=%d/%s] %s", step, self._max_steps_str(), "  ".join(shown))
            for cb in self._iter_callbacks():
                cb.log_metrics(step, metrics)

    def _max_steps_str(self) -> str:
        return str(self.max_duration.value) if self.max_duration.unit.value == "steps" else f"{self.max_duration.value} {self.max_duration.unit}"

    # ------------------------------------------------------------------ cancellation / signals
    def _synchronize_cancellation(self) -> None:
        flag = torch.tensor([1 if self._canceled else 0], dtype=torch.int32)
        group = dist_utils.control_group()
        if group is not None:
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
        self._canceled_synced = bool(flag.item())
        if self._canceled_synced and not self._canceled:
            self.cancel_run("canceled on another rank")

    def _install_signal_handlers(self) -> None:
        def handler(signum, frame):
            del frame
            self.cancel_run(f"received signal {signal.Signals(signum).name}")

        for sig in (signal.SIGTERM, signal.SIGINT):
            try:
                self._old_handlers[sig] = signal.signal(sig, handler)
            except ValueError:  # not the main thread
                pass

    def _restore_signal_handlers(self) -> None:
        for sig, old in self._old_handlers.items():
            try:
                signal.signal(sig, old)
            except ValueError:
                pass
        self._old_handlers.clear()

    # ------------------------------------------------------------------ the optimizer step
    def _default_loss(self, model, micro_batch, cache):
        ids, labels = micro_batch
        loss, z = model(ids, labels, cache, z_loss_multiplier=self.z_loss_multiplier)
        return loss

    def _to_device(self, micro_batch: Any) -> Any:
        dev = self._model.store.device
        if isinstance(micro_batch, (tuple, list)):
            return type(micro_batch)(self._to_device(t) for t in micro_batch)
        if isinstance(micro_batch, torch.Tensor):
            return micro_batch.to(dev, non_blocking=True)
        return micro_batch

    def setup(self, model, num_microbatches: int = 1, buffer_cache: Any = None) -> "Trainer":
        """Attach a model and build its optimizer without entering :meth:`fit`, so that :meth:`train_batch` can be
        driven step by step (benchmarks, notebooks)."""
        self._model = model
        self._cache = buffer_cache
        self._optimizer = self.optim.build(model, num_microbatches)
        return self

    def train_batch(self, batch: Sequence[Any]) -> torch.Tensor:
        """One optimizer step over the micro-batches of ``batch`` (host tensors, ideally pinned).  Returns the mean
        loss over the micro-batches and over all ranks (the global-batch loss, as the reference reports it) as a
        device scalar; the host is not synchronised (the cross-rank mean is one asynchronous scalar all-reduce)."""
        model, optim = self._model, self._optimizer
        if len(batch) != optim.num_microbatches:
            optim.num_microbatches = len(batch)
            optim.update_grad_scale()
        loss_fun = self.loss_fun or self._default_loss
        total = None
        for micro_batch in batch:
            with _nvtx("process_microbatch"):
                mb = self._to_device(micro_batch)
                with _nvtx("compute_loss_and_grads"):
                    loss = loss_fun(model, mb, self._cache)
                    loss.backward()
                optim.accumulate()
                total = loss.detach() if total is None else total + loss.detach()
        with _nvtx("step_optimizer"):
            optim.step()
        mean = total / len(batch)
        world = dist_utils.get_world_size()
        if world > 1 and dist.is_initialized():
            dist.all_reduce(mean)
            mean = mean / world
        return mean

    # ------------------------------------------------------------------ fit
    def fit(self, model, data_loader: DataLoader, load_path: Optional[PathOrStr] = None, buffer_cache: Any = None):
        self._model = model
        self._cache = buffer_cache
        self._data_loader = data_loader
        dist_utils.barrier("pre-train-setup")
        gc_was_enabled = gc.isenabled()
        gc.disable()
        self._install_signal_handlers()
        try:
            batches = iter(data_loader)
            first_batch = next(batches)
            k = len(first_batch)
            self._optimizer = self.optim.build(model, k)
            if load_path is None:
                load_path = self._find_latest_checkpoint()
            if load_path is not None:
                self._restore_checkpoint(load_path)
                batches = iter(data_loader)
                first_batch = next(batches)
            elif self.checkpoint_interval is not None:
                self._save_checkpoint(block=True)
            for cb in self._iter_callbacks():
                cb.pre_train()
            dist_utils.barrier("pre-train-loop")
            pending = first_batch
            while not self.training_complete:
                pending, batches = self._fit_epoch(pending, batches, data_loader)
                if pending is None and not self.training_complete:
                    self._epoch += 1
                    batches = iter(data_loader)
                    try:
                        pending = next(batches)
                    except StopIteration:
                        break
            for cb in self._iter_callbacks():
                cb.post_train()
            if self.checkpoint_interval is not None and self._last_checkpoint != self._step:
                self._save_checkpoint(block=True)
            self._shutdown(wait=True)
        except BaseException as exc:  # noqa: BLE001
            self._error = exc if not isinstance(exc, KeyboardInterrupt) else None
            for cb in self._iter_callbacks():
                try:
                    cb.on_error(exc)
                except Exception:  # pragma: no cover
                    log.exception("callback on_error failed")
            self._shutdown(wait=False)
            raise
        finally:
            self._restore_signal_handlers()
            if gc_was_enabled:
                gc.enable()
        return model

    def _fit_epoch(self, pending, batches, data_loader):
        for cb in self._iter_callbacks():
            cb.pre_epoch()
        last_time = time.perf_counter()
        batch = pending
        while batch is not None and not self.training_complete:
            self._step += 1
            self._step_this_run += 1
            if self._step_this_run % self.cancel_check_interval == 0:
                self._synchronize_cancellation()
            for cb in self._iter_callbacks():
                cb.pre_step()
            for cb in self._iter_callbacks():
                cb.pre_load_batch()
            for cb in self._iter_callbacks():
                cb.post_load_batch(batch)
            with _nvtx("train_batch"):
                loss = self.train_batch(batch)
            self.record_metric(TrainMetrics.loss, loss)
            self._record_kernel_status()
            self.record_metric(TrainMetrics.lr, self._optimizer.last_lr)
            if self._optimizer.grad_norm is not None:
                self.record_metric(TrainMetrics.g_norm, self._optimizer.grad_norm)
            peak = get_peak_local_device_memory_usage()
            if peak is not None:
                self.record_metric("system/peak device mem usage (MiB)", peak / 2**20)
            if self.global_tokens_per_batch is not None:
                n = self.global_tokens_per_batch(batch) if callable(self.global_tokens_per_batch) else self.global_tokens_per_batch
                self._tokens_seen = (self._tokens_seen or 0) + int(n)
            for cb in self._iter_callbacks():
                cb.post_train_batch()
            with _nvtx("log_metrics"):
                self._log_metrics(exclude_current=True)
            if self._step_this_run % self.gc_interval == 0:
                gc.collect()
            for cb in self._iter_callbacks():
                cb.post_step()
            self._poll_checkpoint()
            now = time.perf_counter()
            self._record_throughput(now - last_time, batch)
            last_time = now
            # checkpoint BEFORE the next batch is drawn, so that the saved data-loader state points at it
            if self.checkpoint_interval is not None and self._step % self.checkpoint_interval == 0:
                self._save_checkpoint(block=not self.async_checkpointing)
            t_load = time.perf_counter()
            with _nvtx("load_batch"):
                try:
                    nxt = next(batches)
                except StopIteration:
                    nxt = None
            self.record_metric("throughput/data loading time (s)", time.perf_counter() - t_load, step=self._step)
            batch = nxt
        for cb in self._iter_callbacks():
            cb.post_epoch()
        return batch, batches

    def _record_throughput(self, dt: float, batch: Sequence[Any]) -> None:
        if self._step_this_run == 1:
            log.info("First step (includes kernel-library load and allocator warm-up) took %s",
                     utils.format_timedelta(timedelta(seconds=dt)))
            return
        bps = 1.0 / max(dt, 1e-9)
        self.record_metric("throughput/BPS", bps)
        if self._step_this_run > 10:
            self._bps.update(bps)
            self.record_metric("throughput/BPS average", self._bps.mean)
            if self._bps.n >= 5:
                self.record_metric("throughput/BPS stddev", self._bps.std)
        if self.global_tokens_per_batch is not None:
            n = self.global_tokens_per_batch(batch) if callable(self.global_tokens_per_batch) else self.global_tokens_per_batch
            devices = dist_utils.get_global_device_count()
            self.record_metric("throughput/TPS", bps * n)
            self.record_metric("throughput/TPS device", bps * n / devices)
            if self._bps.n >= 1:
                self.record_metric("throughput/TPS average", self._bps.mean * n)
                self.record_metric("throughput/TPS device average", self._bps.mean * n / devices)
            if self._bps.n >= 5:
                self.record_metric("throughput/TPS stddev", self._bps.std * n)
                self.record_metric("throughput/TPS device stddev", self._bps.std * n / devices)

    def _shutdown(self, wait: bool) -> None:
        try:
            if wait:
                self._log_metrics(exclude_current=False)
                self._maybe_wait_for_checkpoint()
            elif self._save_handle is not None and dist_utils.get_world_size() == 1:
                # error path of a single-process run: a save that was in flight is still completed and finalized
                # (with several ranks the finalization needs barriers the failing job can no longer promise)
                try:
                    self._maybe_wait_for_checkpoint()
                except Exception:  # pragma: no cover
                    log.exception("finalizing the in-flight checkpoint failed")
        finally:
            for cb in self._iter_callbacks():
                try:
                    cb.close()
                except Exception:  # pragma: no cover
                    log.exception("callback close failed")
        if wait:
            dist_utils.barrier("shutdown")

    # ------------------------------------------------------------------ checkpoints
    def _poll_checkpoint(self) -> None:
        """Finalize an asynchronous save as soon as every rank's writer thread has finished (agreed over the host
        control group, one small gather per step while a save is in flight) instead of at the next save: the
        checkpoint becomes visible to ``_find_latest_checkpoint`` within a step of being written."""
        if self._save_handle is None:
            return
        done = bool(self._save_handle.done())
        if dist_utils.get_world_size() > 1:
            done = all(dist_utils.allgather_value(done))
        if done:
            self._maybe_wait_for_checkpoint()

    def _maybe_wait_for_checkpoint(self) -> None:
        if self._save_handle is not None:
            handle, self._save_handle = self._save_handle, None
            handle.wait()
            for cb in self._iter_callbacks():
                cb.post_checkpoint_saved(str(self._last_checkpoint_path))

    def _get_state(self) -> TrainState:
        return TrainState(
            step=self._step, epoch=self._epoch, global_train_tokens_seen=self._tokens_seen, model=self._model,
            optim=self._optimizer,
            data_loader_state=self._data_loader.get_state() if self._data_loader is not None else {},
            callbacks_state={name: cb.get_state() for name, cb in self.callbacks.items()},
        )

    def _save_checkpoint(self, block: bool) -> None:
        self._maybe_wait_for_checkpoint()
        path = fs.join_path(self.save_folder, f"step{self._step}")
        self._last_checkpoint_path = path
        log.info("Saving checkpoint for step %d to %s", self._step, path)
        state = self._get_state()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        # nothing is written from a state that a failed kernel may have corrupted (this step's words included)
        self._check_kernel_status(exclude_current=False)
        if block:
            self.checkpointer.save(path, state, overwrite=self.save_overwrite)
            for cb in self._iter_callbacks():
                cb.post_checkpoint_saved(str(path))
        else:
            self._save_handle = self.checkpointer.save_async(path, state, overwrite=self.save_overwrite)
        self._last_checkpoint = self._step

    def _find_latest_checkpoint(self) -> Optional[PathOrStr]:
        best, best_step = None, -1
        for entry in fs.list_directory(self.save_folder):
            m = re.match(r"^step(\d+)$", Path(fs.normalize_path(entry)).name)
            if m and int(m.group(1)) > best_step and fs.file_exists(fs.join_path(entry, "_CHECKPOINT_METADATA")):
                best, best_step = entry, int(m.group(1))
        return dist_utils.synchronize_value(best)

    def _restore_checkpoint(self, path: PathOrStr) -> None:
        log.info("Restoring checkpoint from %s", path)
        state = self.checkpointer.load(path, self._get_state())
        self._step = state.step
        self._epoch = state.epoch
        self._tokens_seen = state.global_train_tokens_seen
        self._last_checkpoint = state.step
        if self._data_loader is not None and state.data_loader_state:
            self._data_loader.load_state(state.data_loader_state)
        for name, cb_state in state.callbacks_state.items():
            if name in self.callbacks:
                self.callbacks[name].load_state(cb_state)
        for cb in self._iter_callbacks():
            cb.post_checkpoint_loaded(str(path))

    # ------------------------------------------------------------------ working files
    def persist_working_file(self, name: PathOrStr) -> Optional[PathOrStr]:
        """Copy ``work_dir/name`` to ``save_folder/name`` (file-system rank 0 only)."""
        src = Path(self.work_dir) / name
        dst = fs.join_path(self.save_folder, str(name))
        if fs.normalize_path(src) == fs.normalize_path(dst) or not src.is_file():
            return dst
        if dist_utils.get_process_filesystem_rank() == 0:
            fs.copy_file(src, dst, save_overwrite=True)
        return dst

    def persist_working_subdir(self, name: PathOrStr) -> Optional[PathOrStr]:
        src = Path(self.work_dir) / name
        dst = fs.join_path(self.save_folder, str(name))
        if fs.normalize_path(src) == fs.normalize_path(dst) or not src.is_dir():
            return dst
        if dist_utils.get_process_filesystem_rank() == 0:
            fs.copy_dir(src, dst, save_overwrite=True)
        return dst

    def write_file(self, name: str, contents: str) -> PathOrStr:
        path = Path(self.work_dir) / name
        if path.exists() and not self.save_overwrite:
            raise FileExistsError(path)
        fs.write_text(path, contents)
        return self.persist_working_file(name)
