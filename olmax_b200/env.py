"""
Process-environment configuration applied before the first device use (role of ``olmax/env.py:31-259``).

The reference tunes XLA, NCCL, CUDA and JAX through environment variables.  Here the compute path is our own CUDA
kernels on one process per GPU, so the knobs that matter are :class:`RuntimeConfig` (how the framework overlaps and
fuses communication) plus the NCCL / CUDA variables.  :class:`XLAConfig` and :class:`JAXConfig` are kept so that
configs and command lines written for the reference still parse; the fields with an equivalent here are mapped in
:meth:`EnvConfig.apply` and the others are reported as ignored.
"""

from __future__ import annotations

import dataclasses
import logging
from dataclasses import dataclass
from typing import List, Optional, Tuple

from .types import GPUArchitecture
from .utils import bytes_to_mib, mib_to_bytes, set_env_var

__all__ = ["RuntimeConfig", "XLAConfig", "NCCLConfig", "CUDAConfig", "JAXConfig", "EnvConfig"]

log = logging.getLogger(__name__)


@dataclass
class RuntimeConfig:
    """Knobs of this framework's own runtime."""

    comm_backend: str = "auto"
    """``nccl``: collectives through NCCL; ``fused``: peer-memory kernels fused with the GEMMs; ``auto``: fused when
    symmetric memory is available on every rank of the shard group, else nccl.  Read by the parameter store
    (``OLMAX_B200_COMM_BACKEND``) unless a model is built with an explicit ``comm_backend``."""
    reshard_after_forward: bool = True
    """Free gathered weights after the forward use and gather again for backward (the entrypoint passes it to
    ``TransformerConfig.build``)."""
    peer_barrier: str = "flags"
    """How the peer-memory backend separates its phases: ``flags`` (the bounded flag-word barrier kernel, default) or
    ``nccl`` (a one-element all-reduce); ``OLMAX_B200_BARRIER``."""
    rs_wire: str = "bf16"
    """Format of the partial weight gradients that the fused reduce-scatter stores into the owners' staging slots:
    ``bf16`` (default: half the NVLink bytes and half the fold's reads; each rank's partial sum is rounded once, sums
    and the accumulator stay fp32) or ``fp32``; ``OLMAX_B200_RS_WIRE``.  The reference takes its gradients with respect
    to the bf16 copy of the parameters and casts them to fp32 afterwards (``olmax/train/trainer.py:728-739``), so its
    reduce-scatter moves bf16 as well."""
    peer_wait_timeout_ms: int = 600_000
    """Upper bound of the flag barrier's wait for another GPU (``OLMAX_B200_BARRIER_TIMEOUT_S``); a wait that runs out
    raises on the host instead of hanging the GPU.  The waits inside the GEMMs have a fixed iteration limit."""
    nvtx: bool = True
    """Emit NVTX ranges named like the reference's profiler scopes around the trainer's phases (``OLMAX_B200_NVTX``)."""

    @classmethod
    def recommended(cls, gpu_architecture: Optional[GPUArchitecture] = None, **overrides) -> "RuntimeConfig":
        del gpu_architecture
        return cls(**overrides)

    def apply(self) -> None:
        set_env_var("OLMAX_B200_COMM_BACKEND", self.comm_backend, override=True)
        set_env_var("OLMAX_B200_BARRIER", self.peer_barrier, override=True)
        set_env_var("OLMAX_B200_RS_WIRE", self.rs_wire, override=True)
        set_env_var("OLMAX_B200_BARRIER_TIMEOUT_S", str(self.peer_wait_timeout_ms / 1000.0), override=True)
        set_env_var("OLMAX_B200_NVTX", "1" if self.nvtx else "0", override=True)


@dataclass
class XLAConfig:
    """Accepted for command-line compatibility with the reference; see the module docstring."""

    python_client_mem_fraction: float = 0.95
    gpu_enable_latency_hiding_scheduler: bool = True
    gpu_enable_pipelined_all_gather: bool = True
    gpu_enable_pipelined_reduce_scatter: bool = True
    gpu_enable_pipelined_all_reduce: bool = True
    gpu_enable_all_gather_combine_by_dim: bool = False
    gpu_enable_reduce_scatter_combine_by_dim: bool = False
    gpu_all_gather_combine_threshold_bytes: Optional[int] = None
    gpu_reduce_scatter_combine_threshold_bytes: Optional[int] = None
    gpu_all_reduce_combine_threshold_bytes: Optional[int] = None
    gpu_enable_nccl_user_buffers: bool = False
    gpu_enable_nccl_comm_splitting: bool = True
    gpu_enable_nccl_per_stream_comms: Optional[bool] = None
    gpu_enable_while_loop_double_buffering: bool = True
    gpu_enable_command_buffer: Optional[str] = None
    gpu_enable_triton_gemm: bool = False
    gpu_graph_level: Optional[int] = None
    gpu_enable_highest_priority_async_stream: Optional[bool] = None
    disable_hlo_passes: Optional[str] = None

    @classmethod
    def recommended(cls, gpu_architecture: Optional[GPUArchitecture] = None, **overrides) -> "XLAConfig":
        del gpu_architecture
        return cls(**overrides)

    def _mib(self, name: str) -> Optional[float]:
        v = getattr(self, name)
        return None if v is None else bytes_to_mib(v)

    @property
    def gpu_all_gather_combine_threshold_mib(self) -> Optional[float]:
        return self._mib("gpu_all_gather_combine_threshold_bytes")

    @gpu_all_gather_combine_threshold_mib.setter
    def gpu_all_gather_combine_threshold_mib(self, value: Optional[float]) -> None:
        self.gpu_all_gather_combine_threshold_bytes = None if value is None else mib_to_bytes(value)

    @property
    def gpu_reduce_scatter_combine_threshold_mib(self) -> Optional[float]:
        return self._mib("gpu_reduce_scatter_combine_threshold_bytes")

    @gpu_reduce_scatter_combine_threshold_mib.setter
    def gpu_reduce_scatter_combine_threshold_mib(self, value: Optional[float]) -> None:
        self.gpu_reduce_scatter_combine_threshold_bytes = None if value is None else mib_to_bytes(value)

    @property
    def gpu_all_reduce_combine_threshold_mib(self) -> Optional[float]:
        return self._mib("gpu_all_reduce_combine_threshold_bytes")

    @gpu_all_reduce_combine_threshold_mib.setter
    def gpu_all_reduce_combine_threshold_mib(self, value: Optional[float]) -> None:
        self.gpu_all_reduce_combine_threshold_bytes = None if value is None else mib_to_bytes(value)

    def get_env_flags(self) -> List[str]:
        """The ``--xla_*`` flag strings these settings would stand for (informational)."""
        flags = []
        for f in dataclasses.fields(self):
            if f.name == "python_client_mem_fraction":
                continue
            value = getattr(self, f.name)
            if value is None:
                continue
            text = str(value).lower() if isinstance(value, bool) else str(value)
            flags.append(f"--xla_{f.name}={text}")
        return flags

    def apply(self) -> None:
        non_default = [
            f.name for f in dataclasses.fields(self) if getattr(self, f.name) != getattr(XLAConfig(), f.name)
        ]
        if non_default:
            log.info("XLA settings have no effect in this framework (no XLA): %s", ", ".join(non_default))


@dataclass
class NCCLConfig:
    LL128_buffsize: int = -2
    LL_buffsize: int = -2
    proto: str = "Simple,LL,LL128"
    debug: str = "WARN"
    nvls_enable: Optional[int] = None
    tuner_config_path: Optional[str] = None
    shimnet_guest_config_checker_config_file: Optional[str] = None

    @classmethod
    def recommended(cls, gpu_architecture: Optional[GPUArchitecture] = None, **overrides) -> "NCCLConfig":
        del gpu_architecture
        return cls(**overrides)

    def get_env_vars(self) -> List[Tuple[str, str]]:
        out = []
        for f in dataclasses.fields(self):
            value = getattr(self, f.name)
            if value is not None:
                out.append((f"NCCL_{f.name.upper()}", str(value)))
        return out

    def apply(self) -> None:
        for name, value in self.get_env_vars():
            set_env_var(name, value, override=True)


@dataclass
class CUDAConfig:
    device_max_connections: Optional[int] = None
    module_loading: Optional[str] = None

    @classmethod
    def recommended(cls, gpu_architecture: Optional[GPUArchitecture] = None, **overrides) -> "CUDAConfig":
        # One hardware queue serialises kernel and copy submission order, which helped comm/compute overlap before
        # Blackwell; on Blackwell the default is kept (``olmax/env.py:184-194``).
        if gpu_architecture != GPUArchitecture.blackwell:
            return cls(device_max_connections=1, **overrides)
        return cls(**overrides)

    def get_env_vars(self) -> List[Tuple[str, str]]:
        out = []
        for f in dataclasses.fields(self):
            value = getattr(self, f.name)
            if value is not None:
                out.append((f"CUDA_{f.name.upper()}", str(value)))
        return out

    def apply(self) -> None:
        for name, value in self.get_env_vars():
            set_env_var(name, value, override=True)


@dataclass
class JAXConfig:
    """Accepted for compatibility.  ``disable_jit`` maps to eager debugging (no CUDA graphs); the rest is ignored."""

    disable_jit: Optional[bool] = None
    compiler_enable_remat_pass: Optional[bool] = None
    platforms: Optional[str] = None

    @classmethod
    def recommended(cls, gpu_architecture: Optional[GPUArchitecture] = None, **overrides) -> "JAXConfig":
        if gpu_architecture is not None:
            return cls(platforms="cuda,cpu", **overrides)
        return cls(**overrides)

    def apply(self) -> None:
        if self.disable_jit:
            log.info("jax.disable_jit has no counterpart here (kernels are launched eagerly): ignored")


@dataclass
class EnvConfig:
    xla: XLAConfig = dataclasses.field(default_factory=XLAConfig)
    jax: JAXConfig = dataclasses.field(default_factory=JAXConfig)
    nccl: NCCLConfig = dataclasses.field(default_factory=NCCLConfig)
    cuda: CUDAConfig = dataclasses.field(default_factory=CUDAConfig)
    runtime: RuntimeConfig = dataclasses.field(default_factory=RuntimeConfig)

    @classmethod
    def recommended(cls, gpu_architecture: Optional[GPUArchitecture] = None) -> "EnvConfig":
        return cls(
            xla=XLAConfig.recommended(gpu_architecture),
            jax=JAXConfig.recommended(gpu_architecture),
            nccl=NCCLConfig.recommended(gpu_architecture),
            cuda=CUDAConfig.recommended(gpu_architecture),
            runtime=RuntimeConfig.recommended(gpu_architecture),
        )

    def apply(self) -> None:
        self.xla.apply()
        self.jax.apply()
        self.nccl.apply()
        self.cuda.apply()
        self.runtime.apply()
