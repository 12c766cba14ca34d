"""
Beaker cluster integration (``olmax/launch/beaker.py:1-327``): :class:`BeakerRuntime` reads the ``BEAKER_*``
environment of a running job (replica rank / count, leader host, node GPU type) and derives the distributed config and
environment overrides; :func:`main` submits a command as a multi-replica experiment through ``gantry`` when that
package is installed.  Differences from the reference: one process per GPU, so each replica (node) starts
``local_device_count`` ranks through :mod:`olmax_b200.launch.local` and the global rank is
``replica_rank * local_device_count + local_rank``.
"""

from __future__ import annotations

import argparse
import os
import sys
from dataclasses import dataclass
from typing import List, Optional, Sequence

from ..env import EnvConfig, NCCLConfig
from ..exceptions import OLMaxEnvironmentError
from ..parallel.dist_utils import DistConfig
from ..types import DeviceType, GPUArchitecture

__all__ = ["BeakerRuntime", "main"]

COORDINATOR_PORT = 29400


@dataclass
class BeakerNode:
    hostname: str
    device_type: Optional[DeviceType]
    gpu_count: int


@dataclass
class BeakerRuntime:
    workload_id: str
    replica_rank: int
    replica_count: int
    leader_hostname: str
    node: BeakerNode
    cluster: Optional[str] = None

    @classmethod
    def from_env(cls) -> Optional["BeakerRuntime"]:
        """None outside Beaker."""
        if "BEAKER_JOB_ID" not in os.environ and "BEAKER_WORKLOAD_ID" not in os.environ:
            return None
        gpu_name = os.environ.get("BEAKER_NODE_GPU_TYPE", "")
        device_type = None
        for d in DeviceType:
            if d.value.replace("NVIDIA_", "").replace("_", "").lower() in gpu_name.replace(" ", "").replace("-", "").lower():
                device_type = d
                break
        gpus = int(os.environ.get("BEAKER_ASSIGNED_GPU_COUNT", "0") or 0)
        if gpus == 0:
            try:
                import torch

                gpus = torch.cuda.device_count()
            except Exception:
                gpus = 0
        return cls(
            workload_id=os.environ.get("BEAKER_WORKLOAD_ID", os.environ.get("BEAKER_JOB_ID", "")),
            replica_rank=int(os.environ.get("BEAKER_REPLICA_RANK", "0")),
            replica_count=int(os.environ.get("BEAKER_REPLICA_COUNT", "1")),
            leader_hostname=os.environ.get("BEAKER_LEADER_REPLICA_HOSTNAME", "127.0.0.1"),
            node=BeakerNode(os.environ.get("BEAKER_NODE_HOSTNAME", ""), device_type, gpus),
            cluster=os.environ.get("BEAKER_CLUSTER"),
        )

    @property
    def local_device_count(self) -> int:
        return max(1, self.node.gpu_count)

    @property
    def global_device_count(self) -> int:
        return self.local_device_count * self.replica_count

    def get_dist_config(self, local_rank: int = 0) -> DistConfig:
        return DistConfig(
            coordinator_address=f"{self.leader_hostname}:{COORDINATOR_PORT}",
            num_processes=self.global_device_count,
            process_id=self.replica_rank * self.local_device_count + local_rank,
            local_rank=local_rank,
        )

    def get_env_config(self) -> EnvConfig:
        arch = self.node.device_type.architecture if self.node.device_type is not None else None
        env = EnvConfig.recommended(arch)
        if self.cluster and "augusta" in self.cluster.lower():
            # GCP TCPXO fabric: tuner / shim configuration shipped in the cluster image
            env.nccl = NCCLConfig.recommended(
                arch,
                tuner_config_path="/var/lib/tcpxo/lib64/a3plus_tuner_config_ll128.textproto",
                shimnet_guest_config_checker_config_file="/var/lib/tcpxo/lib64/a3plus_guest_config_ll128.textproto",
            )
        return env

    def set_description(self, description: str) -> None:
        try:
            from beaker import Beaker

            Beaker.from_env().workload.update(self.workload_id, description=description)
        except Exception:
            pass


def main(argv: Optional[Sequence[str]] = None) -> None:
    parser = argparse.ArgumentParser(prog="python -m olmax_b200.launch.beaker",
                                     usage="python -m olmax_b200.launch.beaker [OPTIONS] -- CMD ...")
    parser.add_argument("--name", default="olmax-b200")
    parser.add_argument("--gpus", type=int, default=8)
    parser.add_argument("--nodes", type=int, default=1)
    parser.add_argument("--gpu-type", default="b200", choices=["b200", "h100", "a100"])
    parser.add_argument("--cluster", action="append", default=None)
    parser.add_argument("--workspace", default=None)
    parser.add_argument("--budget", default=None)
    parser.add_argument("--priority", default="normal")
    parser.add_argument("--debug", action="store_true")
    parser.add_argument("cmd", nargs=argparse.REMAINDER)
    opts = parser.parse_args(argv)
    cmd: List[str] = opts.cmd[1:] if opts.cmd and opts.cmd[0] == "--" else opts.cmd
    if not cmd:
        parser.error("no command given")
    try:
        from gantry.api import launch_experiment
    except ImportError as e:
        raise OLMaxEnvironmentError("submitting to Beaker needs the beaker-gantry package, which is not installed") from e
    launch_experiment(
        args=cmd, name=opts.name, gpus=opts.gpus, replicas=opts.nodes if opts.nodes > 1 else None,
        leader_selection=opts.nodes > 1, host_networking=opts.nodes > 1, propagate_failure=opts.nodes > 1,
        propagate_preemption=opts.nodes > 1, synchronized_start_timeout="5m" if opts.nodes > 1 else None,
        clusters=opts.cluster, workspace=opts.workspace, budget=opts.budget, priority=opts.priority,
        env_secrets=["BEAKER_TOKEN"], env_vars=[("OLMAX_B200_DEBUG", "1")] if opts.debug else None,
    )


if __name__ == "__main__":
    main()
