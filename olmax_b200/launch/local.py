"""
Local launcher: start one process per GPU (or per CPU rank) on this host and run a module or script in each, with the
torchrun-style environment the framework reads (``RANK``, ``LOCAL_RANK``, ``WORLD_SIZE``, ``LOCAL_WORLD_SIZE``,
``MASTER_ADDR=127.0.0.1``, ``MASTER_PORT``).  A rank that exits non-zero takes the others down, the first failure's
code is returned, and SIGINT / SIGTERM are forwarded so trainers can checkpoint and stop.

    python -m olmax_b200.launch.local --nproc 8 -- -m olmax_b200.launch.train_transformer --recipe=olmo2_7B_bench
"""

from __future__ import annotations

import argparse
import os
import signal
import socket
import subprocess
import sys
import time
from typing import List, Optional, Sequence

__all__ = ["find_free_port", "launch", "main"]


def find_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launch(cmd: Sequence[str], nproc: int, port: Optional[int] = None, env_extra: Optional[dict] = None,
           poll_interval: float = 0.2) -> int:
    port = port or find_free_port()
    procs: List[subprocess.Popen] = []
    for rank in range(nproc):
        env = dict(os.environ)
        env.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(nproc), "LOCAL_WORLD_SIZE": str(nproc),
                    "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
        env.update(env_extra or {})
        procs.append(subprocess.Popen([sys.executable, *cmd], env=env))

    def forward(signum, frame):
        del frame
        for p in procs:
            if p.poll() is None:
                p.send_signal(signum)

    old = {s: signal.signal(s, forward) for s in (signal.SIGINT, signal.SIGTERM)}
    rc = 0
    try:
        alive = set(range(nproc))
        while alive:
            for i in list(alive):
                code = procs[i].poll()
                if code is None:
                    continue
                alive.discard(i)
                if code != 0 and rc == 0:
                    rc = code
                    for j in alive:
                        procs[j].terminate()
            time.sleep(poll_interval)
    finally:
        for s, h in old.items():
            signal.signal(s, h)
        for p in procs:
            if p.poll() is None:
                p.kill()
    return rc


def main(argv: Optional[Sequence[str]] = None) -> int:
    parser = argparse.ArgumentParser(prog="python -m olmax_b200.launch.local")
    parser.add_argument("--nproc", type=int, required=True, help="processes (= GPUs) to start on this host")
    parser.add_argument("--port", type=int, default=None)
    parser.add_argument("cmd", nargs=argparse.REMAINDER, help="-- followed by python arguments (e.g. -m package.module ...)")
    opts = parser.parse_args(argv)
    cmd = opts.cmd[1:] if opts.cmd and opts.cmd[0] == "--" else opts.cmd
    if not cmd:
        parser.error("no command given")
    return launch(cmd, opts.nproc, opts.port)


if __name__ == "__main__":
    sys.exit(main())
