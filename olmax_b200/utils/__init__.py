"""
General utilities: logging set-up, exception hook, environment helpers, formatting, polling, running statistics.
Public surface of ``olmax/utils.py:23-246``; the dataclass codec lives in :mod:`olmax_b200.utils.dataclass_codec` and
tensor-tree helpers in :mod:`olmax_b200.utils.tree`.
"""

from __future__ import annotations

import logging
import math
import os
import sys
import time
from datetime import timedelta
from functools import lru_cache
from typing import Callable, Optional

from ..exceptions import OLMaxError

__all__ = [
    "setup_logging",
    "install_excepthook",
    "prepare_cli_environment",
    "set_env_var",
    "log_once",
    "mib_to_bytes",
    "bytes_to_mib",
    "format_scalar",
    "format_float",
    "format_timedelta",
    "wait_for",
    "RunningAverage",
]

log = logging.getLogger(__name__)
_LOGGING_CONFIGURED = False


def _rank_prefix() -> str:
    rank = os.environ.get("RANK")
    return f"[rank {rank}] " if rank is not None and os.environ.get("OLMAX_LOG_RANK_PREFIX", "0") == "1" else ""


def setup_logging(level: int = logging.INFO, force_plain: bool = False) -> None:
    """
    Rich handler when attached to a terminal (or ``OLMAX_RICH_LOGGING=1``), tab-separated plain records otherwise
    (``olmax/utils.py:23-54``).  Safe to call more than once.
    """
    global _LOGGING_CONFIGURED
    handler: logging.Handler
    use_rich = not force_plain and (sys.stderr.isatty() or os.environ.get("OLMAX_RICH_LOGGING") == "1")
    if use_rich:
        try:
            from rich.logging import RichHandler

            handler = RichHandler(show_path=False, rich_tracebacks=False, markup=False)
            handler.setFormatter(logging.Formatter(_rank_prefix() + "%(message)s"))
        except Exception:  # rich missing or broken terminal
            use_rich = False
    if not use_rich:
        handler = logging.StreamHandler(sys.stderr)
        handler.setFormatter(
            logging.Formatter(_rank_prefix() + "%(asctime)s\t%(name)s\t%(levelname)s\t%(message)s", "%Y-%m-%d %H:%M:%S")
        )
    root = logging.getLogger()
    for h in list(root.handlers):
        if getattr(h, "_olmax_handler", False):
            root.removeHandler(h)
    handler._olmax_handler = True  # type: ignore[attr-defined]
    root.addHandler(handler)
    root.setLevel(level)
    logging.captureWarnings(True)
    _LOGGING_CONFIGURED = True


def install_excepthook() -> None:
    """Log uncaught exceptions; framework errors (:class:`OLMaxError`) are logged without a traceback."""

    def hook(exc_type, exc, tb):
        if issubclass(exc_type, KeyboardInterrupt):
            sys.__excepthook__(exc_type, exc, tb)
        elif issubclass(exc_type, OLMaxError):
            log.error("%s: %s", exc_type.__name__, exc)
        else:
            log.critical("Uncaught %s: %s", exc_type.__name__, exc, exc_info=(exc_type, exc, tb))

    sys.excepthook = hook


def prepare_cli_environment(log_level: int = logging.INFO) -> None:
    """Call first in a CLI entry point: exception hook + logging (``olmax/utils.py:106-111``)."""
    install_excepthook()
    setup_logging(log_level)


def set_env_var(name: str, value: str, override: bool = False, secret: bool = False) -> None:
    """Set ``os.environ[name]`` unless it is already set to something else and ``override`` is False."""
    shown = "****" if secret else value
    current = os.environ.get(name)
    if current is not None and current != value:
        if override:
            log.warning("Overriding env var '%s' to '%s'", name, shown)
            os.environ[name] = value
        else:
            log.warning("Env var '%s' already set to '%s'; keeping it", name, "****" if secret else current)
    else:
        os.environ[name] = value


@lru_cache(maxsize=None)
def log_once(logger_name: str, level: int, msg: str) -> None:
    logging.getLogger(logger_name).log(level, msg)


def mib_to_bytes(mib: float) -> int:
    return int(mib * 1024 * 1024)


def bytes_to_mib(n: int) -> float:
    return n / (1024 * 1024)


def format_float(value: float) -> str:
    if value == 0 or not math.isfinite(value):
        return f"{value}"
    mag = abs(value)
    if mag < 1e-4 or mag >= 1e7:
        return f"{value:.3E}"
    if mag >= 1000:
        return f"{int(round(value)):,d}"
    if mag >= 100:
        return f"{value:.1f}"
    if mag >= 10:
        return f"{value:.2f}"
    if mag >= 1:
        return f"{value:.3f}"
    return f"{value:.4f}"


def format_scalar(value) -> str:
    if hasattr(value, "item"):
        value = value.item()
    if isinstance(value, bool):
        return str(value)
    if isinstance(value, int):
        return f"{value:,d}"
    return format_float(float(value))


def format_timedelta(td: timedelta) -> str:
    secs = td.total_seconds()
    if secs < 1:
        return f"{secs * 1000:.0f}ms"
    parts = []
    days, rem = divmod(int(secs), 86400)
    hours, rem = divmod(rem, 3600)
    minutes, seconds = divmod(rem, 60)
    if days:
        parts.append(f"{days}d")
    if hours:
        parts.append(f"{hours}h")
    if minutes:
        parts.append(f"{minutes}m")
    if seconds or not parts:
        parts.append(f"{seconds}s")
    return " ".join(parts)


def wait_for(condition: Callable[[], bool], description: str, timeout: float = 10.0, interval: float = 0.5) -> None:
    """Poll ``condition`` until true; raise ``TimeoutError`` naming ``description`` after ``timeout`` seconds."""
    start = time.monotonic()
    while not condition():
        if time.monotonic() - start > timeout:
            raise TimeoutError(f"{description} timed out after {timeout:.1f}s")
        time.sleep(interval)


class RunningAverage:
    """Streaming mean / variance (Welford).  ``olmax/utils.py:209-246``."""

    def __init__(self) -> None:
        self.n = 0
        self._mean = 0.0
        self._m2 = 0.0

    def update(self, x: float) -> None:
        self.n += 1
        delta = x - self._mean
        self._mean += delta / self.n
        self._m2 += delta * (x - self._mean)

    @property
    def mean(self) -> float:
        if self.n == 0:
            raise ValueError("no samples")
        return self._mean

    @property
    def var(self) -> float:
        if self.n < 2:
            raise ValueError("need at least two samples")
        return self._m2 / (self.n - 1)

    @property
    def std(self) -> float:
        return math.sqrt(self.var)

    def reset(self) -> None:
        self.n, self._mean, self._m2 = 0, 0.0, 0.0
