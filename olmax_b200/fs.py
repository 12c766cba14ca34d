"""
File-system abstraction over local paths and remote URLs (public surface of ``olmax/fs.py:27-519``).

Local paths and ``file://`` URLs are fully implemented with the standard library.  ``gs://``, ``s3://``, ``r2://``,
``weka://`` and ``http(s)://`` go through back-ends that import their SDK (google-cloud-storage, boto3, requests)
only when first used and raise :class:`OLMaxEnvironmentError` when it is missing, so the framework imports and runs
without any cloud dependency.  Every remote call is wrapped in :func:`retriable` (3 attempts, exponential back-off
capped at 3 s), like the reference.
"""

from __future__ import annotations

import abc
import concurrent.futures
import functools
import io
import logging
import os
import re
import shutil
import tempfile
import time
from pathlib import Path
from typing import Callable, Generator, List, Optional, Tuple, TypeVar, Union
from urllib.parse import urlparse

from .exceptions import OLMaxEnvironmentError, OLMaxNetworkError, OLMaxUploadError
from .types import PathOrStr

__all__ = [
    "normalize_path", "is_url", "join_path", "get_file_size", "get_bytes_range", "upload", "copy_file", "copy_dir",
    "dir_is_empty", "file_exists", "remove_file", "clear_directory", "list_directory", "glob_directory",
    "get_temp_dir_for_target_dir", "init_client", "retriable", "read_text", "write_text",
]

log = logging.getLogger(__name__)
F = TypeVar("F", bound=Callable)

_REMOTE_SCHEMES = ("gs", "s3", "r2", "weka", "http", "https")


# ----------------------------------------------------------------------------------------------------------------------
# path helpers
# ----------------------------------------------------------------------------------------------------------------------
def is_url(path: PathOrStr) -> bool:
    return re.match(r"^[a-z0-9]+://.*", str(path)) is not None


def normalize_path(path: PathOrStr) -> str:
    """String form without a trailing slash; ``file://`` is stripped so that local URLs become plain paths."""
    s = str(path).rstrip("/") if str(path) not in ("/",) else "/"
    if s.startswith("file://"):
        s = s[len("file://"):]
    return s


def join_path(base: PathOrStr, *parts: PathOrStr) -> Union[Path, str]:
    if is_url(base):
        out = normalize_path(base)
        for p in parts:
            out = f"{out}/{str(p).strip('/')}"
        return out
    return Path(normalize_path(base)).joinpath(*[str(p) for p in parts])


def _split(url: str) -> Tuple[str, str, str]:
    p = urlparse(url)
    return p.scheme, p.netloc, p.path.lstrip("/")


# ----------------------------------------------------------------------------------------------------------------------
# retry
# ----------------------------------------------------------------------------------------------------------------------
def retriable(max_attempts: int = 3, retriable_errors: Tuple[type, ...] = (OSError, OLMaxNetworkError),
              retry_condition: Optional[Callable[[Exception], bool]] = None, max_backoff: float = 3.0):
    """Retry the wrapped call on the given errors with exponential back-off (0.5 s, 1 s, 2 s ... capped)."""

    def decorator(fn: F) -> F:
        @functools.wraps(fn)
        def wrapped(*args, **kwargs):
            attempt = 0
            while True:
                attempt += 1
                try:
                    return fn(*args, **kwargs)
                except retriable_errors as e:  # type: ignore[misc]
                    if isinstance(e, (FileNotFoundError, FileExistsError, IsADirectoryError, NotADirectoryError)):
                        raise
                    if retry_condition is not None and not retry_condition(e):
                        raise
                    if attempt >= max_attempts:
                        raise
                    delay = min(0.5 * 2 ** (attempt - 1), max_backoff)
                    log.warning("%s failed (attempt %d/%d): %s; retrying in %.1fs", fn.__name__, attempt, max_attempts, e, delay)
                    time.sleep(delay)

        return wrapped  # type: ignore[return-value]

    return decorator


# ----------------------------------------------------------------------------------------------------------------------
# remote back-ends (lazy)
# ----------------------------------------------------------------------------------------------------------------------
class _Backend(abc.ABC):
    """What a remote store has to offer; ``bucket`` / ``key`` are the host and path parts of the URL."""

    @abc.abstractmethod
    def size(self, bucket: str, key: str) -> int: ...

    @abc.abstractmethod
    def read_range(self, bucket: str, key: str, start: int, n: int) -> bytes: ...

    @abc.abstractmethod
    def exists(self, bucket: str, key: str) -> bool: ...

    def upload(self, src: Path, bucket: str, key: str, overwrite: bool) -> None:
        raise OLMaxUploadError(f"{type(self).__name__} is read-only")

    def remove(self, bucket: str, key: str) -> None:
        raise OLMaxUploadError(f"{type(self).__name__} is read-only")

    def list(self, bucket: str, prefix: str, recursive: bool) -> List[str]:
        raise OLMaxNetworkError(f"{type(self).__name__} cannot list a directory")


class _S3Backend(_Backend):
    """S3-compatible stores: ``s3`` (AWS), ``r2`` (Cloudflare, ``R2_ENDPOINT_URL`` / ``R2_PROFILE``), ``weka``
    (``WEKA_ENDPOINT_URL`` / ``WEKA_PROFILE``)."""

    def __init__(self, scheme: str):
        try:
            import boto3
            from botocore.config import Config
        except ImportError as e:
            raise OLMaxEnvironmentError(f"'{scheme}://' paths need boto3, which is not installed") from e
        kwargs = {}
        prefix = {"s3": "S3", "r2": "R2", "weka": "WEKA"}[scheme]
        endpoint = os.environ.get(f"{prefix}_ENDPOINT_URL")
        if scheme in ("r2", "weka") and not endpoint:
            raise OLMaxEnvironmentError(f"'{scheme}://' paths need the {prefix}_ENDPOINT_URL environment variable")
        if endpoint:
            kwargs["endpoint_url"] = endpoint
        session = boto3.Session(profile_name=os.environ.get(f"{prefix}_PROFILE"))
        self.client = session.client("s3", config=Config(retries={"max_attempts": 10, "mode": "standard"}), **kwargs)
        self.scheme = scheme

    def size(self, bucket, key):
        return int(self.client.head_object(Bucket=bucket, Key=key)["ContentLength"])

    def read_range(self, bucket, key, start, n):
        return self.client.get_object(Bucket=bucket, Key=key, Range=f"bytes={start}-{start + n - 1}")["Body"].read()

    def exists(self, bucket, key):
        try:
            self.client.head_object(Bucket=bucket, Key=key)
            return True
        except Exception:
            return False

    def upload(self, src, bucket, key, overwrite):
        if not overwrite and self.exists(bucket, key):
            raise FileExistsError(f"{self.scheme}://{bucket}/{key} already exists")
        self.client.upload_file(str(src), bucket, key)

    def remove(self, bucket, key):
        self.client.delete_object(Bucket=bucket, Key=key)

    def list(self, bucket, prefix, recursive):
        prefix = prefix.rstrip("/") + "/" if prefix else ""
        out, token = [], None
        while True:
            kw = {"Bucket": bucket, "Prefix": prefix}
            if not recursive:
                kw["Delimiter"] = "/"
            if token:
                kw["ContinuationToken"] = token
            resp = self.client.list_objects_v2(**kw)
            out += [f"{self.scheme}://{bucket}/{o['Key']}" for o in resp.get("Contents", [])]
            out += [f"{self.scheme}://{bucket}/{p['Prefix'].rstrip('/')}" for p in resp.get("CommonPrefixes", [])]
            if not resp.get("IsTruncated"):
                return out
            token = resp.get("NextContinuationToken")


class _GCSBackend(_Backend):
    def __init__(self):
        try:
            from google.cloud import storage
        except ImportError as e:
            raise OLMaxEnvironmentError("'gs://' paths need google-cloud-storage, which is not installed") from e
        self.client = storage.Client()

    def _blob(self, bucket, key):
        return self.client.bucket(bucket).blob(key)

    def size(self, bucket, key):
        blob = self._blob(bucket, key)
        blob.reload()
        return int(blob.size)

    def read_range(self, bucket, key, start, n):
        return self._blob(bucket, key).download_as_bytes(start=start, end=start + n - 1)

    def exists(self, bucket, key):
        return self._blob(bucket, key).exists()

    def upload(self, src, bucket, key, overwrite):
        blob = self._blob(bucket, key)
        if not overwrite and blob.exists():
            raise FileExistsError(f"gs://{bucket}/{key} already exists")
        blob.upload_from_filename(str(src))

    def remove(self, bucket, key):
        self._blob(bucket, key).delete()

    def list(self, bucket, prefix, recursive):
        prefix = prefix.rstrip("/") + "/" if prefix else ""
        it = self.client.list_blobs(bucket, prefix=prefix, delimiter=None if recursive else "/")
        out = [f"gs://{bucket}/{b.name}" for b in it]
        out += [f"gs://{bucket}/{p.rstrip('/')}" for p in getattr(it, "prefixes", [])]
        return out


class _HTTPBackend(_Backend):
    def __init__(self):
        try:
            import requests
        except ImportError as e:
            raise OLMaxEnvironmentError("http(s) paths need requests, which is not installed") from e
        self.requests = requests

    def _url(self, scheme, bucket, key):
        return f"{scheme}://{bucket}/{key}"

    def size(self, bucket, key, scheme="https"):
        r = self.requests.head(self._url(scheme, bucket, key), allow_redirects=True)
        if r.status_code == 404:
            raise FileNotFoundError(self._url(scheme, bucket, key))
        if r.status_code >= 400:
            raise OLMaxNetworkError(f"HEAD {self._url(scheme, bucket, key)} -> {r.status_code}")
        return int(r.headers["Content-Length"])

    def read_range(self, bucket, key, start, n, scheme="https"):
        r = self.requests.get(self._url(scheme, bucket, key), headers={"Range": f"bytes={start}-{start + n - 1}"})
        if r.status_code == 404:
            raise FileNotFoundError(self._url(scheme, bucket, key))
        if r.status_code >= 400:
            raise OLMaxNetworkError(f"GET {self._url(scheme, bucket, key)} -> {r.status_code}")
        return r.content

    def exists(self, bucket, key, scheme="https"):
        return self.requests.head(self._url(scheme, bucket, key), allow_redirects=True).status_code < 400


_BACKENDS: dict = {}


def init_client(path: PathOrStr) -> None:
    """Create the client for the scheme of ``path`` up front (e.g. before forking workers)."""
    if is_url(path):
        _backend(urlparse(str(path)).scheme)


def _backend(scheme: str) -> _Backend:
    if scheme not in _BACKENDS:
        if scheme in ("s3", "r2", "weka"):
            _BACKENDS[scheme] = _S3Backend(scheme)
        elif scheme == "gs":
            _BACKENDS[scheme] = _GCSBackend()
        elif scheme in ("http", "https"):
            _BACKENDS[scheme] = _HTTPBackend()
        else:
            raise NotImplementedError(f"no file-system back-end for '{scheme}://' paths")
    return _BACKENDS[scheme]


# ----------------------------------------------------------------------------------------------------------------------
# public API
# ----------------------------------------------------------------------------------------------------------------------
@retriable()
def get_file_size(path: PathOrStr) -> int:
    if is_url(path) and not str(path).startswith("file://"):
        scheme, bucket, key = _split(str(path))
        be = _backend(scheme)
        return be.size(bucket, key, scheme) if isinstance(be, _HTTPBackend) else be.size(bucket, key)
    return os.stat(normalize_path(path)).st_size


@retriable()
def get_bytes_range(path: PathOrStr, bytes_start: int, num_bytes: int) -> bytes:
    if is_url(path) and not str(path).startswith("file://"):
        scheme, bucket, key = _split(str(path))
        be = _backend(scheme)
        if isinstance(be, _HTTPBackend):
            return be.read_range(bucket, key, bytes_start, num_bytes, scheme)
        return be.read_range(bucket, key, bytes_start, num_bytes)
    with open(normalize_path(path), "rb") as f:
        f.seek(bytes_start)
        return f.read(num_bytes)


def upload(source: PathOrStr, target: str, save_overwrite: bool = False) -> None:
    """Upload a local file to a remote URL."""
    src = Path(normalize_path(source))
    if not src.is_file():
        raise FileNotFoundError(src)
    scheme, bucket, key = _split(target)
    if scheme in ("http", "https"):
        raise OLMaxUploadError("cannot upload to an http(s) URL")
    try:
        retriable()(_backend(scheme).upload)(src, bucket, key, save_overwrite)
    except (FileExistsError, OLMaxEnvironmentError, NotImplementedError):
        raise
    except Exception as e:
        raise OLMaxUploadError(f"uploading {src} to {target} failed: {e}") from e


def copy_file(source: PathOrStr, target: PathOrStr, save_overwrite: bool = False) -> None:
    """Copy local -> local (hard link when possible, else copy) or local -> remote (upload)."""
    if is_url(target) and not str(target).startswith("file://"):
        upload(source, str(target), save_overwrite)
        return
    if is_url(source) and not str(source).startswith("file://"):
        size = get_file_size(source)
        tgt = Path(normalize_path(target))
        if tgt.exists() and not save_overwrite:
            raise FileExistsError(tgt)
        tgt.parent.mkdir(parents=True, exist_ok=True)
        with open(tgt, "wb") as f:
            chunk = 64 * 1024 * 1024
            for off in range(0, size, chunk):
                f.write(get_bytes_range(source, off, min(chunk, size - off)))
        return
    src, tgt = Path(normalize_path(source)), Path(normalize_path(target))
    if tgt.exists():
        if not save_overwrite:
            raise FileExistsError(tgt)
        tgt.unlink()
    tgt.parent.mkdir(parents=True, exist_ok=True)
    try:
        os.link(src, tgt)
    except OSError:
        shutil.copy2(src, tgt)


def copy_dir(source: PathOrStr, target: PathOrStr, save_overwrite: bool = False, num_threads: Optional[int] = None,
             quiet: bool = True) -> None:
    """Copy every file under a local directory to a local or remote directory with a thread pool (<= 16 threads)."""
    src = Path(normalize_path(source))
    if not src.is_dir():
        raise NotADirectoryError(src)
    files = [p for p in src.rglob("*") if p.is_file()]
    workers = num_threads or min(16, max(1, len(files)))
    with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
        futs = [pool.submit(copy_file, p, join_path(target, str(p.relative_to(src))), save_overwrite) for p in files]
        for fut in concurrent.futures.as_completed(futs):
            fut.result()
    if not quiet:
        log.info("Copied %d files from %s to %s", len(files), src, target)


def dir_is_empty(path: PathOrStr) -> bool:
    if is_url(path) and not str(path).startswith("file://"):
        return len(list_directory(path)) == 0
    p = Path(normalize_path(path))
    return not p.exists() or not any(p.iterdir())


def file_exists(path: PathOrStr) -> bool:
    if is_url(path) and not str(path).startswith("file://"):
        scheme, bucket, key = _split(str(path))
        be = _backend(scheme)
        return be.exists(bucket, key, scheme) if isinstance(be, _HTTPBackend) else be.exists(bucket, key)
    return Path(normalize_path(path)).is_file()


def remove_file(path: PathOrStr) -> None:
    if is_url(path) and not str(path).startswith("file://"):
        scheme, bucket, key = _split(str(path))
        _backend(scheme).remove(bucket, key)
        return
    Path(normalize_path(path)).unlink(missing_ok=True)


def clear_directory(path: PathOrStr, force: bool = False) -> None:
    """Remove everything under ``path``.  As a safety net a remote prefix must be at least two levels deep
    (``scheme://bucket/a/b``) unless ``force`` is given (``olmax/fs.py:333-341``)."""
    if is_url(path) and not str(path).startswith("file://"):
        scheme, bucket, key = _split(str(path))
        if not force and len([p for p in key.split("/") if p]) < 2:
            raise ValueError(f"refusing to clear the shallow remote prefix '{path}' without force=True")
        for f in list_directory(path, recurse=True):
            remove_file(f)
        return
    p = Path(normalize_path(path))
    if p.is_dir():
        shutil.rmtree(p)


def list_directory(path: PathOrStr, recurse: bool = False, include_files: bool = True,
                   include_dirs: bool = True) -> List[str]:
    if is_url(path) and not str(path).startswith("file://"):
        scheme, bucket, key = _split(str(path))
        return sorted(_backend(scheme).list(bucket, key, recurse))
    p = Path(normalize_path(path))
    if not p.is_dir():
        return []
    it = p.rglob("*") if recurse else p.iterdir()
    out = []
    for c in it:
        if (c.is_file() and include_files) or (c.is_dir() and include_dirs):
            out.append(str(c))
    return sorted(out)


def _glob_to_regex(pattern: str) -> "re.Pattern[str]":
    """``*`` matches within a path component, ``**`` across components (``olmax/fs.py:412-440``)."""
    out, i = "", 0
    while i < len(pattern):
        if pattern.startswith("**/", i):
            out += "(?:.*/)?"
            i += 3
        elif pattern.startswith("**", i):
            out += ".*"
            i += 2
        elif pattern[i] == "*":
            out += "[^/]*"
            i += 1
        elif pattern[i] == "?":
            out += "[^/]"
            i += 1
        else:
            out += re.escape(pattern[i])
            i += 1
    return re.compile("^" + out + "$")


def glob_directory(pattern: str) -> List[str]:
    """All files matching a glob such as ``/data/**/*.npy`` or ``s3://bucket/run/step*/trainer``."""
    pattern = normalize_path(pattern)
    wild = re.search(r"[*?]", pattern)
    if wild is None:
        return [pattern] if (file_exists(pattern) or Path(pattern).exists()) else []
    base = pattern[: wild.start()].rsplit("/", 1)[0] or "/"
    rx = _glob_to_regex(pattern)
    return [f for f in list_directory(base, recurse=True) if rx.match(normalize_path(f))]


def read_text(path: PathOrStr) -> str:
    return get_bytes_range(path, 0, get_file_size(path)).decode()


def write_text(path: PathOrStr, text: str, save_overwrite: bool = True) -> None:
    if is_url(path) and not str(path).startswith("file://"):
        with tempfile.NamedTemporaryFile("w", delete=False) as f:
            f.write(text)
        try:
            upload(f.name, str(path), save_overwrite)
        finally:
            os.unlink(f.name)
        return
    p = Path(normalize_path(path))
    if p.exists() and not save_overwrite:
        raise FileExistsError(p)
    p.parent.mkdir(parents=True, exist_ok=True)
    tmp = p.with_name(p.name + f".tmp{os.getpid()}")
    tmp.write_text(text)
    os.replace(tmp, p)


class _TempDirForTarget:
    """See :func:`get_temp_dir_for_target_dir`."""

    def __init__(self, target: Path, tmp: Path):
        self.target, self.tmp = target, tmp


def get_temp_dir_for_target_dir(target_dir: PathOrStr):
    """
    Context manager for writing a directory atomically from several ranks that share a file system: file-system rank 0
    creates ``<target>.tmp``, everyone writes into it, and after a barrier rank 0 renames it to ``target``
    (``olmax/fs.py:443-506``).  Yields the temporary path.
    """
    import contextlib

    from .parallel import dist_utils
    from .utils import wait_for

    @contextlib.contextmanager
    def manager() -> Generator[Path, None, None]:
        target = Path(normalize_path(target_dir))
        tmp = target.with_name(target.name + ".tmp")
        if dist_utils.get_process_filesystem_rank() == 0:
            if tmp.exists():
                shutil.rmtree(tmp)
            tmp.mkdir(parents=True, exist_ok=True)
        dist_utils.barrier("tmpdir-created")
        wait_for(tmp.exists, f"waiting for {tmp} to become visible", timeout=30.0, interval=0.1)
        try:
            yield tmp
        finally:
            dist_utils.barrier("tmpdir-written")
        if dist_utils.get_process_filesystem_rank() == 0:
            if target.exists():
                shutil.rmtree(target)
            os.replace(tmp, target)
        dist_utils.barrier("tmpdir-renamed")
        wait_for(target.exists, f"waiting for {target} to become visible", timeout=30.0, interval=0.1)

    return manager()
