"""
Reader and writer for the OCDBT key-value database format ("Optionally-Cooperative Distributed B+Tree", the
``ocdbt`` kvstore driver of TensorStore), which is what Orbax packs the zarr arrays of a checkpoint item into when
``use_ocdbt=True`` (the reference: ``olmax/checkpoint/utils.py:153-159``).

Written from the published description of the storage format; neither TensorStore nor a checkpoint produced by it
is available where this code was developed, so compatibility with TensorStore is by construction from that
description, not by test against it.  What the tests do establish: whatever this writer produces, this reader reads
back (single and multi-level trees, inline and out-of-line values, merged multi-process databases, zstd-compressed
nodes), and hand-assembled byte fixtures of every structure parse to the expected values.

On-disk structures (all integers little-endian unless noted; ``varint`` = unsigned LEB128):

* every encoded structure (manifest, version-tree node, B+tree node) is::

      magic        uint32 BIG-endian   0x0cdb3a2a manifest, 0x0cdb1234 version-tree node, 0x0cdb20de B+tree node
      length       uint64              bytes of the whole structure, header and checksum included
      version      varint              0
      compression  uint8               0 = body stored as is, 1 = body is one zstd frame
      body
      crc32c       uint32              CRC-32C of everything before it

* manifest body: ``config`` (uuid[16], manifest_kind varint, max_inline_value_bytes varint, max_decoded_node_bytes
  varint, version_tree_arity_log2 uint8, compression_method varint [+ zstd level int32 when 1]), then the data-file
  table, the inline version entries and the version-node references;
* data-file table: ``num_files`` varint; for every file after the first the number of leading bytes its path shares
  with the previous one; for every file the length of the rest; for every file how many leading bytes of the full
  path are the ``base_path`` (the remainder is the path relative to it); then the concatenated suffix bytes;
* version entry arrays (column by column): generation numbers, root heights (uint8), root locations (file index,
  offset, length), root statistics (keys, tree bytes, indirect value bytes), commit times (uint64);
* B+tree node body: ``height`` uint8 (0 = leaf), data-file table, ``num_entries`` varint, key prefix lengths (entries
  1..n-1: bytes shared with the previous key), key suffix lengths, [interior: subtree common prefix lengths], key
  suffix bytes; leaf: value lengths, value kinds (uint8; 0 inline, 1 out of line), out-of-line locations (file index,
  offset), inline value bytes; interior: child locations (file index, offset, length) and child statistics.
  Keys inside a child are stored without the first ``subtree_common_prefix_length`` bytes of the parent's key for it.

Directory layout of one database: ``manifest.ocdbt`` plus data files ``d/<32 hex digits>``.  Orbax lets every process
write its own database under ``ocdbt.process_<i>/`` and then merges them: the merged top-level manifest points at a
new B+tree whose leaves reference the values inside the per-process data files (``base_path`` =
``ocdbt.process_<i>/``); :func:`merge_process_databases` does the same.
"""

from __future__ import annotations

import ctypes
import ctypes.util
import os
import struct
import time
import uuid as _uuid
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

from .zarr3 import crc32c

__all__ = ["OcdbtWriter", "OcdbtReader", "merge_process_databases", "ValueRef", "OcdbtFormatError",
           "encode_varint", "decode_varint"]

MAGIC_MANIFEST = 0x0CDB3A2A
MAGIC_VERSION_NODE = 0x0CDB1234
MAGIC_BTREE_NODE = 0x0CDB20DE
MANIFEST_NAME = "manifest.ocdbt"
DEFAULT_MAX_INLINE = 100
DEFAULT_MAX_NODE_BYTES = 8 * 1024 * 1024
DEFAULT_ARITY_LOG2 = 4


class OcdbtFormatError(ValueError):
    pass


# ----------------------------------------------------------------------------------------------------------------------
# primitives
# ----------------------------------------------------------------------------------------------------------------------
def encode_varint(n: int) -> bytes:
    if n < 0:
        raise ValueError("varint is unsigned")
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def decode_varint(buf: bytes, pos: int) -> Tuple[int, int]:
    shift = result = 0
    while True:
        if pos >= len(buf):
            raise OcdbtFormatError("truncated varint")
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7
        if shift > 63:
            raise OcdbtFormatError("varint longer than 64 bits")


class _Cursor:
    def __init__(self, buf: bytes):
        self.buf, self.pos = buf, 0

    def varint(self) -> int:
        v, self.pos = decode_varint(self.buf, self.pos)
        return v

    def varints(self, n: int) -> List[int]:
        return [self.varint() for _ in range(n)]

    def u8(self) -> int:
        v = self.buf[self.pos]
        self.pos += 1
        return v

    def u8s(self, n: int) -> List[int]:
        v = list(self.buf[self.pos : self.pos + n])
        if len(v) != n:
            raise OcdbtFormatError("truncated byte array")
        self.pos += n
        return v

    def take(self, n: int) -> bytes:
        v = self.buf[self.pos : self.pos + n]
        if len(v) != n:
            raise OcdbtFormatError("truncated field")
        self.pos += n
        return v

    def u64s(self, n: int) -> List[int]:
        return list(struct.unpack(f"<{n}Q", self.take(8 * n))) if n else []

    def i32(self) -> int:
        return struct.unpack("<i", self.take(4))[0]

    def done(self) -> bool:
        return self.pos == len(self.buf)


_ZSTD = None


def _zstd():
    """libzstd through ctypes (the image has no Python binding); None when the shared library is missing."""
    global _ZSTD
    if _ZSTD is None:
        name = ctypes.util.find_library("zstd") or "libzstd.so.1"
        try:
            lib = ctypes.CDLL(name)
            lib.ZSTD_compressBound.restype = ctypes.c_size_t
            lib.ZSTD_compressBound.argtypes = [ctypes.c_size_t]
            lib.ZSTD_compress.restype = ctypes.c_size_t
            lib.ZSTD_compress.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
            lib.ZSTD_decompress.restype = ctypes.c_size_t
            lib.ZSTD_decompress.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t]
            lib.ZSTD_getFrameContentSize.restype = ctypes.c_ulonglong
            lib.ZSTD_getFrameContentSize.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
            lib.ZSTD_isError.restype = ctypes.c_uint
            lib.ZSTD_isError.argtypes = [ctypes.c_size_t]
            _ZSTD = lib
        except OSError:
            _ZSTD = False
    return _ZSTD or None


def zstd_compress(data: bytes, level: int = 3) -> bytes:
    lib = _zstd()
    if lib is None:
        raise OcdbtFormatError("zstd compression requested but libzstd is not available")
    bound = lib.ZSTD_compressBound(len(data))
    dst = ctypes.create_string_buffer(bound)
    n = lib.ZSTD_compress(dst, bound, data, len(data), level)
    if lib.ZSTD_isError(n):
        raise OcdbtFormatError("zstd compression failed")
    return dst.raw[:n]


def zstd_decompress(data: bytes) -> bytes:
    lib = _zstd()
    if lib is None:
        raise OcdbtFormatError("a zstd-compressed structure was found but libzstd is not available")
    size = lib.ZSTD_getFrameContentSize(data, len(data))
    if size in (2**64 - 1, 2**64 - 2):   # unknown / error
        raise OcdbtFormatError("zstd frame without a content size")
    dst = ctypes.create_string_buffer(max(1, size))
    n = lib.ZSTD_decompress(dst, size, data, len(data))
    if lib.ZSTD_isError(n) or n != size:
        raise OcdbtFormatError("zstd decompression failed")
    return dst.raw[:size]


def _wrap(magic: int, body: bytes, compress: bool = False) -> bytes:
    """header + (compressed) body + CRC-32C"""
    if compress:
        body = zstd_compress(body)
    tail = encode_varint(0) + bytes([1 if compress else 0]) + body
    length = 4 + 8 + len(tail) + 4
    head = struct.pack(">I", magic) + struct.pack("<Q", length) + tail
    return head + struct.pack("<I", crc32c(head))


def _unwrap(blob: bytes, magic: int, what: str) -> bytes:
    if len(blob) < 18:
        raise OcdbtFormatError(f"{what}: too short")
    if struct.unpack(">I", blob[:4])[0] != magic:
        raise OcdbtFormatError(f"{what}: bad magic {blob[:4].hex()}")
    (length,) = struct.unpack("<Q", blob[4:12])
    if length != len(blob):
        raise OcdbtFormatError(f"{what}: length field {length} != {len(blob)} bytes present")
    (crc,) = struct.unpack("<I", blob[-4:])
    if crc != crc32c(blob[:-4]):
        raise OcdbtFormatError(f"{what}: CRC-32C mismatch")
    version, pos = decode_varint(blob, 12)
    if version != 0:
        raise OcdbtFormatError(f"{what}: unsupported format version {version}")
    compression = blob[pos]
    body = blob[pos + 1 : -4]
    if compression == 1:
        body = zstd_decompress(body)
    elif compression != 0:
        raise OcdbtFormatError(f"{what}: unknown compression format {compression}")
    return body


# ----------------------------------------------------------------------------------------------------------------------
# data-file table
# ----------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class DataFile:
    base_path: str       # "" or "ocdbt.process_3/"
    relative_path: str   # "d/<hex>"

    @property
    def full(self) -> str:
        return self.base_path + self.relative_path


def _encode_file_table(files: Sequence[DataFile]) -> bytes:
    out = bytearray(encode_varint(len(files)))
    full = [f.full.encode() for f in files]
    prefix = [0] * len(files)
    for i in range(1, len(files)):
        n = 0
        a, b = full[i - 1], full[i]
        while n < min(len(a), len(b)) and a[n] == b[n]:
            n += 1
        prefix[i] = n
    for i in range(1, len(files)):
        out += encode_varint(prefix[i])
    for i in range(len(files)):
        out += encode_varint(len(full[i]) - prefix[i])
    for f in files:
        out += encode_varint(len(f.base_path.encode()))
    for i in range(len(files)):
        out += full[i][prefix[i]:]
    return bytes(out)


def _decode_file_table(c: _Cursor) -> List[DataFile]:
    n = c.varint()
    prefix = [0] + c.varints(max(0, n - 1))
    suffix = c.varints(n)
    base_len = c.varints(n)
    files: List[DataFile] = []
    prev = b""
    for i in range(n):
        if prefix[i] > len(prev):
            raise OcdbtFormatError("data-file table: prefix longer than the previous path")
        full = prev[: prefix[i]] + c.take(suffix[i])
        if base_len[i] > len(full):
            raise OcdbtFormatError("data-file table: base path longer than the path")
        files.append(DataFile(full[: base_len[i]].decode(), full[base_len[i]:].decode()))
        prev = full
    return files


# ----------------------------------------------------------------------------------------------------------------------
# B+tree nodes
# ----------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class ValueRef:
    """Where a value lives: inline bytes, or (data file, offset, length)."""
    inline: Optional[bytes] = None
    file: Optional[DataFile] = None
    offset: int = 0
    length: int = 0

    @property
    def size(self) -> int:
        return len(self.inline) if self.inline is not None else self.length


@dataclass
class _Child:
    key: bytes
    common_prefix: int
    file: DataFile
    offset: int
    length: int
    num_keys: int
    tree_bytes: int
    indirect_bytes: int


def _encode_keys(keys: Sequence[bytes]) -> Tuple[List[int], List[int], bytes]:
    prefix, suffix, blob = [], [], bytearray()
    for i, k in enumerate(keys):
        n = 0
        if i:
            p = keys[i - 1]
            while n < min(len(p), len(k)) and p[n] == k[n]:
                n += 1
        if i:
            prefix.append(n)
        suffix.append(len(k) - n)
        blob += k[n:]
    return prefix, suffix, bytes(blob)


def _files_of(items: Iterable[Optional[DataFile]]) -> Tuple[List[DataFile], Dict[DataFile, int]]:
    table: List[DataFile] = []
    index: Dict[DataFile, int] = {}
    for f in items:
        if f is not None and f not in index:
            index[f] = len(table)
            table.append(f)
    return table, index


def encode_leaf(entries: Sequence[Tuple[bytes, ValueRef]], compress: bool = False) -> bytes:
    table, index = _files_of(v.file for _, v in entries)
    prefix, suffix, key_blob = _encode_keys([k for k, _ in entries])
    out = bytearray([0]) + _encode_file_table(table) + encode_varint(len(entries))
    for p in prefix:
        out += encode_varint(p)
    for s in suffix:
        out += encode_varint(s)
    out += key_blob
    for _, v in entries:
        out += encode_varint(v.size)
    out += bytes(0 if v.inline is not None else 1 for _, v in entries)
    for _, v in entries:
        if v.inline is None:
            out += encode_varint(index[v.file])
    for _, v in entries:
        if v.inline is None:
            out += encode_varint(v.offset)
    for _, v in entries:
        if v.inline is not None:
            out += v.inline
    return _wrap(MAGIC_BTREE_NODE, bytes(out), compress)


def encode_interior(height: int, children: Sequence[_Child], compress: bool = False) -> bytes:
    table, index = _files_of(c.file for c in children)
    prefix, suffix, key_blob = _encode_keys([c.key for c in children])
    out = bytearray([height]) + _encode_file_table(table) + encode_varint(len(children))
    for p in prefix:
        out += encode_varint(p)
    for s in suffix:
        out += encode_varint(s)
    for c in children:
        out += encode_varint(c.common_prefix)
    out += key_blob
    for attr in ("offset", "length", "num_keys", "tree_bytes", "indirect_bytes"):
        if attr == "offset":
            for c in children:
                out += encode_varint(index[c.file])
        for c in children:
            out += encode_varint(getattr(c, attr))
    return _wrap(MAGIC_BTREE_NODE, bytes(out), compress)


def decode_node(blob: bytes):
    """-> (height, leaf entries [(key, ValueRef)] or interior children [_Child]); keys are as stored in the node."""
    c = _Cursor(_unwrap(blob, MAGIC_BTREE_NODE, "B+tree node"))
    height = c.u8()
    files = _decode_file_table(c)
    n = c.varint()
    prefix = [0] + c.varints(max(0, n - 1))
    suffix = c.varints(n)
    common = c.varints(n) if height > 0 else []
    keys: List[bytes] = []
    prev = b""
    for i in range(n):
        if prefix[i] > len(prev):
            raise OcdbtFormatError("B+tree node: key prefix longer than the previous key")
        k = prev[: prefix[i]] + c.take(suffix[i])
        keys.append(k)
        prev = k
    if height == 0:
        sizes = c.varints(n)
        kinds = c.u8s(n)
        out_idx = [i for i in range(n) if kinds[i] == 1]
        file_ids = c.varints(len(out_idx))
        offsets = c.varints(len(out_idx))
        refs: List[Optional[ValueRef]] = [None] * n
        for j, i in enumerate(out_idx):
            refs[i] = ValueRef(None, files[file_ids[j]], offsets[j], sizes[i])
        for i in range(n):
            if kinds[i] == 0:
                refs[i] = ValueRef(c.take(sizes[i]))
            elif kinds[i] != 1:
                raise OcdbtFormatError(f"B+tree leaf: unknown value kind {kinds[i]}")
        return 0, list(zip(keys, refs))
    file_ids = c.varints(n)
    offsets, lengths = c.varints(n), c.varints(n)
    num_keys, tree_bytes, indirect = c.varints(n), c.varints(n), c.varints(n)
    return height, [_Child(keys[i], common[i], files[file_ids[i]], offsets[i], lengths[i], num_keys[i], tree_bytes[i],
                           indirect[i]) for i in range(n)]


# ----------------------------------------------------------------------------------------------------------------------
# manifest
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class Version:
    generation: int
    root_height: int
    root_file: Optional[DataFile]   # None: empty tree
    root_offset: int
    root_length: int
    num_keys: int
    tree_bytes: int
    indirect_bytes: int
    commit_time_ns: int


@dataclass
class Manifest:
    uuid: bytes
    versions: List[Version]
    manifest_kind: int = 0
    max_inline_value_bytes: int = DEFAULT_MAX_INLINE
    max_decoded_node_bytes: int = DEFAULT_MAX_NODE_BYTES
    version_tree_arity_log2: int = DEFAULT_ARITY_LOG2
    compression_method: int = 0
    zstd_level: int = 0
    version_nodes: int = 0   # references to out-of-line version-tree nodes (read, counted, not followed)

    @property
    def latest(self) -> Version:
        return max(self.versions, key=lambda v: v.generation)


def encode_manifest(m: Manifest, compress: bool = False) -> bytes:
    out = bytearray(m.uuid)
    out += encode_varint(m.manifest_kind) + encode_varint(m.max_inline_value_bytes) + encode_varint(m.max_decoded_node_bytes)
    out += bytes([m.version_tree_arity_log2]) + encode_varint(m.compression_method)
    if m.compression_method == 1:
        out += struct.pack("<i", m.zstd_level)
    table, index = _files_of(v.root_file for v in m.versions)
    out += _encode_file_table(table)
    vs = m.versions
    out += encode_varint(len(vs))
    for v in vs:
        out += encode_varint(v.generation)
    out += bytes(v.root_height for v in vs)
    # an empty tree has no root: file index / offset / length are all zero and the statistics say zero keys
    for v in vs:
        out += encode_varint(index[v.root_file] if v.root_file is not None else 0)
    for attr in ("root_offset", "root_length", "num_keys", "tree_bytes", "indirect_bytes"):
        for v in vs:
            out += encode_varint(getattr(v, attr))
    out += struct.pack(f"<{len(vs)}Q", *[v.commit_time_ns for v in vs])
    out += encode_varint(0)   # no out-of-line version-tree nodes
    return _wrap(MAGIC_MANIFEST, bytes(out), compress)


def decode_manifest(blob: bytes) -> Manifest:
    c = _Cursor(_unwrap(blob, MAGIC_MANIFEST, "manifest"))
    uid = c.take(16)
    kind, max_inline, max_node = c.varint(), c.varint(), c.varint()
    arity = c.u8()
    method = c.varint()
    level = c.i32() if method == 1 else 0
    if method not in (0, 1):
        raise OcdbtFormatError(f"manifest: unknown compression method {method}")
    files = _decode_file_table(c)
    n = c.varint()
    gens = c.varints(n)
    heights = c.u8s(n)
    fids, offs, lens = c.varints(n), c.varints(n), c.varints(n)
    nkeys, tbytes, ibytes = c.varints(n), c.varints(n), c.varints(n)
    times = c.u64s(n)
    versions = []
    for i in range(n):
        empty = nkeys[i] == 0 and lens[i] == 0
        versions.append(Version(gens[i], heights[i], None if empty else files[fids[i]], offs[i], lens[i], nkeys[i], tbytes[i],
                                ibytes[i], times[i]))
    n_nodes = c.varint()
    if n_nodes:
        # interior references of a large version tree: generation, location (file, offset, length), height,
        # number of generations, commit time.  Older versions are not needed to read the latest one.
        c.varints(n_nodes); c.varints(n_nodes); c.varints(n_nodes); c.varints(n_nodes)
        c.u8s(n_nodes); c.varints(n_nodes); c.u64s(n_nodes)
    if not versions:
        raise OcdbtFormatError("manifest: no version")
    return Manifest(uid, versions, kind, max_inline, max_node, arity, method, level, n_nodes)


# ----------------------------------------------------------------------------------------------------------------------
# writer
# ----------------------------------------------------------------------------------------------------------------------
def _new_data_file_name() -> str:
    return "d/" + _uuid.uuid4().hex


def _build_tree(entries: List[Tuple[bytes, ValueRef]], append, data_file: DataFile, fanout: int, compress: bool):
    """Write leaves and interior levels through ``append(bytes) -> offset``; returns (height, offset, length, keys,
    tree bytes, indirect bytes) of the root, or None for an empty tree."""
    if not entries:
        return None
    level: List[_Child] = []
    for i in range(0, len(entries), fanout):
        part = entries[i : i + fanout]
        blob = encode_leaf(part, compress)
        off = append(blob)
        level.append(_Child(part[0][0], 0, data_file, off, len(blob), len(part), len(blob),
                            sum(v.length for _, v in part if v.inline is None)))
    height = 0
    while len(level) > 1:
        height += 1
        nxt: List[_Child] = []
        for i in range(0, len(level), fanout):
            part = level[i : i + fanout]
            blob = encode_interior(height, part, compress)
            off = append(blob)
            nxt.append(_Child(part[0].key, 0, data_file, off, len(blob), sum(c.num_keys for c in part),
                              len(blob) + sum(c.tree_bytes for c in part), sum(c.indirect_bytes for c in part)))
        level = nxt
    root = level[0]
    return height, root.offset, root.length, root.num_keys, root.tree_bytes, root.indirect_bytes


class OcdbtWriter:
    """Writes ONE database (a directory with ``manifest.ocdbt`` and one data file): ``put`` values, then ``commit``.
    Large values go to the data file as they arrive (nothing is buffered), small ones are stored inline in the leaf."""

    def __init__(self, directory: Path, max_inline_value_bytes: int = DEFAULT_MAX_INLINE, fanout: int = 512,
                 compress_nodes: bool = False):
        self.dir = Path(directory)
        self.dir.mkdir(parents=True, exist_ok=True)
        (self.dir / "d").mkdir(exist_ok=True)
        self.max_inline = max_inline_value_bytes
        self.fanout = max(2, fanout)
        self.compress = compress_nodes
        self.data_file = DataFile("", _new_data_file_name())
        self._fh = open(self.dir / self.data_file.relative_path, "wb")
        self._pos = 0
        self._entries: Dict[bytes, ValueRef] = {}

    def _append(self, data) -> int:
        off = self._pos
        self._fh.write(data)
        self._pos += len(data) if not isinstance(data, memoryview) else data.nbytes
        return off

    def put(self, key: str, value) -> None:
        """``value``: bytes-like (a memoryview of a tensor's storage is written without a copy)."""
        n = value.nbytes if isinstance(value, memoryview) else len(value)
        if n <= self.max_inline:
            self._entries[key.encode()] = ValueRef(bytes(value))
        else:
            self._entries[key.encode()] = ValueRef(None, self.data_file, self._append(value), n)

    def commit(self) -> Manifest:
        entries = sorted(self._entries.items())
        root = _build_tree(entries, self._append, self.data_file, self.fanout, self.compress)
        self._fh.flush()
        os.fsync(self._fh.fileno())
        self._fh.close()
        now = time.time_ns()
        if root is None:
            v = Version(1, 0, None, 0, 0, 0, 0, 0, now)
            (self.dir / self.data_file.relative_path).unlink()
        else:
            v = Version(1, root[0], self.data_file, root[1], root[2], root[3], root[4], root[5], now)
        m = Manifest(_uuid.uuid4().bytes, [v], max_inline_value_bytes=self.max_inline,
                     compression_method=1 if self.compress else 0, zstd_level=3 if self.compress else 0)
        tmp = self.dir / (MANIFEST_NAME + f".tmp{os.getpid()}")
        tmp.write_bytes(encode_manifest(m))
        os.replace(tmp, self.dir / MANIFEST_NAME)
        return m


# ----------------------------------------------------------------------------------------------------------------------
# reader
# ----------------------------------------------------------------------------------------------------------------------
class OcdbtReader:
    """Read-only view of the latest version of a database directory."""

    def __init__(self, directory: Path):
        self.dir = Path(directory)
        path = self.dir / MANIFEST_NAME
        if not path.exists():
            raise FileNotFoundError(f"{path}: not an OCDBT database")
        self.manifest = decode_manifest(path.read_bytes())
        self._index: Optional[Dict[str, ValueRef]] = None
        self._fds: Dict[str, int] = {}

    def _read_at(self, file: DataFile, offset: int, length: int) -> bytes:
        fd = self._fds.get(file.full)
        if fd is None:
            fd = os.open(self.dir / file.full, os.O_RDONLY)
            self._fds[file.full] = fd
        data = os.pread(fd, length, offset)
        if len(data) != length:
            raise OcdbtFormatError(f"{file.full}: short read at {offset}+{length}")
        return data

    def close(self) -> None:
        for fd in self._fds.values():
            os.close(fd)
        self._fds.clear()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _walk(self, file: DataFile, offset: int, length: int, key_prefix: bytes, expect_height: Optional[int]) -> Iterator[Tuple[bytes, ValueRef]]:
        height, items = decode_node(self._read_at(file, offset, length))
        if expect_height is not None and height != expect_height:
            raise OcdbtFormatError(f"B+tree node at {file.full}:{offset} has height {height}, expected {expect_height}")
        if height == 0:
            for k, ref in items:
                yield key_prefix + k, ref
            return
        for child in items:
            if child.common_prefix > len(child.key):
                raise OcdbtFormatError("B+tree interior node: common prefix longer than the key")
            yield from self._walk(child.file, child.offset, child.length, key_prefix + child.key[: child.common_prefix],
                                  height - 1)

    def items(self) -> Dict[str, ValueRef]:
        """key -> ValueRef for every key of the latest version (the tree is walked once and cached)."""
        if self._index is None:
            v = self.manifest.latest
            idx: Dict[str, ValueRef] = {}
            if v.root_file is not None:
                last = None
                for k, ref in self._walk(v.root_file, v.root_offset, v.root_length, b"", v.root_height):
                    if last is not None and k <= last:
                        raise OcdbtFormatError("B+tree keys are not strictly increasing")
                    last = k
                    idx[k.decode()] = ref
                if len(idx) != v.num_keys:
                    raise OcdbtFormatError(f"manifest says {v.num_keys} keys, the tree holds {len(idx)}")
            self._index = idx
        return self._index

    def keys(self, prefix: str = "") -> List[str]:
        return [k for k in self.items() if k.startswith(prefix)]

    def __contains__(self, key: str) -> bool:
        return key in self.items()

    def get(self, key: str, offset: int = 0, length: Optional[int] = None) -> bytes:
        ref = self.items().get(key)
        if ref is None:
            raise KeyError(key)
        n = ref.size - offset if length is None else length
        if offset < 0 or n < 0 or offset + n > ref.size:
            raise ValueError(f"{key}: range {offset}+{n} outside the value ({ref.size} bytes)")
        if ref.inline is not None:
            return ref.inline[offset : offset + n]
        return self._read_at(ref.file, ref.offset + offset, n)


# ----------------------------------------------------------------------------------------------------------------------
# merging per-process databases
# ----------------------------------------------------------------------------------------------------------------------
def merge_process_databases(directory: Path, process_dirs: Sequence[str], fanout: int = 512,
                            compress_nodes: bool = False) -> Manifest:
    """Write ``directory/manifest.ocdbt`` whose tree holds every key of the databases in the sub-directories
    ``process_dirs`` (e.g. ``ocdbt.process_0``): out-of-line values stay where they are and are referenced through a
    data-file ``base_path``; inline values are copied into the new leaves.  A key written by several processes must
    have been written with identical bytes (replicated metadata); the first one wins."""
    directory = Path(directory)
    merged: Dict[bytes, ValueRef] = {}
    for sub in process_dirs:
        with OcdbtReader(directory / sub) as r:
            for k, ref in r.items().items():
                kb = k.encode()
                if kb in merged:
                    continue
                if ref.inline is None:
                    ref = ValueRef(None, DataFile(sub.rstrip("/") + "/" + ref.file.base_path, ref.file.relative_path), ref.offset,
                                   ref.length)
                merged[kb] = ref
    (directory / "d").mkdir(parents=True, exist_ok=True)
    data_file = DataFile("", _new_data_file_name())
    pos = 0
    with open(directory / data_file.relative_path, "wb") as fh:
        def append(b: bytes) -> int:
            nonlocal pos
            off = pos
            fh.write(b)
            pos += len(b)
            return off

        root = _build_tree(sorted(merged.items()), append, data_file, max(2, fanout), compress_nodes)
        fh.flush()
        os.fsync(fh.fileno())
    now = time.time_ns()
    if root is None:
        (directory / data_file.relative_path).unlink()
        v = Version(1, 0, None, 0, 0, 0, 0, 0, now)
    else:
        v = Version(1, root[0], data_file, root[1], root[2], root[3], root[4], root[5], now)
    m = Manifest(_uuid.uuid4().bytes, [v], compression_method=1 if compress_nodes else 0, zstd_level=3 if compress_nodes else 0)
    tmp = directory / (MANIFEST_NAME + f".tmp{os.getpid()}")
    tmp.write_bytes(encode_manifest(m))
    os.replace(tmp, directory / MANIFEST_NAME)
    return m
