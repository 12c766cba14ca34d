"""
Typed dataclass <-> plain-data codec with a polymorphic registry.

The reference builds its config system on the third-party ``dataclass_extensions`` package (``Registrable``,
``encode``, ``decode``; used from ``olmax/config.py:61-77`` and every ``*Config`` class).  That package is not
available offline, so this module provides the same capabilities with an independent implementation:

* :func:`encode` turns a dataclass tree into JSON/YAML-safe data (dicts, lists, scalars).  Instances of a
  :class:`Registrable` subclass get a ``"type"`` key holding their registered name.
* :func:`decode` rebuilds a typed tree from such data by walking the annotations: nested dataclasses, ``Optional`` and
  other unions, lists, tuples (fixed and variadic), sequences, dicts, enums, paths, ``torch.dtype`` and numpy dtypes.
* :class:`Registrable` gives a base class a name -> subclass registry; ``decode`` consults the ``"type"`` key to pick
  the subclass, and falls back to the class registered as default.
"""

from __future__ import annotations

import collections.abc
import dataclasses
import enum
import os
import pathlib
import types
import typing
from typing import Any, Callable, ClassVar, Dict, Optional, Type, TypeVar

__all__ = ["Registrable", "encode", "decode", "register_encoder", "register_decoder", "DecodeError"]

T = TypeVar("T")
R = TypeVar("R", bound="Registrable")

TYPE_KEY = "type"


class DecodeError(ValueError):
    """The data cannot be decoded as the requested type."""


class Registrable:
    """
    Mixin that lets a (dataclass) base class keep a registry of named subclasses::

        @dataclass
        class Schedule(Registrable): ...

        @Schedule.register("constant")
        @dataclass
        class Constant(Schedule): ...

    ``Schedule.by_name("constant")`` returns the class, ``Schedule.registered_name(Constant)`` the name.
    """

    _registries: ClassVar[Dict[type, Dict[str, type]]] = {}
    _defaults: ClassVar[Dict[type, str]] = {}

    @classmethod
    def _registry_root(cls) -> type:
        # the root is the class that directly lists Registrable among its bases
        for klass in cls.__mro__:
            if Registrable in klass.__bases__:
                return klass
        raise TypeError(f"{cls} is not a Registrable")

    @classmethod
    def register(cls: Type[R], name: str, default: bool = False, exist_ok: bool = False) -> Callable[[Type[R]], Type[R]]:
        root = cls._registry_root()
        registry = Registrable._registries.setdefault(root, {})

        def wrap(subclass: Type[R]) -> Type[R]:
            if not exist_ok and name in registry and registry[name] is not subclass:
                raise ValueError(f"'{name}' is already registered for {root.__name__} as {registry[name].__name__}")
            registry[name] = subclass
            if default:
                Registrable._defaults[root] = name
            return subclass

        return wrap

    @classmethod
    def by_name(cls: Type[R], name: str) -> Type[R]:
        registry = Registrable._registries.get(cls._registry_root(), {})
        if name not in registry:
            raise KeyError(
                f"'{name}' is not a registered {cls._registry_root().__name__}; known: {sorted(registry)}"
            )
        return typing.cast(Type[R], registry[name])

    @classmethod
    def registered_name(cls, subclass: Optional[type] = None) -> Optional[str]:
        target = subclass if subclass is not None else cls
        for name, klass in Registrable._registries.get(cls._registry_root(), {}).items():
            if klass is target:
                return name
        return None

    @classmethod
    def list_available(cls) -> list:
        return sorted(Registrable._registries.get(cls._registry_root(), {}))

    @classmethod
    def default_name(cls) -> Optional[str]:
        return Registrable._defaults.get(cls._registry_root())


# ------------------------------------------------------------------------------------------------------------------
# encode
# ------------------------------------------------------------------------------------------------------------------

_ENCODERS: Dict[type, Callable[[Any], Any]] = {}
_DECODERS: Dict[type, Callable[[Any], Any]] = {}


def register_encoder(fn: Callable[[Any], Any], *klasses: type) -> None:
    """Encode instances of ``klasses`` with ``fn`` (e.g. ``register_encoder(str, torch.dtype)``)."""
    for k in klasses:
        _ENCODERS[k] = fn


def register_decoder(fn: Callable[[Any], Any], *klasses: type) -> None:
    """Decode values annotated as one of ``klasses`` with ``fn``."""
    for k in klasses:
        _DECODERS[k] = fn


def encode(obj: Any) -> Any:
    """Dataclass tree -> plain data."""
    for klass, fn in _ENCODERS.items():
        if isinstance(obj, klass):
            return fn(obj)
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        out: Dict[str, Any] = {}
        if isinstance(obj, Registrable):
            name = type(obj).registered_name()
            if name is not None:
                out[TYPE_KEY] = name
        for f in dataclasses.fields(obj):
            if f.name.startswith("_") or not f.init:
                continue
            out[f.name] = encode(getattr(obj, f.name))
        return out
    if isinstance(obj, enum.Enum):
        return obj.value
    if isinstance(obj, (str, int, float, bool)) or obj is None:
        return obj
    if isinstance(obj, os.PathLike):
        return os.fspath(obj)
    if isinstance(obj, dict):
        return {str(k): encode(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple, set, frozenset)):
        return [encode(v) for v in obj]
    return obj


# ------------------------------------------------------------------------------------------------------------------
# decode
# ------------------------------------------------------------------------------------------------------------------


def _type_hints(klass: type) -> Dict[str, Any]:
    try:
        return typing.get_type_hints(klass)
    except Exception:
        # local classes with forward references that cannot be resolved: fall back to raw annotations
        return {f.name: f.type for f in dataclasses.fields(klass)}


def _decode_dataclass(klass: type, data: Any, path: str) -> Any:
    if isinstance(data, klass):
        return data
    if not isinstance(data, dict):
        raise DecodeError(f"{path}: expected a mapping for {klass.__name__}, got {type(data).__name__}")
    data = dict(data)
    target = klass
    if isinstance(klass, type) and issubclass(klass, Registrable):
        name = data.pop(TYPE_KEY, None)
        if name is None and klass.registered_name() is None:
            name = klass.default_name()
        if name is not None:
            target = klass.by_name(name)
            if not issubclass(target, klass) and klass is not klass._registry_root():
                raise DecodeError(f"{path}: '{name}' is not a kind of {klass.__name__}")
    hints = _type_hints(target)
    kwargs: Dict[str, Any] = {}
    known = {f.name for f in dataclasses.fields(target) if f.init}
    for key, value in data.items():
        if key not in known:
            # A field of a different registered subclass left over after a `type` override: drop it, like the
            # reference does when only `--x.type=...` is overridden and the remaining fields are kept where valid.
            if target is not klass or (isinstance(klass, type) and issubclass(klass, Registrable)):
                continue
            raise DecodeError(f"{path}: unknown field '{key}' for {target.__name__}")
        kwargs[key] = _decode(hints.get(key, Any), value, f"{path}.{key}" if path else key)
    try:
        return target(**kwargs)
    except TypeError as e:
        raise DecodeError(f"{path}: cannot build {target.__name__}: {e}") from e


def _is_union(tp: Any) -> bool:
    origin = typing.get_origin(tp)
    return origin is typing.Union or origin is types.UnionType


def _decode(tp: Any, data: Any, path: str) -> Any:
    if tp is Any or tp is typing.Any or tp is object:
        return data
    if isinstance(tp, TypeVar):
        bound = tp.__bound__
        return _decode(bound, data, path) if bound is not None else data
    for klass, fn in _DECODERS.items():
        if tp is klass:
            return data if isinstance(data, klass) else fn(data)
    if _is_union(tp):
        args = typing.get_args(tp)
        if data is None and type(None) in args:
            return None
        # exact-type matches first (so that 2 stays an int in `int | Sequence[int]`), then structural attempts
        for arg in args:
            if arg is type(None):
                continue
            if isinstance(arg, type) and not dataclasses.is_dataclass(arg) and type(data) is arg:
                return data
        errors = []
        for arg in args:
            if arg is type(None):
                continue
            try:
                return _decode(arg, data, path)
            except (DecodeError, KeyError, TypeError, ValueError) as e:
                errors.append(str(e))
        raise DecodeError(f"{path}: {data!r} matches no member of {tp}: {errors}")
    origin = typing.get_origin(tp)
    if origin is typing.Literal:
        if data not in typing.get_args(tp):
            raise DecodeError(f"{path}: {data!r} is not one of {typing.get_args(tp)}")
        return data
    if origin is not None:
        args = typing.get_args(tp)
        if origin in (list, collections.abc.MutableSequence):
            if not isinstance(data, (list, tuple)):
                raise DecodeError(f"{path}: expected a list, got {type(data).__name__}")
            elem = args[0] if args else Any
            return [_decode(elem, v, f"{path}.{i}") for i, v in enumerate(data)]
        if origin in (collections.abc.Sequence, collections.abc.Iterable, collections.abc.Collection):
            if isinstance(data, str) or not isinstance(data, (list, tuple)):
                raise DecodeError(f"{path}: expected a sequence, got {type(data).__name__}")
            elem = args[0] if args else Any
            return tuple(_decode(elem, v, f"{path}.{i}") for i, v in enumerate(data))
        if origin is tuple:
            if not isinstance(data, (list, tuple)):
                raise DecodeError(f"{path}: expected a tuple, got {type(data).__name__}")
            if len(args) == 2 and args[1] is Ellipsis:
                return tuple(_decode(args[0], v, f"{path}.{i}") for i, v in enumerate(data))
            if args and len(args) != len(data):
                raise DecodeError(f"{path}: expected {len(args)} items, got {len(data)}")
            return tuple(_decode(a, v, f"{path}.{i}") for i, (a, v) in enumerate(zip(args, data)))
        if origin in (dict, collections.abc.Mapping, collections.abc.MutableMapping):
            if not isinstance(data, dict):
                raise DecodeError(f"{path}: expected a mapping, got {type(data).__name__}")
            kt, vt = args if len(args) == 2 else (Any, Any)
            return {_decode(kt, k, path): _decode(vt, v, f"{path}.{k}") for k, v in data.items()}
        if origin in (set, frozenset):
            elem = args[0] if args else Any
            return origin(_decode(elem, v, path) for v in data)
        if isinstance(origin, type) and dataclasses.is_dataclass(origin):
            return _decode_dataclass(origin, data, path)
        return data
    if isinstance(tp, type):
        if dataclasses.is_dataclass(tp):
            return _decode_dataclass(tp, data, path)
        if issubclass(tp, enum.Enum):
            if isinstance(data, tp):
                return data
            try:
                return tp(data)
            except ValueError:
                try:
                    return tp[data]
                except KeyError:
                    raise DecodeError(f"{path}: {data!r} is not a valid {tp.__name__}") from None
        if tp is bool:
            if isinstance(data, bool):
                return data
            raise DecodeError(f"{path}: expected a bool, got {data!r}")
        if tp is int:
            if isinstance(data, bool) or not isinstance(data, int):
                if isinstance(data, float) and data.is_integer():
                    return int(data)
                raise DecodeError(f"{path}: expected an int, got {data!r}")
            return data
        if tp is float:
            if isinstance(data, bool) or not isinstance(data, (int, float)):
                if isinstance(data, str):
                    try:
                        return float(data)  # YAML reads "1e-5" (no dot) as a string
                    except ValueError:
                        pass
                raise DecodeError(f"{path}: expected a float, got {data!r}")
            return float(data)
        if tp is str:
            if not isinstance(data, str):
                raise DecodeError(f"{path}: expected a str, got {data!r}")
            return data
        if issubclass(tp, pathlib.PurePath):
            return tp(data)
        if tp is os.PathLike:
            if isinstance(data, (str, os.PathLike)):
                return data
            raise DecodeError(f"{path}: expected a path, got {data!r}")
        if tp is type(None):
            if data is None:
                return None
            raise DecodeError(f"{path}: expected None, got {data!r}")
        if tp in (list, tuple, dict, set):
            return tp(data)
        if isinstance(data, tp):
            return data
        raise DecodeError(f"{path}: cannot decode {data!r} as {tp.__name__}")
    return data


def decode(klass: Type[T], data: Any) -> T:
    """Plain data -> typed tree rooted at ``klass``."""
    return typing.cast(T, _decode(klass, data, ""))
