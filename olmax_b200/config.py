"""
Command-line overrides for dataclass configs (same surface as ``olmax/config.py:39-112``).

``parse_config_from_args(config, args=[...])`` encodes the dataclass tree to plain data, applies every override of
the form ``--a.b.0.c=VALUE`` (leading dashes optional, ``-`` in names becomes ``_``, a bare ``--flag`` means
``true``, list elements addressed by index, values parsed as YAML) and decodes the result back into typed objects.
Overriding only ``x.type`` keeps the other fields where they still apply; overriding ``x`` with a mapping replaces it.
"""

from __future__ import annotations

import dataclasses
import os
import sys
from typing import Any, List, Optional, Sequence, Tuple, Type, TypeVar

import torch
import yaml

from .utils.dataclass_codec import decode, encode, register_decoder, register_encoder

__all__ = ["parse_config_from_args", "config_to_dict", "config_to_yaml"]

C = TypeVar("C")


def _dtype_to_str(dt: torch.dtype) -> str:
    return str(dt).replace("torch.", "")


def _dtype_from_str(name: Any) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    aliases = {"float": "float32", "half": "float16", "bf16": "bfloat16", "fp32": "float32", "fp16": "float16"}
    key = aliases.get(str(name), str(name)).replace("torch.", "")
    dt = getattr(torch, key, None)
    if not isinstance(dt, torch.dtype):
        raise ValueError(f"unknown dtype '{name}'")
    return dt


register_encoder(_dtype_to_str, torch.dtype)
register_decoder(_dtype_from_str, torch.dtype)


def parse_config_from_args(
    config: Any,
    config_class: Optional[Type[C]] = None,
    /,
    *,
    args: Optional[Sequence[str]] = None,
) -> C:
    """
    ``config`` is either a dataclass instance or the path of a YAML file (then ``config_class`` is required).
    ``args`` defaults to ``sys.argv[1:]``.
    """
    if args is None and sys.argv:
        args = sys.argv[1:]

    if dataclasses.is_dataclass(config) and not isinstance(config, type):
        if config_class is None:
            config_class = type(config)
        elif not isinstance(config, config_class):
            raise ValueError(f"expected a {config_class.__name__}, got {type(config).__name__}")
        data = encode(config)
    elif isinstance(config, (str, os.PathLike)):
        if config_class is None:
            raise ValueError(f"config_class is required to type the config file '{config}'")
        with open(config) as f:
            data = yaml.safe_load(f)
    else:
        raise ValueError(f"cannot parse a config from {config!r}")

    for key, value in (_parse_override(a) for a in (args or ())):
        _assign(data, key.split("."), value, key)
    return decode(config_class, data)


def config_to_dict(config: Any) -> Any:
    return encode(config)


def config_to_yaml(config: Any) -> str:
    return yaml.safe_dump(encode(config), sort_keys=False)


def _assign(node: Any, parts: List[str], value: Any, full_key: str) -> None:
    head, rest = parts[0], parts[1:]
    if isinstance(node, list):
        idx = int(head)
        if rest:
            _assign(node[idx], rest, value, full_key)
        else:
            node[idx] = value
    elif isinstance(node, dict):
        if rest:
            if head not in node or node[head] is None:
                node[head] = {}
            _assign(node[head], rest, value, full_key)
        else:
            node[head] = value
    else:
        raise ValueError(f"cannot apply override '{full_key}': '{head}' addresses into {type(node).__name__}")


def _parse_override(arg: str) -> Tuple[str, Any]:
    name, sep, raw = arg.partition("=")
    if not sep:
        raw = "true"
    name = name.strip().lstrip("-").replace("-", "_")
    if not name:
        raise ValueError(f"malformed override '{arg}'")
    value: Any = "" if (not raw or raw.isspace()) else yaml.safe_load(raw)
    return name, value
