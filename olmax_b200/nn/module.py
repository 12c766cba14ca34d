"""
Module base class (role of ``olmax/nn/module.py:18-145``).

Modules are ``torch.nn.Module``s whose weights live in a :class:`~olmax_b200.parallel.param_store.ParamStore`
instead of ``nn.Parameter``s: a module registers its weights while it is constructed inside a :class:`BuildContext`
and keeps the returned handles.  Every module has a dotted ``checkpoint_name`` (``layers.3.attention`` ...) that names
its parameters in checkpoints and is what activation-checkpointing policies match against.
"""

from __future__ import annotations

import contextlib
from typing import Dict, Iterator, List, Optional, Tuple

import torch

from ..parallel.param_store import ParamHandle, ParamStore

__all__ = ["BuildContext", "Module", "current_build_context", "build_module"]

_CTX_STACK: List["BuildContext"] = []


class BuildContext:
    """Carries the parameter store, the FSDP unit and the name prefix while a model is being constructed."""

    def __init__(self, store: ParamStore, unit: str = "root", prefix: str = ""):
        self.store = store
        self.unit = unit
        self.prefix = prefix

    @contextlib.contextmanager
    def scope(self, name: str, unit: Optional[str] = None):
        child = BuildContext(self.store, unit if unit is not None else self.unit,
                             f"{self.prefix}.{name}" if self.prefix else name)
        _CTX_STACK.append(child)
        try:
            yield child
        finally:
            _CTX_STACK.pop()

    def __enter__(self):
        _CTX_STACK.append(self)
        return self

    def __exit__(self, *exc):
        _CTX_STACK.pop()
        return False

    def param(self, name: str, shape, **kwargs) -> ParamHandle:
        full = f"{self.prefix}.{name}" if self.prefix else name
        return self.store.register(full, shape, unit=self.unit, **kwargs)


def current_build_context() -> BuildContext:
    if not _CTX_STACK:
        raise RuntimeError("modules must be constructed inside a BuildContext (see TransformerConfig.build)")
    return _CTX_STACK[-1]


class Module(torch.nn.Module):
    def __init__(self):
        super().__init__()
        ctx = current_build_context()
        self.checkpoint_name: str = ctx.prefix
        self._store = ctx.store
        self._handles: Dict[str, ParamHandle] = {}

    @property
    def store(self) -> ParamStore:
        return self._store

    @property
    def mesh(self):
        return self._store.mesh

    def add_param(self, name: str, shape, **kwargs) -> ParamHandle:
        h = current_build_context().param(name, shape, **kwargs)
        self._handles[name] = h
        return h

    def param_handles(self, recurse: bool = True) -> Iterator[Tuple[str, ParamHandle]]:
        mods = self.modules() if recurse else [self]
        seen = set()
        for m in mods:
            if isinstance(m, Module):
                for h in m._handles.values():
                    if h.name not in seen:
                        seen.add(h.name)
                        yield h.name, h

    def get_checkpoint_names(self) -> List[str]:
        return [m.checkpoint_name for m in self.modules() if isinstance(m, Module) and m.checkpoint_name]


def build_module(factory, *, seed: int = 0, mesh=None, mesh_resource=None, param_dtype: torch.dtype = torch.float32,
                 compute_dtype: Optional[torch.dtype] = None, device: Optional[torch.device] = None,
                 comm_backend: Optional[str] = None, unit: str = "root"):
    """
    Build a single module (or any tree of modules) outside a Transformer: creates a parameter store on ``mesh`` (default:
    the current mesh, else FSDP over the whole job), runs ``factory()`` inside a build context, initialises the
    parameters and returns the module.  ``module.store`` gives access to gradients and full parameters, e.g.::

        lin = build_module(lambda: Linear(64, 32))
        y = lin(x); y.sum().backward(); lin.store.finish_backward()
        dw = lin.store.full_gradient("weight")
    """
    from ..parallel import dist_utils
    from ..parallel.mesh import MeshResource, get_mesh

    if mesh is None:
        mesh = get_mesh() if mesh_resource is None else None
    if mesh is None:
        resource = mesh_resource or MeshResource.FSDP(dist_utils.get_world_size())
        mesh = resource.build(device=device)
    device = torch.device(device) if device is not None else mesh.device
    if compute_dtype is None:
        compute_dtype = torch.bfloat16 if device.type == "cuda" else param_dtype
    store = ParamStore(mesh, param_dtype=param_dtype, compute_dtype=compute_dtype, device=device,
                       comm_backend=comm_backend)
    with BuildContext(store, unit=unit):
        module = factory()
    store.finalize(seed=seed)
    return module
