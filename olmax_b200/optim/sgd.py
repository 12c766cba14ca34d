"""Plain SGD step over a ParamStore (``olmax/optim/sgd.py:12-19``), mostly for tests."""

from __future__ import annotations


def sgd_step(store, lr: float) -> None:
    store.reduce_replicated_grads()
    store.master.add_(store.grad.to(store.master.dtype), alpha=-lr)
    store.zero_grad()
    store.sync_shadow()
