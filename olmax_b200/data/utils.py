"""
Synthetic token batches (``olmax/data/utils.py:12-66``).

``generate_batches_of_sequential_tokens`` is the reference's generator: every instance is
``(arange(S) + random_offset) % V`` with targets ``inputs + 1`` (not wrapped, so a target can equal V: such a token
contributes zero loss but still counts in the mean).  ``generate_batches_of_uniform_tokens`` draws ids uniformly and
uses the ids shifted by one as labels (the last label of a row is ``ignore_index``).  Both derive per-batch and
per-micro-batch streams by folding indices into the seed, produce only this rank's data shard, and return pinned CPU
tensors so that the host-to-device copy can be asynchronous.  With context parallelism (``cp_size > 1``) a rank
receives, of every instance of its data shard, the two chunks it holds in dual-chunk-swap order
(``olmax/data/utils.py:25-31``).
"""

from __future__ import annotations

from typing import Iterator, List, Optional, Tuple

import torch

from ..utils.tree import fold_in

__all__ = ["generate_batches_of_sequential_tokens", "generate_batches_of_uniform_tokens"]

MicroBatch = Tuple[torch.Tensor, torch.Tensor]


def _maybe_pin(t: torch.Tensor, pin: bool) -> torch.Tensor:
    if pin and torch.cuda.is_available():
        return t.pin_memory()
    return t


def _shard(t: torch.Tensor, dp_rank: int, dp_size: int, cp_rank: int = 0, cp_size: int = 1) -> torch.Tensor:
    assert t.shape[0] % dp_size == 0, "global micro-batch must be divisible by the data-parallel size"
    per = t.shape[0] // dp_size
    t = t[dp_rank * per : (dp_rank + 1) * per]
    if cp_size > 1:
        from ..parallel.context import shard_sequence_for_cp

        return shard_sequence_for_cp(t, cp_size, cp_rank, seq_dim=1)
    return t.contiguous()


def generate_batches_of_sequential_tokens(
    seed: int,
    *,
    vocab_size: int,
    sequence_length: int,
    global_microbatch_instances: int,
    num_microbatches: int = 1,
    dp_rank: int = 0,
    dp_size: int = 1,
    cp_rank: int = 0,
    cp_size: int = 1,
    start_batch: int = 0,
    num_batches: Optional[int] = None,
    pin_memory: bool = True,
) -> Iterator[List[MicroBatch]]:
    b = start_batch
    while num_batches is None or b < start_batch + num_batches:
        batch: List[MicroBatch] = []
        for mb in range(num_microbatches):
            gen = torch.Generator().manual_seed(fold_in(fold_in(seed, b), mb))
            offs = torch.randint(0, max(1, vocab_size - 1), (global_microbatch_instances, 1), generator=gen)
            inputs = (torch.arange(sequence_length).view(1, -1) + offs) % vocab_size
            targets = inputs + 1
            batch.append((_maybe_pin(_shard(inputs, dp_rank, dp_size, cp_rank, cp_size), pin_memory),
                          _maybe_pin(_shard(targets, dp_rank, dp_size, cp_rank, cp_size), pin_memory)))
        yield batch
        b += 1


def generate_batches_of_uniform_tokens(
    seed: int,
    *,
    vocab_size: int,
    sequence_length: int,
    global_microbatch_instances: int,
    num_microbatches: int = 1,
    dp_rank: int = 0,
    dp_size: int = 1,
    cp_rank: int = 0,
    cp_size: int = 1,
    start_batch: int = 0,
    num_batches: Optional[int] = None,
    ignore_index: int = -100,
    pin_memory: bool = True,
) -> Iterator[List[MicroBatch]]:
    b = start_batch
    while num_batches is None or b < start_batch + num_batches:
        batch: List[MicroBatch] = []
        for mb in range(num_microbatches):
            gen = torch.Generator().manual_seed(fold_in(fold_in(seed, b), mb))
            ids = torch.randint(0, vocab_size, (global_microbatch_instances, sequence_length), generator=gen)
            labels = torch.full_like(ids, ignore_index)
            labels[:, :-1] = ids[:, 1:]
            batch.append((_maybe_pin(_shard(ids, dp_rank, dp_size, cp_rank, cp_size), pin_memory),
                          _maybe_pin(_shard(labels, dp_rank, dp_size, cp_rank, cp_size), pin_memory)))
        yield batch
        b += 1
