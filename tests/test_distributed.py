"""
Multi-process (gloo, CPU) tests of the sharding layer: the loss and the gradients of a model sharded over a mesh equal
those of the same model on one process, for FSDP, HSDP, DDP and FSDP x TP (with sequence parallelism); initialisation
is independent of the sharding; collectives and host-side synchronisation helpers behave.
"""

import pytest
import torch

from olmax_b200.testing import run_distributed_test


def _model(mesh_resource, seed=0, layer="default", tie=False, kv=None, cp_strategy=None, window=None, softcap=None,
           ac=None, vocab_parallel=False, final_softcap=None):
    from olmax_b200.models import (DefaultTransformerConfig, DefaultTransformerLayerConfig, GemmaTransformerLayerConfig,
                                   ReorderedNormTransformerLayerConfig)
    from olmax_b200.nn import MultiheadSelfAttentionConfig, RMSNormConfig

    layer_cls = {"default": DefaultTransformerLayerConfig, "reordered_norm": ReorderedNormTransformerLayerConfig,
                 "gemma": GemmaTransformerLayerConfig}[layer]
    attn = MultiheadSelfAttentionConfig(n_heads=4, n_kv_heads=kv, head_dim=16,
                                        qk_norm=RMSNormConfig() if layer != "default" else None, use_head_qk_norm=True,
                                        cp_strategy=cp_strategy, window_size=window, logit_softcap=softcap)
    from olmax_b200.nn import LMHeadConfig

    cfg = DefaultTransformerConfig(vocab_size=64, d_model=64, hidden_size=96, num_layers=2, layer=layer_cls(attention=attn),
                                   tie_embeddings=tie, scale_embeddings=tie, ce_chunk_rows=16, layer_ac_policy=_policy(ac),
                                   lm_head=LMHeadConfig(vocab_parallel=vocab_parallel, logit_softcap=final_softcap))
    return cfg.build(seed=seed, mesh_resource=mesh_resource)


def _policy(ac):
    from olmax_b200.activation_checkpointing import NothingSaveable, SaveAnythingExceptTheseNames

    return {None: None, "full": NothingSaveable(), "mlp": SaveAnythingExceptTheseNames(names=["layers.*.mlp"]),
            "attention": SaveAnythingExceptTheseNames(names=["layers.*.attention"])}[ac]


def _global_batch(ignore_last=True):
    g = torch.Generator().manual_seed(123)
    ids = torch.randint(0, 64, (8, 16), generator=g)
    labels = torch.roll(ids, -1, 1)
    if ignore_last:
        labels[:, -1] = -100
    return ids, labels


def _single_process_reference(layer, tie, kv):
    from olmax_b200.parallel import MeshResource

    model = _model(MeshResource.FSDP(1), layer=layer, tie=tie, kv=kv)
    ids, labels = _global_batch()
    model.store.set_grad_scale(1.0)
    loss, _ = model(ids, labels)
    loss.backward()
    model.store.finish_backward()
    grads = {n: model.store.full_gradient(n) for n, _ in model.store.named_parameters()}
    params = {n: model.store.full_parameter(n) for n, _ in model.store.named_parameters()}
    return loss.item(), grads, params


def _sharded_worker(mesh_kind, layer, tie, kv):
    import torch.distributed as dist

    from olmax_b200.parallel import MeshResource, dist_utils

    world = dist_utils.get_world_size()
    res = {"fsdp": lambda: MeshResource.FSDP(world), "hsdp": lambda: MeshResource.HSDP(2, world, 2),
           "ddp": lambda: MeshResource.DDP(world), "tp": lambda: MeshResource.FSDP_with_TP(2, world)}[mesh_kind]()
    model = _model(res, layer=layer, tie=tie, kv=kv)
    mesh = model.mesh
    ids, labels = _global_batch()
    dp, r = mesh.data_parallel_size, mesh.data_parallel_rank
    per = ids.shape[0] // dp
    model.store.set_grad_scale(1.0 / world)
    loss, _ = model(ids[r * per : (r + 1) * per], labels[r * per : (r + 1) * per])
    loss.backward()
    model.store.finish_backward()
    model.store.reduce_replicated_grads()
    t = loss.detach().clone()
    dist.all_reduce(t, group=dist_utils.control_group())
    grads = {n: model.store.full_gradient(n) for n, _ in model.store.named_parameters()}
    params = {n: model.store.full_parameter(n) for n, _ in model.store.named_parameters()}
    return (t / world).item(), grads, params, dict(model.store.stats)


@pytest.mark.parametrize("mesh_kind,world,layer,tie,kv", [
    ("fsdp", 2, "default", False, None),
    ("fsdp", 4, "reordered_norm", False, 2),
    ("hsdp", 4, "default", False, None),
    ("ddp", 2, "gemma", True, 2),
    ("tp", 2, "default", False, None),
    ("tp", 4, "gemma", True, 2),
])
def test_sharded_model_matches_single_process(mesh_kind, world, layer, tie, kv):
    want_loss, want_grads, want_params = _single_process_reference(layer, tie, kv)
    results = run_distributed_test(_sharded_worker, world_size=world, func_args=(mesh_kind, layer, tie, kv))
    for loss, grads, params, stats in results:
        assert loss == pytest.approx(want_loss, rel=1e-5)
        for n in want_grads:
            assert torch.equal(params[n], want_params[n]), f"init of {n} depends on the sharding"
            assert torch.allclose(grads[n], want_grads[n], rtol=1e-3, atol=1e-6), n
    if mesh_kind == "fsdp":
        assert results[0][3]["all_gather_bytes"] > 0 and results[0][3]["reduce_scatter_bytes"] > 0


def _cp_reference(layer, kv, window, softcap):
    from olmax_b200.parallel import MeshResource

    model = _model(MeshResource.FSDP(1), layer=layer, kv=kv, window=window, softcap=softcap)
    ids, labels = _global_batch(ignore_last=False)
    model.store.set_grad_scale(1.0)
    loss, _ = model(ids, labels)
    loss.backward()
    model.store.finish_backward()
    return loss.item(), {n: model.store.full_gradient(n) for n, _ in model.store.named_parameters()}


def _cp_worker(mesh_kind, cp, strategy, layer, kv, window, softcap):
    import torch.distributed as dist

    from olmax_b200.parallel import MeshResource, dist_utils
    from olmax_b200.parallel.context import shard_sequence_for_cp

    world = dist_utils.get_world_size()
    res = MeshResource.FSDP_with_CP(world, cp) if mesh_kind == "fsdp_cp" else MeshResource.HSDP_with_CP(2, world, 2)
    model = _model(res, layer=layer, kv=kv, cp_strategy=strategy, window=window, softcap=softcap)
    mesh = model.mesh
    assert mesh.cp.size == cp
    ids, labels = _global_batch(ignore_last=False)   # equal token counts on every rank: mean of means = global mean
    dp, r = mesh.data_parallel_size, mesh.data_parallel_rank
    per = ids.shape[0] // dp
    local_ids = shard_sequence_for_cp(ids[r * per : (r + 1) * per], cp, mesh.cp.rank)
    local_labels = shard_sequence_for_cp(labels[r * per : (r + 1) * per], cp, mesh.cp.rank)
    model.store.set_grad_scale(1.0 / world)
    loss, _ = model(local_ids, local_labels)
    loss.backward()
    model.store.finish_backward()
    model.store.reduce_replicated_grads()
    t = loss.detach().clone()
    dist.all_reduce(t, group=dist_utils.control_group())
    return (t / world).item(), {n: model.store.full_gradient(n) for n, _ in model.store.named_parameters()}


@pytest.mark.parametrize("mesh_kind,world,cp,strategy,layer,kv,window,softcap", [
    ("fsdp_cp", 2, 2, "all_gather", "default", None, None, None),
    ("fsdp_cp", 2, 2, "ring", "reordered_norm", 2, None, 20.0),
    ("fsdp_cp", 4, 2, "ring", "default", None, None, None),          # batch 2 x context 2
    ("fsdp_cp", 4, 4, "ring", "gemma", 2, None, None),
    ("fsdp_cp", 4, 4, "all_gather", "default", 2, 5, None),          # sliding window narrower than a chunk pair
    ("fsdp_cp", 2, 2, "ring", "default", None, 5, None),             # ring with a narrow window falls back to all-gather
    ("hsdp_cp", 4, 2, "all_gather", "default", None, None, None),    # CP over the shard axis of an HSDP mesh
])
def test_context_parallel_matches_single_process(mesh_kind, world, cp, strategy, layer, kv, window, softcap):
    want_loss, want_grads = _cp_reference(layer, kv, window, softcap)
    results = run_distributed_test(_cp_worker, world_size=world,
                                   func_args=(mesh_kind, cp, strategy, layer, kv, window, softcap))
    for loss, grads in results:
        assert loss == pytest.approx(want_loss, rel=1e-5)
        for n in want_grads:
            assert torch.allclose(grads[n], want_grads[n], rtol=1e-3, atol=1e-6), n


def test_dual_chunk_swap_reordering():
    from olmax_b200.parallel.context import (cp_local_positions, inverse_reorder_causal_load_balancing,
                                             reorder_causal_load_balancing, shard_sequence_for_cp)

    x = torch.arange(2 * 16).view(2, 16)
    y = reorder_causal_load_balancing(x, 2, seq_dim=1)
    assert y[0].tolist() == [0, 1, 2, 3, 12, 13, 14, 15, 4, 5, 6, 7, 8, 9, 10, 11]
    assert torch.equal(inverse_reorder_causal_load_balancing(y, 2, seq_dim=1), x)
    for r in range(2):
        assert torch.equal(shard_sequence_for_cp(x, 2, r), y.chunk(2, dim=1)[r])
        assert torch.equal(cp_local_positions(16, 2, r), y[0].chunk(2)[r])
    # every rank gets the same amount of causal work: sum of (position + 1) over its tokens
    work = [int((cp_local_positions(64, 4, r) + 1).sum()) for r in range(4)]
    assert len(set(work)) == 1
    with pytest.raises(ValueError):
        reorder_causal_load_balancing(torch.zeros(1, 6), 2, seq_dim=1)


def _recompute_worker(mesh_kind, ac, cp_strategy):
    import torch.distributed as dist

    from olmax_b200.parallel import MeshResource, dist_utils
    from olmax_b200.parallel.context import shard_sequence_for_cp

    world = dist_utils.get_world_size()
    res = MeshResource.FSDP_with_TP(2, world) if mesh_kind == "tp" else MeshResource.FSDP_with_CP(world, 2)
    model = _model(res, layer="gemma", kv=2, ac=ac, cp_strategy=cp_strategy)
    mesh = model.mesh
    ids, labels = _global_batch(ignore_last=False)
    if mesh.cp.size > 1:
        ids, labels = (shard_sequence_for_cp(t, mesh.cp.size, mesh.cp.rank) for t in (ids, labels))
    model.store.set_grad_scale(1.0 / world)
    loss, _ = model(ids, labels)
    loss.backward()
    model.store.finish_backward()
    model.store.reduce_replicated_grads()
    t = loss.detach().clone()
    dist.all_reduce(t, group=dist_utils.control_group())
    return (t / world).item(), {n: model.store.full_gradient(n) for n, _ in model.store.named_parameters()}


@pytest.mark.parametrize("mesh_kind,ac,cp_strategy", [("tp", "full", None), ("tp", "mlp", None), ("cp", "attention", "ring"),
                                                      ("cp", "full", "all_gather")])
def test_recomputation_repeats_the_collectives_consistently(mesh_kind, ac, cp_strategy):
    """Recomputing a block in backward re-runs its collectives (sequence-parallel gathers, the K/V ring) on every rank
    in the same order: loss and gradients equal the run without recomputation."""
    base = run_distributed_test(_recompute_worker, world_size=2, func_args=(mesh_kind, None, cp_strategy))
    remat = run_distributed_test(_recompute_worker, world_size=2, func_args=(mesh_kind, ac, cp_strategy))
    for (l0, g0), (l1, g1) in zip(base, remat):
        assert l1 == pytest.approx(l0, rel=1e-6)
        for n in g0:
            assert torch.allclose(g1[n], g0[n], rtol=1e-5, atol=1e-7), n


def _vocab_parallel_worker(vocab_parallel, world_kind):
    import torch.distributed as dist

    from olmax_b200.parallel import MeshResource, dist_utils

    world = dist_utils.get_world_size()
    res = MeshResource.FSDP_with_TP(2, world)
    model = _model(res, layer="reordered_norm", kv=2, vocab_parallel=vocab_parallel, final_softcap=30.0)
    assert model.lm_head.vocab_parallel == vocab_parallel
    assert model.lm_head.weight.meta.tp_dim == (0 if vocab_parallel else None)
    mesh = model.mesh
    ids, labels = _global_batch()
    labels[1, 3] = 64   # out of range but counted
    per = ids.shape[0] // mesh.data_parallel_size
    ids = ids[mesh.data_parallel_rank * per : (mesh.data_parallel_rank + 1) * per]
    labels = labels[mesh.data_parallel_rank * per : (mesh.data_parallel_rank + 1) * per]
    model.store.set_grad_scale(1.0 / world)
    loss, zl = model(ids, labels, z_loss_multiplier=1e-3)
    loss.backward()
    model.store.finish_backward()
    model.store.reduce_replicated_grads()
    t = loss.detach().clone()
    dist.all_reduce(t, group=dist_utils.control_group())
    logits = model(ids)   # the inference path gathers the vocabulary slices
    return (t / world).item(), {n: model.store.full_gradient(n) for n, _ in model.store.named_parameters()}, logits


@pytest.mark.parametrize("world", [2, 4])
def test_vocab_parallel_loss_matches_replicated_head(world):
    """Splitting the LM head's vocabulary over the TP group (every member computes its slice of the logits for the
    gathered rows; softmax statistics are combined across the members) gives the loss, the z-loss-inclusive gradients
    and the logits of the head that is replicated over the TP group."""
    base = run_distributed_test(_vocab_parallel_worker, world_size=world, func_args=(False, "tp"))
    vp = run_distributed_test(_vocab_parallel_worker, world_size=world, func_args=(True, "tp"))
    for (l0, g0, z0), (l1, g1, z1) in zip(base, vp):
        assert l1 == pytest.approx(l0, rel=1e-5)
        assert set(g0) == set(g1)
        for n in g0:
            assert torch.allclose(g1[n], g0[n], rtol=1e-4, atol=1e-7), n
        assert torch.allclose(z1, z0, rtol=1e-4, atol=1e-5)


def _collectives_worker():
    import torch.distributed as dist

    from olmax_b200.parallel import MeshResource, collectives as coll, dist_utils

    rank, world = dist_utils.get_rank(), dist_utils.get_world_size()
    mesh = MeshResource.HSDP(2, world, 2).build()
    assert mesh.shard.size == 2 and mesh.replicate.size == world // 2
    assert mesh.shard.ranks == [rank - rank % 2, rank - rank % 2 + 1]
    x = torch.full((2, 3), float(rank))
    g = coll.all_gather(x, mesh.shard, dim=0)
    assert g.shape == (4, 3) and g[0, 0] == mesh.shard.ranks[0] and g[2, 0] == mesh.shard.ranks[1]
    full = torch.arange(8.0).view(4, 2) + rank
    rs = coll.reduce_scatter(full.clone(), mesh.shard, dim=0)
    want = sum(torch.arange(8.0).view(4, 2) + r for r in mesh.shard.ranks)[mesh.shard.rank * 2 : mesh.shard.rank * 2 + 2]
    assert torch.equal(rs, want)
    h = torch.full((4,), 1.0 + rank, dtype=torch.bfloat16)
    coll.all_reduce(h, mesh.world, mean=True)
    assert torch.allclose(h.float(), torch.full((4,), sum(1.0 + r for r in range(world)) / world), rtol=1e-2)
    # host-side helpers
    dist_utils.barrier("t")
    assert dist_utils.synchronize_value({"a": rank}, src=0) == {"a": 0}
    assert dist_utils.allgather_value(rank * 10) == [r * 10 for r in range(world)]
    assert dist_utils.get_process_filesystem_rank() == rank  # OLMAX_SHARED_FS_DIRS is set by the harness
    return True


def test_collectives_and_host_sync():
    assert all(run_distributed_test(_collectives_worker, world_size=4))


def test_reduce_divide_factor_and_mesh_math():
    from olmax_b200.parallel import MeshResource, get_reduce_divide_factor

    assert [get_reduce_divide_factor(n) for n in (1, 2, 4, 8, 16, 32, 64)] == [1, 2, 2, 4, 4, 8, 8]
    m = MeshResource.FSDP_with_TP(2, 8)
    assert m.data_parallel_size == 4 and m.fsdp_size == 4 and m.tp_size == 2
    assert m.coordinates(5) == {"fsdp": 2, "tp": 1} and m.rank_of({"fsdp": 2, "tp": 1}) == 5
    assert m.group_ranks("tp", 5) == [4, 5] and m.group_ranks("fsdp", 5) == [1, 3, 5, 7]
    h = MeshResource.HSDP(4, 8, 8)
    assert h.replicate_axes == ("fsdp_replicate",) and h.group_ranks("fsdp_shard", 6) == [4, 5, 6, 7]
    assert MeshResource.DDP(4).replicate_axes == ("data",) and MeshResource.DDP(4).fsdp_size == 1
    cp = MeshResource.FSDP_with_CP(8, 2)
    assert cp.data_parallel_size == 4 and cp.fsdp_size == 8 and cp.cp_size == 2
    with pytest.raises(Exception):
        MeshResource(axes=((2, "a"),), batch_sharding_axis="b")


def _hsdp_accumulation_worker(num_microbatches):
    from olmax_b200.optim import AdamWConfig, ConstantSchedule
    from olmax_b200.parallel import MeshResource, dist_utils

    world = dist_utils.get_world_size()
    model = _model(MeshResource.HSDP(2, world, 2))
    optim = AdamWConfig(lr=ConstantSchedule(1e-3)).build(model, num_microbatches)
    ids, labels = _global_batch()
    dp, r = model.mesh.data_parallel_size, model.mesh.data_parallel_rank
    per = ids.shape[0] // dp
    mine_ids, mine_labels = ids[r * per : (r + 1) * per], labels[r * per : (r + 1) * per]
    per_step = []
    for _ in range(2):
        before = dict(model.store.stats)
        for mb in range(num_microbatches):
            loss, _ = model(mine_ids.chunk(num_microbatches)[mb], mine_labels.chunk(num_microbatches)[mb])
            loss.backward()
            assert optim.accumulate() == (mb == num_microbatches - 1)
        optim.step()
        per_step.append({k: model.store.stats[k] - before[k] for k in before})
    return per_step, model.store.grad.numel(), model.mesh.replicate.size


def test_hsdp_all_reduces_once_per_optimizer_step():
    """The cross-replica all-reduce runs after the LAST micro-batch only (the reference all-reduces after every
    micro-batch, its README's known issue): its byte count per optimizer step does not depend on the number of
    micro-batches, while the reduce-scatter inside the shard group runs once per micro-batch."""
    one = run_distributed_test(_hsdp_accumulation_worker, world_size=4, func_args=(1,))
    two = run_distributed_test(_hsdp_accumulation_worker, world_size=4, func_args=(2,))
    for (steps1, numel, rep), (steps2, _, _) in zip(one, two):
        want = 2 * (rep - 1) * numel * 4 // rep
        assert all(s["all_reduce_bytes"] == want for s in steps1 + steps2)
        assert all(s2["reduce_scatter_bytes"] == 2 * s1["reduce_scatter_bytes"] for s1, s2 in zip(steps1, steps2))


def test_split_phase_barrier_protocol_with_threads_as_peers():
    """Host model of the reduce-scatter staging protocol of the peer-memory backend, with CPU threads standing in for
    the GPUs and a shared array for their peer-mapped memory: every member stores its contribution to unit u into the
    owners' slots of staging buffer u % 3, then waits for the members' epoch of the PREVIOUS unit, folds that unit and
    only then publishes its epoch for u (publish after fold).  Random delays shuffle the interleavings; every fold must
    see exactly the contributions of its unit, which fails if a buffer could be rewritten before its owner has folded it."""
    import random
    import threading
    import time

    import numpy as np

    n, units, n_buf, width = 4, 40, 3, 8
    flags = np.zeros((n, n), dtype=np.int64)              # flags[owner][member] = newest epoch `member` published
    stage = np.zeros((n, n_buf, n, width))                # stage[owner][buffer][member slot][...]
    results = [[] for _ in range(n)]
    errors = []

    def member(me):
        rng = random.Random(me)
        pending = None                                    # (unit, epoch) whose fold is still to come
        epoch = 0
        try:
            for u in range(units):
                time.sleep(rng.random() * 1e-3)
                for owner in range(n):                    # "weight-gradient epilogue": stores into the owners' slots
                    stage[owner, u % n_buf, me, :] = 1000 * u + me
                if pending is not None:
                    pu, pe = pending
                    deadline = time.time() + 20
                    while flags[me].min() < pe:           # bounded wait
                        if time.time() > deadline:
                            raise TimeoutError(f"member {me} waiting for epoch {pe}: {flags[me]}")
                        time.sleep(1e-5)
                    results[me].append((pu, stage[me, pu % n_buf].sum(axis=0).copy()))
                epoch += 1
                for owner in range(n):                    # publish AFTER the fold
                    flags[owner, me] = epoch
                pending = (u, epoch)
            pu, pe = pending
            while flags[me].min() < pe:
                time.sleep(1e-5)
            results[me].append((pu, stage[me, pu % n_buf].sum(axis=0).copy()))
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=member, args=(r,)) for r in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    assert not errors, errors
    for me in range(n):
        assert [u for u, _ in results[me]] == list(range(units))
        for u, total in results[me]:
            assert np.all(total == n * 1000 * u + sum(range(n))), (me, u, total)
    assert (flags == units).all()                        # epochs advanced in step on every member
