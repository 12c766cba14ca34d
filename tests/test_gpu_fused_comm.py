"""
Fused compute + communication paths.

* The all-gather fused into the GEMM is exercised on ONE GPU by letting the "peer" shard pointers address other local
  buffers: the staging buffer holds only this rank's slot, the kernel's copy warps fetch the rest while tiles of the
  local slot compute, and the result must equal a plain GEMM on the assembled weight.
* On two GPUs (skipped when fewer are visible) a sharded model trained through the peer-memory backend (all-gather in
  the GEMM, reduce-scatter in the weight-gradient epilogue, embedding rows read from their owner) must match the NCCL
  backend.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

from olmax_b200.testing import rel_err, run_distributed_test


def _check():
    from olmax_b200.ops import _lib

    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("rank,N,R", [(0, 2048, 4), (2, 2048, 4), (5, 11008, 8)])   # 11008 / 8: 1376-row shards
def test_all_gather_fused_gemm_single_gpu_emulation(rank, N, R):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from olmax_b200.ops import kernels as K

    dev = torch.device("cuda")
    torch.manual_seed(20)
    M, Kd = 1024, 512
    rows = N // R
    w = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16)
    a = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16)
    peers = [w[r * rows : (r + 1) * rows].clone() for r in range(R)]          # what each "GPU" owns
    table = K.pointer_table([p.data_ptr() for p in peers], dev)
    flags = torch.zeros(R * 64, dtype=torch.int32, device=dev)

    def staging():
        buf = torch.full((R, rows * Kd + 128), float("nan"), device=dev, dtype=torch.bfloat16)
        buf[rank, : rows * Kd] = peers[rank].reshape(-1)
        return buf

    # forward: N-sharded K-major B
    st = staging()
    c = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
    K.gemm(a, st, c, M, N, Kd, ldb=Kd, N_s=rows, b_shard_stride=st.stride(0), ag_src=table, ag_flags=flags, ag_rank=rank)
    assert rel_err(c, a.float() @ w.float().t()) < 5e-3
    assert not torch.isnan(st[:, : rows * Kd].float()).any()       # every slot was filled
    got = torch.cat([st[r, : rows * Kd].view(rows, Kd) for r in range(R)])
    assert torch.equal(got, w)
    # dgrad: contraction over the shards (MN-major B)
    st = staging()
    dy = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
    dx = torch.zeros(M, Kd, device=dev, dtype=torch.bfloat16)
    K.gemm(dy, st, dx, M, Kd, N, b_mn=True, ldb=Kd, Kc_s=rows, b_shard_stride=st.stride(0), ag_src=table,
           ag_flags=flags, ag_rank=rank)
    assert rel_err(dx, dy.float() @ w.float()) < 5e-3
    # gated MLP: two operands fetched by the same launch
    w2 = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) * 0.1
    peers2 = [w2[r * rows : (r + 1) * rows].clone() for r in range(R)]
    table2 = K.pointer_table([p.data_ptr() for p in peers2], dev)
    st1, st2 = staging(), torch.full((R, rows * Kd + 128), float("nan"), device=dev, dtype=torch.bfloat16)
    st2[rank, : rows * Kd] = peers2[rank].reshape(-1)
    act = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    g, u = torch.empty_like(act), torch.empty_like(act)
    K.gemm(a, st1, act, M, N, Kd, ldb=Kd, N_s=rows, b_shard_stride=st1.stride(0), epi=K.EPI_SWIGLU, b2=st2, c2=g, c3=u,
           ag_src=table, ag_src2=table2, ag_flags=flags, ag_rank=rank)
    gf, uf = a.float() @ w.float().t(), a.float() @ w2.float().t()
    assert rel_err(g, gf) < 5e-3 and rel_err(u, uf) < 5e-3
    assert rel_err(act, torch.nn.functional.silu(gf) * uf) < 1e-2
    _check()


@pytest.mark.parametrize("rank,tp", [(0, 2), (1, 2), (2, 4)])
def test_tensor_parallel_fused_kernels_single_gpu_emulation(rank, tp):
    """The activation-side fusions of tensor parallelism on ONE GPU, the "peers" being other local buffers:
    all-gather of the A operand's row shards inside the GEMM, the gated dual-B GEMM on such an operand, the
    reduce-scatter epilogue (row block s stored to c_shards[s], with and without a local partial sum folded in) and the
    bf16 slot fold."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from olmax_b200.ops import kernels as K

    dev = torch.device("cuda")
    torch.manual_seed(30 + rank)
    M, N, Kd = 1024 * tp, 1280, 512
    M_s = M // tp
    x = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16)
    peers = [x[r * M_s : (r + 1) * M_s].clone() for r in range(tp)]
    table = K.pointer_table([p.data_ptr() for p in peers], dev)
    flags = torch.zeros(tp * 64, dtype=torch.int32, device=dev)

    def full_with_local_rows():
        buf = torch.full((M, Kd), float("nan"), device=dev, dtype=torch.bfloat16)
        buf[rank * M_s : (rank + 1) * M_s] = peers[rank]
        return buf

    # all-gather -> GEMM
    xf = full_with_local_rows()
    y = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
    K.gemm(xf, w, y, M, N, Kd, M_s=M_s, ag_src=table, ag_flags=flags, ag_rank=rank, ag_on_a=True)
    assert torch.equal(xf, x)                                   # every row shard arrived
    assert rel_err(y, x.float() @ w.float().t()) < 5e-3
    # ... with the gated epilogue
    w2 = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) * 0.1
    xf = full_with_local_rows()
    act, g, u = (torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in range(3))
    K.gemm(xf, w, act, M, N, Kd, M_s=M_s, epi=K.EPI_GEGLU, b2=w2, c2=g, c3=u, ag_src=table, ag_flags=flags, ag_rank=rank,
           ag_on_a=True)
    gf, uf = x.float() @ w.float().t(), x.float() @ w2.float().t()
    assert rel_err(g, gf) < 5e-3 and rel_err(u, uf) < 5e-3
    assert rel_err(act, torch.nn.functional.gelu(gf, approximate="tanh") * uf) < 1e-2
    # ... as the A operand of a dgrad-layout GEMM (MN-major B)
    wt = torch.randn(Kd, N, device=dev, dtype=torch.bfloat16)
    xf = full_with_local_rows()
    y2 = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
    K.gemm(xf, wt, y2, M, N, Kd, b_mn=True, M_s=M_s, ag_src=table, ag_flags=flags, ag_rank=rank, ag_on_a=True)
    assert rel_err(y2, x.float() @ wt.float()) < 5e-3

    # GEMM -> reduce-scatter: row block s goes to "GPU" s's slot
    slots = [torch.full((M_s * N + 64,), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(tp)]
    ctable = K.pointer_table([t.data_ptr() for t in slots], dev)
    want = x.float() @ w.float().t()
    K.gemm(x, w, slots[0], M, N, Kd, ldc=N, M_s=M_s, c_shards=ctable, m_shard_rot=(rank + 1) % tp)
    for r in range(tp):
        assert rel_err(slots[r][: M_s * N].view(M_s, N), want[r * M_s : (r + 1) * M_s]) < 5e-3
    # ... folding in a local partial sum (which must stay untouched)
    prior = torch.randn(M, N, device=dev, dtype=torch.bfloat16) * 10
    prior0 = prior.clone()
    K.gemm(x, w, prior, M, N, Kd, ldc=N, epi=K.EPI_BF16_ACC, M_s=M_s, c_shards=ctable, m_shard_rot=(rank + 1) % tp)
    assert torch.equal(prior, prior0)
    for r in range(tp):
        assert rel_err(slots[r][: M_s * N].view(M_s, N), (want + prior0.float())[r * M_s : (r + 1) * M_s]) < 5e-3
    # fold of the staging slots
    stage = torch.randn(tp, M_s * N, device=dev, dtype=torch.bfloat16)
    out = torch.randn(M_s * N, device=dev, dtype=torch.bfloat16)
    out0 = out.clone()
    K.fold_slots_bf16(out, stage, M_s * N, tp, M_s * N, skip=-1, accumulate=False)
    assert rel_err(out, stage.float().sum(0)) < 5e-3
    out = out0.clone()
    K.fold_slots_bf16(out, stage, M_s * N, tp, M_s * N, skip=rank, accumulate=True)
    keep = [r for r in range(tp) if r != rank]
    assert rel_err(out, out0.float() + stage[keep].float().sum(0)) < 5e-3
    _check()


def test_small_shard_helpers():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from olmax_b200.ops import kernels as K

    dev = torch.device("cuda")
    R, n = 4, 96
    shards = [torch.randn(n, device=dev).to(torch.bfloat16) for _ in range(R)]
    table = K.pointer_table([s.data_ptr() for s in shards], dev)
    dst = torch.zeros(R, n + 32, device=dev, dtype=torch.bfloat16)
    K.gather_shards(table, dst, dst.stride(0), n, R, 1)
    for r in range(R):
        assert torch.equal(dst[r, :n], shards[r] if r != 1 else torch.zeros_like(shards[r]))
    grads = [torch.zeros(n, device=dev) for _ in range(R)]
    gtable = K.pointer_table([g.data_ptr() for g in grads], dev)
    src = torch.randn(R * n, device=dev)
    K.scatter_add_shards(src, gtable, n, R, 0.5)
    K.scatter_add_shards(src, gtable, n, R, 0.5)
    assert torch.allclose(torch.cat(grads), src, rtol=1e-6)
    # raw copy (every unroll variant, a ragged tail) and the one-to-many push
    big = torch.randn(1_000_003 * 8, device=dev).to(torch.bfloat16)            # 16,000,048 bytes: a multiple of 16
    for unroll in (4, 8, 16):
        out = torch.zeros_like(big)
        K.copy_bytes(out.data_ptr(), big.data_ptr(), big.numel() * 2, dev, blocks=37, unroll=unroll)
        assert torch.equal(out, big)
    dsts = [torch.zeros_like(big) for _ in range(3)]
    ptable = K.pointer_table([d.data_ptr() for d in dsts], dev)
    K.push_copy(ptable, big, big.numel() * 2, 3, skip=1)
    assert torch.equal(dsts[0], big) and torch.equal(dsts[2], big) and not dsts[1].any()
    _check()


def _train_worker(backend, mesh_kind="fsdp", barrier="nccl", wire="bf16"):
    import os

    import torch.distributed as dist

    os.environ["OLMAX_B200_BARRIER"] = barrier   # read when the peer-memory context is built
    os.environ["OLMAX_B200_RS_WIRE"] = wire      # likewise: format of the staged partial gradients

    from olmax_b200.models import DefaultTransformerConfig, ReorderedNormTransformerLayerConfig
    from olmax_b200.nn import MultiheadSelfAttentionConfig, RMSNormConfig
    from olmax_b200.ops import _lib
    from olmax_b200.optim import AdamWConfig, ConstantSchedule
    from olmax_b200.parallel import MeshResource, dist_utils

    world, rank = dist_utils.get_world_size(), dist_utils.get_rank()
    dev = torch.device("cuda", rank)
    attn = MultiheadSelfAttentionConfig(n_heads=4, head_dim=128, qk_norm=RMSNormConfig(), use_head_qk_norm=False)
    cfg = DefaultTransformerConfig(vocab_size=4096, d_model=512, hidden_size=1408, num_layers=2,
                                   layer=ReorderedNormTransformerLayerConfig(attention=attn), ce_chunk_rows=256)
    res = {"fsdp": lambda: MeshResource.FSDP(world), "ddp": lambda: MeshResource.DDP(world),
           "hsdp": lambda: MeshResource.HSDP(2, world, 2)}[mesh_kind]()
    model = cfg.build(seed=5, mesh_resource=res, device=dev, comm_backend=backend)
    assert (model.store.symm is not None) == (backend == "fused")
    optim = AdamWConfig(lr=ConstantSchedule(1e-3), max_grad_norm=1.0).build(model, 2)
    g = torch.Generator().manual_seed(100 + rank)
    cache = model.get_buffer_cache(256, dev)
    losses = []
    for step in range(3):
        for mb in range(2):
            ids = torch.randint(0, 4096, (2, 256), generator=g).to(dev)
            labels = torch.roll(ids, -1, 1)
            loss, _ = model(ids, labels, cache)
            loss.backward()
            optim.accumulate()
        if step == 0:
            model.store.sync_peers()   # the peers' direct additions (embedding, norm weights) have landed after this
            first_grads = model.store.grad.clone()
        optim.step()
        losses.append(loss.item())
    torch.cuda.synchronize()
    _lib.check_status(dev)
    if model.store.symm is not None:
        model.store.symm.check_canaries()   # nobody stored outside its staging slots; barrier epochs are in step
    full = {n: model.store.full_parameter(n).cpu() for n, _ in model.store.named_parameters()}
    return losses, first_grads.cpu(), full


@pytest.mark.parametrize("mesh_kind,world,barrier,wire", [
    ("fsdp", 2, "nccl", "bf16"), ("fsdp", 2, "flags", "bf16"), ("ddp", 2, "nccl", "bf16"), ("hsdp", 4, "nccl", "bf16"),
    ("fsdp", 2, "flags", "fp32"),   # partial weight gradients cross NVLink as fp32
])
def test_peer_memory_backend_matches_nccl(mesh_kind, world, barrier, wire):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    fused = run_distributed_test(_train_worker, world_size=world, backend="nccl",
                                 func_args=("fused", mesh_kind, barrier, wire), timeout=300)
    nccl = run_distributed_test(_train_worker, world_size=world, backend="nccl", func_args=("nccl", mesh_kind), timeout=300)
    for r in range(world):
        lf, gf, pf = fused[r]
        ln, gn, pn = nccl[r]
        assert all(abs(a - b) < 2e-2 * abs(b) for a, b in zip(lf, ln)), (lf, ln)
        assert rel_err(gf, gn) < 2e-2
        for name in pn:
            assert rel_err(pf[name], pn[name]) < 1e-2, name


def _tp_worker(mesh_kind, backend="nccl"):
    from olmax_b200.models import DefaultTransformerConfig, GemmaTransformerLayerConfig
    from olmax_b200.nn import LMHeadConfig, MultiheadSelfAttentionConfig
    from olmax_b200.ops import _lib
    from olmax_b200.optim import AdamWConfig, ConstantSchedule
    from olmax_b200.parallel import MeshResource, dist_utils

    world, rank = dist_utils.get_world_size(), dist_utils.get_rank()
    dev = torch.device("cuda", rank)
    from olmax_b200.parallel.context import shard_sequence_for_cp

    res = {"tp": lambda: MeshResource.FSDP_with_TP(2, world), "fsdp": lambda: MeshResource.FSDP(world),
           "cp_ring": lambda: MeshResource.FSDP_with_CP(world, 2), "cp_all_gather": lambda: MeshResource.FSDP_with_CP(world, 2),
           }[mesh_kind]()
    attn = MultiheadSelfAttentionConfig(n_heads=4, n_kv_heads=2, head_dim=128, logit_softcap=50.0,
                                        cp_strategy=mesh_kind[3:] if mesh_kind.startswith("cp_") else None)
    cfg = DefaultTransformerConfig(vocab_size=4096, d_model=512, hidden_size=1024, num_layers=2,
                                   layer=GemmaTransformerLayerConfig(attention=attn), lm_head=LMHeadConfig(logit_softcap=30.0),
                                   tie_embeddings=True, scale_embeddings=True, sliding_window=128, sliding_window_pattern=2,
                                   ce_chunk_rows=256)
    model = cfg.build(seed=5, mesh_resource=res, device=dev, comm_backend=backend)
    mesh = model.mesh
    assert (model.store.tp_symm is not None) == (backend == "fused" and mesh.tp.size > 1)
    # the FSDP axis of a mesh that also has a TP axis runs on the peer-memory backend too
    assert (model.store.symm_ag is not None) == (backend == "fused" and mesh.shard.size > 1)
    optim = AdamWConfig(lr=ConstantSchedule(1e-3)).build(model, 1)
    gen = torch.Generator().manual_seed(7)
    cache = model.get_buffer_cache(256, dev)
    losses = []
    for step in range(3):
        ids = torch.randint(0, 4096, (4, 256), generator=gen)      # the same global batch on every rank
        per = 4 // mesh.data_parallel_size
        mine = ids[mesh.data_parallel_rank * per : (mesh.data_parallel_rank + 1) * per]
        labels = torch.roll(mine, -1, 1)
        if mesh.cp.size > 1:   # this rank's two chunks of every sequence
            mine = shard_sequence_for_cp(mine, mesh.cp.size, mesh.cp.rank)
            labels = shard_sequence_for_cp(labels, mesh.cp.size, mesh.cp.rank)
        loss, _ = model(mine.to(dev), labels.to(dev), cache)
        loss.backward()
        optim.accumulate()
        optim.step()
        t = loss.detach().clone()
        torch.distributed.all_reduce(t)
        losses.append(t.item() / world)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    return losses, {n: model.store.full_parameter(n).cpu() for n, _ in model.store.named_parameters()}


def test_tensor_parallel_matches_fsdp_on_two_gpus():
    """FSDP x TP (heads and MLP hidden split over 2 GPUs, sequence-parallel norms) trains like plain FSDP."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    tp = run_distributed_test(_tp_worker, world_size=2, backend="nccl", func_args=("tp",), timeout=300)
    fsdp = run_distributed_test(_tp_worker, world_size=2, backend="nccl", func_args=("fsdp",), timeout=300)
    lt, pt = tp[0]
    lf, pf = fsdp[0]
    assert all(abs(a - b) < 2e-2 * abs(b) for a, b in zip(lt, lf)), (lt, lf)
    for name in pf:
        assert rel_err(pt[name], pf[name]) < 1e-2, name


@pytest.mark.parametrize("world", [2, 4])
def test_fused_tensor_parallel_matches_nccl_tensor_parallel(world):
    """TP with the collectives fused into the GEMMs (all-gather of the activation rows in the q / gate-up / dgrad
    GEMMs, reduce-scatter in the o / down / dgrad epilogues, over peer memory) trains like TP over NCCL collectives;
    world 4 = FSDP 2 x TP 2."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    fused = run_distributed_test(_tp_worker, world_size=world, backend="nccl", func_args=("tp", "fused"), timeout=300)
    nccl = run_distributed_test(_tp_worker, world_size=world, backend="nccl", func_args=("tp", "nccl"), timeout=300)
    for r in range(world):
        lf, pf = fused[r]
        ln, pn = nccl[r]
        assert all(abs(a - b) < 2e-2 * abs(b) for a, b in zip(lf, ln)), (lf, ln)
        for name in pn:
            assert rel_err(pf[name], pn[name]) < 1e-2, name


def _vp_worker(backend, vocab_parallel):
    from olmax_b200.models import DefaultTransformerConfig, ReorderedNormTransformerLayerConfig
    from olmax_b200.nn import LMHeadConfig, MultiheadSelfAttentionConfig
    from olmax_b200.ops import _lib
    from olmax_b200.optim import AdamWConfig, ConstantSchedule
    from olmax_b200.parallel import MeshResource, dist_utils

    world, rank = dist_utils.get_world_size(), dist_utils.get_rank()
    dev = torch.device("cuda", rank)
    attn = MultiheadSelfAttentionConfig(n_heads=4, n_kv_heads=2, head_dim=128)
    cfg = DefaultTransformerConfig(vocab_size=4096, d_model=512, hidden_size=1024, num_layers=2,
                                   layer=ReorderedNormTransformerLayerConfig(attention=attn),
                                   lm_head=LMHeadConfig(logit_softcap=30.0, vocab_parallel=vocab_parallel), ce_chunk_rows=256)
    model = cfg.build(seed=5, mesh_resource=MeshResource.FSDP_with_TP(2, world), device=dev, comm_backend=backend)
    assert model.lm_head.vocab_parallel == vocab_parallel
    optim = AdamWConfig(lr=ConstantSchedule(1e-3)).build(model, 1)
    gen = torch.Generator().manual_seed(7)
    cache = model.get_buffer_cache(256, dev)
    mesh = model.mesh
    losses = []
    for step in range(3):
        ids = torch.randint(0, 4096, (4, 256), generator=gen)
        per = 4 // mesh.data_parallel_size
        mine = ids[mesh.data_parallel_rank * per : (mesh.data_parallel_rank + 1) * per]
        labels = torch.roll(mine, -1, 1)
        labels[:, -1] = -100
        loss, _ = model(mine.to(dev), labels.to(dev), cache, z_loss_multiplier=1e-4)
        loss.backward()
        optim.accumulate()
        optim.step()
        t = loss.detach().clone()
        torch.distributed.all_reduce(t)
        losses.append(t.item() / world)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    return losses, {n: model.store.full_parameter(n).cpu() for n, _ in model.store.named_parameters()}


@pytest.mark.parametrize("world,backend", [(2, "fused"), (2, "nccl"), (4, "fused")])
def test_vocab_parallel_head_trains_like_the_replicated_head(world, backend):
    """The LM head's vocabulary split over the TP pair (statistics exchanged through peer memory on the fused backend,
    through NCCL otherwise) trains like the head replicated over the pair."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    vp = run_distributed_test(_vp_worker, world_size=world, backend="nccl", func_args=(backend, True), timeout=300)
    base = run_distributed_test(_vp_worker, world_size=world, backend="nccl", func_args=("nccl", False), timeout=300)
    lv, pv = vp[0]
    lb, pb = base[0]
    assert all(abs(a - b) < 2e-2 * abs(b) for a, b in zip(lv, lb)), (lv, lb)
    for name in pb:
        assert rel_err(pv[name], pb[name]) < 1e-2, name


def test_fused_fsdp_with_tied_embeddings_matches_nccl():
    """A tied LM head stages its weight gradient under the embedding unit during the forward pass; the peer-memory
    reduce-scatter has to fold it before any layer's gradients reuse that staging buffer."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    fused = run_distributed_test(_tp_worker, world_size=2, backend="nccl", func_args=("fsdp", "fused"), timeout=300)
    nccl = run_distributed_test(_tp_worker, world_size=2, backend="nccl", func_args=("fsdp", "nccl"), timeout=300)
    for r in range(2):
        lf, pf = fused[r]
        ln, pn = nccl[r]
        assert all(abs(a - b) < 2e-2 * abs(b) for a, b in zip(lf, ln)), (lf, ln)
        for name in pn:
            assert rel_err(pf[name], pn[name]) < 1e-2, name


@pytest.mark.parametrize("strategy", ["all_gather", "ring"])
def test_context_parallel_matches_fsdp_on_two_gpus(strategy):
    """Sequences split over 2 GPUs (dual-chunk-swap order; K/V all-gathered or travelling around the ring; the
    sliding-window layers of the ring run use the all-gather composition) train like plain FSDP."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    cp = run_distributed_test(_tp_worker, world_size=2, backend="nccl", func_args=("cp_" + strategy,), timeout=300)
    fsdp = run_distributed_test(_tp_worker, world_size=2, backend="nccl", func_args=("fsdp",), timeout=300)
    lc, pc = cp[0]
    lf, pf = fsdp[0]
    assert all(abs(a - b) < 2e-2 * abs(b) for a, b in zip(lc, lf)), (lc, lf)
    for name in pf:
        assert rel_err(pc[name], pf[name]) < 1e-2, name


def test_peer_barrier_times_out_and_reports():
    """A member that never arrives: the bounded wait runs out, the kernel records the error and returns, the host
    raises, and the GPU stays usable (the "missing peer" is a flag word that nothing sets; both flag arrays are local)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from olmax_b200.ops import _lib, kernels as K

    dev = torch.device("cuda")
    mine = torch.zeros(64, dtype=torch.int32, device=dev)
    absent = torch.zeros(64, dtype=torch.int32, device=dev)
    table = K.pointer_table([mine.data_ptr(), absent.data_ptr()], dev)
    K.peer_barrier(table, 0, 2, 1, timeout_s=0.05)
    torch.cuda.synchronize()
    assert absent[0].item() == 1 and mine[0].item() == 1 and mine[1].item() == 0   # we published, the peer never did
    with pytest.raises(K.KernelError, match="peer flag wait timed out"):
        _lib.check_status()
    # the error words were cleared by the check and the device still works; an arrived peer lets the barrier pass
    mine[1] = 2
    K.peer_barrier(table, 0, 2, 2, timeout_s=0.05)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.ones(4, device=dev).sum().item() == 4
