"""GPU numerics: every CUDA kernel against the PyTorch fp32 restatement of the same op."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from olmax_b200.ops import reference as ref
from olmax_b200.testing import rel_err


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from olmax_b200.ops import kernels

    return kernels


def _check_status():
    from olmax_b200.ops import _lib

    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("M,N,Kd", [(128, 256, 64), (1000, 776, 520), (2048, 1376, 1024)])
def test_gemm_layouts(K, M, N, Kd):
    dev = "cuda"
    torch.manual_seed(0)
    a = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16)
    b = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16)
    want = a.float() @ b.float().t()
    c = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
    K.gemm(a, b, c, M, N, Kd)
    assert rel_err(c, want) < 5e-3
    bt = b.t().contiguous()
    c.zero_()
    K.gemm(a, bt, c, M, N, Kd, b_mn=True)
    assert rel_err(c, want) < 5e-3
    at = a.t().contiguous()
    cf = torch.zeros(M, N, device=dev, dtype=torch.float32)
    K.gemm(at, bt, cf, M, N, Kd, a_mn=True, b_mn=True, epi=K.EPI_F32)
    assert rel_err(cf, want) < 1e-4
    K.gemm(at, bt, cf, M, N, Kd, a_mn=True, b_mn=True, epi=K.EPI_F32_ACC, alpha=0.5)
    assert rel_err(cf, 1.5 * want) < 1e-4
    K.gemm(at, bt, cf, M, N, Kd, a_mn=True, b_mn=True, epi=K.EPI_F32_RED, alpha=0.5)
    assert rel_err(cf, 2.0 * want) < 1e-4
    c.copy_(want.to(torch.bfloat16))
    K.gemm(a, b, c, M, N, Kd, epi=K.EPI_BF16_ACC)
    assert rel_err(c, 2.0 * want) < 8e-3
    _check_status()


@pytest.mark.parametrize("M,N,Kd", [(4096, 4608, 1024), (2304, 5120, 2048), (1152, 20000, 256)])
def test_gemm_cta_pair_tiles_and_split_k_tail(K, M, N, Kd):
    """Shapes with enough 256 x 256 tiles that the CTA-pair kernel (tcgen05.mma.cta_group::2) runs, ragged in M and N,
    in all three layouts; the accumulating fp32 epilogue also with its last wave cut into k slices."""
    dev = "cuda"
    torch.manual_seed(3)
    a = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16)
    b = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16)
    want = a.float() @ b.float().t()
    c = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
    K.gemm(a, b, c, M, N, Kd)
    assert rel_err(c, want) < 5e-3
    bt = b.t().contiguous()
    c.zero_()
    K.gemm(a, bt, c, M, N, Kd, b_mn=True)
    assert rel_err(c, want) < 5e-3
    at = a.t().contiguous()
    cf = torch.zeros(M, N, device=dev, dtype=torch.float32)
    K.gemm(at, bt, cf, M, N, Kd, a_mn=True, b_mn=True, epi=K.EPI_F32_ACC)
    K.gemm(at, bt, cf, M, N, Kd, a_mn=True, b_mn=True, epi=K.EPI_F32_ACC, alpha=0.5)
    assert rel_err(cf, 1.5 * want) < 1e-4
    cf2 = torch.zeros(M, N, device=dev, dtype=torch.float32)
    K.gemm(at, bt, cf2, M, N, Kd, a_mn=True, b_mn=True, epi=K.EPI_F32_ACC, alpha=1.5, no_split_k=True)
    assert rel_err(cf2, 1.5 * want) < 1e-4
    _check_status()


def test_gemm_sharded_operands(K):
    dev = "cuda"
    torch.manual_seed(1)
    M, N, Kd, R = 512, 1024, 512, 4
    a = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16)
    stage = torch.zeros(R, (N // R) * Kd + 64, device=dev, dtype=torch.bfloat16)
    for r in range(R):
        stage[r, : (N // R) * Kd] = w[r * (N // R) : (r + 1) * (N // R)].reshape(-1)
    c = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
    K.gemm(a, stage, c, M, N, Kd, ldb=Kd, N_s=N // R, b_shard_stride=stage.stride(0))
    assert rel_err(c, a.float() @ w.float().t()) < 5e-3
    dy = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
    dx = torch.zeros(M, Kd, device=dev, dtype=torch.bfloat16)
    K.gemm(dy, stage, dx, M, Kd, N, b_mn=True, ldb=Kd, Kc_s=N // R, b_shard_stride=stage.stride(0))
    assert rel_err(dx, dy.float() @ w.float()) < 5e-3
    # weight gradient written as R row blocks `stride` apart
    g = torch.zeros(R, (N // R) * Kd + 64, device=dev, dtype=torch.float32)
    K.gemm(dy, a, g, N, Kd, M, a_mn=True, b_mn=True, epi=K.EPI_F32_ACC, ldc=Kd, M_s=N // R, c_shard_stride=g.stride(0))
    got = torch.cat([g[r, : (N // R) * Kd].view(N // R, Kd) for r in range(R)])
    assert rel_err(got, dy.float().t() @ a.float()) < 1e-4
    # the same through a device pointer table (the form used for peer GPUs' buffers)
    g.zero_()
    table = K.pointer_table([g[r].data_ptr() for r in range(R)], torch.device(dev))
    K.gemm(dy, a, g, N, Kd, M, a_mn=True, b_mn=True, epi=K.EPI_F32_RED, ldc=Kd, M_s=N // R, c_shards=table)
    got = torch.cat([g[r, : (N // R) * Kd].view(N // R, Kd) for r in range(R)])
    assert rel_err(got, dy.float().t() @ a.float()) < 1e-4
    _check_status()


@pytest.mark.parametrize("rows", [128, 352, 640, 1152, 1376])
def test_gemm_every_sharded_layout_over_shard_sizes(K, rows):
    """The five GEMM forms of a linear layer whose weight is split into R row shards of ``rows`` rows (forward, gated
    forward, dgrad, weight gradient accumulated into a sharded buffer, weight gradient stored to per-owner buffers),
    for shard sizes that are and are not multiples of 64 / 128 / 256: the sizes 8-way sharding produces for real
    models (1376 = 11008 / 8, 640 = 5120 / 8, 1152 = 4608 / 4, 128 = 1024 / 8)."""
    dev = "cuda"
    torch.manual_seed(rows)
    R, Kd, M, gap = 4, 256, 512, 1024
    N = R * rows
    x = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16) * 0.25
    W = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) * 0.1
    W2 = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) * 0.1
    stride = rows * Kd + gap

    def pieces(w):
        buf = torch.zeros(R * stride, device=dev, dtype=torch.bfloat16)
        for r in range(R):
            buf[r * stride : r * stride + rows * Kd] = w[r * rows : (r + 1) * rows].reshape(-1)
        return buf

    b1, b2 = pieces(W), pieces(W2)
    y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    K.gemm(x, b1, y, M, N, Kd, ldb=Kd, ldc=N, N_s=rows, b_shard_stride=stride)
    assert rel_err(y, x.float() @ W.float().t()) < 5e-3, "forward"
    act, cg, cu = torch.empty_like(y), torch.empty_like(y), torch.empty_like(y)
    K.gemm(x, b1, act, M, N, Kd, ldb=Kd, ldc=N, N_s=rows, b_shard_stride=stride, epi=K.EPI_SWIGLU, b2=b2, c2=cg, c3=cu)
    g, u = x.float() @ W.float().t(), x.float() @ W2.float().t()
    assert rel_err(cg, g) < 5e-3 and rel_err(cu, u) < 5e-3 and rel_err(act, torch.nn.functional.silu(g) * u) < 1e-2, "gated"
    dy = torch.randn(M, N, device=dev, dtype=torch.bfloat16) * 0.25
    dx = torch.empty(M, Kd, device=dev, dtype=torch.bfloat16)
    K.gemm(dy, b1, dx, M, Kd, N, b_mn=True, ldb=Kd, ldc=Kd, Kc_s=rows, b_shard_stride=stride)
    assert rel_err(dx, dy.float() @ W.float()) < 5e-3, "dgrad"
    want = dy.float().t() @ x.float()
    acc = torch.zeros(R, stride, device=dev, dtype=torch.float32)
    K.gemm(dy, x, acc, N, Kd, M, a_mn=True, b_mn=True, epi=K.EPI_F32_ACC, ldc=Kd, M_s=rows, c_shard_stride=stride)
    got = torch.cat([acc[r, : rows * Kd].view(rows, Kd) for r in range(R)])
    assert rel_err(got, want) < 1e-4, "wgrad into a sharded accumulator"
    outs = [torch.full((rows, Kd), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(R)]
    table = K.pointer_table([o.data_ptr() for o in outs], torch.device(dev))
    K.gemm(dy, x, outs[0], N, Kd, M, a_mn=True, b_mn=True, epi=K.EPI_BF16, ldc=Kd, M_s=rows, c_shards=table)
    assert rel_err(torch.cat(outs), want) < 5e-3, "wgrad stored to the owners"
    _check_status()


def test_gemm_column_shards_that_end_inside_a_store_chunk(K):
    """Forward GEMM over weights gathered as 8 row shards of 1376 rows (11008 / 8): a shard's last tile holds 96 output
    columns, so the epilogue must not write whole 64-column chunks across the shard's end."""
    dev = "cuda"
    torch.manual_seed(3)
    R, N, Kd, M = 8, 11008, 512, 1024
    Ns, gap = N // R, 4096
    x = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16) * 0.25
    W = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) * 0.05
    stride = Ns * Kd + gap
    buf = torch.zeros(R * stride, device=dev, dtype=torch.bfloat16)
    for r in range(R):
        buf[r * stride : r * stride + Ns * Kd] = W[r * Ns : (r + 1) * Ns].reshape(-1)
    y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    K.gemm(x, buf, y, M, N, Kd, ldb=Kd, ldc=N, N_s=Ns, b_shard_stride=stride)
    assert rel_err(y, x.float() @ W.float().t()) < 5e-3
    dy = torch.randn(M, N, device=dev, dtype=torch.bfloat16) * 0.25
    dx = torch.empty(M, Kd, device=dev, dtype=torch.bfloat16)
    K.gemm(dy, buf, dx, M, Kd, N, b_mn=True, ldb=Kd, ldc=Kd, Kc_s=Ns, b_shard_stride=stride)   # contraction over the shards
    assert rel_err(dx, dy.float() @ W.float()) < 5e-3
    _check_status()


@pytest.mark.parametrize("N,Kd,M,R,epi_name", [
    (4096, 4096, 8192, 4, "bf16"),
    (4096, 4096, 8192, 2, "f32"),
    (11008, 1024, 4096, 8, "bf16"),    # 1376-row shards: partly filled tiles at every shard boundary
    (1024, 5120, 2048, 8, "bf16"),     # 128-row shards (k / v of a grouped-query model over 8 owners): single-CTA tiles
])
def test_gemm_store_to_shards(K, N, Kd, M, R, epi_name):
    """Weight-gradient GEMM whose row blocks are stored into per-owner buffers in either wire format (the fused
    reduce-scatter's epilogue, here with all owners on this GPU)."""
    dev = "cuda"
    torch.manual_seed(13)
    dy = torch.randn(M, N, device=dev, dtype=torch.bfloat16) * 0.25
    x = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16) * 0.25
    dtype = torch.bfloat16 if epi_name == "bf16" else torch.float32
    rows = N // R
    outs = [torch.full((rows, Kd), float("nan"), device=dev, dtype=dtype) for _ in range(R)]
    table = K.pointer_table([o.data_ptr() for o in outs], torch.device(dev))
    K.gemm(dy, x, outs[0], N, Kd, M, a_mn=True, b_mn=True, epi=K.EPI_BF16 if epi_name == "bf16" else K.EPI_F32, ldc=Kd,
           M_s=rows, c_shards=table)
    got = torch.cat(outs).float()
    assert torch.isfinite(got).all()
    assert rel_err(got, dy.float().t() @ x.float()) < (5e-3 if epi_name == "bf16" else 1e-4)
    _check_status()


@pytest.mark.parametrize("gelu", [False, True])
def test_gemm_gated_epilogue(K, gelu):
    dev = "cuda"
    torch.manual_seed(2)
    M, N, Kd = 512, 384, 256
    a = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16) * 0.5
    wg = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) * 0.1
    wu = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) * 0.1
    g = a.float() @ wg.float().t()
    u = a.float() @ wu.float().t()
    act = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    cg, cu = torch.empty_like(act), torch.empty_like(act)
    K.gemm(a, wg, act, M, N, Kd, epi=K.EPI_GEGLU if gelu else K.EPI_SWIGLU, b2=wu, c2=cg, c3=cu)
    want = ref.activation("gelu_tanh" if gelu else "silu", g) * u
    assert rel_err(act, want) < 8e-3
    assert rel_err(cg, g) < 5e-3 and rel_err(cu, u) < 5e-3
    _check_status()


@pytest.mark.parametrize("B,S,H,Hkv,causal,window,softcap", [
    (1, 256, 2, 2, True, -1, 0.0),
    (2, 512, 4, 2, True, -1, 0.0),
    (1, 333, 2, 1, True, -1, 0.0),
    (1, 640, 2, 2, True, 200, 0.0),
    (1, 384, 2, 2, True, -1, 20.0),
    (1, 256, 2, 2, False, -1, 0.0),
    (1, 128, 2, 2, True, -1, 0.0),        # one query tile: the second tile of the pair is inactive
    (2, 2048, 16, 4, True, -1, 0.0),      # more work items than SMs: several items per persistent CTA
    (3, 1024, 5, 5, True, 300, 0.0),      # 15 (batch, head) slices: a partly filled scheduling group; window
    (1, 900, 3, 1, False, -1, 0.0),       # no mask, ragged length, equal-weight items
    (1, 2048, 8, 2, True, 512, 30.0),     # window + soft-cap + grouped heads together (the Gemma-like layer)
])
def test_flash_attention(K, B, S, H, Hkv, causal, window, softcap):
    dev = "cuda"
    torch.manual_seed(3)
    q = torch.randn(B, S, H, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, S, Hkv, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, S, Hkv, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    o, lse = K.flash_attn_fwd(q.detach(), k.detach(), v.detach(), causal=causal, window=window, softcap=softcap)
    o_ref, lse_ref = ref.attention(q.float(), k.float(), v.float(), causal, window, softcap)
    assert rel_err(o, o_ref) < 6e-3
    assert rel_err(lse, lse_ref) < 1e-3
    d_o = torch.randn_like(o)
    gq, gk, gv = torch.autograd.grad(o_ref, (q, k, v), d_o.float())
    dq, dk, dv = K.flash_attn_bwd(q.detach(), k.detach(), v.detach(), o, lse, d_o, causal=causal, window=window, softcap=softcap)
    assert rel_err(dq, gq) < 1e-2 and rel_err(dk, gk) < 1e-2 and rel_err(dv, gv) < 1e-2
    _check_status()


@pytest.mark.parametrize("S,Sk,q_off,window,softcap", [
    (256, 512, 256, -1, 0.0),      # late query chunk against the causally visible prefix
    (128, 128, 384, -1, 0.0),      # ring block far below the diagonal: every key visible
    (256, 640, 384, 300, 0.0),     # sliding window over a left-trimmed prefix
    (200, 456, 256, -1, 15.0),     # ragged lengths + soft-cap
])
def test_flash_attention_rectangular_blocks(K, S, Sk, q_off, window, softcap):
    """Query rows at key-axis offset ``q_off`` against a key block of another length (context-parallel blocks), read
    through strided slices of larger tensors as the context-parallel code does."""
    dev = "cuda"
    torch.manual_seed(5)
    B, H, Hkv = 2, 4, 2
    q_all = torch.randn(B, S + 64, H, 128, device=dev, dtype=torch.bfloat16)
    k_all = torch.randn(B, Sk + 128, Hkv, 128, device=dev, dtype=torch.bfloat16)
    v_all = torch.randn(B, Sk + 128, Hkv, 128, device=dev, dtype=torch.bfloat16)
    q, k, v = q_all[:, 64:], k_all[:, 128:], v_all[:, 128:]
    qr, kr, vr = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    o, lse = K.flash_attn_fwd(q, k, v, causal=True, window=window, softcap=softcap, q_off=q_off)
    o_ref, lse_ref = ref.attention(qr, kr, vr, True, window, softcap, q_off=q_off)
    assert rel_err(o, o_ref) < 6e-3 and rel_err(lse, lse_ref) < 1e-3
    d_o = torch.randn_like(o)
    gq, gk, gv = torch.autograd.grad(o_ref, (qr, kr, vr), d_o.float())
    dq, dk, dv = K.flash_attn_bwd(q, k, v, o, lse, d_o, causal=True, window=window, softcap=softcap, q_off=q_off)
    assert rel_err(dq, gq) < 1e-2 and rel_err(dk, gk) < 1e-2 and rel_err(dv, gv) < 1e-2
    # the explicit block backward of the oracle agrees with autograd (it is the CPU path of context parallelism)
    rq, rk, rv = ref.attention_bwd(q.float(), k.float(), v.float(), o_ref.detach(), lse_ref.detach(), d_o.float(), True,
                                   window, softcap, q_off=q_off)
    assert rel_err(rq, gq) < 1e-4 and rel_err(rk, gk) < 1e-4 and rel_err(rv, gv) < 1e-4
    _check_status()


def test_flash_attention_rejects_unsupported_geometry(K):
    q = torch.randn(1, 128, 2, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(1, 512, 2, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(Exception):   # keys beyond the last query row's position: no query would see the last tiles
        K.flash_attn_fwd(q, k, k, causal=True, q_off=0)


def test_blockwise_attention_composes_to_full_attention(K):
    """The two compositions context parallelism uses (prefix blocks; ring blocks merged by log-sum-exp), evaluated
    for every rank in turn on one GPU, reproduce plain causal attention and its gradients."""
    from olmax_b200.ops import functional as F
    from olmax_b200.parallel.context import _merge, _ring_pairs, cp_local_positions

    dev, cp, S, B, H, Hkv = "cuda", 2, 1024, 1, 4, 2
    c = S // (2 * cp)
    torch.manual_seed(6)
    q, k, v = (torch.randn(B, S, h, 128, device=dev, dtype=torch.bfloat16) for h in (H, Hkv, Hkv))
    d_o = torch.randn_like(q)
    o_full, lse_full = K.flash_attn_fwd(q, k, v)
    dq_full, dk_full, dv_full = K.flash_attn_bwd(q, k, v, o_full, lse_full, d_o)
    local = [cp_local_positions(S, cp, r, device=dev) for r in range(cp)]
    dq = torch.zeros(q.shape, device=dev)
    dk, dv = torch.zeros(k.shape, device=dev), torch.zeros(v.shape, device=dev)
    for r in range(cp):
        ql = q[:, local[r]]
        o_acc = torch.zeros(ql.shape, device=dev)
        lse_acc = torch.full((B, H, 2 * c), float("-inf"), device=dev)
        for j in range(cp):
            kl, vl = k[:, local[j]], v[:, local[j]]
            for qh, kh, dist_c in _ring_pairs(r, j, cp):
                qs, ks = slice(qh * c, (qh + 1) * c), slice(kh * c, (kh + 1) * c)
                oo, ll = F.attention_block_fwd(ql[:, qs], kl[:, ks], vl[:, ks], q_off=dist_c * c)
                o_acc[:, qs], lse_acc[:, :, qs] = _merge(o_acc[:, qs], lse_acc[:, :, qs], oo, ll)
        assert rel_err(o_acc, o_full[:, local[r]]) < 6e-3
        assert rel_err(lse_acc, lse_full[:, :, local[r]]) < 1e-3
        o_l, dol = o_acc.to(torch.bfloat16), d_o[:, local[r]]
        for j in range(cp):
            kl, vl = k[:, local[j]], v[:, local[j]]
            for qh, kh, dist_c in _ring_pairs(r, j, cp):
                qs, ks = slice(qh * c, (qh + 1) * c), slice(kh * c, (kh + 1) * c)
                g = F.attention_block_bwd(ql[:, qs], kl[:, ks], vl[:, ks], o_l[:, qs], lse_acc[:, :, qs].contiguous(),
                                          dol[:, qs], q_off=dist_c * c)
                dq[:, local[r][qs]] += g[0].float()
                dk[:, local[j][ks]] += g[1].float()
                dv[:, local[j][ks]] += g[2].float()
    assert rel_err(dq, dq_full) < 1e-2 and rel_err(dk, dk_full) < 1e-2 and rel_err(dv, dv_full) < 1e-2
    _check_status()


@pytest.mark.parametrize("rows,d,bias", [(300, 512, True), (70, 4096, True), (33, 8192, False), (257, 128, True),
                                           (65, 2048, True)])
def test_layernorm(K, rows, d, bias):
    dev = "cuda"
    torch.manual_seed(8)
    x = (torch.randn(rows, d, device=dev) * 2 + 0.5).to(torch.bfloat16)
    w = (torch.randn(d, device=dev) * 0.1 + 1).to(torch.bfloat16)
    b = (torch.randn(d, device=dev) * 0.1).to(torch.bfloat16) if bias else None
    y = torch.empty_like(x)
    mean = torch.empty(rows, device=dev)
    rstd = torch.empty(rows, device=dev)
    K.layernorm_fwd(x, w, b, y, mean, rstd, rows=rows, d=d, eps=1e-5)
    xr, wr = x.float().requires_grad_(True), w.float().requires_grad_(True)
    br = b.float().requires_grad_(True) if bias else None
    want = torch.nn.functional.layer_norm(xr, (d,), wr, br, 1e-5)
    assert rel_err(y, want) < 5e-3
    assert rel_err(mean, x.float().mean(-1)) < 1e-4
    dy = torch.randn_like(y)
    leaves = [xr, wr] + ([br] if bias else [])
    grads = torch.autograd.grad(want, leaves, dy.float())
    dx = torch.empty_like(x)
    dw = torch.zeros(d, device=dev)
    db = torch.zeros(d, device=dev) if bias else None
    K.layernorm_bwd(dy, x, w, mean, rstd, dx, rows=rows, d=d, dw=dw, db=db, scale=0.5)
    assert rel_err(dx, grads[0]) < 1e-2
    assert rel_err(dw, 0.5 * grads[1]) < 1e-2
    if bias:
        assert rel_err(db, 0.5 * grads[2]) < 1e-2
    _check_status()


@pytest.mark.parametrize("rows,d,heads", [(300, 512, 1), (64, 4096, 1), (100, 128, 6), (77, 2048, 1), (40, 5120, 1)])
def test_rmsnorm(K, rows, d, heads):
    dev = "cuda"
    torch.manual_seed(4)
    width = d * heads
    x = torch.randn(rows, width, device=dev, dtype=torch.bfloat16)
    res = torch.randn(rows, width, device=dev, dtype=torch.bfloat16)
    w = (torch.randn(d, device=dev) * 0.1 + 1).to(torch.bfloat16)
    n_rows = rows * heads
    xv = x.view(rows, heads, d)

    def want(t):
        return ref.rms_norm(t.float().view(rows, heads, d), w.float(), 1e-5).view(rows, width)

    y = torch.empty_like(x)
    rstd = torch.empty(n_rows, device=dev, dtype=torch.float32)
    K.rmsnorm_fwd(x, w, y, rows=n_rows, d=d, eps=1e-5, rstd=rstd, heads=heads, ld_x=width, ld_y=width)
    assert rel_err(y, want(x)) < 5e-3
    K.rmsnorm_fwd(x, w, y, rows=n_rows, d=d, eps=1e-5, res=res, heads=heads, ld_x=width, ld_res=width, ld_y=width)
    assert rel_err(y, want(x) + res.float()) < 5e-3
    h = torch.empty_like(x)
    K.rmsnorm_fwd(x, w, y, rows=n_rows, d=d, eps=1e-5, res=res, sum_out=h, rstd=rstd, heads=heads, ld_x=width,
                  ld_res=width, ld_y=width, add_before=True)
    hs = (x.float() + res.float()).to(torch.bfloat16)
    assert rel_err(h, hs) < 1e-3 and rel_err(y, want(hs)) < 5e-3
    # backward of the plain form
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    yy = ref.rms_norm(xf.view(rows, heads, d), wf, 1e-5).view(rows, width)
    dy = torch.randn_like(x)
    gx, gw = torch.autograd.grad(yy, (xf, wf), dy.float())
    K.rmsnorm_fwd(x, w, y, rows=n_rows, d=d, eps=1e-5, rstd=rstd, heads=heads, ld_x=width, ld_y=width)
    dx = torch.empty_like(x)
    dw = torch.zeros(d, device=dev, dtype=torch.float32)
    K.rmsnorm_bwd(dy, x, w, rstd, dx, rows=n_rows, d=d, dw=dw, heads=heads, ld_dy=width, ld_x=width, ld_dx=width)
    assert rel_err(dx, gx) < 6e-3 and rel_err(dw, gw) < 6e-3
    _check_status()


def test_rope_and_glu(K):
    dev = "cuda"
    torch.manual_seed(5)
    x = torch.randn(2, 96, 3, 128, device=dev, dtype=torch.bfloat16)
    cos, sin = ref.rope_tables(96, 128, 500000.0, device=dev)
    y = torch.empty_like(x)
    K.rope(x, y, cos, sin)
    assert rel_err(y, ref.apply_rope(x.float(), cos, sin)) < 4e-3
    back = torch.empty_like(x)
    K.rope(y, back, cos, sin, sign=-1.0)
    assert rel_err(back, x) < 8e-3
    g = torch.randn(64, 512, device=dev, dtype=torch.bfloat16)
    u = torch.randn_like(g)
    da = torch.randn_like(g)
    for gelu, name in ((False, "silu"), (True, "gelu_tanh")):
        a = torch.empty_like(g)
        K.glu_fwd(g, u, a, gelu)
        gf, uf = g.float().requires_grad_(True), u.float().requires_grad_(True)
        want = ref.activation(name, gf) * uf
        assert rel_err(a, want) < 5e-3
        wg, wu = torch.autograd.grad(want, (gf, uf), da.float())
        dg, du, a2 = torch.empty_like(g), torch.empty_like(g), torch.empty_like(g)
        K.glu_bwd(g, u, da, dg, du, a2, gelu)
        assert rel_err(dg, wg) < 6e-3 and rel_err(du, wu) < 6e-3 and rel_err(a2, want) < 5e-3
    _check_status()


@pytest.mark.parametrize("B,S,n,hd,head_wise", [
    (2, 96, 32, 128, False),     # norm over the whole 4096-wide projection (256 pairs: one per thread)
    (2, 96, 8, 128, False),      # 1024-wide k projection of a grouped-query model
    (1, 200, 4, 128, True),      # head-wise norm
    (2, 64, 3, 64, True),        # head dim 64
    (1, 50, 64, 128, False),     # 8192-wide projection (two pairs per thread)
])
def test_fused_rmsnorm_rope_matches_the_two_kernels_and_the_fp32_reference(K, B, S, n, hd, head_wise):
    dev = "cuda"
    torch.manual_seed(9)
    T, width = B * S, n * hd
    heads, d = (n, hd) if head_wise else (1, width)
    x = torch.randn(T, width, device=dev, dtype=torch.bfloat16)
    w = (torch.randn(d, device=dev) * 0.1 + 1).to(torch.bfloat16)
    cos, sin = ref.rope_tables(S, hd, 500000.0, device=dev)
    rows = T * heads
    y, rstd = torch.empty_like(x), torch.empty(rows, device=dev, dtype=torch.float32)
    K.rmsnorm_rope_fwd(x, w, y, rstd, cos, sin, rows=rows, d=d, hd=hd, heads=heads, seq_len=S, eps=1e-5, ld_x=width,
                       ld_y=width)
    # the same through the separate kernels, which round the normalised value to bf16 before the rotation
    yn, rstd2, y2 = torch.empty_like(x), torch.empty_like(rstd), torch.empty_like(x)
    K.rmsnorm_fwd(x, w, yn, rows=rows, d=d, eps=1e-5, rstd=rstd2, heads=heads, ld_x=width, ld_y=width)
    K.rope(yn.view(B, S, n, hd), y2.view(B, S, n, hd), cos, sin)
    assert rel_err(y, y2) < 4e-3 and rel_err(rstd, rstd2) < 1e-5
    xf, wf = x.float().requires_grad_(True), w.float().requires_grad_(True)
    want = ref.apply_rope(ref.rms_norm(xf.view(T, heads, d), wf, 1e-5).view(B, S, n, hd), cos, sin)
    assert rel_err(y.view(B, S, n, hd), want) < 6e-3
    dy = torch.randn_like(x)
    gx, gw = torch.autograd.grad(want, (xf, wf), dy.float().view(B, S, n, hd))
    dx, dw = torch.empty_like(x), torch.zeros(d, device=dev, dtype=torch.float32)
    K.rmsnorm_rope_bwd(dy, x, w, rstd, dx, cos, sin, rows=rows, d=d, hd=hd, heads=heads, seq_len=S, dw=dw, dw_scale=0.5,
                       ld_dy=width, ld_x=width, ld_dx=width)
    assert rel_err(dx, gx) < 1e-2 and rel_err(dw, 0.5 * gw) < 1e-2
    _check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reduce_slots_folds_fp32_and_bf16_staging(K, dtype):
    dev = "cuda"
    torch.manual_seed(12)
    R, n, stride = 4, 8 * 1000, 8 * 1300
    stage = torch.randn(R * stride, device=dev).to(dtype)
    acc = torch.randn(n, device=dev)
    want = acc + 0.25 * stage.view(R, stride)[:, :n].float().sum(0)
    K.reduce_slots(stage, acc, n, R, stride, 0.25)
    assert rel_err(acc, want) < 1e-6
    _check_status()


def test_embedding_kernels(K):
    dev = torch.device("cuda")
    torch.manual_seed(6)
    V, d, R = 512, 256, 4
    w = torch.randn(V, d, device=dev, dtype=torch.bfloat16)
    ids = torch.randint(0, V, (300,), device=dev)
    shards = [w[r * (V // R) : (r + 1) * (V // R)].contiguous() for r in range(R)]
    table = K.pointer_table([s.data_ptr() for s in shards], dev)
    out = torch.empty(300, d, device=dev, dtype=torch.bfloat16)
    K.embed_gather(ids, table, V // R, R, out, d, 2.0)
    assert rel_err(out, w[ids].float() * 2.0) < 1e-3
    grads = [torch.zeros(V // R, d, device=dev, dtype=torch.float32) for _ in range(R)]
    gtable = K.pointer_table([g.data_ptr() for g in grads], dev)
    dout = torch.randn(300, d, device=dev, dtype=torch.bfloat16)
    K.embed_scatter(ids, gtable, V // R, R, dout, d, 0.5)
    want = torch.zeros(V, d, device=dev)
    want.index_add_(0, ids, dout.float() * 0.5)
    assert rel_err(torch.cat(grads), want) < 1e-5
    _check_status()


@pytest.mark.parametrize("softcap,z", [(0.0, 0.0), (30.0, 1e-4)])
def test_cross_entropy_kernel(K, softcap, z):
    dev = "cuda"
    torch.manual_seed(7)
    rows, V = 200, 4104
    logits = (torch.randn(rows, V, device=dev) * 3).contiguous()
    labels = torch.randint(0, V, (rows,), device=dev)
    labels[::7] = -100
    labels[3::11] = V   # out of range but not ignored (the sequential synthetic data produces these): counted in the mean
                        # and in the z-loss, no cross-entropy term
    lf = logits.clone().requires_grad_(True)
    loss, zl = ref.fused_cross_entropy(lf, labels, z_loss_multiplier=z, logit_softcap=softcap)
    (gl,) = torch.autograd.grad(loss + zl, lf)
    stats = torch.zeros(2, device=dev)
    inv = torch.empty(2, device=dev)
    counter = torch.zeros(2, device=dev, dtype=torch.int32)
    K.count_valid(labels, -100, V, inv, counter)
    dl = torch.empty(rows, V, device=dev, dtype=torch.bfloat16)
    K.ce_fwd_bwd(logits, labels, dl, stats, inv, V=V, softcap=softcap, z_loss=z)
    got = stats[0] * inv[0]
    assert abs(got.item() - loss.item()) < 2e-3 * max(1.0, abs(loss.item()))
    assert abs((stats[1] * inv[0] * z).item() - zl.item()) < 2e-3 * max(1e-6, abs(zl.item()))
    assert rel_err(dl, gl) < 8e-3
    _check_status()


@pytest.mark.parametrize("softcap,z", [(0.0, 0.0), (30.0, 1e-3)])
def test_vocab_parallel_cross_entropy_kernels(K, softcap, z):
    """Two vocabulary slices of one logits matrix, processed like two members of a group on one GPU: per-slice
    statistics, then each slice's gradient from both members' statistics, against the unsplit cross entropy."""
    dev = "cuda"
    torch.manual_seed(11)
    rows, V, n = 96, 2 * 1032, 2
    Vl = V // n
    logits = (torch.randn(rows, V, device=dev) * 3).contiguous()
    labels = torch.randint(0, V, (rows,), device=dev)
    labels[::5] = -100
    labels[2::9] = V
    lf = logits.clone().requires_grad_(True)
    loss, zl = ref.fused_cross_entropy(lf, labels, z_loss_multiplier=z, logit_softcap=softcap)
    (gl,) = torch.autograd.grad(loss + zl, lf)
    # rows come from two sources (48 rows each) with their own counts, as under sequence parallelism
    per = rows // n
    cnt = torch.stack([(labels[i * per : (i + 1) * per] != -100).sum() for i in range(n)]).float().clamp(min=1)
    inv = (1.0 / cnt).to(dev)
    slices = [logits[:, i * Vl : (i + 1) * Vl].contiguous() for i in range(n)]
    stats = [torch.empty(rows * 4, device=dev) for _ in range(n)]
    for i in range(n):
        K.ce_vp_stats(slices[i], labels, stats[i], V=Vl, vocab_offset=i * Vl, softcap=softcap)
    table = K.pointer_table([t.data_ptr() for t in stats], torch.device(dev))
    total, ztotal = 0.0, 0.0
    grads = []
    for i in range(n):
        sums = torch.zeros(2, device=dev)
        dl = torch.empty(rows, Vl, device=dev, dtype=torch.bfloat16)
        K.ce_vp_grad(slices[i], labels, dl, table, n, inv, sums, V=Vl, vocab_offset=i * Vl, V_total=V, rows_per_src=per,
                     row0=0, my_src=i, softcap=softcap, z_loss=z)
        grads.append(dl.float())
        total += (sums[0] * inv[i]).item() / n          # mean over the two sources of their own mean losses
        ztotal += (sums[1] * inv[i] * z).item() / n
    # reference with the same per-source normalisation: mean of the two halves' mean losses
    halves = [ref.fused_cross_entropy(logits[i * per : (i + 1) * per], labels[i * per : (i + 1) * per],
                                      z_loss_multiplier=z, logit_softcap=softcap) for i in range(n)]
    want = sum(h[0].item() for h in halves) / n
    assert abs(total - want) < 2e-3 * max(1.0, abs(want))
    assert abs(ztotal - sum(h[1].item() for h in halves) / n) < 2e-3 * max(1e-6, abs(ztotal))
    lf2 = logits.clone().requires_grad_(True)
    obj = sum(sum(ref.fused_cross_entropy(lf2[i * per : (i + 1) * per], labels[i * per : (i + 1) * per],
                                          z_loss_multiplier=z, logit_softcap=softcap)) for i in range(n))
    (g2,) = torch.autograd.grad(obj, lf2)
    assert rel_err(torch.cat(grads, dim=1), g2) < 8e-3
    _check_status()


def test_adamw_and_norm_kernels(K):
    dev = "cuda"
    torch.manual_seed(8)
    n = 100003
    p = torch.randn(n, device=dev)
    g = torch.randn(n, device=dev) * 0.1
    m = torch.zeros(n, device=dev)
    v = torch.zeros(n, device=dev)
    shadow = torch.empty(n, device=dev, dtype=torch.bfloat16)
    ss = torch.zeros(1, device=dev, dtype=torch.float64)
    K.sumsq(g, ss)
    assert abs(ss.item() - g.double().pow(2).sum().item()) < 1e-6 * ss.item() + 1e-9
    coef = torch.empty(2, device=dev)
    K.clip_coef(ss, 1.0, 1.0, coef)
    norm = g.norm().item()
    assert abs(coef[1].item() - norm) < 1e-4 * norm and abs(coef[0].item() - 1.0 / max(1.0, norm)) < 1e-5
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.95, 1e-8, 0.1
    for t in range(1, 4):
        ge = g * coef[0]
        mr = b1 * mr + (1 - b1) * ge
        vr = b2 * vr + (1 - b2) * ge * ge
        pr = pr - lr * ((mr / (1 - b1**t)) / ((vr / (1 - b2**t)).sqrt() + eps) + wd * pr)
        gg = g.clone()
        K.adamw(p, m, v, gg, shadow, lr=lr, b1=b1, b2=b2, eps=eps, wd=wd, bias_corr1=1 - b1**t, bias_corr2=1 - b2**t,
                gscale=coef, zero_grad=True)
        assert gg.abs().max().item() == 0.0
    assert rel_err(p, pr) < 1e-5 and rel_err(shadow, pr) < 4e-3
    _check_status()
