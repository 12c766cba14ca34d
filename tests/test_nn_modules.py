"""
Single-module tests on CPU (the ideas of the reference's ``src/test/nn/*_test.py``): every module built on its own
parameter store gives the values and gradients of the plain PyTorch expression over its full parameters, and the
shape contracts of embedding / RoPE / attention / LM head / layers / model hold.
"""

import math

import pytest
import torch

from olmax_b200.nn import (Embedding, GatedMLP, LayerNorm, Linear, LMHead, MultiheadSelfAttention,
                           MultiheadSelfAttentionConfig, RMSNorm, RMSNormConfig, RotaryPositionalEmbedding,
                           RotaryPositionalEmbeddingConfig)
from olmax_b200.nn import functional as NF
from olmax_b200.nn.module import build_module
from olmax_b200.ops import reference as ref
from olmax_b200.parallel import MeshResource


def _build(factory, seed=0):
    return build_module(factory, seed=seed, mesh_resource=MeshResource.FSDP(1), device=torch.device("cpu"))


def _grads(module):
    module.store.finish_backward()
    return {n: module.store.full_gradient(n) for n, _ in module.store.named_parameters()}


def _params(module, requires_grad=True):
    return {n: module.store.full_parameter(n).clone().requires_grad_(requires_grad) for n, _ in module.store.named_parameters()}


@pytest.mark.parametrize("bias", [False, True])
def test_linear_value_and_grad(bias):
    lin = _build(lambda: Linear(24, 16, bias=bias))
    p = _params(lin)
    assert p["weight"].shape == (16, 24) and p["weight"].abs().max() <= 3 * 0.02 + 1e-6   # truncated normal
    x = torch.randn(5, 24, requires_grad=True)
    y = lin(x)
    y.square().sum().backward()
    want = NF.linear(x.detach(), p["weight"], p.get("bias"))
    assert torch.allclose(y, want, atol=1e-6)
    want.square().sum().backward()
    g = _grads(lin)
    assert torch.allclose(g["weight"], p["weight"].grad, atol=1e-5)
    if bias:
        assert torch.allclose(g["bias"], p["bias"].grad, atol=1e-5)


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
def test_gated_mlp_value_and_grad(act):
    mlp = _build(lambda: GatedMLP(16, 40, activation=act))
    p = _params(mlp)
    x = torch.randn(7, 16, requires_grad=True)
    y = mlp(x)
    y.sum().backward()
    xr = x.detach().clone().requires_grad_(True)
    f = torch.nn.functional.silu if act == "silu" else (lambda t: torch.nn.functional.gelu(t, approximate="tanh"))
    want = (f(xr @ p["gate_proj.weight"].t()) * (xr @ p["up_proj.weight"].t())) @ p["down_proj.weight"].t()
    assert torch.allclose(y, want, atol=1e-6)
    want.sum().backward()
    g = _grads(mlp)
    for n in p:
        assert torch.allclose(g[n], p[n].grad, atol=1e-5), n
    assert torch.allclose(x.grad, xr.grad, atol=1e-5)
    with pytest.raises(ValueError):
        _build(lambda: GatedMLP(16, 40, bias=True))


@pytest.mark.parametrize("kind", ["rms", "layer", "layer_nobias"])
def test_normalizers_value_and_grad(kind):
    make = {"rms": lambda: RMSNorm(32, eps=1e-5), "layer": lambda: LayerNorm(32, eps=1e-5, use_bias=True),
            "layer_nobias": lambda: LayerNorm(32, use_bias=False)}[kind]
    norm = _build(make)
    p = _params(norm)
    assert torch.all(p["weight"] == 1) and ("bias" not in p or torch.all(p["bias"] == 0))
    # move the parameters off their initial values so that the gradients are not trivially structured
    for n in p:
        norm.store.load_full(n, p[n].detach() + 0.1 * torch.randn(32))
    norm.store.sync_shadow()
    p = _params(norm)
    x = torch.randn(3, 5, 32, requires_grad=True)
    y = norm(x)
    (y * torch.arange(32.0)).sum().backward()
    xr = x.detach().clone().requires_grad_(True)
    if kind == "rms":
        want = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * p["weight"]
    else:
        want = torch.nn.functional.layer_norm(xr, (32,), p["weight"], p.get("bias"), 1e-5)
    assert torch.allclose(y, want, atol=1e-5)
    (want * torch.arange(32.0)).sum().backward()
    g = _grads(norm)
    for n in p:
        assert torch.allclose(g[n], p[n].grad, atol=1e-4), n
    assert torch.allclose(x.grad, xr.grad, atol=1e-4)


def test_normalizer_residual_modes_and_heads():
    for make in (lambda: RMSNorm(16), lambda: LayerNorm(16, use_bias=True)):
        norm = _build(make)
        x, r = torch.randn(4, 16), torch.randn(4, 16)
        assert torch.allclose(norm(x, residual=r, mode="post"), r + norm(x), atol=1e-6)
        h, y = norm(x, residual=r, mode="pre")
        assert torch.allclose(h, x + r) and torch.allclose(y, norm(x + r), atol=1e-6)
        wide = torch.randn(4, 3 * 16)   # three heads normalised separately
        per_head = torch.cat([norm(wide[:, i * 16 : (i + 1) * 16]) for i in range(3)], dim=-1)
        assert torch.allclose(norm(wide, heads=3), per_head, atol=1e-6)
    with pytest.raises(ValueError):
        _build(lambda: RMSNorm(16, use_bias=True))


def test_embedding_gather_and_grad():
    emb = _build(lambda: Embedding(50, 8, scale=2.0))
    w = emb.store.full_parameter("weight")
    ids = torch.tensor([[1, 4, 4], [0, 49, 1]])
    anchor = torch.zeros(1, requires_grad=True)
    out = emb(ids.reshape(-1), anchor)
    assert out.shape == (6, 8) and torch.allclose(out, 2.0 * w[ids.reshape(-1)])
    out.sum().backward()
    g = _grads(emb)["weight"]
    counts = torch.bincount(ids.reshape(-1), minlength=50).float()
    assert torch.allclose(g, 2.0 * counts.view(-1, 1).expand(50, 8))


def test_rope_shapes_values_and_cache():
    rope = RotaryPositionalEmbedding(16, theta=10000.0)
    x = torch.randn(2, 12, 3, 16)
    from olmax_b200.nn import BufferCache

    cache = BufferCache()
    y = rope(x, cache)
    assert y.shape == x.shape and len(cache) == 1
    assert torch.allclose(y[:, 0], x[:, 0], atol=1e-6)                       # position 0 is not rotated
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4)         # a rotation preserves the norm
    # rotate-half convention with frequencies theta^(-2i/d)
    inv = 10000.0 ** (-torch.arange(0, 8).float() / 8)
    ang = torch.arange(12).float().view(-1, 1) * inv
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
    rot = torch.cat([-x[..., 8:], x[..., :8]], -1)
    want = x * cos.view(1, 12, 1, 16) + rot * sin.view(1, 12, 1, 16)
    assert torch.allclose(y, want, atol=1e-5)
    assert rope(x, cache) is not None and len(cache) == 1                    # the tables are reused
    # context-parallel tables are the rows of the full tables at the rank's positions
    c0, s0 = rope.get_local_tables(6, 2, 0, x.device, cache)
    full_c, _ = rope.get_tables(12, x.device, cache)
    assert torch.equal(c0, full_c[[0, 1, 2, 9, 10, 11]])


def test_lm_head_logits_loss_and_tying():
    head = _build(lambda: LMHead(16, 40, logit_softcap=30.0))
    w = head.store.full_parameter("proj.weight")
    x = torch.randn(6, 16)
    logits = head(x)
    assert logits.dtype == torch.float32 and logits.shape == (6, 40)
    assert torch.allclose(logits, 30.0 * torch.tanh((x @ w.t()) / 30.0), atol=1e-5)
    labels = torch.tensor([1, 2, -100, 39, 0, 5])
    loss, z = head.loss(x.clone().requires_grad_(True), labels, z_loss_multiplier=1e-2, chunk_rows=4)
    want = torch.nn.functional.cross_entropy(logits, labels, ignore_index=-100)
    lse = torch.logsumexp(logits, -1)[labels != -100]
    assert torch.allclose(z, 1e-2 * lse.pow(2).mean(), rtol=1e-5)
    assert torch.allclose(loss, want + z, rtol=1e-5)
    with pytest.raises(ValueError):
        _build(lambda: LMHead(16, 40, bias=True))


def test_cross_entropy_helpers_agree():
    logits = torch.randn(4, 9, 20)
    labels = torch.randint(0, 20, (4, 9))
    labels[0, :3] = -100
    a = NF.cross_entropy_loss(logits, labels)
    b, z = NF.fused_cross_entropy_loss(logits, labels, z_loss_multiplier=1e-3)
    want = torch.nn.functional.cross_entropy(logits.view(-1, 20), labels.view(-1), ignore_index=-100)
    assert torch.allclose(a, want, atol=1e-6) and torch.allclose(b, want, atol=1e-6) and z > 0
    per_tok = NF.cross_entropy_loss(logits, labels, reduction="none")
    assert per_tok.shape == labels.shape and torch.all(per_tok[0, :3] == 0)
    assert torch.allclose(NF.cross_entropy_loss(logits, labels, reduction="sum"), per_tok.sum(), rtol=1e-6)


def test_scan_module_equals_loop():
    layers = [torch.nn.Linear(8, 8) for _ in range(3)]
    x = torch.randn(2, 8)
    want = x
    for layer in layers:
        want = layer(want)
    assert torch.equal(NF.scan_module(layers, x), want)


@pytest.mark.parametrize("kv,qk_norm,headwise,window,softcap", [
    (None, False, False, None, None),
    (2, True, True, None, None),
    (None, True, False, None, None),
    (2, False, False, 4, 20.0),
])
def test_attention_module_matches_plain_expression(kv, qk_norm, headwise, window, softcap):
    cfg = MultiheadSelfAttentionConfig(n_heads=4, n_kv_heads=kv, head_dim=8, qk_norm=RMSNormConfig() if qk_norm else None,
                                       use_head_qk_norm=headwise, rope=RotaryPositionalEmbeddingConfig(theta=1e4),
                                       window_size=window, logit_softcap=softcap)
    att = _build(lambda: cfg.build(32))
    p = _params(att, requires_grad=False)
    B, S, Hkv = 2, 10, kv or 4
    x = torch.randn(B * S, 32)
    y = att(x, B)
    assert y.shape == (B * S, 32)
    q, k, v = x @ p["q_proj.weight"].t(), x @ p["k_proj.weight"].t(), x @ p["v_proj.weight"].t()
    if qk_norm and not headwise:
        q, k = ref.rms_norm(q, p["q_norm.weight"], 1e-5), ref.rms_norm(k, p["k_norm.weight"], 1e-5)
        assert p["k_norm.weight"].numel() == Hkv * 8          # sized by the KV heads
    q, k, v = q.view(B, S, 4, 8), k.view(B, S, Hkv, 8), v.view(B, S, Hkv, 8)
    if qk_norm and headwise:
        q, k = ref.rms_norm(q, p["q_norm.weight"], 1e-5), ref.rms_norm(k, p["k_norm.weight"], 1e-5)
    cos, sin = ref.rope_tables(S, 8, 1e4)
    q, k = ref.apply_rope(q, cos, sin), ref.apply_rope(k, cos, sin)
    o, _ = ref.attention(q, k, v, True, window if window is not None else -1, softcap or 0.0, 1 / math.sqrt(8))
    want = o.reshape(B * S, 32) @ p["o_proj.weight"].t()
    assert torch.allclose(y, want, atol=1e-5)
    # causality: changing a later token does not change earlier outputs
    x2 = x.clone()
    x2[S - 1] += 1.0
    assert torch.allclose(att(x2, B)[: S - 1], y[: S - 1], atol=1e-6)


def test_layer_variants_and_model_shapes():
    from olmax_b200.models import (DefaultTransformerConfig, DefaultTransformerLayerConfig, GemmaTransformerLayerConfig,
                                   ReorderedNormTransformerLayerConfig)

    attn = MultiheadSelfAttentionConfig(n_heads=2, head_dim=8)
    ids = torch.randint(0, 32, (2, 6))
    for layer_cls, n_norms in ((DefaultTransformerLayerConfig, 2), (ReorderedNormTransformerLayerConfig, 2),
                               (GemmaTransformerLayerConfig, 4)):
        cfg = DefaultTransformerConfig(vocab_size=32, d_model=16, hidden_size=24, num_layers=2, layer=layer_cls(attention=attn))
        model = cfg.build(seed=1, mesh_resource=MeshResource.FSDP(1), device=torch.device("cpu"))
        names = [n for n, _ in model.store.named_parameters()]
        assert sum(n.startswith("layers.0.") and n.endswith("norm.weight") for n in names) == n_norms
        assert {"embedding.weight", "norm.weight", "lm_head.proj.weight"} <= set(names)
        logits = model(ids)
        assert logits.shape == (2, 6, 32) and logits.dtype == torch.float32
        loss, _ = model(ids, torch.roll(ids, -1, 1))
        assert loss.ndim == 0 and abs(loss.item() - math.log(32)) < 0.5      # near-uniform prediction at init
        assert model.num_params() == sum(model.store.full_parameter(n).numel() for n in names)


def test_param_store_layout_validation():
    from olmax_b200.exceptions import OLMaxConfigurationError

    lin = _build(lambda: Linear(24, 16, bias=True))
    store = lin.store
    store.validate_layout()                                   # a finalized store is consistent
    metas = {m.name: m for m in store.metas}
    assert metas["weight"].offset % 64 == 0 and metas["bias"].offset % 64 == 0
    assert metas["bias"].offset >= metas["weight"].offset + metas["weight"].numel_local
    saved = metas["bias"].unit_offset
    metas["bias"].unit_offset = metas["weight"].unit_offset   # two parameters on top of each other
    metas["bias"].offset = metas["weight"].offset
    with pytest.raises(OLMaxConfigurationError, match="overlaps"):
        store.validate_layout()
    metas["bias"].unit_offset, metas["bias"].offset = saved + 8, store.units[0].offset + saved + 8
    with pytest.raises(OLMaxConfigurationError, match="misplaced"):
        store.validate_layout()


def test_gated_mlp_selective_recomputation_keeps_only_its_input():
    """recompute=True: same values and gradients, and the autograd node holds one tensor (x) instead of three."""
    from olmax_b200.ops import functional as F

    mlp = _build(lambda: GatedMLP(16, 40))
    w = (mlp.gate_proj.weight, mlp.up_proj.weight, mlp.down_proj.weight)
    x = torch.randn(7, 16)
    outs = {}
    for recompute in (False, True):
        mlp.store.zero_grad()
        xi = x.clone().requires_grad_(True)
        y = F.gated_mlp(xi, *w, "silu", recompute=recompute)
        saved = len(y.grad_fn.saved_tensors)
        y.square().sum().backward()
        outs[recompute] = (y.detach(), xi.grad.clone(), mlp.store.grad.clone(), saved)
    assert outs[False][3] == 3 and outs[True][3] == 1
    for a, b in zip(outs[False][:3], outs[True][:3]):
        assert torch.allclose(a, b, atol=1e-6)
    with torch.no_grad():      # nothing to recompute without a backward pass
        assert F.gated_mlp(x, *w, "silu", recompute=True).shape == (7, 16)


@pytest.mark.parametrize("kv,qk_norm,window,softcap", [(None, True, None, None), (2, False, 4, 20.0)])
def test_attention_block_recomputation_keeps_input_output_and_statistics(kv, qk_norm, window, softcap):
    """recompute=True: same values and gradients; the block's node holds x, the attention output and the row
    statistics instead of q, k, v and everything the projections, norms and rotation keep."""
    cfg = MultiheadSelfAttentionConfig(n_heads=4, n_kv_heads=kv, head_dim=8, qk_norm=RMSNormConfig() if qk_norm else None,
                                       rope=RotaryPositionalEmbeddingConfig(theta=1e4), window_size=window,
                                       logit_softcap=softcap)
    att = _build(lambda: cfg.build(32))
    B, S = 2, 10
    x = torch.randn(B * S, 32)
    outs = {}
    for recompute in (False, True):
        att.recompute = recompute
        att.store.zero_grad()
        xi = x.clone().requires_grad_(True)
        y = att(xi * 1.0, B)          # the block input is a non-leaf, as inside a layer
        y.square().sum().backward()
        outs[recompute] = (y.detach(), xi.grad.clone(), att.store.grad.clone())
    for a, b in zip(outs[False], outs[True]):
        assert torch.allclose(a, b, atol=1e-5), (a - b).abs().max()
    # the node of the recomputed block saves three tensors: x, o, lse
    att.recompute = True
    y = att((x.clone().requires_grad_(True)) * 1.0, B)
    node = y.grad_fn
    seen, stack, found = set(), [node], None
    while stack:
        n = stack.pop()
        if n is None or n in seen:
            continue
        seen.add(n)
        if "RecomputedAttention" in type(n).__name__:
            found = n
            break
        stack.extend(f for f, _ in n.next_functions)
    assert found is not None and len(found.saved_tensors) == 3
    with torch.no_grad():      # nothing to recompute without a backward pass
        assert att(x, B).shape == (B * S, 32)


def test_cross_entropy_counts_out_of_range_labels_in_mean_and_z_loss():
    """A label outside [0, V) that is not ``ignore_index`` (the sequential synthetic data yields label == V) has no
    cross-entropy term but stays in the mean and in the z-loss, as in the reference's ``fused_cross_entropy_loss``
    (``src/olmax/nn/functional.py:94-121``: the one-hot vanishes, ``log_normalizer * where`` does not)."""
    from olmax_b200.ops import reference as ref

    torch.manual_seed(0)
    logits = torch.randn(6, 10)
    labels = torch.tensor([1, 10, -100, 3, 10, 9])
    loss, z = ref.fused_cross_entropy(logits, labels, z_loss_multiplier=0.1)
    lse = torch.logsumexp(logits, -1)
    has_ce = torch.tensor([1.0, 0, 0, 1, 0, 1])
    counted = torch.tensor([1.0, 1, 0, 1, 1, 1])
    want_loss = ((lse - logits[torch.arange(6), labels.clamp(0, 9)]) * has_ce).sum() / counted.sum()
    want_z = 0.1 * (lse.pow(2) * counted).sum() / counted.sum()
    assert torch.allclose(loss, want_loss) and torch.allclose(z, want_z)
