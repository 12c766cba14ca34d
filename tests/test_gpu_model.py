"""GPU end-to-end: model loss / gradients on the CUDA kernels (bf16) against the CPU restatement (fp32 math on the
same bf16-rounded weights), for every layer family; an optimizer step; the driver's smoke entry point."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from olmax_b200.activation_checkpointing import NothingSaveable, SaveAnythingExceptTheseNames
from olmax_b200.models import (
    DefaultTransformerConfig,
    DefaultTransformerLayerConfig,
    GemmaTransformerLayerConfig,
    ReorderedNormTransformerLayerConfig,
)
from olmax_b200.nn import LMHeadConfig, MultiheadSelfAttentionConfig, RMSNormConfig, RotaryPositionalEmbeddingConfig
from olmax_b200.optim import AdamWConfig, ConstantSchedule
from olmax_b200.parallel import MeshResource


def _make(dev, layer_cls, qk=False, headwise=True, kv=None, softcap=None, fsoft=None, tie=False, window=None, ac=None):
    attn = MultiheadSelfAttentionConfig(n_heads=4, n_kv_heads=kv, head_dim=128,
                                        rope=RotaryPositionalEmbeddingConfig(theta=10000.0),
                                        qk_norm=RMSNormConfig() if qk else None, use_head_qk_norm=headwise,
                                        logit_softcap=softcap)
    cfg = DefaultTransformerConfig(vocab_size=2048, d_model=512, hidden_size=1024, num_layers=2,
                                   layer=layer_cls(attention=attn), lm_head=LMHeadConfig(logit_softcap=fsoft),
                                   tie_embeddings=tie, scale_embeddings=tie, sliding_window=window,
                                   sliding_window_pattern=2, layer_ac_policy=ac, ce_chunk_rows=256)
    return cfg.build(seed=1, mesh_resource=MeshResource.FSDP(1), device=torch.device(dev))


CASES = {
    "llama": dict(layer_cls=DefaultTransformerLayerConfig),
    "olmo2_full_qk": dict(layer_cls=ReorderedNormTransformerLayerConfig, qk=True, headwise=False),
    "olmo2_head_qk_gqa": dict(layer_cls=ReorderedNormTransformerLayerConfig, qk=True, headwise=True, kv=2),
    "gemma": dict(layer_cls=GemmaTransformerLayerConfig, kv=2, softcap=50.0, fsoft=30.0, tie=True, window=100),
    "llama_remat": dict(layer_cls=DefaultTransformerLayerConfig, ac=NothingSaveable()),
    "gemma_mlp_remat": dict(layer_cls=GemmaTransformerLayerConfig, kv=2, softcap=50.0,
                            ac=SaveAnythingExceptTheseNames(names=["layers.*.mlp"])),
    "olmo2_attention_remat": dict(layer_cls=ReorderedNormTransformerLayerConfig, qk=True, headwise=True,
                                  ac=SaveAnythingExceptTheseNames(names=["layers.*.attention"])),
}


@pytest.mark.parametrize("name", list(CASES))
def test_model_matches_cpu_restatement(name):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from olmax_b200.ops import _lib

    kw = CASES[name]
    torch.manual_seed(0)
    ids = torch.randint(0, 2048, (2, 256))
    labels = torch.roll(ids, -1, 1)
    labels[:, -1] = -100
    mc, mg = _make("cpu", **kw), _make("cuda", **kw)
    mg.store.master.copy_(mc.store.master.to("cuda"))
    mg.store.sync_shadow()
    mc.store.master.copy_(mg.store.shadow.float().cpu())
    mc.store.sync_shadow()
    out = {}
    for m, dev in ((mc, "cpu"), (mg, "cuda")):
        m.store.set_grad_scale(1.0)
        cache = m.get_buffer_cache(256, torch.device(dev))
        loss, _ = m(ids.to(dev), labels.to(dev), cache)
        loss.backward()
        m.store.finish_backward()
        out[dev] = (loss.item(), m.store.grad.float().cpu().clone())
    _lib.check_status()
    assert abs(out["cpu"][0] - out["cuda"][0]) < 5e-3 * abs(out["cpu"][0])
    gc_, gg = out["cpu"][1], out["cuda"][1]
    assert ((gc_ - gg).norm() / gc_.norm()).item() < 4e-2
    for n, h in mc.store.named_parameters():
        a = gc_[h.meta.offset : h.meta.offset + h.meta.numel_local]
        b = gg[h.meta.offset : h.meta.offset + h.meta.numel_local]
        assert ((a - b).norm() / (a.norm() + 1e-20)).item() < 8e-2, n


def test_optimizer_step_matches_cpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    mc, mg = _make("cpu", DefaultTransformerLayerConfig), _make("cuda", DefaultTransformerLayerConfig)
    mg.store.master.copy_(mc.store.master.to("cuda"))
    mg.store.sync_shadow()
    oc = AdamWConfig(lr=ConstantSchedule(1e-3), weight_decay=0.1, max_grad_norm=1.0, no_decay_modules=["embedding.weight"])
    opt_c, opt_g = oc.build(mc), oc.build(mg)
    g = torch.randn(mc.store.numel_local) * 0.01
    for _ in range(3):
        mc.store.grad.copy_(g)
        mg.store.grad.copy_(g.cuda())
        opt_c.step()
        opt_g.step()
    err = ((mc.store.master - mg.store.master.cpu()).norm() / mc.store.master.norm()).item()
    assert err < 1e-5
    assert abs(opt_c.grad_norm.item() - opt_g.grad_norm.item()) < 1e-3 * opt_c.grad_norm.item()
    assert mg.store.grad.abs().max().item() == 0.0
    assert ((mg.store.shadow.float() - mg.store.master).abs().max() / mg.store.master.abs().max()).item() < 1e-2


def test_smoke_entry_point():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    import __graft_entry__

    __graft_entry__.smoke()
