"""Schedules, weight-decay mask, AdamW semantics (vs torch.optim.AdamW, clipping, accumulation), synthetic data."""

import math
import warnings

import pytest
import torch

from olmax_b200.data import generate_batches_of_sequential_tokens, generate_batches_of_uniform_tokens
from olmax_b200.models import TransformerRecipeType
from olmax_b200.optim import (
    AdamWConfig,
    ConstantSchedule,
    OptimConfig,
    WarmupCosineDecaySchedule,
    WarmupStableDecaySchedule,
    clip_grads_by_global_norm,
)
from olmax_b200.parallel import MeshResource


def test_warmup_stable_decay_schedule():
    s = WarmupStableDecaySchedule(warmup_steps=10, stable_steps=10, decay_steps=10, peak_value=1.0).build()
    r = [s(i) for i in range(32)]
    assert r[0] == 0.0 and r[5] == 0.5 and r[10] == 1.0 and r[20] == 1.0 and r[25] == 0.5 and r[30] == 0.0 and r[31] == 0.0


def test_warmup_cosine_decay_schedule():
    s = WarmupCosineDecaySchedule(warmup_steps=10, decay_steps=100, peak_value=1.0, init_value=0.1, end_value=0.2).build()
    assert s(0) == pytest.approx(0.1) and s(10) == pytest.approx(1.0)
    assert s(60) == pytest.approx(0.2 + 0.8 * 0.5)  # half way through the decay (decay_steps excludes the warm-up)
    assert s(110) == pytest.approx(0.2) and s(500) == pytest.approx(0.2)
    assert ConstantSchedule(3.0).build()(17) == 3.0


def test_weight_decay_mask():
    names = ["embedding.weight", "layers.0.mlp.gate_proj.weight", "layers.0.attention_norm.weight", "norm.weight"]
    mask = OptimConfig.build_weight_decay_mask(names, ["embedding.weight", "*norm.weight"])
    assert mask == {names[0]: False, names[1]: True, names[2]: False, names[3]: False}
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        OptimConfig.build_weight_decay_mask(names, ["does.not.match"])
    assert any("did not match" in str(x.message) for x in w)


def _tiny(seed=0):
    return TransformerRecipeType.tiny_llama.build_recipe().model.build(seed=seed, mesh_resource=MeshResource.FSDP(1))


def test_adamw_matches_torch_adamw():
    model = _tiny()
    st = model.store
    cfg = AdamWConfig(lr=ConstantSchedule(1e-2), b1=0.9, b2=0.95, eps=1e-8, weight_decay=0.1,
                      no_decay_modules=["embedding.weight"])
    opt = cfg.build(model)
    decay, nodecay = st.decay_runs()
    ref_p = st.master.clone().requires_grad_(True)
    groups = [{"params": [ref_p], "weight_decay": 0.0}]
    ref = torch.optim.AdamW(groups, lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    wd_mask = torch.zeros_like(ref_p)
    for s, e in decay:
        wd_mask[s:e] = 1.0
    torch.manual_seed(0)
    for _ in range(4):
        g = torch.randn_like(st.master) * 0.01
        st.grad.copy_(g)
        # torch's decoupled decay multiplies p by (1 - lr * wd) before the Adam update; same as ours to first order
        with torch.no_grad():
            ref_p.mul_(1 - 1e-2 * 0.1 * wd_mask)
        ref_p.grad = g.clone()
        ref.step()
        opt.step()
    assert torch.allclose(st.master, ref_p.detach(), rtol=2e-4, atol=2e-6)
    assert opt.count == 4 and st.grad.abs().max() == 0


def test_clipping_and_microbatch_accumulation():
    m1, m2 = _tiny(3), _tiny(3)
    ids = torch.randint(0, 1024, (4, 64))
    labels = torch.roll(ids, -1, 1)
    cfg = AdamWConfig(lr=ConstantSchedule(1e-3), max_grad_norm=0.5)
    o1, o2 = cfg.build(m1, 1), cfg.build(m2, 2)
    # one micro-batch of 4 sequences == two micro-batches of 2 sequences (mean of means over equal sizes)
    loss, _ = m1(ids, labels)
    loss.backward()
    assert o1.accumulate()
    g1 = m1.store.grad.clone()
    for part in (slice(0, 2), slice(2, 4)):
        l2, _ = m2(ids[part], labels[part])
        l2.backward()
        due = o2.accumulate()
    assert due
    assert torch.allclose(g1, m2.store.grad, rtol=1e-4, atol=1e-7)
    o1.step()
    o2.step()
    assert o1.grad_norm.item() == pytest.approx(g1.double().norm().item(), rel=1e-5)
    # the first Adam update is lr * g / (|g| + eps): entries whose gradient is ~eps amplify rounding differences
    diff = (m1.store.master - m2.store.master).abs()
    assert (diff > 1e-5).float().mean().item() < 0.01 and diff.max().item() <= 2.1e-3
    clipped, norm = clip_grads_by_global_norm({"a": g1.double()}, 0.5)
    assert clipped["a"].norm().item() == pytest.approx(min(0.5, norm.item()), rel=1e-4)


def test_grad_norm_is_only_computed_when_asked_for():
    model = _tiny()
    plain = AdamWConfig(lr=ConstantSchedule(1e-3)).build(model)
    assert not plain.tracks_grad_norm and plain.grad_norm is None          # as in the reference: no clipping, no norm
    assert AdamWConfig(lr=ConstantSchedule(1e-3), max_grad_norm=1.0).build(model).tracks_grad_norm
    tracked = AdamWConfig(lr=ConstantSchedule(1e-3), track_grad_norm=True).build(model)
    model.store.grad.fill_(0.5)
    want = model.store.grad.double().norm().item()
    tracked.step()
    assert tracked.grad_norm.item() == pytest.approx(want, rel=1e-5)


def test_synthetic_data_generators():
    a = next(generate_batches_of_sequential_tokens(0, vocab_size=100, sequence_length=16, global_microbatch_instances=8,
                                                   num_microbatches=2, pin_memory=False))
    assert len(a) == 2 and a[0][0].shape == (8, 16)
    ids, tg = a[0]
    assert torch.equal(tg, ids + 1) and ids.max() < 100
    assert torch.equal((ids[:, 1:] - ids[:, :-1]) % 100, torch.ones(8, 15, dtype=torch.long))
    # sharding: rank r of 4 sees rows [2r, 2r+2) of the same global batch; streams are reproducible and resumable
    full = next(generate_batches_of_uniform_tokens(5, vocab_size=50, sequence_length=8, global_microbatch_instances=8,
                                                   pin_memory=False))[0]
    part = next(generate_batches_of_uniform_tokens(5, vocab_size=50, sequence_length=8, global_microbatch_instances=8,
                                                   dp_rank=2, dp_size=4, pin_memory=False))[0]
    assert torch.equal(part[0], full[0][4:6]) and torch.equal(part[1], full[1][4:6])
    assert torch.equal(full[1][:, :-1], full[0][:, 1:]) and (full[1][:, -1] == -100).all()
    gen = generate_batches_of_uniform_tokens(5, vocab_size=50, sequence_length=8, global_microbatch_instances=2,
                                             pin_memory=False)
    first, second = next(gen), next(gen)
    resumed = next(generate_batches_of_uniform_tokens(5, vocab_size=50, sequence_length=8, global_microbatch_instances=2,
                                                      start_batch=1, pin_memory=False))
    assert torch.equal(second[0][0], resumed[0][0]) and not torch.equal(first[0][0], second[0][0])
