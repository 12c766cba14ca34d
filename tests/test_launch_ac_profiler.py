"""Launchers (Beaker runtime from its environment, local one-process-per-device launcher), activation-checkpointing
policies (registry names, glob resolution, same loss and gradients with and without recomputation) and the profiler
callback's schedule."""

import sys

import pytest
import torch

from olmax_b200.activation_checkpointing import (ActivationCheckpointingPolicy, NoPolicy, NothingSaveable,
                                                 SaveAnythingExceptTheseNames, SaveOnlyTheseNames)
from olmax_b200.parallel import MeshResource


def test_beaker_runtime_from_env(monkeypatch):
    from olmax_b200.launch.beaker import BeakerRuntime
    from olmax_b200.types import DeviceType

    for k in ("BEAKER_JOB_ID", "BEAKER_WORKLOAD_ID"):
        monkeypatch.delenv(k, raising=False)
    assert BeakerRuntime.from_env() is None
    monkeypatch.setenv("BEAKER_WORKLOAD_ID", "wl-1")
    monkeypatch.setenv("BEAKER_REPLICA_RANK", "1")
    monkeypatch.setenv("BEAKER_REPLICA_COUNT", "2")
    monkeypatch.setenv("BEAKER_LEADER_REPLICA_HOSTNAME", "node-a")
    monkeypatch.setenv("BEAKER_NODE_GPU_TYPE", "NVIDIA B200")
    monkeypatch.setenv("BEAKER_ASSIGNED_GPU_COUNT", "8")
    monkeypatch.setenv("BEAKER_CLUSTER", "ai2/titan")
    rt = BeakerRuntime.from_env()
    assert rt.node.device_type == DeviceType.NVIDIA_B200
    assert rt.local_device_count == 8 and rt.global_device_count == 16
    dc = rt.get_dist_config(local_rank=3)
    assert dc.coordinator_address == "node-a:29400" and dc.num_processes == 16 and dc.process_id == 11 and dc.local_rank == 3
    env = rt.get_env_config()
    assert env.nccl is not None and env.cuda is not None
    monkeypatch.setenv("BEAKER_CLUSTER", "ai2/augusta")
    assert "tcpxo" in (BeakerRuntime.from_env().get_env_config().nccl.tuner_config_path or "")


def test_beaker_submit_needs_gantry():
    from olmax_b200.exceptions import OLMaxEnvironmentError
    from olmax_b200.launch import beaker

    try:
        import gantry  # noqa: F401
    except ImportError:
        with pytest.raises(OLMaxEnvironmentError, match="beaker-gantry"):
            beaker.main(["--nodes", "2", "--", "python", "-c", "pass"])
    with pytest.raises(SystemExit):
        beaker.main(["--nodes", "2"])     # no command


def test_local_launcher_starts_ranks_and_propagates_failure(tmp_path):
    from olmax_b200.launch.local import launch

    out = tmp_path / "ranks"
    out.mkdir()
    script = ("import os, pathlib; r = os.environ['RANK']; "
              f"pathlib.Path(r'{out}').joinpath(r).write_text(os.environ['WORLD_SIZE'] + ' ' + os.environ['LOCAL_RANK'] "
              "+ ' ' + os.environ['MASTER_ADDR'])")
    assert launch(["-c", script], nproc=3) == 0
    assert sorted(p.name for p in out.iterdir()) == ["0", "1", "2"]
    assert (out / "2").read_text() == "3 2 127.0.0.1"
    # one rank fails: the launcher returns its exit code and stops the others
    bad = "import os, sys, time; sys.exit(7) if os.environ['RANK'] == '1' else time.sleep(30)"
    assert launch(["-c", bad], nproc=2) == 7


def test_policy_registry_and_name_resolution():
    names = ["layers.0", "layers.0.attention", "layers.0.mlp", "layers.1", "layers.1.attention", "layers.1.mlp"]
    for type_name in ("default", "everything_saveable", "nothing_saveable", "dots_saveable",
                      "dots_with_no_batch_dims_saveable", "save_anything_except_these_names", "save_any_names_but_these",
                      "save_only_these_names"):
        assert type_name in ActivationCheckpointingPolicy.list_available()
    assert not NoPolicy().should_recompute("layers.0")
    assert NothingSaveable().should_recompute("layers.0")
    p = SaveAnythingExceptTheseNames(names=["layers.*.mlp"])
    p.resolve_names(names)
    assert p.should_recompute("layers.1.mlp") and not p.should_recompute("layers.1.attention")
    q = SaveOnlyTheseNames(names=["layers.0.attention"])     # an exact name works (the reference only accepts globs)
    q.resolve_names(names)
    assert not q.should_recompute("layers.0.attention") and q.should_recompute("layers.0.mlp")
    with pytest.raises(Exception):
        SaveOnlyTheseNames(names=["no.such.*"]).resolve_names(names)


@pytest.mark.parametrize("policy", [NothingSaveable(), SaveAnythingExceptTheseNames(names=["layers.*.mlp"]),
                                    SaveOnlyTheseNames(names=["layers.*.attention"])])
def test_recomputation_does_not_change_loss_or_gradients(policy):
    from olmax_b200.models import DefaultTransformerConfig, GemmaTransformerLayerConfig
    from olmax_b200.nn import MultiheadSelfAttentionConfig

    attn = MultiheadSelfAttentionConfig(n_heads=2, n_kv_heads=1, head_dim=16)

    def run(pol):
        cfg = DefaultTransformerConfig(vocab_size=48, d_model=32, hidden_size=64, num_layers=2,
                                       layer=GemmaTransformerLayerConfig(attention=attn), layer_ac_policy=pol)
        model = cfg.build(seed=2, mesh_resource=MeshResource.FSDP(1), device=torch.device("cpu"))
        calls = {"attention": 0, "mlp": 0}
        # forward executions of the sub-blocks, recomputation included (pre-hooks: a recomputation stops as soon as the
        # last tensor the backward pass needs has been produced, so it may never reach the end of the block)
        for layer in model.layers:
            layer.attention.register_forward_pre_hook(lambda *a: calls.__setitem__("attention", calls["attention"] + 1))
            layer.mlp.register_forward_pre_hook(lambda *a: calls.__setitem__("mlp", calls["mlp"] + 1))
        ids = torch.randint(0, 48, (2, 12), generator=torch.Generator().manual_seed(1))
        loss, _ = model(ids, torch.roll(ids, -1, 1))
        loss.backward()
        model.store.finish_backward()
        if pol is not None and not isinstance(pol, NothingSaveable):
            assert all(layer.mlp.recompute for layer in model.layers)
        else:
            assert not any(layer.mlp.recompute for layer in model.layers)
        return loss.item(), model.store.grad.clone(), calls

    want_loss, want_grad, base_calls = run(None)
    assert base_calls == {"attention": 2, "mlp": 2}
    loss, grad, calls = run(policy)
    assert loss == pytest.approx(want_loss, rel=1e-6)
    assert torch.allclose(grad, want_grad, rtol=1e-5, atol=1e-7)
    # a recomputed layer runs its blocks twice (forward + one recomputation); a recomputed MLP block runs once as a module
    # and repeats only its gate/up GEMM inside its autograd node (it keeps nothing but its input for backward)
    want_calls = {NothingSaveable: {"attention": 4, "mlp": 4}, SaveAnythingExceptTheseNames: {"attention": 2, "mlp": 2},
                  SaveOnlyTheseNames: {"attention": 2, "mlp": 2}}[type(policy)]
    assert calls == want_calls


def test_profiler_callback_schedule(tmp_path):
    """skip_first steps untouched, then `active` steps traced into work_dir/profiler, then the directory is persisted."""
    from olmax_b200.train.callbacks.profiler import ProfilerCallback

    cb = ProfilerCallback(skip_first=2, active=2)
    persisted = []

    class FakeTrainer:
        step = 0
        work_dir = tmp_path

        def persist_working_subdir(self, name):
            persisted.append((self.step, str(name)))

    cb.trainer = FakeTrainer()
    active_steps = []
    for step in range(1, 7):
        cb.trainer.step = step
        cb.pre_step()
        if cb._prof is not None:
            active_steps.append(step)
        torch.ones(8).sum()
        cb.post_step()
    assert active_steps == [3, 4]                 # steps 1-2 skipped, 3-4 traced
    assert persisted == [(4, "profiler")]
    traces = list((tmp_path / "profiler").glob("trace_rank*.json"))
    assert len(traces) == 1 and traces[0].stat().st_size > 0
    cb.close()                                    # idempotent once stopped
    assert len(persisted) == 1
