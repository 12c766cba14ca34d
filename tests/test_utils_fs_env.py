"""Utilities, the file-system layer (local paths), environment configs, tree helpers."""

import logging
import os
from pathlib import Path

import pytest
import torch

from olmax_b200 import fs
from olmax_b200.env import CUDAConfig, EnvConfig, NCCLConfig, XLAConfig
from olmax_b200.exceptions import OLMaxEnvironmentError
from olmax_b200.types import DeviceType, GPUArchitecture
from olmax_b200.utils import RunningAverage, format_float, format_timedelta, set_env_var, wait_for
from olmax_b200.utils.tree import cast_tree, count_params, fold_in, get_global_norm, shaped_rng_split, zeros_like_tree


def test_running_average():
    ra = RunningAverage()
    for x in (1.0, 2.0, 3.0, 4.0):
        ra.update(x)
    assert ra.mean == pytest.approx(2.5)
    assert ra.var == pytest.approx(5.0 / 3.0)
    with pytest.raises(ValueError):
        RunningAverage().mean


def test_format_and_wait():
    from datetime import timedelta

    assert format_float(12345.6) == "12,346" and format_float(0.00001234) == "1.234E-05"
    assert format_timedelta(timedelta(seconds=3725)) == "1h 2m 5s"
    state = {"n": 0}

    def cond():
        state["n"] += 1
        return state["n"] >= 3

    wait_for(cond, "cond", timeout=2, interval=0.01)
    with pytest.raises(TimeoutError):
        wait_for(lambda: False, "never", timeout=0.05, interval=0.01)


def test_set_env_var(monkeypatch):
    monkeypatch.delenv("OB_TEST_VAR", raising=False)
    set_env_var("OB_TEST_VAR", "a")
    set_env_var("OB_TEST_VAR", "b")
    assert os.environ["OB_TEST_VAR"] == "a"
    set_env_var("OB_TEST_VAR", "b", override=True)
    assert os.environ["OB_TEST_VAR"] == "b"


def test_tree_helpers():
    tree = {"a": torch.ones(2, 3), "b": [torch.full((4,), 2.0), torch.arange(3)]}
    n, b = count_params(tree)
    assert n == 13 and b == 6 * 4 + 4 * 4 + 3 * 8
    assert get_global_norm({"a": tree["a"], "b": tree["b"][0]}).item() == pytest.approx((6 + 16) ** 0.5)
    cast = cast_tree(tree, torch.bfloat16)
    assert cast["a"].dtype == torch.bfloat16 and cast["b"][1].dtype == torch.int64
    assert zeros_like_tree(tree)["b"][0].sum() == 0
    assert fold_in(0, 1) != fold_in(0, 2) and fold_in(3, 5) == fold_in(3, 5)
    seeds = shaped_rng_split(7, (2, 3))
    assert len(seeds) == 2 and len(seeds[0]) == 3 and len({s for row in seeds for s in row}) == 6


def test_fs_local(tmp_path):
    src = tmp_path / "a" / "b"
    src.mkdir(parents=True)
    (src / "x.txt").write_text("hello world")
    (src / "y.bin").write_bytes(bytes(range(100)))
    assert fs.get_file_size(src / "x.txt") == 11
    assert fs.get_bytes_range(src / "y.bin", 10, 5) == bytes(range(10, 15))
    assert fs.file_exists(src / "x.txt") and not fs.file_exists(src / "nope")
    assert not fs.dir_is_empty(src) and fs.dir_is_empty(tmp_path / "missing")
    fs.copy_dir(tmp_path / "a", tmp_path / "c")
    assert (tmp_path / "c" / "b" / "x.txt").read_text() == "hello world"
    with pytest.raises(FileExistsError):
        fs.copy_file(src / "x.txt", tmp_path / "c" / "b" / "x.txt")
    fs.copy_file(src / "x.txt", tmp_path / "c" / "b" / "x.txt", save_overwrite=True)
    assert fs.glob_directory(str(tmp_path / "**" / "*.txt")) == sorted(
        [str(src / "x.txt"), str(tmp_path / "c" / "b" / "x.txt")])
    assert fs.glob_directory(str(tmp_path / "a" / "*" / "y.bin")) == [str(src / "y.bin")]
    assert str(fs.join_path("s3://bucket/run", "step1", "f")) == "s3://bucket/run/step1/f"
    assert fs.is_url("gs://b/x") and not fs.is_url("/tmp/x")
    assert fs.normalize_path("file:///tmp/x/") == "/tmp/x"
    fs.remove_file(src / "x.txt")
    assert not (src / "x.txt").exists()
    fs.clear_directory(tmp_path / "c")
    assert not (tmp_path / "c").exists()
    with pytest.raises(ValueError):
        fs.clear_directory("s3://bucket/shallow")
    with fs.get_temp_dir_for_target_dir(tmp_path / "final") as tmp:
        (tmp / "f").write_text("1")
    assert (tmp_path / "final" / "f").read_text() == "1"


def test_fs_retriable_and_missing_sdk():
    calls = {"n": 0}

    @fs.retriable(max_attempts=3, max_backoff=0.01)
    def flaky():
        calls["n"] += 1
        if calls["n"] < 3:
            raise OSError("transient")
        return "ok"

    assert flaky() == "ok" and calls["n"] == 3

    @fs.retriable(max_attempts=2, max_backoff=0.01)
    def always():
        raise OSError("down")

    with pytest.raises(OSError):
        always()
    try:
        import boto3  # noqa: F401
    except ImportError:
        with pytest.raises(OLMaxEnvironmentError):
            fs.get_file_size("s3://bucket/key")


def test_env_configs(monkeypatch):
    for k in ("NCCL_DEBUG", "NCCL_PROTO", "CUDA_DEVICE_MAX_CONNECTIONS"):
        monkeypatch.delenv(k, raising=False)
    env = EnvConfig.recommended(GPUArchitecture.hopper)
    assert env.cuda.device_max_connections == 1
    assert EnvConfig.recommended(GPUArchitecture.blackwell).cuda.device_max_connections is None
    assert DeviceType.NVIDIA_B200.architecture == GPUArchitecture.blackwell
    env.nccl.debug = "INFO"
    env.apply()
    assert os.environ["NCCL_DEBUG"] == "INFO" and os.environ["NCCL_PROTO"] == "Simple,LL,LL128"
    assert os.environ["CUDA_DEVICE_MAX_CONNECTIONS"] == "1"
    x = XLAConfig()
    x.gpu_all_gather_combine_threshold_mib = 1024
    assert x.gpu_all_gather_combine_threshold_bytes == 1024 * 1024 * 1024
    assert "--xla_gpu_enable_triton_gemm=false" in x.get_env_flags()
    assert ("NCCL_LL128_BUFFSIZE", "-2") in NCCLConfig().get_env_vars()


def test_kernel_utils_without_a_gpu():
    import torch

    from olmax_b200.kernel_utils import assert_kernels, host_library_path, kernel_library_path, kernels_available

    assert kernel_library_path().name == "libolmax_b200.so" and host_library_path().name == "libolmax_ckpt.so"
    if torch.cuda.is_available():
        assert kernels_available()
        assert_kernels("anything")
    else:
        assert not kernels_available()
        with pytest.raises(RuntimeError, match="flash attention requires a CUDA device"):
            assert_kernels("flash attention")


def test_tree_compat_helpers():
    import torch

    from olmax_b200.parallel import shard_map
    from olmax_b200.utils.tree import (abs_sq, is_in_jit, maybe_rng_split, uncommit_single_device_arrays, vmap_multiple,
                                       with_optional_sharding_contraint)

    assert maybe_rng_split(None, 3) == [None, None, None]
    a, b = maybe_rng_split(7, 2)
    assert a != b and maybe_rng_split(7, 2) == [a, b]
    f = vmap_multiple(lambda v: v.sum(), 2)
    x = torch.arange(24.0).view(2, 3, 4)
    assert torch.equal(f(x), x.sum(-1))
    z = torch.tensor([3 + 4j])
    assert abs_sq(z).item() == 25 and abs_sq(torch.tensor([-2.0])).item() == 4
    assert is_in_jit() is False
    tree = {"w": torch.ones(2)}
    assert uncommit_single_device_arrays(tree) is tree and with_optional_sharding_contraint(tree, None, None) is tree
    g = lambda t: t + 1  # noqa: E731
    assert shard_map(g, None, in_specs=(), out_specs=()) is g


def test_runtime_config_maps_to_the_environment(monkeypatch):
    from olmax_b200.env import RuntimeConfig

    for k in ("OLMAX_B200_COMM_BACKEND", "OLMAX_B200_BARRIER", "OLMAX_B200_BARRIER_TIMEOUT_S", "OLMAX_B200_NVTX"):
        monkeypatch.delenv(k, raising=False)
    RuntimeConfig(comm_backend="nccl", peer_barrier="flags", peer_wait_timeout_ms=2500, nvtx=False).apply()
    assert os.environ["OLMAX_B200_COMM_BACKEND"] == "nccl" and os.environ["OLMAX_B200_BARRIER"] == "flags"
    assert float(os.environ["OLMAX_B200_BARRIER_TIMEOUT_S"]) == 2.5 and os.environ["OLMAX_B200_NVTX"] == "0"
    for k in ("OLMAX_B200_COMM_BACKEND", "OLMAX_B200_BARRIER", "OLMAX_B200_BARRIER_TIMEOUT_S", "OLMAX_B200_NVTX"):
        monkeypatch.delenv(k, raising=False)
