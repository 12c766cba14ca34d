"""
Kernel micro-benchmarks with CUDA-event timing (and the small cases used for ncu captures).

    python -m olmax_b200.ops.microbench gemm            # the GEMM shapes of a 7B layer, all three layouts
    python -m olmax_b200.ops.microbench attn            # flash attention forward / backward, B=2 S=4096 H=32
    python -m olmax_b200.ops.microbench elementwise     # rmsnorm / rope / glu / adamw / cross-entropy bandwidth
    python -m olmax_b200.ops.microbench gemm --small    # one launch per variant on an 8192x4096x4096 case (for ncu)
    python -m olmax_b200.ops.microbench elementwise --small   # one rmsnorm fwd + bwd launch on [8192, 4096] (for ncu)
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m olmax_b200.ops.microbench p2p
                                                        # NVLink: remote loads (pull) vs remote stores (push)

Every figure is the mean over ``--iters`` launches after 3 warm-up launches, timed with CUDA events on the launching
stream with a synchronize on both sides; operands of a timed loop exceed the 126 MB L2 or rotate over several buffers.
Achieved rates are printed next to the fraction of the measured peaks in ``MEASURED_PEAKS.json`` when that file exists.
"""

from __future__ import annotations

import argparse
import json
import math
import sys
from pathlib import Path

import torch

from . import _lib
from . import kernels as K

ROOT = Path(__file__).resolve().parents[2]


def _peaks():
    try:
        return json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "fallback": True}


def _time(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def bench_gemm(iters: int, small: bool):
    dev = torch.device("cuda")
    peak = _peaks()["bf16_tflops"]
    shapes = {
        "fwd_qkvo   NT": (8192, 4096, 4096, False, False, K.EPI_BF16),
        "fwd_down   NT": (8192, 4096, 11008, False, False, K.EPI_BF16),
        "fwd_logits NT f32": (2048, 100352, 4096, False, False, K.EPI_F32),
        "dgrad_up   NN": (8192, 4096, 11008, False, True, K.EPI_BF16),
        "dgrad_qkvo NN": (8192, 4096, 4096, False, True, K.EPI_BF16),
        "wgrad_up   TN f32+=": (11008, 4096, 8192, True, True, K.EPI_F32_ACC),
        "wgrad_qkvo TN f32+=": (4096, 4096, 8192, True, True, K.EPI_F32_ACC),
        "wgrad_down TN f32+=": (4096, 11008, 8192, True, True, K.EPI_F32_ACC),
    }
    if small:
        shapes = {"NT": (8192, 4096, 4096, False, False, K.EPI_BF16), "NN": (8192, 4096, 4096, False, True, K.EPI_BF16),
                  "TN f32+=": (4096, 4096, 8192, True, True, K.EPI_F32_ACC)}
    out = {}
    for name, (M, N, Kd, a_mn, b_mn, epi) in shapes.items():
        a = torch.randn((Kd, M) if a_mn else (M, Kd), device=dev, dtype=torch.bfloat16)
        b = torch.randn((Kd, N) if b_mn else (N, Kd), device=dev, dtype=torch.bfloat16)
        c = torch.zeros(M, N, device=dev, dtype=torch.float32 if epi in (K.EPI_F32, K.EPI_F32_ACC) else torch.bfloat16)
        fn = lambda: K.gemm(a, b, c, M, N, Kd, a_mn=a_mn, b_mn=b_mn, epi=epi)
        if small:
            fn()
            torch.cuda.synchronize()
            continue
        ms = _time(fn, iters)
        tf = 2.0 * M * N * Kd / ms / 1e9
        # the library GEMM on the same operands and layout (comparison only; fp32 outputs compare against a bf16 matmul)
        am, bm = (a.t() if a_mn else a), (b if b_mn else b.t())
        lib_out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        ms_lib = _time(lambda: torch.matmul(am, bm, out=lib_out), iters)
        tf_lib = 2.0 * M * N * Kd / ms_lib / 1e9
        out[name] = {"M": M, "N": N, "K": Kd, "ms": round(ms, 4), "tflops": round(tf, 1), "of_measured_burst": round(tf / peak, 3),
                     "cublas_ms": round(ms_lib, 4), "cublas_tflops": round(tf_lib, 1)}
        print(f"{name:24s} {M:6d}x{N:6d}x{Kd:6d}  {ms:7.3f} ms  {tf:7.1f} TFLOP/s  {tf / peak:5.2f} of measured"
              f"   | torch.matmul {ms_lib:7.3f} ms {tf_lib:7.1f} TFLOP/s", flush=True)
    # gated-MLP epilogue (two B operands)
    if not small:
        M, N, Kd = 8192, 11008, 4096
        a = torch.randn(M, Kd, device=dev, dtype=torch.bfloat16)
        wg = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) * 0.02
        wu = torch.randn(N, Kd, device=dev, dtype=torch.bfloat16) * 0.02
        act, g, u = (torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in range(3))
        ms = _time(lambda: K.gemm(a, wg, act, M, N, Kd, epi=K.EPI_SWIGLU, b2=wu, c2=g, c3=u), iters)
        tf = 4.0 * M * N * Kd / ms / 1e9
        out["fwd_gate_up SwiGLU"] = {"ms": round(ms, 4), "tflops": round(tf, 1), "of_measured_burst": round(tf / peak, 3)}
        print(f"{'fwd_gate_up SwiGLU':24s} {M:6d}x{2 * N:6d}x{Kd:6d}  {ms:7.3f} ms  {tf:7.1f} TFLOP/s  {tf / peak:5.2f} of measured")
    _lib.check_status()
    return out


def bench_attn(iters: int, small: bool):
    dev = torch.device("cuda")
    peak = _peaks()["bf16_tflops"]
    B, S, H = (2, 4096, 16) if small else (2, 4096, 32)
    q = torch.randn(B, S, H, 128, device=dev, dtype=torch.bfloat16)
    k, v = torch.randn_like(q), torch.randn_like(q)
    o, lse = K.flash_attn_fwd(q, k, v)
    d_o = torch.randn_like(o)
    if small:
        K.flash_attn_bwd(q, k, v, o, lse, d_o)
        torch.cuda.synchronize()
        _lib.check_status()
        return {}
    fl = 4.0 * B * H * S * S * 128 / 2
    ms_f = _time(lambda: K.flash_attn_fwd(q, k, v), iters)
    ms_b = _time(lambda: K.flash_attn_bwd(q, k, v, o, lse, d_o), iters)
    out = {"fwd": {"ms": round(ms_f, 4), "tflops": round(fl / ms_f / 1e9, 1), "of_measured_burst": round(fl / ms_f / 1e9 / peak, 3)},
           "bwd": {"ms": round(ms_b, 4), "tflops": round(2.5 * fl / ms_b / 1e9, 1),
                   "of_measured_burst": round(2.5 * fl / ms_b / 1e9 / peak, 3)}}
    print(f"flash fwd  B{B} S{S} H{H} D128 causal: {ms_f:.3f} ms  {out['fwd']['tflops']} TFLOP/s")
    print(f"flash bwd  B{B} S{S} H{H} D128 causal: {ms_b:.3f} ms  {out['bwd']['tflops']} TFLOP/s (2.5x forward FLOPs)")
    _lib.check_status()
    return out


def bench_elementwise(iters: int, small: bool):
    dev = torch.device("cuda")
    bw = _peaks()["hbm_gbs"]
    out = {}

    def report(name, ms, nbytes):
        gbs = nbytes / ms / 1e6
        out[name] = {"ms": round(ms, 4), "GB/s": round(gbs, 1), "of_measured_copy": round(gbs / bw, 3)}
        print(f"{name:28s} {ms:7.3f} ms  {gbs:8.1f} GB/s  {gbs / bw:5.2f} of measured copy bandwidth", flush=True)

    if small:   # one launch of each normalisation kernel on [8192, 4096] (201 MB of traffic in the backward: beyond L2)
        rows, d = 8192, 4096
        x = torch.randn(rows, d, device=dev, dtype=torch.bfloat16)
        w = torch.ones(d, device=dev, dtype=torch.bfloat16)
        y, dx = torch.empty_like(x), torch.empty_like(x)
        rstd = torch.empty(rows, device=dev, dtype=torch.float32)
        dw = torch.zeros(d, device=dev, dtype=torch.float32)
        K.rmsnorm_fwd(x, w, y, rows=rows, d=d, eps=1e-5, rstd=rstd)
        K.rmsnorm_bwd(y, x, w, rstd, dx, rows=rows, d=d, dw=dw)
        torch.cuda.synchronize()
        _lib.check_status()
        return {}
    rows, d = 32768, 4096          # 256 MiB per tensor: larger than L2
    x = torch.randn(rows, d, device=dev, dtype=torch.bfloat16)
    res = torch.randn_like(x)
    w = torch.ones(d, device=dev, dtype=torch.bfloat16)
    y = torch.empty_like(x)
    rstd = torch.empty(rows, device=dev, dtype=torch.float32)
    report("rmsnorm_fwd", _time(lambda: K.rmsnorm_fwd(x, w, y, rows=rows, d=d, eps=1e-5, rstd=rstd), iters), 2 * x.numel() * 2)
    report("rmsnorm_fwd + residual", _time(lambda: K.rmsnorm_fwd(x, w, y, rows=rows, d=d, eps=1e-5, res=res, rstd=rstd), iters),
           3 * x.numel() * 2)
    dw = torch.zeros(d, device=dev, dtype=torch.float32)
    dx = torch.empty_like(x)
    report("rmsnorm_bwd", _time(lambda: K.rmsnorm_bwd(y, x, w, rstd, dx, rows=rows, d=d, dw=dw), iters), 3 * x.numel() * 2)
    q = torch.randn(8, 4096, 32, 128, device=dev, dtype=torch.bfloat16)
    from . import reference as ref

    cos, sin = ref.rope_tables(4096, 128, 500000.0, device=dev)
    qo = torch.empty_like(q)
    report("rope", _time(lambda: K.rope(q, qo, cos, sin), iters), 2 * q.numel() * 2)
    g = torch.randn(16384, 11008, device=dev, dtype=torch.bfloat16)
    u, da = torch.randn_like(g), torch.randn_like(g)
    dg, du, a2 = torch.empty_like(g), torch.empty_like(g), torch.empty_like(g)
    report("glu_bwd (silu)", _time(lambda: K.glu_bwd(g, u, da, dg, du, a2, False), iters), 6 * g.numel() * 2)
    n = 256 * 1024 * 1024
    p_, m_, v_, g_ = (torch.zeros(n, device=dev) for _ in range(4))
    sh = torch.empty(n, device=dev, dtype=torch.bfloat16)
    report("adamw (fp32 + bf16 copy)", _time(lambda: K.adamw(p_, m_, v_, g_, sh, lr=1e-3, b1=0.9, b2=0.95, eps=1e-8, wd=0.1,
                                                           bias_corr1=0.1, bias_corr2=0.05, zero_grad=True), iters), n * 34)
    ss = torch.zeros(1, device=dev, dtype=torch.float64)
    report("sumsq", _time(lambda: K.sumsq(g_, ss), iters), n * 4)
    V, r = 100352, 2048
    logits = torch.randn(r, V, device=dev)
    labels = torch.randint(0, V, (r,), device=dev)
    dl = torch.empty(r, V, device=dev, dtype=torch.bfloat16)
    stats, inv = torch.zeros(2, device=dev), torch.ones(2, device=dev)
    report("cross_entropy fwd+grad", _time(lambda: K.ce_fwd_bwd(logits, labels, dl, stats, inv, V=V), iters), r * V * (4 + 4 + 2))
    _lib.check_status()
    return out


def bench_p2p(iters: int, small: bool):
    """Peer-memory copy rates of our copy kernel between two GPUs (both ranks copy at the same time, so every figure
    is per direction with the opposite direction busy): pull = remote loads + local stores, push = local loads +
    remote stores.  Timed on the device, max over the two ranks."""
    import os

    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem

    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if not dist.is_initialized():
        dist.init_process_group("nccl")
    assert dist.get_world_size() == 2, "run with 2 ranks"
    dev = torch.device("cuda", torch.cuda.current_device())
    nbytes = (32 if small else 256) * 2**20
    buf = symm_mem.empty(nbytes // 2, dtype=torch.bfloat16, device=dev)
    buf.normal_()
    h = symm_mem.rendezvous(buf, dist.group.WORLD)
    peer = int(h.buffer_ptrs[1 - rank])
    local = torch.empty(nbytes // 2, dtype=torch.bfloat16, device=dev)
    out = {}
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    for mode in ("pull", "push"):
        for blocks_per_sm in (1, 2, 4, 8):
            for unroll in (4, 8, 16):
                dst, src = (local.data_ptr(), peer) if mode == "pull" else (peer, local.data_ptr())
                fn = lambda: K.copy_bytes(dst, src, nbytes, dev, blocks=blocks_per_sm * sms, unroll=unroll)
                dist.barrier()
                ms = _time(fn, iters)
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                gbs = nbytes / t.item() / 1e6
                out[f"{mode} blocks/SM={blocks_per_sm} unroll={unroll}"] = {"ms": round(t.item(), 4), "GB/s": round(gbs, 1)}
                if rank == 0:
                    print(f"{mode:5s} {blocks_per_sm} CTAs/SM x 512 thr, {unroll:2d} x 16 B in flight/thread: {t.item():7.3f} ms "
                          f"{gbs:7.1f} GB/s per direction", flush=True)
    dist.barrier()
    _lib.check_status()
    return out if rank == 0 else {}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attn", "elementwise", "p2p"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--small", action="store_true", help="one launch per variant on a small case (for ncu)")
    ap.add_argument("--json", default=None, help="also write the results to this file")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        print("needs a CUDA device")
        return 1
    fn = {"gemm": bench_gemm, "attn": bench_attn, "elementwise": bench_elementwise, "p2p": bench_p2p}[args.what]
    out = fn(args.iters, args.small)
    if args.json and out:
        Path(args.json).write_text(json.dumps(out, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
