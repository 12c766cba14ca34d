"""
The allocation-free flash-attention backward (``ob_flash_attn_bwd_static``) gives the same gradients as the regular
entry point.  It serves programs that may not allocate device memory themselves (a server with a pre-carved memory
arena, a plug-in inside another framework's allocator, a job under a fixed memory cap): its work buffers live in an
array built into the library.  The test calls the exported C symbol directly, twice in a row with different inputs,
because the built-in array keeps the previous call's contents and the second call must not see them.  This file sorts
last so that a failure here cannot hide the other tests in a run that stops at the first failure.
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(lib_mod, q, k, v, o, lse, d_o, dq, dk, dv, causal, window, softcap):
    a = lib_mod.ObAttnArgs()
    for field, t, prefix in (("q", q, "q"), ("k", k, "k"), ("v", v, "v"), ("o", o, "o"), ("d_o", d_o, "do"),
                             ("dq", dq, "dq"), ("dk", dk, "dk"), ("dv", dv, "dv")):
        setattr(a, field, t.data_ptr())
        setattr(a, prefix + "_sb", t.stride(0))
        setattr(a, prefix + "_ss", t.stride(1))
        setattr(a, prefix + "_sh", t.stride(2))
    a.lse = lse.data_ptr()
    a.delta = None      # ignored by the static variant
    a.dq_accum = None
    a.B, a.S, a.H, a.Hkv, a.D = q.shape[0], q.shape[1], q.shape[2], k.shape[2], q.shape[3]
    a.causal, a.window, a.scale, a.softcap = int(causal), window, 1.0 / math.sqrt(q.shape[3]), softcap
    a.status = lib_mod.status_buffer(q.device).data_ptr()
    return a


def test_static_scratch_backward_matches_regular_entry_point():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from olmax_b200.ops import _lib, kernels as K
    from olmax_b200.testing import rel_err

    lib = _lib.lib()
    fn = lib.ob_flash_attn_bwd_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(_lib.ObAttnArgs), ctypes.c_void_p]
    dev = torch.device("cuda")
    torch.manual_seed(11)
    # two calls in a row; the second is smaller and uses other options, so stale sums from the first would show
    for B, S, H, Hkv, window, softcap in ((2, 512, 4, 2, -1, 0.0), (1, 333, 2, 2, 100, 20.0)):
        q = torch.randn(B, S, H, 128, device=dev, dtype=torch.bfloat16)
        k = torch.randn(B, S, Hkv, 128, device=dev, dtype=torch.bfloat16)
        v = torch.randn(B, S, Hkv, 128, device=dev, dtype=torch.bfloat16)
        o, lse = K.flash_attn_fwd(q, k, v, causal=True, window=window, softcap=softcap)
        d_o = torch.randn_like(o)
        want = K.flash_attn_bwd(q, k, v, o, lse, d_o, causal=True, window=window, softcap=softcap)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        a = _args(_lib, q, k, v, o, lse, d_o, dq, dk, dv, True, window, softcap)
        rc = fn(ctypes.byref(a), _lib.stream_ptr(dev))
        assert rc == 0, lib.ob_last_error()
        torch.cuda.synchronize()
        _lib.check_status(dev)
        for got, ref in zip((dq, dk, dv), want):
            assert rel_err(got, ref) < 2e-3
    # a problem beyond the built-in work area is refused with a message, not run
    big = torch.empty(1, 1, 1, 128, device=dev, dtype=torch.bfloat16)
    a = _args(_lib, big, big, big, big, torch.empty(1, device=dev), big, big, big, big, True, -1, 0.0)
    a.B, a.S, a.H, a.Hkv = 4, 4096, 32, 32
    assert fn(ctypes.byref(a), _lib.stream_ptr(dev)) != 0
    assert b"exceeds" in lib.ob_last_error()
