"""Allocation-free attention backward (``bcom_attention_bwd_no_alloc``), called through its
exported C symbol the way a host that cannot allocate device memory would call it — a
runtime that gave all GPU memory to one arena at start-up, or code running under another
framework's allocator lock.  Its result must match the ordinary entry point
(``bcom_attention_bwd``, caller-provided scratch) on two calls in a row: the built-in scratch
array keeps the first call's contents, so the second call checks that the entry point clears
what has to start at zero.  Collected last so that a failure here cannot hide other tests.
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from bitscom_b200 import _build

    lib = _build.load_library("bcom_llama")
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.bcom_attention_fwd.argtypes = [vp, vp, vp, ci, ci, ci, ci, cf, vp]
    lib.bcom_attention_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, cf, vp]
    lib.bcom_attention_bwd_no_alloc.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, cf, vp]
    lib.bcom_no_alloc_scratch_bytes.restype = ctypes.c_ulonglong
    return lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def test_no_alloc_backward_matches_regular_entry_point_twice():
    lib = _lib()
    B, S, nh, hd = 2, 256, 4, 128
    H = nh * hd
    scale = 1.0 / math.sqrt(hd)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.bcom_no_alloc_scratch_bytes() == 36 << 20

    for call in range(2):
        g = torch.Generator(device="cuda").manual_seed(100 + call)
        qkv = (torch.randn(B * S, 3 * H, device="cuda", generator=g) * 0.7).to(torch.bfloat16)
        d_out = (torch.randn(B * S, H, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
        out = torch.empty(B * S, H, dtype=torch.bfloat16, device="cuda")
        lse = torch.empty(B, nh, S, dtype=torch.float32, device="cuda")
        assert lib.bcom_attention_fwd(_p(qkv), _p(out), _p(lse), B, S, nh, hd, scale, stream) == 0

        # ordinary entry point: the caller owns the scratch
        want = torch.empty_like(qkv)
        dq_acc = torch.zeros(B * S, H, dtype=torch.float32, device="cuda")
        delta = torch.empty(B, nh, S, dtype=torch.float32, device="cuda")
        assert lib.bcom_attention_bwd(_p(qkv), _p(out), _p(d_out), _p(lse), _p(want), _p(dq_acc),
                                      _p(delta), B, S, nh, hd, scale, stream) == 0

        # allocation-free entry point: inputs and outputs only
        got = torch.empty_like(qkv)
        torch.cuda.synchronize()
        allocated = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]   # sees a cudaMalloc made by ANY library
        rc = lib.bcom_attention_bwd_no_alloc(_p(qkv), _p(out), _p(d_out), _p(lse), _p(got),
                                             B, S, nh, hd, scale, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == allocated
        if call == 1:   # the first call may still load the module; the second must not move
            assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.isfinite(got.float()).all()
        diff = (got.float() - want.float()).abs().max().item()
        tol = 3e-2 * max(1.0, want.float().abs().max().item())
        assert diff < tol, f"call {call}: max diff {diff} (tol {tol})"


def test_no_alloc_rejects_problems_larger_than_the_scratch():
    lib = _lib()
    B, S, nh, hd = 1, 4096, 32, 128   # 64 MiB accumulator: more than the built-in array
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    x = torch.zeros(16, dtype=torch.bfloat16, device="cuda")  # never touched
    rc = lib.bcom_attention_bwd_no_alloc(_p(x), _p(x), _p(x), _p(x), _p(x), B, S, nh, hd,
                                         0.1, stream)
    assert rc == 1006
    torch.cuda.synchronize()


def test_no_alloc_entry_point_can_be_the_first_call_of_the_library_in_a_process():
    """A fresh process whose FIRST use of the library is the allocation-free entry point (so
    the module load and the symbol lookup happen inside it): it must succeed, and a second
    call must agree with the ordinary entry point."""
    import os
    import subprocess
    import sys
    import textwrap

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = textwrap.dedent(f"""
        import ctypes, math, sys, torch
        sys.path.insert(0, {root!r})
        sys.path.insert(0, {os.path.join(root, "tests")!r})
        import test_zz_no_alloc as T
        lib = T._lib()
        B, S, nh, hd = 1, 256, 2, 128
        H, scale = nh * hd, 1.0 / math.sqrt(hd)
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        qkv = (torch.randn(B * S, 3 * H, device="cuda") * 0.7).to(torch.bfloat16)
        d_out = (torch.randn(B * S, H, device="cuda") * 0.5).to(torch.bfloat16)
        out = torch.zeros(B * S, H, dtype=torch.bfloat16, device="cuda")
        lse = torch.zeros(B, nh, S, dtype=torch.float32, device="cuda")
        got = torch.empty_like(qkv)
        # first touch of the library: placeholder statistics, only the return code matters
        rc = lib.bcom_attention_bwd_no_alloc(T._p(qkv), T._p(out), T._p(d_out), T._p(lse),
                                             T._p(got), B, S, nh, hd, scale, st)
        torch.cuda.synchronize()
        assert rc == 0, rc
        assert lib.bcom_attention_fwd(T._p(qkv), T._p(out), T._p(lse), B, S, nh, hd, scale, st) == 0
        want = torch.empty_like(qkv)
        dq = torch.zeros(B * S, H, dtype=torch.float32, device="cuda")
        delta = torch.empty(B, nh, S, dtype=torch.float32, device="cuda")
        assert lib.bcom_attention_bwd(T._p(qkv), T._p(out), T._p(d_out), T._p(lse), T._p(want),
                                      T._p(dq), T._p(delta), B, S, nh, hd, scale, st) == 0
        assert lib.bcom_attention_bwd_no_alloc(T._p(qkv), T._p(out), T._p(d_out), T._p(lse),
                                               T._p(got), B, S, nh, hd, scale, st) == 0
        torch.cuda.synchronize()
        diff = (got.float() - want.float()).abs().max().item()
        assert diff < 3e-2 * max(1.0, want.float().abs().max().item()), diff
        print("ok")
    """)
    run = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True,
                         timeout=300, cwd=root)
    assert run.returncode == 0 and "ok" in run.stdout, run.stdout[-1000:] + run.stderr[-3000:]
