"""The decode attention entry point that allocates nothing, called through its exported C symbol.

Some hosts of the kernel library cannot allocate device memory (their own pool owns it all, or
an allocation in their loop is not acceptable); for them qv_attn_decode_bf16_static keeps the
workspace of the key slices in an array inside the library.  Here it is checked against the
regular entry point, on two calls in a row with different shapes (the second call finds the
first call's leftovers in the shared array), and its size limit is checked to refuse cleanly.

Why equality with the regular entry point is the claim: both run the same kernels on the same
inputs with the same slice counts, the only difference being where the slices' partial results
lie, so the outputs must agree bit for bit; that the regular entry point computes the right
attention is held against float64 arithmetic in tests/test_kernels_gpu.py.  The call must also
leave the device's memory as it found it: nothing allocated, nothing freed.

This file sorts last on purpose: a run that stops at the first failure has then run every
other test already.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

from qorvix_b200.csrc import ops
from qorvix_b200.csrc.build import load_library

pytestmark = pytest.mark.gpu
DEV = "cuda"
SCRATCH_FLOATS = 2 * 1024 * 1024


def _case(T, H, Hkv, hd, page, ctx_lens, seed):
    g = torch.Generator().manual_seed(seed)
    n_blocks = [-(-c // page) for c in ctx_lens]
    n_pages = sum(n_blocks) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    bt = torch.zeros((T, max(n_blocks)), dtype=torch.int32)
    for i, nb in enumerate(n_blocks):
        bt[i, :nb] = torch.tensor([perm.pop() for _ in range(nb)], dtype=torch.int32)
    cache = torch.randn(n_pages, 2, Hkv, page, hd, generator=g).to(torch.bfloat16).to(DEV)
    q = (torch.randn(T, H * hd, generator=g) * 1.5).to(torch.bfloat16).to(DEV)
    pos = torch.tensor([c - 1 for c in ctx_lens], dtype=torch.int32, device=DEV)
    seg = torch.arange(T, dtype=torch.int32, device=DEV)
    return q, cache, bt.to(DEV), pos, seg


def _static_call(lib, out, q, cache, pos, seg, bt, H, Hkv, hd, page, scale, splits):
    p = lambda t: c_void_p(t.data_ptr())
    lib.qv_attn_decode_bf16_static.restype = c_int
    return lib.qv_attn_decode_bf16_static(
        p(out), c_int(out.stride(0)), p(q), c_int(q.stride(0)), p(cache), p(pos), p(seg), p(bt), c_int(bt.shape[1]),
        c_int(q.shape[0]), c_int(H), c_int(Hkv), c_int(hd), c_int(page), c_int(0), c_float(scale), c_int(splits),
        c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_entry_point_matches_the_regular_one_twice_in_a_row():
    lib = load_library("attention_bf16")
    shapes = [dict(T=5, H=32, Hkv=8, hd=128, page=16, ctx_lens=[700, 1, 64, 333, 1024], splits=6, seed=1),
              dict(T=3, H=6, Hkv=2, hd=48, page=32, ctx_lens=[90, 400, 17], splits=3, seed=2)]
    for s in shapes:
        q, cache, bt, pos, seg = _case(s["T"], s["H"], s["Hkv"], s["hd"], s["page"], s["ctx_lens"], s["seed"])
        scale = 1.0 / math.sqrt(s["hd"])
        want = torch.zeros_like(q)
        assert ops.attention_decode_bf16(want, q, cache, pos, seg, bt, s["H"], s["Hkv"], s["hd"], s["page"], 0, scale, s["splits"])
        got = torch.full_like(q, float("nan"))
        torch.cuda.synchronize()
        held, (free_before, _) = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()
        rc = _static_call(lib, got, q, cache, pos, seg, bt, s["H"], s["Hkv"], s["hd"], s["page"], scale, s["splits"])
        assert rc == 0, rc
        torch.cuda.synchronize()
        if s is not shapes[0]:           # (the library's first launch on a device may load its kernels)
            assert torch.cuda.memory_allocated() == held and torch.cuda.mem_get_info()[0] == free_before
        assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        assert torch.equal(got, want)        # same kernels, same order of sums: in fact identical


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = load_library("attention_bf16")
    T, H, Hkv, hd, page, splits = 64, 32, 8, 128, 16, 16
    assert T * H * splits * (hd + 2) > SCRATCH_FLOATS
    q, cache, bt, pos, seg = _case(T, H, Hkv, hd, page, [40] * T, 3)
    out = torch.zeros_like(q)
    rc = _static_call(lib, out, q, cache, pos, seg, bt, H, Hkv, hd, page, 0.1, splits)
    assert rc == -4
    lib.qv_attn_decode_static_strerror.restype = ctypes.c_char_p
    assert b"built-in workspace" in lib.qv_attn_decode_static_strerror(c_int(rc))
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0       # nothing was launched
