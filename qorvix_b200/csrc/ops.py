"""Python face of the CUDA kernels: each function checks its tensors and launches one kernel
of this folder on torch's current stream.  Nothing here computes on the CPU or calls a
library kernel; a missing or unbuildable library raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import KernelBuildError, load_library

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dt_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


# Every entry point's C signature.  With the types declared once, a call passes plain Python
# numbers (None for a null pointer) and ctypes builds no wrapper object per argument.
_V, _I, _F, _L = c_void_p, c_int, c_float, c_longlong
_ARGTYPES = {
    "qv_error_string": [_I],
    "qv_embed": [_V, _V, _V, _I, _I, _I, _I, _V],
    "qv_add_rmsnorm": [_V, _V, _V, _V, _V, _I, _I, _F, _I, _I, _I, _V],
    "qv_rope_kv_write": [_V, _I, _V, _V, _I, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _V],
    "qv_swiglu": [_V, _V, _I, _I, _I, _I, _V],
    "qv_cast": [_V, _V, _L, _I, _I, _V],
    "qv_cast_rows": [_V, _L, _V, _L, _I, _I, _I, _I, _V],
    "qv_gemm_simt": [_V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _V],
    "qv_gemm_bf16_tc": [_V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _V, _I, _I, _V],
    "qv_packed_weight_bytes": [_I, _I],
    "qv_pack_weight_tiles": [_V, _V, _I, _I, _I, _V],
    "qv_gemm_bf16_packed": [_V, _V, _V, _I, _I, _I, _I, _I, _I, _V, _I, _I, _V],
    "qv_gemm_bf16_qkv_rope": [_V, _V, _V, _I, _I, _I, _I, _V, _V, _I, _V, _V, _V, _I, _V, _I, _I, _I, _I, _V],
    "qv_gemm_bf16_norm": [_V, _V, _V, _I, _I, _I, _I, _I, _I, _V, _I, _V, _I, _V, _V, _V, _I, _F, _F, _V],
    "qv_gemm_bf16_set_prefill_bn": [_I],
    "qv_gemm_bf16_set_split_workspace": [_V, _V, _I],
    "qv_gemm_bf16_split_slot_bytes": [],
    "qv_attention_generic": [_V, _I, _V, _I, _V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _F, _I, _V],
    "qv_attn_prefill_bf16": [_V, _I, _V, _I, _V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _V],
    "qv_attn_prefill_tc": [_V, _I, _V, _I, _I, _V, _L, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _V, _V],
    "qv_attn_set_decode_variant": [_I],
    "qv_attn_set_error_word": [_V],
    "qv_attn_decode_bf16": [_V, _I, _V, _I, _V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _F, _I, _V, _V],
    "qv_argmax": [_V, _V, _I, _I, _L, _V],
    "qv_sample": [_V, _V, _I, _I, _L, _V, _V, _V, _V, _V, _V, _I, _V, _V, _V, _V],
}
_RESTYPES = {"qv_error_string": ctypes.c_char_p, "qv_packed_weight_bytes": c_longlong, "qv_gemm_bf16_split_slot_bytes": c_longlong}
_typed_libs = {}


def _lib(name: str):
    """The library `name` (compiled and loaded on first use) with its entry points' types declared."""
    lib = _typed_libs.get(name)
    if lib is None:
        lib = load_library(name)
        for fn, types in _ARGTYPES.items():
            if hasattr(lib, fn):
                f = getattr(lib, fn)
                f.argtypes = types
                f.restype = _RESTYPES.get(fn, c_int)
        _typed_libs[name] = lib
    return lib


def _ptr(t):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_get_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current stream's handle (the raw getters cost a fraction of building a Stream object)."""
    if _raw_stream is not None and _get_device is not None:
        return _raw_stream(_get_device())
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel operands must live on a CUDA device; there is no CPU path")


_launches = 0


def launch_count() -> int:
    """Kernels of this package launched so far (replays of captured steps add their kernels)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(rc: int, what: str):
    global _launches
    _launches += 1
    if rc != 0:
        lib = _lib("elementwise")
        msg = lib.qv_error_string(rc).decode()
        raise KernelError(f"{what}: {msg} (code {rc})")


def _i32(t, name):
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")


# ------------------------------------------------------------------ elementwise

def embed(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> None:
    """out[t] (float32) = table[ids[t]]."""
    _need_cuda(out, table, ids)
    _i32(ids, "ids")
    T, d = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous()
    assert table.shape[1] == d and ids.numel() >= T
    rc = _lib("elementwise").qv_embed(
        _ptr(out), _ptr(table), _ptr(ids), T, d, table.shape[0], dt_code(table.dtype), _stream())
    _check(rc, "embed")


def add_rmsnorm(out, residual, delta, weight, eps: float, row_idx=None, write_residual=True) -> None:
    """x = residual[s] (+ delta[s]); residual[s] = x if write_residual; out[r] = rmsnorm(x) * weight
    with s = row_idx[r] if row_idx is given, else r.  residual and weight are float32."""
    _need_cuda(out, residual, delta, weight, row_idx)
    rows, d = out.shape
    assert residual.dtype == torch.float32 and weight.dtype == torch.float32
    assert residual.is_contiguous() and out.is_contiguous() and weight.numel() == d and residual.shape[1] == d
    if delta is not None:
        assert delta.is_contiguous() and delta.shape == residual.shape
    if row_idx is not None:
        _i32(row_idx, "row_idx")
        assert row_idx.numel() >= rows
        write_residual = False
    else:
        assert residual.shape[0] >= rows
    ddt = dt_code(delta.dtype) if delta is not None else dt_code(out.dtype)
    rc = _lib("elementwise").qv_add_rmsnorm(
        _ptr(out), _ptr(residual), _ptr(delta), _ptr(weight), _ptr(row_idx), rows, d, eps, 1 if (write_residual and
        delta is not None) else 0, ddt, dt_code(out.dtype), _stream())
    _check(rc, "add_rmsnorm")


def rope_kv_write(qkv, cache_layer, cos_sin, tok_pos, tok_seg, block_table, H, Hkv, hd, rot, page) -> None:
    """Rotates q (in place) and k, writes k and v of every token into its cache slot.
    qkv [T, (H+2Hkv)*hd]; cache_layer [pages, 2, Hkv, page, hd] or None; cos_sin [rows, rot/2, 2] float32."""
    _need_cuda(qkv, cache_layer, cos_sin, tok_pos, tok_seg, block_table)
    T = qkv.shape[0]
    assert qkv.stride(1) == 1 and qkv.shape[1] == (H + 2 * Hkv) * hd
    if cos_sin is None:
        assert rot == 0, "a rotation needs its cos/sin table"
    else:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1] * 2 == rot
    _i32(tok_pos, "tok_pos"); _i32(tok_seg, "tok_seg"); _i32(block_table, "block_table")
    if cache_layer is not None:
        assert cache_layer.dtype == qkv.dtype and cache_layer.is_contiguous()
        assert tuple(cache_layer.shape[1:]) == (2, Hkv, page, hd)
    rc = _lib("elementwise").qv_rope_kv_write(
        _ptr(qkv), qkv.stride(0), _ptr(cache_layer), _ptr(cos_sin), cos_sin.shape[0] if cos_sin is not None else 1,
        _ptr(tok_pos), _ptr(tok_seg), _ptr(block_table), block_table.shape[-1], T, H, Hkv, hd, rot, page,
        dt_code(qkv.dtype), _stream())
    _check(rc, "rope_kv_write")


def swiglu(out, gu, interleaved: bool = False) -> None:
    """gu [T, 2f] -> out [T, f] = silu(gate) * up.  gu is [gate | up], or with `interleaved` groups of
    32 columns: 16 gate values, then the 16 up values of the same features."""
    _need_cuda(out, gu)
    T, f = out.shape
    assert gu.shape == (T, 2 * f) and gu.is_contiguous() and out.is_contiguous() and gu.dtype == out.dtype
    rc = _lib("elementwise").qv_swiglu(
        _ptr(out), _ptr(gu), T, f, 1 if interleaved else 0, dt_code(out.dtype), _stream())
    _check(rc, "swiglu")


def cast(out, src) -> None:
    _need_cuda(out, src)
    assert out.numel() == src.numel() and out.is_contiguous() and src.is_contiguous()
    rc = _lib("elementwise").qv_cast(
        _ptr(out), _ptr(src), src.numel(), dt_code(src.dtype), dt_code(out.dtype), _stream())
    _check(rc, "cast")


def cast_rows(out, src) -> None:
    """out[r, c] = src[r, c] for 2-D tensors whose rows are contiguous (any row stride), float32 or
    bfloat16 each: a dense copy of a slice, with a change of type if the two differ."""
    _need_cuda(out, src)
    assert out.dim() == 2 and out.shape == src.shape and out.stride(1) == 1 and src.stride(1) == 1
    rc = _lib("elementwise").qv_cast_rows(_ptr(out), out.stride(0), _ptr(src), src.stride(0), src.shape[0], src.shape[1],
                                          dt_code(src.dtype), dt_code(out.dtype), _stream())
    _check(rc, "cast_rows")


# ------------------------------------------------------------------ matrix products

def gemm_simt(c, a, w, accumulate=False) -> None:
    """c[M,N] (+)= a[M,K] @ w[N,K]^T with float32 multiply-adds on the CUDA cores."""
    _need_cuda(c, a, w)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    rc = _lib("gemm_simt").qv_gemm_simt(
        _ptr(c), _ptr(a), _ptr(w), M, N, K, a.stride(0), w.stride(0), c.stride(0), dt_code(a.dtype),
        dt_code(w.dtype), dt_code(c.dtype), 1 if accumulate else 0, _stream())
    _check(rc, "gemm_simt")


_tc_state = {}


def _tc_buffers(device):
    """Per device: the error word of the tensor-core kernels."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _tc_state.get(key)
    if st is None:
        st = dict(err=torch.zeros(1, dtype=torch.int32, device=device))
        _tc_state[key] = st
    return st


_split_registered = [None]      # the workspace the library knows (its address), 0 after it was told to share no tiles
_split_enabled = [os.environ.get("QORVIX_SHARE_TILES", "1") != "0"]


def _gemm_buffers(device):
    """`_tc_buffers` plus, for the products: the workspace through which CTAs of the many-token
    kernel hand the partial sums of a tile they share to its owner (one slot and one flag per SM),
    registered with the library once; products run on one stream at a time."""
    st = _tc_buffers(device)
    if not _split_enabled[0]:
        return st
    if "split_slots" not in st:
        ctas = sm_count()
        st["split_slots"] = torch.empty(ctas * int(_lib("gemm_bf16").qv_gemm_bf16_split_slot_bytes()) // 4, dtype=torch.float32, device=device)
        st["split_flags"] = torch.zeros(ctas, dtype=torch.int32, device=device)
    key = st["split_slots"].data_ptr()
    if _split_registered[0] != key:
        _lib("gemm_bf16").qv_gemm_bf16_set_split_workspace(_ptr(st["split_slots"]), _ptr(st["split_flags"]), st["split_flags"].numel())
        _split_registered[0] = key
    return st


def prepare_products(device) -> None:
    """Allocates and registers what the bfloat16 products need beside their operands (error word, workspace
    of shared tiles), so that no first call inside a stream capture has to."""
    _gemm_buffers(torch.device(device))


def gemm_share_tiles(enabled: bool) -> None:
    """Switches the sharing of tiles between CTAs of the many-token kernel off, or on again (for comparison)."""
    _split_enabled[0] = bool(enabled)
    if not enabled and _split_registered[0]:
        _lib("gemm_bf16").qv_gemm_bf16_set_split_workspace(None, None, 0)
        _split_registered[0] = 0


def gemm_bf16_tc(c, a, w, force_splits: int = 0, swiglu: bool = False) -> bool:
    """c[M,N] (bf16 or f32) = a[M,K] @ w[N,K]^T on the tcgen05 tensor cores.  With `swiglu`, w holds
    gate and up rows interleaved in groups of 16 and c[M,N/2] = silu(gate) * up.  False when the
    shape is one the kernel refuses (K not a multiple of 8, unaligned rows); nothing is written then."""
    _need_cuda(c, a, w)
    M, K = a.shape
    N = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    assert c.shape == ((M, N // 2) if swiglu else (M, N))
    assert a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    st = _gemm_buffers(a.device)
    rc = _lib("gemm_bf16").qv_gemm_bf16_tc(
        _ptr(c), _ptr(a), _ptr(w), M, N, K, a.stride(0), w.stride(0), c.stride(0), dt_code(c.dtype),
        _ptr(st["err"]), force_splits, 1 if swiglu else 0, _stream())
    if rc == -2:
        return False
    _check(rc, "gemm_bf16_tc")
    return True


def pack_weight(w: torch.Tensor) -> torch.Tensor:
    """The bfloat16 matrix w [N, K] as the 16 KB tiles (128 rows x 64 k, in the shared-memory layout of
    the MMA) that gemm_bf16_packed streams with contiguous copies.  K must be a multiple of 8."""
    _need_cuda(w)
    assert w.dtype == torch.bfloat16 and w.dim() == 2 and w.stride(1) == 1
    N, K = w.shape
    lib = _lib("gemm_bf16")
    out = torch.empty(lib.qv_packed_weight_bytes(N, K) // 2, device=w.device, dtype=torch.bfloat16)
    _check(lib.qv_pack_weight_tiles(_ptr(out), _ptr(w), N, K, w.stride(0), _stream()), "pack_weight_tiles")
    return out


def gemm_bf16_packed(c, a, packed, N: int, force_splits: int = 0, swiglu: bool = False) -> bool:
    """As gemm_bf16_tc, with the weights given by pack_weight (for any number of rows of a)."""
    _need_cuda(c, a, packed)
    M, K = a.shape
    assert a.dtype == torch.bfloat16 and packed.dtype == torch.bfloat16
    assert c.shape == ((M, N // 2) if swiglu else (M, N)) and a.stride(1) == 1 and c.stride(1) == 1
    st = _gemm_buffers(a.device)
    rc = _lib("gemm_bf16").qv_gemm_bf16_packed(
        _ptr(c), _ptr(a), _ptr(packed), M, N, K, a.stride(0), c.stride(0), dt_code(c.dtype), _ptr(st["err"]),
        force_splits, 1 if swiglu else 0, _stream())
    if rc == -2:
        return False
    _check(rc, "gemm_bf16_packed")
    return True


def gemm_bf16_norm(c, a, packed, N: int, swiglu: bool = False, residual=None, norm_weight=None, ssq_out=None,
                   ssq_in=None, stream_width: int = 0, eps: float = 0.0) -> bool:
    """A product of up to 64 tokens with the neighbouring RMS norm folded in.
    residual (float32 [M, N]) given: residual += a w^T; c (bfloat16) = residual * norm_weight; ssq_out
    (float32 [ceil(N/128), 64]) = sums of squares of the updated rows per tile of 128 features.
    ssq_in (such sums of a stream of `stream_width` features) given: row t of a w^T is scaled by
    rsqrt(sum(ssq_in[:, t]) / stream_width + eps) before it is stored (or goes through SwiGLU).
    False, with nothing written, when the kernel does not take the product."""
    _need_cuda(c, a, packed, residual, norm_weight, ssq_out, ssq_in)
    M, K = a.shape
    if M > 64 or a.dtype != torch.bfloat16 or packed is None:
        return False
    assert c.shape == ((M, N // 2) if swiglu else (M, N)) and a.stride(1) == 1 and c.stride(1) == 1
    tiles_in = 0
    if residual is not None:
        assert residual.dtype == torch.float32 and residual.stride(1) == 1 and tuple(residual.shape) == (M, N)
        assert norm_weight.dtype == torch.float32 and norm_weight.numel() == N
        assert ssq_out.dtype == torch.float32 and ssq_out.is_contiguous() and tuple(ssq_out.shape) == (-(-N // 128), 64)
    if ssq_in is not None:
        assert ssq_in.dtype == torch.float32 and ssq_in.is_contiguous() and ssq_in.shape[1] == 64 and stream_width > 0
        tiles_in = ssq_in.shape[0]
    st = _gemm_buffers(a.device)
    rc = _lib("gemm_bf16").qv_gemm_bf16_norm(
        _ptr(c), _ptr(a), _ptr(packed), M, N, K, a.stride(0), c.stride(0), dt_code(c.dtype), _ptr(st["err"]),
        1 if swiglu else 0, _ptr(residual), residual.stride(0) if residual is not None else 0, _ptr(norm_weight),
        _ptr(ssq_out), _ptr(ssq_in), tiles_in, 1.0 / stream_width if stream_width else 0.0, eps, _stream())
    if rc == -2:
        return False
    _check(rc, "gemm_bf16_norm")
    return True


def new_norm_stats(features: int, device) -> torch.Tensor:
    """The buffer gemm_bf16_norm leaves a stream's sums of squares in (per tile of 128 features of the
    few-token kernel, for its 64 token columns); what it holds is between the producing and the
    consuming launch of that kernel."""
    return torch.empty((-(-features // 128), 64), device=device, dtype=torch.float32)


def _rules():
    """The kernel-choice rules live in C++ (csrc/host/dispatch.hpp), one statement for this module and
    for the native executor; they are reached through the host runtime library."""
    from ..cache import native
    return native.lib()


def folded_norm_enabled(tokens: int) -> bool:
    """Whether the RMS norms of a step of `tokens` tokens ride in the epilogues of the products around
    them: up to 16 tokens, unless QORVIX_FOLDED_NORM=0 (never) or =64 (up to 64 tokens; for comparison)."""
    return bool(_rules().qvh_folded_norm_enabled(int(tokens)))


def fused_rope_enabled(tokens: int) -> bool:
    """Whether the QKV projection of a step of `tokens` tokens takes the rotation and the cache write
    into its epilogue: above 64 tokens, unless QORVIX_FUSED_ROPE=0 (for comparison)."""
    return bool(_rules().qvh_fused_rope_enabled(int(tokens)))


def gemm_qkv_rope(qkv, x, packed, cache_layer, cos_sin, tok_pos, tok_seg, block_table, H, Hkv, hd, page) -> bool:
    """The QKV projection of more than 64 tokens with the rotation of q and k and the cache write of k
    and v in the product's epilogue: qkv[:, :H*hd] gets the rotated queries, the key and value columns
    of qkv are not written.  False (nothing written) when the sizes are not ones it takes: head sizes
    other than 64 and 128, a partial rotation, no packed weights, 64 tokens or fewer."""
    if x.dtype != torch.bfloat16 or qkv.dtype != torch.bfloat16 or packed is None or cos_sin is None:
        return False
    M, K = x.shape
    if cos_sin.shape[1] * 2 != hd or cache_layer.dtype != torch.bfloat16:
        return False
    _need_cuda(qkv, x, packed, cache_layer, cos_sin, tok_pos, tok_seg, block_table)
    assert x.stride(1) == 1 and qkv.stride(1) == 1 and qkv.shape == (M, (H + 2 * Hkv) * hd)
    assert cache_layer.is_contiguous() and tuple(cache_layer.shape[1:]) == (2, Hkv, page, hd)
    assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
    _i32(tok_pos, "tok_pos"); _i32(tok_seg, "tok_seg"); _i32(block_table, "block_table")
    st = _gemm_buffers(x.device)
    rc = _lib("gemm_bf16").qv_gemm_bf16_qkv_rope(
        _ptr(qkv), _ptr(x), _ptr(packed), M, K, x.stride(0), qkv.stride(0), _ptr(st["err"]), _ptr(cos_sin),
        cos_sin.shape[0], _ptr(tok_pos), _ptr(tok_seg), _ptr(block_table), block_table.shape[-1], _ptr(cache_layer),
        H, Hkv, hd, page, _stream())
    if rc == -2:
        return False
    _check(rc, "gemm_qkv_rope")
    return True


def gemm_bf16_set_prefill_tile_width(bn: int) -> None:
    """Columns of the persistent kernel's tiles: 0 (default) lets each product choose, else a multiple
    of 16 (32 with the fused activation) up to 256.  For comparison and tests."""
    _lib("gemm_bf16").qv_gemm_bf16_set_prefill_bn(bn)


def check_kernel_errors() -> None:
    """Raises if a kernel gave up on a bounded wait since the last check (synchronises)."""
    for key, st in _tc_state.items():
        code = int(st["err"].item())
        if code:
            st["err"].zero_()
            raise KernelError(f"a tensor-core kernel on device {key} gave up waiting on a barrier (code {code})")


# ------------------------------------------------------------------ attention

def attention_generic(out, q, cache_layer, tok_pos, tok_seg, block_table, H, Hkv, hd, page, window, scale) -> None:
    """out[t, h*hd:(h+1)*hd] = causal GQA attention of query (t, h) over its request's pages.
    q may be a column slice of the qkv buffer (row stride given by its stride)."""
    _need_cuda(out, q, cache_layer, tok_pos, tok_seg, block_table)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == cache_layer.dtype
    assert cache_layer.is_contiguous() and tuple(cache_layer.shape[1:]) == (2, Hkv, page, hd)
    _i32(tok_pos, "tok_pos"); _i32(tok_seg, "tok_seg"); _i32(block_table, "block_table")
    rc = _lib("attention_generic").qv_attention_generic(
        _ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(cache_layer), _ptr(tok_pos), _ptr(tok_seg),
        _ptr(block_table), block_table.shape[-1], T, H, Hkv, hd, page, window, scale, dt_code(q.dtype), _stream())
    _check(rc, "attention_generic")


# ------------------------------------------------------------------ dispatch

def packed_weights_enabled() -> bool:
    """Whether bfloat16 weight matrices are stored as packed tiles (QORVIX_PACKED_WEIGHTS=0: as rows)."""
    import os
    return os.environ.get("QORVIX_PACKED_WEIGHTS", "1") != "0"


def gemm(out, x, w, packed=None, n: int = 0) -> None:
    """out = x @ w^T with the kernel that fits the dtypes and the shape.  w is the matrix as rows
    [n, K] (or None when only its packed tiles are kept, `packed` with `n` rows): bfloat16 operands
    go to the tensor-core kernels (over the packed tiles when there are any), everything else to the
    CUDA-core kernel."""
    if x.dtype == torch.bfloat16 and packed is not None and gemm_bf16_packed(out, x, packed, n or w.shape[0]):
        return
    if w is None:
        # Only the packed tiles are kept and the kernel that reads them refused x as it is (float32
        # values, rows that do not start on 16 bytes, a row stride that is no multiple of 8): an
        # aligned bfloat16 copy of x, which that kernel takes.
        xb = torch.empty(x.shape, device=x.device, dtype=torch.bfloat16)
        cast_rows(xb, x)
        if packed is not None and gemm_bf16_packed(out, xb, packed, n):
            return
        raise KernelError("the product's shape is one the tensor-core kernel refuses and the weight rows were not kept")
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and gemm_bf16_tc(out, x, w):
        return
    gemm_simt(out, x, w)


def gemm_swiglu(out, x, w_interleaved, packed=None, n: int = 0) -> None:
    """out[M,f] = silu(x Wg^T) * (x Wu^T) with gate and up rows interleaved in groups of 16 in
    w_interleaved [2f, K]: one tensor-core kernel when it takes the shape, else the product followed
    by the activation kernel."""
    n = n or w_interleaved.shape[0]
    if x.dtype == torch.bfloat16 and out.dtype == torch.bfloat16:
        if packed is not None and gemm_bf16_packed(out, x, packed, n, swiglu=True):
            return
        if (w_interleaved is not None and w_interleaved.dtype == torch.bfloat16
                and gemm_bf16_tc(out, x, w_interleaved, swiglu=True)):
            return
    gu = torch.empty((x.shape[0], n), device=x.device, dtype=out.dtype)
    gemm(gu, x, w_interleaved, packed, n)
    swiglu(out, gu, interleaved=True)


def attention_prefill_bf16(out, q, cache_layer, seg_q_start, seg_pos0, block_table, S, max_q_len, H, Hkv, hd, page,
                           window, scale, variant: int = 0) -> bool:
    """Flash attention of prompt portions (any mix of segments) over the paged bfloat16 cache.
    False when the kernel refuses the sizes."""
    _need_cuda(out, q, cache_layer, seg_q_start, seg_pos0, block_table)
    assert q.dtype == out.dtype == cache_layer.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and cache_layer.is_contiguous()
    assert tuple(cache_layer.shape[1:]) == (2, Hkv, page, hd)
    _i32(seg_q_start, "seg_q_start"); _i32(seg_pos0, "seg_pos0"); _i32(block_table, "block_table")
    rc = _lib("attention_bf16").qv_attn_prefill_bf16(
        _ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(cache_layer), _ptr(seg_q_start), _ptr(seg_pos0),
        _ptr(block_table), block_table.shape[-1], S, max_q_len, H, Hkv, hd, page, window, scale, variant, _stream())
    if rc == -2:
        return False
    _check(rc, "attention_prefill_bf16")
    return True


def attention_prefill_tc(out, q, cache_layer, seg_q_start, seg_pos0, block_table, S, max_q_len, H, Hkv, hd, page,
                         window, scale, max_ctx_len: int = 0) -> bool:
    """Flash attention of prompt portions with tcgen05 tensor-core products (head sizes 64 and 128).
    max_ctx_len: the longest context (cached + new tokens) among the portions, where the host knows it; it
    only steers how the kernel cuts its work.  False when the kernel refuses the sizes."""
    _need_cuda(out, q, cache_layer, seg_q_start, seg_pos0, block_table)
    assert q.dtype == out.dtype == cache_layer.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and cache_layer.is_contiguous()
    assert tuple(cache_layer.shape[1:]) == (2, Hkv, page, hd)
    _i32(seg_q_start, "seg_q_start"); _i32(seg_pos0, "seg_pos0"); _i32(block_table, "block_table")
    st = _tc_buffers(q.device)
    rc = _lib("attention_tc").qv_attn_prefill_tc(
        _ptr(out), out.stride(0), _ptr(q), q.stride(0), q.shape[0], _ptr(cache_layer), cache_layer.shape[0],
        _ptr(seg_q_start), _ptr(seg_pos0), _ptr(block_table), block_table.shape[-1], S, max_q_len, int(max_ctx_len), H, Hkv,
        hd, page, window, scale, _ptr(st["err"]), _stream())
    if rc == -2:
        return False
    _check(rc, "attention_prefill_tc")
    return True


_decode_variant_forced = None
_sm_count = None


def sm_count() -> int:
    """Streaming multiprocessors of the current device (asked once); without a device, as on a
    machine that only plans steps, the B200's 148."""
    global _sm_count
    if _sm_count is None:
        _sm_count = 148
        if torch.cuda.is_available():
            _sm_count = int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
    return _sm_count


def decode_variant(T: int, Hkv: int) -> int:
    """Which decode kernel a step of T tokens takes: 0 reads keys and values through a ring in shared
    memory that bulk copies fill (the faster one when many (token, kv head) pairs stream long key
    ranges), 1 through per-thread loads (less set-up; better when there are few pairs)."""
    if _decode_variant_forced is not None:
        return _decode_variant_forced
    return _rules().qvh_decode_variant(int(T), int(Hkv))


def decode_splits(T: int, Hkv: int, max_ctx: int, known: bool = True) -> int:
    """How many slices of the keys each (token, kv head) is cut into: the count whose waves of CTAs
    take the least time when max_ctx is the step's real longest context (`known`), else the count that
    fills one wave.  A function of the step's shape only (a captured step keeps it)."""
    return _rules().qvh_decode_splits(int(T), int(Hkv), int(max_ctx), 1 if known else 0, decode_variant(T, Hkv), sm_count())


def attention_decode_bf16(out, q, cache_layer, tok_pos, tok_seg, block_table, H, Hkv, hd, page, window, scale,
                          splits: int = 1) -> bool:
    """Attention of single query tokens (split over `splits` slices of the keys).  False when refused."""
    _need_cuda(out, q, cache_layer, tok_pos, tok_seg, block_table)
    T = q.shape[0]
    assert q.dtype == out.dtype == cache_layer.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and cache_layer.is_contiguous()
    assert tuple(cache_layer.shape[1:]) == (2, Hkv, page, hd)
    _i32(tok_pos, "tok_pos"); _i32(tok_seg, "tok_seg"); _i32(block_table, "block_table")
    partial = None
    if splits > 1:
        partial = torch.empty(T * H * splits * (hd + 2), dtype=torch.float32, device=q.device)
    lib = _lib("attention_bf16")
    lib.qv_attn_set_decode_variant(decode_variant(T, Hkv))
    if not getattr(lib, "_qv_err_set", False):
        # the word that the kernel's bounded waits report into (see check_kernel_errors)
        lib.qv_attn_set_error_word(_ptr(_tc_buffers(q.device)["err"]))
        lib._qv_err_set = True
    rc = lib.qv_attn_decode_bf16(_ptr(
        out), out.stride(0), _ptr(q), q.stride(0), _ptr(cache_layer), _ptr(tok_pos), _ptr(tok_seg),
        _ptr(block_table), block_table.shape[-1], T, H, Hkv, hd, page, window, scale, splits, _ptr(partial),
        _stream())
    if rc == -2:
        return False
    _check(rc, "attention_decode_bf16")
    if splits > 1:
        add_launches(1)                              # the merge of the slices
    return True


def attention_set_decode_variant(variant) -> None:
    """Forces the decode kernel (0: bulk copies into shared memory, 1: per-thread loads) or, with
    None, gives the choice back to decode_variant().  For comparison and tests."""
    global _decode_variant_forced
    _decode_variant_forced = variant


def _attention_portions_bf16(out, q, cache_layer, seg_q_start, seg_pos0, block_table, S, max_q_len, H, Hkv, hd, page,
                             window, scale, max_ctx_len=0) -> bool:
    """Prompt portions: tcgen05 kernel for long portions at head sizes 64/128, else mma.sync kernels."""
    if max_q_len >= 32 and attention_prefill_tc(out, q, cache_layer, seg_q_start, seg_pos0, block_table, S, max_q_len,
                                                H, Hkv, hd, page, window, scale, max_ctx_len):
        return True
    return attention_prefill_bf16(out, q, cache_layer, seg_q_start, seg_pos0, block_table, S, max_q_len, H, Hkv, hd,
                                  page, window, scale)


def attention(out, q, cache_layer, ctx, block_table, H, Hkv, hd, page, window, scale) -> None:
    """Attention of every token of the step over its request's pages.  bfloat16: the tensor-core
    kernels when they take the sizes (split-KV for single tokens, flash attention for portions; a
    step whose single-token segments come first is served by both, each on its part); float32,
    and sizes they refuse: the CUDA-core kernel."""
    if q.dtype == torch.bfloat16:
        T = q.shape[0]
        if ctx.max_q_len == 1:
            splits = decode_splits(T, Hkv, ctx.max_ctx_len, known=not ctx.captured)
            if attention_decode_bf16(out, q, cache_layer, ctx.tok_pos, ctx.tok_seg, block_table, H, Hkv, hd, page,
                                     window, scale, splits):
                return
        else:
            n1 = 0                                    # leading segments of one token (decoded tokens)
            while n1 < ctx.num_segments and ctx.seg_len[n1] == 1:
                n1 += 1
            S = ctx.num_segments
            # the longest context among the segments of more than one token (what the flash kernel cuts its work by)
            deep = max((p0 + n for p0, n in zip(ctx.seg_start_pos, ctx.seg_len) if n > 1), default=0)
            if n1 >= 4 and n1 < S:
                rest_q = max(ctx.seg_len[n1:])
                splits = decode_splits(n1, Hkv, ctx.max_ctx_len, known=not ctx.captured)
                ok = attention_decode_bf16(out[:n1], q[:n1], cache_layer, ctx.tok_pos, ctx.tok_seg, block_table, H, Hkv,
                                           hd, page, window, scale, splits)
                if ok and _attention_portions_bf16(out, q, cache_layer, ctx.seg_q_start[n1:], ctx.seg_pos0[n1:],
                                                   block_table[n1:], S - n1, rest_q, H, Hkv, hd, page, window, scale, deep):
                    return
            elif _attention_portions_bf16(out, q, cache_layer, ctx.seg_q_start, ctx.seg_pos0, block_table, S,
                                          ctx.max_q_len, H, Hkv, hd, page, window, scale, deep):
                return
    attention_generic(out, q, cache_layer, ctx.tok_pos, ctx.tok_seg, block_table, H, Hkv, hd, page, window, scale)


# ------------------------------------------------------------------ sampling

def argmax(out_ids, logits) -> None:
    """out_ids[r] = index of the first maximum of logits[r] (float32)."""
    _need_cuda(out_ids, logits)
    _i32(out_ids, "out_ids")
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out_ids.numel() >= logits.shape[0]
    rc = _lib("sampling").qv_argmax(
        _ptr(out_ids), _ptr(logits), logits.shape[0], logits.shape[1], logits.stride(0), _stream())
    _check(rc, "argmax")


def sample(out_ids, logits, temperature, top_k, top_p, min_p, uniform, recent=None, rep_pen=None,
           freq_pen=None, pres_pen=None) -> None:
    """One token per row of logits (float32; rewritten in place by the penalties).  Per-row
    parameters are device tensors: temperature/top_p/min_p/uniform float32, top_k int32; recent is
    int32 [rows, n] of the tokens the penalties look at (-1: empty)."""
    _need_cuda(out_ids, logits, temperature, top_k, top_p, min_p, uniform, recent, rep_pen, freq_pen, pres_pen)
    _i32(out_ids, "out_ids"); _i32(top_k, "top_k")
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    for t in (temperature, top_p, min_p, uniform):
        assert t.dtype == torch.float32 and t.is_contiguous() and t.numel() >= rows
    recent_n = 0
    if recent is not None:
        _i32(recent, "recent")
        recent_n = recent.shape[1]
        for t in (rep_pen, freq_pen, pres_pen):
            assert t is not None and t.dtype == torch.float32 and t.numel() >= rows
    rc = _lib("sampling").qv_sample(
        _ptr(out_ids), _ptr(logits), rows, V, logits.stride(0), _ptr(temperature), _ptr(top_k), _ptr(top_p),
        _ptr(min_p), _ptr(uniform), _ptr(recent), recent_n, _ptr(rep_pen), _ptr(freq_pen), _ptr(pres_pen),
        _stream())
    _check(rc, "sample")
