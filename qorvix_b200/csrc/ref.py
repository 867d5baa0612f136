"""Python face of the plain C++ twins (csrc/ref/): a whole-model forward over a model folder and
one function per operation, all on the host.  `qorvix gpu-check` and the tests compare the engine
and its kernels with these; nothing on the product's step path uses them."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_longlong, c_void_p

import numpy as np

from .build import load_library

_lib = None


def lib():
    global _lib
    if _lib is None:
        L = load_library("ref")
        fp, ip, dp = POINTER(c_float), POINTER(c_int), POINTER(c_double)
        sig = {
            "qvr_last_error": (c_char_p, []), "qvr_model_open": (c_void_p, [c_char_p]), "qvr_model_close": (None, [c_void_p]),
            "qvr_model_vocab": (c_int, [c_void_p]), "qvr_forward": (c_int, [c_void_p, ip, c_int, fp]),
            "qvr_rmsnorm": (None, [fp, fp, fp, c_int, c_int, c_double]), "qvr_gemm": (None, [fp, fp, fp, c_int, c_int, c_int]),
            "qvr_rope": (None, [fp, c_int, ip, c_int, c_int, c_int, dp]),
            "qvr_inverse_frequencies": (None, [dp, c_int, c_double, c_int, c_double, c_double, c_double, c_longlong]),
            "qvr_attention_paged": (None, [fp, c_int, fp, c_int, fp, ip, ip, ip, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_double]),
            "qvr_swiglu": (None, [fp, fp, fp, c_longlong]), "qvr_argmax": (c_int, [fp, c_int]),
            "qvr_candidates": (c_int, [fp, c_int, c_double, c_int, c_double, c_double, ip, dp, c_int]),
            "qvr_sample": (c_int, [fp, c_int, c_double, c_int, c_double, c_double, c_double, c_double, c_double, c_int, ip, c_int, c_double]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(POINTER(c_float))


def _i(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(POINTER(c_int))


class RefModel:
    """The plain C++ decoder over a model folder (config.json + safetensors)."""

    def __init__(self, model_dir):
        self._lib = lib()
        self._h = self._lib.qvr_model_open(str(model_dir).encode())
        if not self._h:
            raise ValueError(self._lib.qvr_last_error().decode())
        self.vocab_size = self._lib.qvr_model_vocab(self._h)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.qvr_model_close(self._h)
            self._h = None

    def logits(self, tokens) -> np.ndarray:
        """float32 [len(tokens), vocab] of one whole sequence."""
        toks, tp = _i(list(tokens))
        out = np.empty((len(toks), self.vocab_size), dtype=np.float32)
        if self._lib.qvr_forward(self._h, tp, len(toks), out.ctypes.data_as(POINTER(c_float))) != 0:
            raise ValueError(self._lib.qvr_last_error().decode())
        return out


def rmsnorm(x, w, eps):
    x, xp = _f(x); w, wp = _f(w)
    out = np.empty_like(x)
    lib().qvr_rmsnorm(out.ctypes.data_as(POINTER(c_float)), xp, wp, x.shape[0], x.shape[1], float(eps))
    return out


def gemm(a, w):
    a, ap = _f(a); w, wp = _f(w)
    out = np.empty((a.shape[0], w.shape[0]), dtype=np.float32)
    lib().qvr_gemm(out.ctypes.data_as(POINTER(c_float)), ap, wp, a.shape[0], w.shape[0], a.shape[1])
    return out


def inverse_frequencies(rotary_dim, theta, scaling=None):
    out = np.empty(rotary_dim // 2, dtype=np.float64)
    if scaling is None:
        lib().qvr_inverse_frequencies(out.ctypes.data_as(POINTER(c_double)), rotary_dim, float(theta), 0, 1.0, 1.0, 4.0, 0)
    else:
        lib().qvr_inverse_frequencies(out.ctypes.data_as(POINTER(c_double)), rotary_dim, float(theta), 1, float(scaling.factor),
                                      float(scaling.low_freq_factor), float(scaling.high_freq_factor),
                                      int(scaling.original_max_position_embeddings))
    return out


def rope(vec, positions, n_heads, head_dim, rotary_dim, inv_freq):
    """vec [rows, n_heads * head_dim] rotated (a copy is returned)."""
    v, vp = _f(np.array(vec, copy=True)); pos, pp = _i(positions)
    f = np.ascontiguousarray(inv_freq, dtype=np.float64)
    lib().qvr_rope(vp, v.shape[0], pp, n_heads, head_dim, rotary_dim, f.ctypes.data_as(POINTER(c_double)))
    return v


def attention_paged(q, cache, tok_pos, tok_seg, block_table, H, Hkv, hd, page, window, scale):
    """q [T, H*hd]; cache [pages, 2, Hkv, page, hd]; block_table [S, max_blocks]."""
    q, qp = _f(q); cache, cp = _f(cache)
    pos, pp = _i(tok_pos); seg, sp = _i(tok_seg); bt, bp = _i(block_table)
    out = np.empty_like(q)
    lib().qvr_attention_paged(out.ctypes.data_as(POINTER(c_float)), q.shape[1], qp, q.shape[1], cp, pp, sp, bp, bt.shape[1], q.shape[0],
                              H, Hkv, hd, page, window, float(scale))
    return out


def swiglu(gate, up):
    g, gp = _f(gate); u, up_ = _f(up)
    out = np.empty_like(g)
    lib().qvr_swiglu(out.ctypes.data_as(POINTER(c_float)), gp, up_, g.size)
    return out


def argmax(x) -> int:
    x, xp = _f(x)
    return lib().qvr_argmax(xp, x.size)


def candidates(logits, temperature, top_k=0, top_p=1.0, min_p=0.0):
    l, lp = _f(logits)
    ids = np.empty(l.size, dtype=np.int32); probs = np.empty(l.size, dtype=np.float64)
    n = lib().qvr_candidates(lp, l.size, float(temperature), int(top_k), float(top_p), float(min_p),
                             ids.ctypes.data_as(POINTER(c_int)), probs.ctypes.data_as(POINTER(c_double)), l.size)
    return ids[:n].copy(), probs[:n].copy()


def sample(logits, u, temperature, top_k=0, top_p=1.0, min_p=0.0, recent=(), repetition_penalty=1.0, frequency_penalty=0.0,
           presence_penalty=0.0, penalty_last_n=64) -> int:
    l, lp = _f(np.array(logits, copy=True))
    rec, rp = _i(list(recent) or [0])
    return lib().qvr_sample(lp, l.size, float(temperature), int(top_k), float(top_p), float(min_p), float(repetition_penalty),
                            float(frequency_penalty), float(presence_penalty), int(penalty_last_n), rp, len(recent), float(u))
