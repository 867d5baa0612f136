"""Plain, slow Llama decoder: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite. It shares no code with the product
package: it has its own config.json reader, its own safetensors reader and its own
math, written from the formulas of the reference engine (paths are relative to the
reference project):

  * embedding           runtime/src/text_model.cpp:118-122, runtime/include/qorvix/runtime/weights.hpp:90-97
  * rmsnorm             runtime/src/ops.cpp:8-13
  * projections         runtime/src/ops.cpp:34-56 (out[r] = dot(W[r,:], x), no bias)
  * rope (split-half)   runtime/src/ops.cpp:127-148
  * attention (GQA)     runtime/src/text_model.cpp:78-116
  * softmax             runtime/src/ops.cpp:83-94
  * swiglu              runtime/src/ops.cpp:96-100
  * block order         runtime/src/text_model.cpp:133-176
  * sampler             runtime/src/sampler.cpp:13-101
  * greedy generation   runtime/src/text_model.cpp:178-195

The llama3 frequency scaling has no counterpart in the reference (it parses the
rope-scaling keys for display only, gguf/src/gguf_file.cpp:233-243); `llama3_inv_freq`
rests on the published formula alone.

`tests/golden/make_golden.py` compiled the reference's own CPU TextModel once and
stored its logits for a tiny random model; `tests/test_plain_reference.py` checks this
file against those numbers.

All arithmetic is float64 unless `dtype` says otherwise, so that it is a stricter
oracle than either engine path.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

_ST_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "I32": (torch.int32, 4), "I64": (torch.int64, 8), "F64": (torch.float64, 8),
}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """Minimal reader: 8-byte little-endian header length, JSON header, raw bytes."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen].decode("utf-8"))
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dt, _ = _ST_DTYPES[meta["dtype"]]
        b, e = meta["data_offsets"]
        buf = bytearray(raw[base + b: base + e])
        t = torch.frombuffer(buf, dtype=dt).clone() if e > b else torch.empty(0, dtype=dt)
        out[name] = t.reshape(meta["shape"])
    return out


def read_model_dir(model_dir):
    """Returns (config dict, weights dict) of a folder with config.json + model.safetensors."""
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    weights = read_safetensors(model_dir / "model.safetensors")
    return cfg, weights


# ----------------------------------------------------------------------------- parts

def embedding(table: torch.Tensor, ids) -> torch.Tensor:
    """x = tokenEmbd[token, :], no scaling (runtime/src/text_model.cpp:120)."""
    return table[torch.as_tensor(ids, dtype=torch.long, device=table.device)]


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """out_i = x_i * (1/sqrt(sum(x^2)/n + eps)) * w_i (runtime/src/ops.cpp:8-13)."""
    n = x.shape[-1]
    sum_sq = (x * x).sum(dim=-1, keepdim=True)
    scale = 1.0 / torch.sqrt(sum_sq / n + eps)
    return x * scale * weight


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """out[r] = dot(W[r,:], x) for every row of x (runtime/src/ops.cpp:34-56)."""
    return x @ w.t()


def plain_inv_freq(head_dim: int, base: float) -> torch.Tensor:
    """f_i = base^(-2i/head_dim), i in [0, head_dim/2) (runtime/src/ops.cpp:132)."""
    i = torch.arange(head_dim // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / head_dim)


def llama3_inv_freq(head_dim: int, base: float, factor: float, low_freq_factor: float,
                    high_freq_factor: float, original_max_position: int) -> torch.Tensor:
    """llama3 frequency scaling (formula only; the reference has none).

    wavelength = 2*pi/f.  Short wavelengths (< orig/high) keep f, long ones
    (> orig/low) use f/factor, those between are blended linearly in
    s = (orig/wavelength - low) / (high - low).
    """
    f = plain_inv_freq(head_dim, base)
    out = torch.empty_like(f)
    low_wavelen = original_max_position / low_freq_factor
    high_wavelen = original_max_position / high_freq_factor
    for i in range(f.numel()):
        fi = float(f[i])
        wavelen = 2.0 * math.pi / fi
        if wavelen < high_wavelen:
            out[i] = fi
        elif wavelen > low_wavelen:
            out[i] = fi / factor
        else:
            s = (original_max_position / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def inv_freq_from_config(cfg: dict) -> torch.Tensor:
    hd = head_dim_of(cfg)
    base = float(cfg.get("rope_theta", 10000.0))
    rs = cfg.get("rope_scaling")
    if not rs:
        return plain_inv_freq(hd, base)
    kind = rs.get("rope_type", rs.get("type"))
    if kind in (None, "default"):
        return plain_inv_freq(hd, base)
    if kind != "llama3":
        raise ValueError(f"plain implementation knows no rope scaling {kind!r}")
    return llama3_inv_freq(hd, base, float(rs["factor"]), float(rs["low_freq_factor"]),
                           float(rs["high_freq_factor"]), int(rs["original_max_position_embeddings"]))


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Split-half rotation of x[T, heads, head_dim] (runtime/src/ops.cpp:141-146):
    pairs (i, i+half): a' = a cos - b sin, b' = a sin + b cos, theta = pos * f_i."""
    half = x.shape[-1] // 2
    theta = positions.to(torch.float64)[:, None] * inv_freq.to(torch.float64)[None, :]
    cos = torch.cos(theta).to(x.dtype).to(x.device)[:, None, :]
    sin = torch.sin(theta).to(x.dtype).to(x.device)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)


def softmax(scores: torch.Tensor) -> torch.Tensor:
    """exp(s - max) / sum (runtime/src/ops.cpp:83-94)."""
    m = scores.max(dim=-1, keepdim=True).values
    e = torch.exp(scores - m)
    return e / e.sum(dim=-1, keepdim=True)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0, rows=None) -> torch.Tensor:
    """Causal grouped-query attention over one whole sequence.

    q[T,H,hd], k,v[T,Hkv,hd] -> [T,H,hd].  kvHead = h / (H/Hkv); score =
    (q.k)/sqrt(hd) for t <= pos; softmax; weighted sum of V
    (runtime/src/text_model.cpp:83-114).  `window` > 0 keeps only the last `window`
    keys (pos - window < t <= pos); the reference has no window, 0 means all keys.
    `rows`: only these positions are computed (the others stay zero), for long sequences of
    which a test looks at a few places.
    """
    T, H, hd = q.shape
    Hkv = k.shape[1]
    group = H // Hkv
    out = torch.zeros_like(q)
    inv_sqrt = 1.0 / math.sqrt(hd)
    for h in range(H):
        kvh = h // group
        for pos in (range(T) if rows is None else rows):
            lo = 0 if window <= 0 else max(0, pos - window + 1)
            s = (k[lo:pos + 1, kvh, :] @ q[pos, h, :]) * inv_sqrt
            p = softmax(s)
            out[pos, h, :] = p @ v[lo:pos + 1, kvh, :]
    return out


def silu(z: torch.Tensor) -> torch.Tensor:
    """z / (1 + e^-z) (runtime/src/ops.cpp:96)."""
    return z / (1.0 + torch.exp(-z))


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up (runtime/src/ops.cpp:98-100)."""
    return silu(gate) * up


# ----------------------------------------------------------------------------- model

def head_dim_of(cfg: dict) -> int:
    hd = cfg.get("head_dim")
    return int(hd) if hd else int(cfg["hidden_size"]) // int(cfg["num_attention_heads"])


def attention_block(x, w, prefix, cfg, positions, inv_freq, rows=None):
    """norm -> q,k,v -> rope(q), rope(k) -> attention -> o-proj (runtime/src/text_model.cpp:146-158).
    With `rows` the output holds those positions only (keys and values are still the whole sequence's)."""
    H = int(cfg["num_attention_heads"])
    Hkv = int(cfg.get("num_key_value_heads") or H)
    hd = head_dim_of(cfg)
    T = x.shape[0]
    xn = rmsnorm(x, w[prefix + "input_layernorm.weight"], float(cfg.get("rms_norm_eps", 1e-5)))
    q = linear(xn, w[prefix + "self_attn.q_proj.weight"]).reshape(T, H, hd)
    k = linear(xn, w[prefix + "self_attn.k_proj.weight"]).reshape(T, Hkv, hd)
    v = linear(xn, w[prefix + "self_attn.v_proj.weight"]).reshape(T, Hkv, hd)
    q = rope(q, positions, inv_freq)
    k = rope(k, positions, inv_freq)
    a = attention(q, k, v, rows=rows).reshape(T, H * hd)
    if rows is not None:
        a = a[torch.as_tensor(list(rows), dtype=torch.long, device=a.device)]
    return linear(a, w[prefix + "self_attn.o_proj.weight"])


def feed_forward_block(x, w, prefix, cfg):
    """norm -> gate, up -> swiglu -> down (runtime/src/text_model.cpp:162-167)."""
    xn = rmsnorm(x, w[prefix + "post_attention_layernorm.weight"], float(cfg.get("rms_norm_eps", 1e-5)))
    g = linear(xn, w[prefix + "mlp.gate_proj.weight"])
    u = linear(xn, w[prefix + "mlp.up_proj.weight"])
    return linear(swiglu(g, u), w[prefix + "mlp.down_proj.weight"])


def lm_head_weight(w: dict, cfg: dict) -> torch.Tensor:
    """output.weight if present, else the embedding table (runtime/include/qorvix/runtime/weights.hpp:119)."""
    if "lm_head.weight" in w and not cfg.get("tie_word_embeddings", False):
        return w["lm_head.weight"]
    return w["model.embed_tokens.weight"]


def forward(cfg: dict, weights: dict, token_ids, dtype=torch.float64, rows=None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence (runtime/src/text_model.cpp:133-176).  With `rows`
    only the logits at those positions, [len(rows), vocab]: the last layer's attention, feed-forward
    and the head then run on those positions alone (the layers before it need every position)."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    T = len(token_ids)
    positions = torch.arange(T)
    inv_freq = inv_freq_from_config(cfg)
    x = embedding(w["model.embed_tokens.weight"], token_ids)
    n_layers = int(cfg["num_hidden_layers"])
    for layer in range(n_layers):
        prefix = f"model.layers.{layer}."
        if rows is not None and layer == n_layers - 1:
            idx = torch.as_tensor(list(rows), dtype=torch.long, device=x.device)
            x = x[idx] + attention_block(x, w, prefix, cfg, positions, inv_freq, rows=list(rows))
        else:
            x = x + attention_block(x, w, prefix, cfg, positions, inv_freq)
        x = x + feed_forward_block(x, w, prefix, cfg)
    xn = rmsnorm(x, w["model.norm.weight"], float(cfg.get("rms_norm_eps", 1e-5)))
    return linear(xn, lm_head_weight(w, cfg))


def argmax(logits: torch.Tensor) -> int:
    """First maximum wins (runtime/src/ops.cpp:150-156)."""
    best = 0
    vals = logits.tolist()
    for i in range(1, len(vals)):
        if vals[i] > vals[best]:
            best = i
    return best


def generate_greedy(cfg: dict, weights: dict, prompt, max_new: int, dtype=torch.float64) -> list[int]:
    """Greedy continuation; recomputes the whole sequence for each token
    (runtime/src/text_model.cpp:178-195)."""
    seq = list(prompt)
    out = []
    for _ in range(max_new):
        logits = forward(cfg, weights, seq, dtype)
        nxt = argmax(logits[-1])
        out.append(nxt)
        seq.append(nxt)
    return out


# ----------------------------------------------------------------------------- sampler

def apply_penalties(logits: np.ndarray, recent, repetition_penalty=1.0, frequency_penalty=0.0,
                    presence_penalty=0.0, penalty_last_n=64) -> np.ndarray:
    """runtime/src/sampler.cpp:13-34."""
    logits = logits.astype(np.float32).copy()
    if penalty_last_n == 0:
        return logits
    if repetition_penalty == 1.0 and frequency_penalty == 0.0 and presence_penalty == 0.0:
        return logits
    window = list(recent)[-penalty_last_n:] if len(recent) > penalty_last_n else list(recent)
    counts = {}
    for t in window:
        counts[t] = counts.get(t, 0) + 1
    for tok, count in counts.items():
        if tok < 0 or tok >= logits.shape[0]:
            continue
        l = logits[tok]
        if repetition_penalty != 1.0:
            l = l / repetition_penalty if l > 0 else l * repetition_penalty
        l -= count * frequency_penalty
        l -= presence_penalty
        logits[tok] = l
    return logits


def candidate_set(logits: np.ndarray, temperature: float, top_k: int = 0, top_p: float = 1.0,
                  min_p: float = 0.0):
    """The (ids, probs) that survive temperature -> softmax -> sort -> top-k -> top-p ->
    min-p, in that order (runtime/src/sampler.cpp:53-87).  top-p keeps the shortest prefix
    whose cumulative un-renormalised probability reaches p."""
    l = logits.astype(np.float64) / temperature
    p = np.exp(l - l.max())
    p = p / p.sum()
    order = np.argsort(-p, kind="stable")
    probs = p[order]
    if 0 < top_k < len(order):
        order, probs = order[:top_k], probs[:top_k]
    if top_p < 1.0:
        cum = np.cumsum(probs)
        keep = len(order)
        for i in range(len(order)):
            if cum[i] >= top_p:
                keep = i + 1
                break
        order, probs = order[:keep], probs[:keep]
    if min_p > 0.0 and len(order):
        thr = min_p * probs[0]
        mask = probs >= thr
        order, probs = order[mask], probs[mask]
    return order, probs


def sample_with_uniform(logits: np.ndarray, u: float, temperature: float, top_k: int = 0,
                        top_p: float = 1.0, min_p: float = 0.0) -> int:
    """Draw with a given uniform number u in [0,1): r = u * total, walk the sorted
    survivors subtracting probabilities (runtime/src/sampler.cpp:92-100)."""
    if temperature <= 0.0:
        return int(np.argmax(logits))
    ids, probs = candidate_set(logits, temperature, top_k, top_p, min_p)
    if len(ids) == 0:
        return int(np.argmax(logits))
    r = u * probs.sum()
    for i, pr in zip(ids, probs):
        r -= pr
        if r <= 0.0:
            return int(i)
    return int(ids[-1])
