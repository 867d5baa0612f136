"""Layer descriptions as data.  An architecture turns its configuration into a ModelSpec: a
list of LayerSpecs (each naming its mixer, feed-forward, norms and arrangement, with all
sizes and constants as fields) and the order in which layers run.  Parts are built from
these specs through the registry in parts/registry.py; no part knows which model it is in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

# tensor table entries: name -> (shape, kind) with kind in {"matrix", "norm"} (how random
# weights are drawn)
TensorTable = Dict[str, Tuple[Tuple[int, ...], str]]


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding.  `rotary_dim` leading dims of each head are rotated in
    split-half pairs (i, i + rotary_dim/2); the reference's NeoX mode (runtime/src/ops.cpp:141-146)."""
    head_dim: int
    rotary_dim: int
    theta: float
    scaling: Optional[object] = None          # config.RopeScaling or None
    kind: str = "rotary"

    def tensors(self) -> TensorTable:
        return {}


@dataclass(frozen=True)
class RMSNormSpec:
    size: int
    eps: float
    weight: str
    kind: str = "rmsnorm"

    def tensors(self) -> TensorTable:
        return {self.weight: ((self.size,), "norm")}


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention with its four projections."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    q_proj: str
    k_proj: str
    v_proj: str
    o_proj: str
    position: Optional[object] = None         # a position-encoding spec, or None
    window: int = 0                           # 0: all keys; n: the last n keys
    kv_from: Optional[int] = None             # read this layer's cache instead of keeping one
    kind: str = "attention"

    def tensors(self) -> TensorTable:
        t = {self.q_proj: ((self.num_heads * self.head_dim, self.hidden_size), "matrix"),
             self.o_proj: ((self.hidden_size, self.num_heads * self.head_dim), "matrix")}
        if self.kv_from is None:
            t[self.k_proj] = ((self.num_kv_heads * self.head_dim, self.hidden_size), "matrix")
            t[self.v_proj] = ((self.num_kv_heads * self.head_dim, self.hidden_size), "matrix")
        if self.position is not None:
            t.update(self.position.tensors())       # a position encoding may have weights of its own
        return t


@dataclass(frozen=True)
class SwiGLUSpec:
    """Dense gated feed-forward: down(silu(gate x) * up x)."""
    hidden_size: int
    intermediate_size: int
    gate_proj: str
    up_proj: str
    down_proj: str
    kind: str = "swiglu"

    def tensors(self) -> TensorTable:
        return {self.gate_proj: ((self.intermediate_size, self.hidden_size), "matrix"),
                self.up_proj: ((self.intermediate_size, self.hidden_size), "matrix"),
                self.down_proj: ((self.hidden_size, self.intermediate_size), "matrix")}


@dataclass(frozen=True)
class LayerSpec:
    """One block: which parts and how they are arranged ('pre_norm': x += mixer(norm(x));
    x += ffn(norm(x)), the reference's order, runtime/src/text_model.cpp:146-168)."""
    mixer: object
    feed_forward: object
    mixer_norm: object
    ffn_norm: object
    block: str = "pre_norm"

    def tensors(self) -> TensorTable:
        t: TensorTable = {}
        for part in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward):
            if part is not None:
                t.update(part.tensors())
        return t


@dataclass
class ModelSpec:
    """A whole decoder: embedding, layers, the order they run in, final norm, output head."""
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: str
    layers: List[LayerSpec]
    final_norm: object
    lm_head: Optional[str]                    # None: the head is the embedding table (tied)
    order: List[int] = None                   # layer indices in execution order; may repeat
    optional_tensors: Tuple[str, ...] = ()    # may be stored but are not used (e.g. a tied head's copy)
    ignored_tensors: Tuple[str, ...] = ()     # name patterns (fnmatch) of stored buffers that are no weights
    max_position: int = 0

    def __post_init__(self):
        if self.order is None:
            self.order = list(range(len(self.layers)))
        for i in self.order:
            if not 0 <= i < len(self.layers):
                raise ValueError(f"layer order names layer {i}, the model has {len(self.layers)}")

    def tensor_table(self) -> TensorTable:
        t: TensorTable = {self.embedding: ((self.vocab_size, self.hidden_size), "matrix")}
        for layer in self.layers:
            t.update(layer.tensors())
        t.update(self.final_norm.tensors())
        if self.lm_head is not None:
            t[self.lm_head] = ((self.vocab_size, self.hidden_size), "matrix")
        return t

    def expected_shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {n: s for n, (s, _) in self.tensor_table().items()}
