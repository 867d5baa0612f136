"""Toy parts of every category, defined here and registered without a change to the framework's
files: a feed-forward with routing, a position encoding that is no rotation and has weights of
its own, a norm with a mean and a bias, and a block arrangement that runs its mixer and its
feed-forward side by side.  One toy model mixes them with the framework's own parts layer by
layer; the engine steps it whole, in portions, beside another request and in captured decode
steps, and the logits are compared with the same arithmetic written out in float64.

The toys compute with torch on the device: they are test fixtures that show the interfaces,
not kernels of the package.
"""
from dataclasses import dataclass

import pytest
import torch

import plain_llama as plain
from helpers import assert_close_logits, random_tokens
from qorvix_b200 import ModelRunner, StepEntry
from qorvix_b200.config import ModelConfig, register_architecture, unregister_architecture
from qorvix_b200.parts import (AttentionSpec, LayerSpec, ModelSpec, RMSNormSpec, RotarySpec, build_part,
                               register_part, unregister_part)
from qorvix_b200.parts.base import Block, FeedForward, Norm, PositionEncoding

pytestmark = pytest.mark.gpu

D, H, HKV, HD, F, E, VOCAB, MAXPOS = 48, 3, 1, 16, 40, 3, 83, 160
EPS = 1e-4


# ------------------------------------------------------------------ a feed-forward with routing

@dataclass(frozen=True)
class RoutedSpec:
    """Top-1 of `experts` two-matrix experts; the chosen expert's output is scaled by its softmax weight."""
    hidden_size: int
    intermediate_size: int
    experts: int
    prefix: str
    kind: str = "toy_routed"

    def tensors(self):
        t = {self.prefix + "router": ((self.experts, self.hidden_size), "matrix")}
        for e in range(self.experts):
            t[f"{self.prefix}e{e}.up"] = ((self.intermediate_size, self.hidden_size), "matrix")
            t[f"{self.prefix}e{e}.down"] = ((self.hidden_size, self.intermediate_size), "matrix")
        return t


class RoutedFeedForward(FeedForward):
    def __init__(self, spec, source, rt):
        self.rt, self.n = rt, spec.experts
        self.router = source.get(spec.prefix + "router").float()
        self.up = [source.get(f"{spec.prefix}e{e}.up").float() for e in range(self.n)]
        self.down = [source.get(f"{spec.prefix}e{e}.down").float() for e in range(self.n)]

    def forward(self, x, ctx):
        x = x.float()
        logits = x @ self.router.t()                              # router logits in float32
        prob = torch.softmax(logits, dim=-1)
        choice = logits.argmax(dim=-1)
        out = torch.zeros_like(x)
        for e in range(self.n):                                   # every expert on every row, masked: no shape depends on the data
            y = torch.relu(x @ self.up[e].t()) @ self.down[e].t()
            out += torch.where((choice == e)[:, None], prob[:, e:e + 1] * y, torch.zeros_like(y))
        return out.to(self.rt.dtype)


def routed_plain(h, w, prefix):
    logits = h @ w[prefix + "router"].t()
    prob = torch.softmax(logits, dim=-1)
    choice = logits.argmax(dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        e = int(choice[t])
        out[t] = prob[t, e] * (torch.relu(h[t] @ w[f"{prefix}e{e}.up"].t()) @ w[f"{prefix}e{e}.down"].t())
    top2 = logits.topk(2, dim=-1).values
    return out, float((top2[:, 0] - top2[:, 1]).min())


# ------------------------------------------------------------------ a position encoding with weights, no rotation

@dataclass(frozen=True)
class LearnedPositionSpec:
    """q and k of every head get a learned vector of their position added."""
    head_dim: int
    positions: int
    q_table: str
    k_table: str
    kind: str = "toy_learned"

    def tensors(self):
        return {self.q_table: ((self.positions, self.head_dim), "matrix"),
                self.k_table: ((self.positions, self.head_dim), "matrix")}


class LearnedPosition(PositionEncoding):
    def __init__(self, spec, source, rt):
        self.q = source.get(spec.q_table).float()
        self.k = source.get(spec.k_table).float()

    def table(self):
        return None                                               # not a rotation the kernels fuse

    def apply(self, qkv, ctx, num_heads, num_kv_heads, head_dim):
        pos = ctx.tok_pos.long()
        heads = qkv.view(qkv.shape[0], -1, head_dim)
        heads[:, :num_heads] = (heads[:, :num_heads].float() + self.q[pos][:, None, :]).to(qkv.dtype)
        if num_kv_heads:
            k = heads[:, num_heads:num_heads + num_kv_heads]
            heads[:, num_heads:num_heads + num_kv_heads] = (k.float() + self.k[pos][:, None, :]).to(qkv.dtype)


# ------------------------------------------------------------------ a norm with a mean and a bias

@dataclass(frozen=True)
class LayerNormSpec:
    size: int
    eps: float
    weight: str
    bias: str
    kind: str = "toy_layernorm"

    def tensors(self):
        return {self.weight: ((self.size,), "norm"), self.bias: ((self.size,), "matrix")}


class LayerNorm(Norm):
    def __init__(self, spec, source, rt):
        self.rt, self.eps = rt, spec.eps
        self.w = source.get(spec.weight, dtype=torch.float32)
        self.b = source.get(spec.bias, dtype=torch.float32)

    def add_norm(self, residual, delta, rows=None):
        if rows is None:
            if delta is not None:
                residual += delta.float()
            x = residual
        else:
            idx = rows.long()
            x = residual[idx] + (delta[idx].float() if delta is not None else 0.0)
        mu = x.mean(dim=-1, keepdim=True)
        var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
        return ((x - mu) * torch.rsqrt(var + self.eps) * self.w + self.b).to(self.rt.dtype)


def layernorm_plain(x, w, b, eps):
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


# ------------------------------------------------------------------ a block that runs mixer and feed-forward side by side

class ParallelBlock(Block):
    """x += mixer(norm(x)) + feed_forward(norm(x)): one norm, both parts read it."""

    def __init__(self, spec, source, rt):
        self.norm = build_part("norm", spec.mixer_norm, source, rt)
        self.mixer = build_part("mixer", spec.mixer, source, rt)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, source, rt)

    def forward(self, residual, pending, ctx, cache):
        h = self.norm.add_norm(residual, pending)
        a = self.mixer.forward(h, ctx, cache)
        f = self.feed_forward.forward(h, ctx)
        return residual, (a.float() + f.float()).to(a.dtype)


# ------------------------------------------------------------------ the toy model

@dataclass(frozen=True)
class ToyCfg(ModelConfig):
    pass


def toy_spec(cfg):
    def att(p, position):
        return AttentionSpec(hidden_size=D, num_heads=H, num_kv_heads=HKV, head_dim=HD, scale=HD ** -0.5, q_proj=p + "q",
                             k_proj=p + "k", v_proj=p + "v", o_proj=p + "o", position=position)
    layers = [
        # side by side, layer norm, learned positions, routed experts
        LayerSpec(mixer=att("l0.", LearnedPositionSpec(HD, MAXPOS, "l0.pos_q", "l0.pos_k")),
                  feed_forward=RoutedSpec(D, F, E, "l0.moe."), mixer_norm=LayerNormSpec(D, EPS, "l0.ln.w", "l0.ln.b"),
                  ffn_norm=None, block="toy_parallel"),
        # the framework's arrangement, norms and rotary attention around the toy feed-forward
        LayerSpec(mixer=att("l1.", RotarySpec(HD, HD, 10000.0)), feed_forward=RoutedSpec(D, F, E, "l1.moe."),
                  mixer_norm=RMSNormSpec(D, EPS, "l1.n1"), ffn_norm=RMSNormSpec(D, EPS, "l1.n2")),
    ]
    return ModelSpec(architecture="ToyPartsLM", vocab_size=VOCAB, hidden_size=D, embedding="emb", layers=layers,
                     final_norm=LayerNormSpec(D, EPS, "fn.w", "fn.b"), lm_head="head", max_position=MAXPOS)


def toy_plain(w, tokens):
    """The toy model on one whole sequence in float64; also the smallest gap between the two best experts."""
    T = len(tokens)
    pos = torch.arange(T)
    x = w["emb"][torch.tensor(tokens)]
    # layer 0
    h = layernorm_plain(x, w["l0.ln.w"], w["l0.ln.b"], EPS)
    q = plain.linear(h, w["l0.q"]).reshape(T, H, HD) + w["l0.pos_q"][pos][:, None, :]
    k = plain.linear(h, w["l0.k"]).reshape(T, HKV, HD) + w["l0.pos_k"][pos][:, None, :]
    v = plain.linear(h, w["l0.v"]).reshape(T, HKV, HD)
    a = plain.linear(plain.attention(q, k, v).reshape(T, H * HD), w["l0.o"])
    f, gap0 = routed_plain(h, w, "l0.moe.")
    x = x + a + f
    # layer 1
    inv = plain.plain_inv_freq(HD, 10000.0)
    h = plain.rmsnorm(x, w["l1.n1"], EPS)
    q = plain.rope(plain.linear(h, w["l1.q"]).reshape(T, H, HD), pos, inv)
    k = plain.rope(plain.linear(h, w["l1.k"]).reshape(T, HKV, HD), pos, inv)
    v = plain.linear(h, w["l1.v"]).reshape(T, HKV, HD)
    x = x + plain.linear(plain.attention(q, k, v).reshape(T, H * HD), w["l1.o"])
    f, gap1 = routed_plain(plain.rmsnorm(x, w["l1.n2"], EPS), w, "l1.moe.")
    x = x + f
    return plain.linear(layernorm_plain(x, w["fn.w"], w["fn.b"], EPS), w["head"]), min(gap0, gap1)


def toy_tensors(seed=14):
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for name, (shape, kind) in toy_spec(None).tensor_table().items():
        t = torch.randn(shape, generator=g)
        if kind == "norm":
            t = 1 + 0.1 * t
        elif name.endswith("router"):
            t = 1.5 * t                       # wide gaps between the experts' logits
        elif len(shape) == 1 or "pos_" in name:
            t = 0.3 * t
        else:
            t = 0.2 * t
        tensors[name] = t.to(torch.bfloat16)
    return tensors


# weights and token seeds found by search: every routing decision of these sequences is clear of a tie
# (the test checks the gap between the two best experts' logits)
SEED_A, SEED_B = 3, 2


@pytest.fixture
def toy():
    register_part("feed_forward", "toy_routed", RoutedFeedForward)
    register_part("position", "toy_learned", LearnedPosition)
    register_part("norm", "toy_layernorm", LayerNorm)
    register_part("block", "toy_parallel", ParallelBlock)
    register_architecture("ToyPartsLM", lambda raw: ToyCfg("ToyPartsLM"), toy_spec)
    yield toy_tensors()
    unregister_architecture("ToyPartsLM")
    for cat, kind in (("feed_forward", "toy_routed"), ("position", "toy_learned"), ("norm", "toy_layernorm"),
                      ("block", "toy_parallel")):
        unregister_part(cat, kind)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_parts_of_every_category_are_registered_built_and_stepped(toy, dtype):
    tensors = toy
    w = {k: v.double() for k, v in tensors.items()}
    a, b = random_tokens(VOCAB, 44, SEED_A), random_tokens(VOCAB, 27, SEED_B)
    ref_a, gap_a = toy_plain(w, a)
    ref_b, gap_b = toy_plain(w, b)
    # a routing decision within rounding of a tie would make the comparison meaningless
    assert min(gap_a, gap_b) > 0.5, (gap_a, gap_b)
    r = ModelRunner(config=ToyCfg("ToyPartsLM"), tensors=tensors, dtype=dtype, max_tokens=192, max_requests=3)
    assert "l0.pos_q" in r.model.spec.tensor_table()             # the position encoding's own weights are loaded by name
    whole = r.step([StepEntry("w", a, list(range(44)))], end=["w"])
    assert_close_logits(whole, ref_a, dtype, "toy parts whole")
    got_a, got_b = [], []
    got_a.append(r.step([StepEntry("a", a[:2], [0, 1])]))
    out = r.step([StepEntry("a", a[2:21], list(range(19))), StepEntry("b", b[:16], list(range(16)))])
    got_a.append(out[:19]); got_b.append(out[19:])
    out = r.step([StepEntry("b", b[16:22], list(range(6))), StepEntry("a", a[21:34], list(range(13)))])
    got_b.append(out[:6]); got_a.append(out[6:])
    for i in range(5):                                            # both decode: captured steps
        out = r.step([StepEntry("a", [a[34 + i]], [0]), StepEntry("b", [b[22 + i]], [0])])
        got_a.append(out[:1]); got_b.append(out[1:])
    for i in range(39, 44):
        got_a.append(r.step([StepEntry("a", [a[i]], [0])]))
    assert_close_logits(torch.cat(got_a), ref_a, dtype, "toy parts, request a in portions")
    assert_close_logits(torch.cat(got_b), ref_b, dtype, "toy parts, request b in portions")


# ------------------------------------------------------------------ a norm of its own that folds into the products

@dataclass(frozen=True)
class OnePlusRMSSpec:
    """x * rsqrt(mean(x^2) + eps) * (1 + w): not the framework's norm, but of the family whose two
    passes over the stream the few-token products can take over."""
    size: int
    eps: float
    weight: str
    kind: str = "toy_one_plus_rms"

    def tensors(self):
        return {self.weight: ((self.size,), "matrix")}


class OnePlusRMS(Norm):
    folds_into_products = True

    def __init__(self, spec, source, rt):
        self.size, self.eps, self.rt = spec.size, spec.eps, rt
        self.w1 = (1.0 + source.get(spec.weight, dtype=torch.float32)).contiguous()

    def scale_weight(self):
        return self.w1

    def add_norm(self, residual, delta, rows=None):
        if delta is not None and not hasattr(delta, "materialise"):
            residual += delta.float()
        x = residual if rows is None else residual[rows.long()]
        return (x * torch.rsqrt((x * x).mean(-1, keepdim=True) + self.eps) * self.w1).to(self.rt.dtype)


def test_a_toy_norm_opts_into_folding_without_a_change_to_the_package(monkeypatch):
    """Llama-shaped layers whose norms are the toy (1 + w) RMS norm above: in decode steps of the
    bfloat16 engine the products around the norms take over its passes (the folding kernel is seen
    to run) and the logits are those of float64 arithmetic with the same norm."""
    from helpers import CallCounter
    from qorvix_b200.parts import SwiGLUSpec
    d, heads, kvh, hd, f, vocab, eps = 512, 4, 2, 128, 1024, 211, 1e-5

    def spec(cfg):
        layers = []
        for i in range(2):
            p = f"l{i}."
            layers.append(LayerSpec(
                mixer=AttentionSpec(hidden_size=d, num_heads=heads, num_kv_heads=kvh, head_dim=hd, scale=hd ** -0.5, q_proj=p + "q",
                                    k_proj=p + "k", v_proj=p + "v", o_proj=p + "o", position=RotarySpec(hd, hd, 10000.0)),
                feed_forward=SwiGLUSpec(d, f, p + "gate", p + "up", p + "down"),
                mixer_norm=OnePlusRMSSpec(d, eps, p + "n1"), ffn_norm=OnePlusRMSSpec(d, eps, p + "n2")))
        return ModelSpec(architecture="ToyNormLM", vocab_size=vocab, hidden_size=d, embedding="emb", layers=layers,
                         final_norm=OnePlusRMSSpec(d, eps, "fn"), lm_head="head", max_position=128)

    g = torch.Generator().manual_seed(5)
    tensors = {}
    for name, (shape, _) in spec(None).tensor_table().items():
        t = torch.randn(shape, generator=g)
        t = 0.2 * t if len(shape) == 1 else (0.08 * t if name.endswith((".q", ".k")) else 0.02 * t)
        tensors[name] = t.to(torch.bfloat16)
    w = {k: v.double() for k, v in tensors.items()}

    def plain_model(tokens):
        T = len(tokens)
        pos = torch.arange(T)
        inv = plain.plain_inv_freq(hd, 10000.0)
        x = w["emb"][torch.tensor(tokens)]
        for i in range(2):
            p = f"l{i}."
            h = plain.rmsnorm(x, 1.0 + w[p + "n1"], eps)
            q = plain.rope(plain.linear(h, w[p + "q"]).reshape(T, heads, hd), pos, inv)
            k = plain.rope(plain.linear(h, w[p + "k"]).reshape(T, kvh, hd), pos, inv)
            v = plain.linear(h, w[p + "v"]).reshape(T, kvh, hd)
            x = x + plain.linear(plain.attention(q, k, v).reshape(T, heads * hd), w[p + "o"])
            h = plain.rmsnorm(x, 1.0 + w[p + "n2"], eps)
            x = x + plain.linear(plain.swiglu(plain.linear(h, w[p + "gate"]), plain.linear(h, w[p + "up"])), w[p + "down"])
        return plain.linear(plain.rmsnorm(x, 1.0 + w["fn"], eps), w["head"])

    register_part("norm", "toy_one_plus_rms", OnePlusRMS)
    register_architecture("ToyNormLM", lambda raw: ToyCfg("ToyNormLM"), spec)
    try:
        toks = random_tokens(vocab, 40, 9)
        ref = plain_model(toks)
        counts = CallCounter(monkeypatch, "gemm_bf16_norm")
        r = ModelRunner(config=ToyCfg("ToyNormLM"), tensors=tensors, dtype="bfloat16", max_tokens=128, max_requests=2, use_graphs=False)
        outs = [r.step([StepEntry("a", toks[:30], list(range(30)))])]
        for i in range(30, 40):
            outs.append(r.step([StepEntry("a", [toks[i]], [0])]))
        assert counts["gemm_bf16_norm"] > 0, "the folding products were meant to serve the toy norm"
        assert_close_logits(torch.cat(outs), ref, "bfloat16", "toy folding norm", sharp=True)
    finally:
        unregister_architecture("ToyNormLM")
        unregister_part("norm", "toy_one_plus_rms")
