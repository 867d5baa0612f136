"""Each part alone against the plain implementation, and a toy mixer with state of its own that
is defined here, registered, built and stepped without a change to the framework's files."""
import math
from dataclasses import dataclass

import pytest
import torch

import plain_llama as plain
from helpers import TINY, assert_close_logits, random_tokens
from qorvix_b200 import ModelRunner, StepEntry
from qorvix_b200.cache import CacheManager, FixedStateSpec
from qorvix_b200.config import ModelConfig, RopeScaling, register_architecture, unregister_architecture
from qorvix_b200.engine.batch import BatchBuilder
from qorvix_b200.parts import (AttentionSpec, LayerSpec, ModelSpec, RMSNormSpec, RotarySpec, Runtime, SwiGLUSpec,
                               build_part, register_part, unregister_part)
from qorvix_b200.parts.base import Mixer
from qorvix_b200.parts.linear import Linear
from qorvix_b200.weights import TensorSource

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)


def close(got, want, dtype):
    """max |got - want| within 2e-2 (bfloat16) or 2e-5 (float32) of max |want|: the measure the
    logits comparisons use."""
    bound = (2e-5 if dtype == torch.float32 else 2e-2) * max(1.0, float(want.abs().max()))
    return float((got.double().cpu() - want).abs().max()) <= bound


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def source(tensors, dtype):
    t = {k: v.to(torch.bfloat16) for k, v in tensors.items()}
    return TensorSource(tensors=t, device=DEV, compute_dtype=dtype), {k: v.double() for k, v in t.items()}


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    rt = Runtime(DEV, dtype, 64)
    src, ref_w = source({"n.weight": 1 + 0.1 * rnd(200, seed=1)}, dtype)
    norm = build_part("norm", RMSNormSpec(200, 3e-6, "n.weight"), src, rt)
    res, delta = rnd(5, 200, seed=2).to(DEV), rnd(5, 200, seed=3).to(dtype).to(DEV)
    before = res.clone()
    out = norm.add_norm(res, delta)
    want = plain.rmsnorm(before.double().cpu() + delta.double().cpu(), ref_w["n.weight"], 3e-6)
    assert torch.allclose(out.double().cpu(), want, **tol(dtype))
    assert torch.allclose(res.double().cpu(), before.double().cpu() + delta.double().cpu(), atol=1e-6)


def test_rotary_part_tables():
    rt = Runtime(DEV, torch.float32, 300)
    sc = RopeScaling("llama3", 8.0, 1.0, 4.0, 64)
    for scaling, ref_freq in ((None, plain.plain_inv_freq(32, 5e5)), (sc, plain.llama3_inv_freq(32, 5e5, 8.0, 1.0, 4.0, 64))):
        rot = build_part("position", RotarySpec(head_dim=32, rotary_dim=32, theta=5e5, scaling=scaling), None, rt)
        assert torch.allclose(rot.inv_freq, ref_freq, rtol=1e-12, atol=0)
        ang = torch.arange(300, dtype=torch.float64)[:, None] * ref_freq[None, :]
        assert torch.allclose(rot.table()[..., 0].double().cpu(), ang.cos(), atol=1e-7)
        assert torch.allclose(rot.table()[..., 1].double().cpu(), ang.sin(), atol=1e-7)
    half = build_part("position", RotarySpec(head_dim=32, rotary_dim=16, theta=1e4), None, rt)      # partial rotation
    assert tuple(half.table().shape) == (300, 8, 2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("f", [172, 512])          # 172: plain layout; 512: gate/up interleaved and fused
def test_swiglu_part(dtype, f):
    d = 64
    rt = Runtime(DEV, dtype, 64)
    src, w = source({"g": rnd(f, d, seed=1, scale=0.2), "u": rnd(f, d, seed=2, scale=0.2), "dn": rnd(d, f, seed=3, scale=0.1)}, dtype)
    ff = build_part("feed_forward", SwiGLUSpec(d, f, "g", "u", "dn"), src, rt)
    x = rnd(37, d, seed=4).to(dtype).to(DEV)
    xd = x.double().cpu()
    want = plain.linear(plain.swiglu(plain.linear(xd, w["g"]), plain.linear(xd, w["u"])), w["dn"])
    assert torch.allclose(ff.forward(x, None).double().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_part_keeps_a_32_bit_matrix_32_bit(dtype):
    w = rnd(100, 72, seed=1, scale=0.1)
    lin = Linear(w.to(DEV))                        # stored in 32-bit: stays so, runs on the CUDA cores
    x = rnd(9, 72, seed=2).to(dtype).to(DEV)
    y = lin(x, out_dtype=dtype)
    assert lin.weight.dtype == torch.float32
    assert torch.allclose(y.double().cpu(), x.double().cpu() @ w.double().t(), **tol(dtype))


def _attention_setup(cfg, dtype, window=0):
    """An Attention part on random weights, a cache manager for it, and a way to run one step."""
    H, Hkv, hd, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.hidden_size
    rt = Runtime(DEV, dtype, 256)
    names = dict(q_proj="q", k_proj="k", v_proj="v", o_proj="o")
    # q and k small enough that scores are of order one: bfloat16 rounding of q and k then stays
    # within the comparison's bound (sharper attention is covered by the replay tests)
    qk = 1.2 / math.sqrt(d)
    tensors = {"q": rnd(H * hd, d, seed=1, scale=qk), "k": rnd(Hkv * hd, d, seed=2, scale=qk),
               "v": rnd(Hkv * hd, d, seed=3, scale=0.2), "o": rnd(d, H * hd, seed=4, scale=0.2)}
    src, w = source(tensors, dtype)
    spec = AttentionSpec(hidden_size=d, num_heads=H, num_kv_heads=Hkv, head_dim=hd, scale=1 / math.sqrt(hd),
                         position=RotarySpec(hd, hd, cfg.rope_theta, cfg.rope_scaling), window=window, **names)
    att = build_part("mixer", spec, src, rt)
    cache = CacheManager([(att.cache_spec(), None)], max_tokens=256, page_size=16, max_requests=2, device=DEV, dtype=dtype)
    return att, cache, w


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,window", [("A", 0), ("B", 0), ("C", 0), ("B", 21)])
def test_attention_part_alone_in_portions(dtype, name, window):
    cfg = TINY[name]
    att, cache, w = _attention_setup(cfg, dtype, window)
    T, d = 90, cfg.hidden_size
    x = rnd(T, d, seed=9).to(dtype)
    H, Hkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    xd = x.double()
    inv = plain.inv_freq_from_config(dict(cfg.to_dict(), rope_scaling=cfg.rope_scaling.to_dict() if cfg.rope_scaling else None))
    pos = torch.arange(T)
    qr = plain.rope(plain.linear(xd, w["q"]).reshape(T, H, hd), pos, inv)
    kr = plain.rope(plain.linear(xd, w["k"]).reshape(T, Hkv, hd), pos, inv)
    want = plain.linear(plain.attention(qr, kr, plain.linear(xd, w["v"]).reshape(T, Hkv, hd), window=window).reshape(T, H * hd), w["o"])
    builder = BatchBuilder(DEV)
    cache.admit("r")
    outs, i = [], 0
    for n in (33, 2, 1, 40, 1, 13):
        assert cache.reserve("r", n)
        segs = [dict(tokens=[0] * n, pos0=cache.length("r"), slot=cache.slot("r"), want=[], first=i == 0)]
        ctx = builder.build(segs, {0: [cache.block_table("r", 0)]}, cache.scratch_page)
        outs.append(att.forward(x[i:i + n].to(DEV), ctx, cache.layer_view(0)))
        cache.commit("r", n)
        i += n
    got = torch.cat(outs)
    assert close(got, want, dtype)


# ------------------------------------------------------------------ a toy mixer with state of its own

@dataclass(frozen=True)
class DecaySpec:
    """Toy mixer: a decaying sum per request, s <- decay * s + x W^T; the output at a token is s."""
    hidden_size: int
    decay: float
    proj: str
    kind: str = "toy_decay"

    def tensors(self):
        return {self.proj: ((self.hidden_size, self.hidden_size), "matrix")}


class DecayMixer(Mixer):
    def __init__(self, spec, source, rt):
        self.spec, self.rt = spec, rt
        self.w = source.get(spec.proj).float()

    def cache_spec(self):
        return FixedStateSpec(shape=(self.spec.hidden_size,), dtype="float32")

    def forward(self, x, ctx, cache):
        u = x.float() @ self.w.t()
        state = cache.tensor                          # [request slots + 1, hidden]
        if ctx.max_q_len == 1:                        # one token per request: all slots at once, from device data
            slots = ctx.seg_slot.long()
            s = self.spec.decay * state[slots] + u
            state[slots] = s
            return s.to(self.rt.dtype)
        out = torch.empty_like(u)
        row = 0
        for n, slot in zip(ctx.seg_len, ctx.seg_slots):
            s = state[slot].clone()
            for t in range(n):
                s = self.spec.decay * s + u[row + t]
                out[row + t] = s
            state[slot] = s
            row += n
        return out.to(self.rt.dtype)


@dataclass(frozen=True)
class ToyConfig(ModelConfig):
    vocab_size: int = 0
    hidden_size: int = 0
    intermediate_size: int = 0
    decay: float = 0.5

    @staticmethod
    def from_dict(d):
        return ToyConfig(architecture=d["architectures"][0], vocab_size=d["vocab_size"], hidden_size=d["hidden_size"],
                         intermediate_size=d["intermediate_size"], decay=d["decay"])


def toy_spec(cfg):
    d = cfg.hidden_size
    attn = AttentionSpec(hidden_size=d, num_heads=4, num_kv_heads=2, head_dim=16, scale=0.25, q_proj="l1.q", k_proj="l1.k",
                         v_proj="l1.v", o_proj="l1.o", position=RotarySpec(16, 16, 10000.0))
    layers = [
        LayerSpec(mixer=DecaySpec(d, cfg.decay, "l0.proj"), feed_forward=SwiGLUSpec(d, cfg.intermediate_size, "l0.g", "l0.u", "l0.d"),
                  mixer_norm=RMSNormSpec(d, 1e-5, "l0.n1"), ffn_norm=RMSNormSpec(d, 1e-5, "l0.n2")),
        LayerSpec(mixer=attn, feed_forward=None, mixer_norm=RMSNormSpec(d, 1e-5, "l1.n1"), ffn_norm=None),
    ]
    # the order is data: the stateful layer runs, then attention, then the stateful layer's twin is not
    # needed: a list may also name a layer twice, which test_layer_order_may_repeat checks
    return ModelSpec(architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=d, embedding="emb", layers=layers,
                     final_norm=RMSNormSpec(d, 1e-5, "fn"), lm_head=None, order=[0, 1], max_position=256)


def toy_plain(cfg, w, tokens):
    """The toy model on one whole sequence, in float64, from the plain parts."""
    w = {k: v.double() for k, v in w.items()}
    x = w["emb"][torch.tensor(tokens)]
    T = len(tokens)
    h = plain.rmsnorm(x, w["l0.n1"], 1e-5)
    u = h @ w["l0.proj"].t()
    s = torch.zeros(cfg.hidden_size, dtype=torch.float64)
    mixed = []
    for t in range(T):
        s = cfg.decay * s + u[t]
        mixed.append(s)
    x = x + torch.stack(mixed)
    h = plain.rmsnorm(x, w["l0.n2"], 1e-5)
    x = x + plain.linear(plain.swiglu(plain.linear(h, w["l0.g"]), plain.linear(h, w["l0.u"])), w["l0.d"])
    h = plain.rmsnorm(x, w["l1.n1"], 1e-5)
    inv = plain.plain_inv_freq(16, 10000.0)
    q = plain.rope(plain.linear(h, w["l1.q"]).reshape(T, 4, 16), torch.arange(T), inv)
    k = plain.rope(plain.linear(h, w["l1.k"]).reshape(T, 2, 16), torch.arange(T), inv)
    a = plain.attention(q * 4 * 0.25, k, plain.linear(h, w["l1.v"]).reshape(T, 2, 16))   # scale 0.25 = 1/sqrt(16)
    x = x + plain.linear(a.reshape(T, 64), w["l1.o"])
    return plain.linear(plain.rmsnorm(x, w["fn"], 1e-5), w["emb"])


@pytest.fixture
def toy():
    register_part("mixer", "toy_decay", DecayMixer)
    register_architecture("ToyDecayLM", ToyConfig.from_dict, toy_spec)
    cfg = ToyConfig(architecture="ToyDecayLM", vocab_size=97, hidden_size=64, intermediate_size=80, decay=0.6)
    spec = toy_spec(cfg)
    g = torch.Generator().manual_seed(5)
    tensors = {}
    for name, (shape, kind) in spec.tensor_table().items():
        t = torch.randn(shape, generator=g)
        tensors[name] = (1 + 0.1 * t if kind == "norm" else 0.15 * t).to(torch.bfloat16)
    yield cfg, tensors
    unregister_architecture("ToyDecayLM")
    unregister_part("mixer", "toy_decay")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(toy, dtype):
    cfg, tensors = toy
    r = ModelRunner(config=cfg, tensors=tensors, dtype=dtype, max_tokens=256, max_requests=3)
    kinds = [type(g.spec).__name__ for g in r.cache.groups]
    assert sorted(kinds) == ["FixedStateSpec", "PagedKVSpec"]          # a state group beside the paged one
    a, b = random_tokens(97, 40, 1), random_tokens(97, 25, 2)
    wf = {k: v.float() for k, v in tensors.items()}
    ref_a, ref_b = toy_plain(cfg, wf, a), toy_plain(cfg, wf, b)
    # whole, then in portions beside another request, the last tokens one by one (captured decode steps)
    whole = r.step([StepEntry("w", a, list(range(40)))], end=["w"])
    assert_close_logits(whole, ref_a, dtype, "toy whole")
    got_a, got_b = [], []
    got_a.append(r.step([StepEntry("a", a[:17], list(range(17)))]))
    out = r.step([StepEntry("a", a[17:30], list(range(13))), StepEntry("b", b[:20], list(range(20)))])
    got_a.append(out[:13]); got_b.append(out[13:])
    for i in range(5):
        out = r.step([StepEntry("a", [a[30 + i]], [0]), StepEntry("b", [b[20 + i]], [0])])
        got_a.append(out[:1]); got_b.append(out[1:])
    for i in range(35, 40):
        got_a.append(r.step([StepEntry("a", [a[i]], [0])]))
    assert_close_logits(torch.cat(got_a), ref_a, dtype, "toy request a in portions")
    assert_close_logits(torch.cat(got_b), ref_b, dtype, "toy request b in portions")
    # a new request in a used slot starts from a zero state
    r.release("a"); r.release("b")
    again = r.step([StepEntry("c", b, list(range(25)))], end=["c"])
    assert_close_logits(again, ref_b, dtype, "toy state slot is zeroed on admission")


def test_layer_order_may_repeat_and_a_layer_may_read_anothers_cache():
    """The order of execution is a list: [0, 1, 1] runs layer 1 twice over the same weights; layer 2
    keeps no keys of its own and reads layer 0's."""
    d, H, hd = 64, 4, 16
    def att(p, kv_from=None):
        return AttentionSpec(hidden_size=d, num_heads=H, num_kv_heads=2, head_dim=hd, scale=0.25, q_proj=p + "q", k_proj=p + "k",
                             v_proj=p + "v", o_proj=p + "o", position=RotarySpec(hd, hd, 10000.0), kv_from=kv_from)
    def layer(p, kv_from=None, ffn=True):
        return LayerSpec(mixer=att(p, kv_from), feed_forward=SwiGLUSpec(d, 96, p + "g", p + "u", p + "d") if ffn else None,
                         mixer_norm=RMSNormSpec(d, 1e-5, p + "n1"), ffn_norm=RMSNormSpec(d, 1e-5, p + "n2") if ffn else None)
    def spec_of(cfg):
        return ModelSpec(architecture="ToyOrderLM", vocab_size=50, hidden_size=d, embedding="emb",
                         layers=[layer("a."), layer("b."), layer("c.", kv_from=0, ffn=False)], final_norm=RMSNormSpec(d, 1e-5, "fn"),
                         lm_head=None, order=[0, 1, 1, 2], max_position=128)
    @dataclass(frozen=True)
    class Cfg(ModelConfig):
        pass
    register_architecture("ToyOrderLM", lambda raw: Cfg("ToyOrderLM"), spec_of)
    try:
        spec = spec_of(None)
        assert "c.k" not in spec.tensor_table() and "c.q" in spec.tensor_table()
        g = torch.Generator().manual_seed(3)
        tensors = {n: ((1 + 0.1 * torch.randn(s, generator=g)) if k == "norm" else 0.2 * torch.randn(s, generator=g)).to(torch.bfloat16)
                   for n, (s, k) in spec.tensor_table().items()}
        r = ModelRunner(config=Cfg("ToyOrderLM"), tensors=tensors, dtype="float32", max_tokens=128, max_requests=2)
        assert len(r.cache.groups) == 1 and r.cache.groups[0].layers == [0, 1, 2]      # one cache per run: a, b, b again
        toks = random_tokens(50, 30, 4)
        whole = r.step([StepEntry("w", toks, list(range(30)))], end=["w"])
        parts = [r.step([StepEntry("p", toks[:11], list(range(11)))]), r.step([StepEntry("p", toks[11:29], list(range(18)))]),
                 r.step([StepEntry("p", toks[29:], [0])])]
        assert torch.equal(torch.cat(parts), whole)
        # plain: the same order by hand
        w = {k: v.double() for k, v in tensors.items()}
        x = w["emb"][torch.tensor(toks)]
        T = 30
        inv = plain.plain_inv_freq(hd, 10000.0)
        def qkv(h, p):
            q = plain.rope(plain.linear(h, w[p + "q"]).reshape(T, H, hd), torch.arange(T), inv)
            k = plain.rope(plain.linear(h, w[p + "k"]).reshape(T, 2, hd), torch.arange(T), inv) if p + "k" in w else None
            v = plain.linear(h, w[p + "v"]).reshape(T, 2, hd) if p + "v" in w else None
            return q, k, v
        kv0 = None
        for p in ("a.", "b.", "b.", "c."):
            h = plain.rmsnorm(x, w[p + "n1"], 1e-5)
            q, k, v = qkv(h, p)
            if p == "a.":
                kv0 = (k, v)
            if p == "c.":
                k, v = kv0
            x = x + plain.linear(plain.attention(q, k, v).reshape(T, H * hd), w[p + "o"])
            if p + "g" in w:
                h = plain.rmsnorm(x, w[p + "n2"], 1e-5)
                x = x + plain.linear(plain.swiglu(plain.linear(h, w[p + "g"]), plain.linear(h, w[p + "u"])), w[p + "d"])
        ref = plain.linear(plain.rmsnorm(x, w["fn"], 1e-5), w["emb"])
        assert_close_logits(whole, ref, "float32", "repeated and shared layers")
    finally:
        unregister_architecture("ToyOrderLM")
