"""Host-side rules that pick kernels and orders: no GPU needed."""
from qorvix_b200 import StepEntry
from qorvix_b200.csrc import ops
from qorvix_b200.engine.runner import single_token_entries_first


def test_single_token_entries_run_first_and_rows_map_back():
    e = [StepEntry("p1", [1, 2, 3], [0, 2]), StepEntry("d1", [4], [0]), StepEntry("p2", [5, 6], []),
         StepEntry("d2", [7], [0]), StepEntry("d3", [8], [])]
    order, back = single_token_entries_first(e)
    assert order == [1, 3, 4, 0, 2]                      # decoded tokens first, each kind in the caller's order
    # the step's output rows are d1, d2, p1[0], p1[2]; the caller wants p1[0], p1[2], d1, d2
    assert back == [2, 3, 0, 1]
    # nothing to undo when the caller's order is already that
    assert single_token_entries_first([e[1], e[3], e[0]]) == ([0, 1, 2], None)
    assert single_token_entries_first([]) == ([], None)


def test_decode_attention_slices():
    # few (token, kv head) pairs: the slices fill one wave of 296 CTAs, at least 256 keys each
    assert ops.decode_variant(8, 8) == 0 and ops.decode_splits(8, 8, 1024) == 4
    assert ops.decode_splits(8, 8, 8192) == 4
    assert ops.decode_splits(8, 8, 300) == 1
    # more pairs than one wave holds: the count whose waves take the least time ...
    assert ops.decode_splits(8, 40, 2048) == 3
    assert ops.decode_splits(64, 8, 8192) == 4
    assert ops.decode_splits(64, 8, 1024) == 1
    # ... but only where the context is known; a captured step keeps one wave
    assert ops.decode_splits(64, 8, 8192, known=False) == 1
    assert ops.decode_splits(8, 8, 8192, known=False) == 4
    # very few pairs take the per-thread-load kernel with about three CTAs per SM
    assert ops.decode_variant(1, 8) == 1 and 1 <= ops.decode_splits(1, 8, 1024) <= 16
    for T in (1, 3, 8, 17, 64):
        for hkv in (1, 2, 8, 40):
            for ctx in (1, 63, 64, 1000, 8192, 100000):
                for known in (True, False):
                    assert 1 <= ops.decode_splits(T, hkv, ctx, known=known) <= 16


def test_switches(monkeypatch):
    monkeypatch.delenv("QORVIX_FOLDED_NORM", raising=False)
    monkeypatch.delenv("QORVIX_FUSED_ROPE", raising=False)
    assert ops.folded_norm_enabled(1) and ops.folded_norm_enabled(16) and not ops.folded_norm_enabled(17)
    assert ops.fused_rope_enabled(65) and not ops.fused_rope_enabled(64)
    monkeypatch.setenv("QORVIX_FOLDED_NORM", "0")
    assert not ops.folded_norm_enabled(8)
    monkeypatch.setenv("QORVIX_FOLDED_NORM", "64")
    assert ops.folded_norm_enabled(64) and not ops.folded_norm_enabled(65)
    monkeypatch.setenv("QORVIX_FUSED_ROPE", "0")
    assert not ops.fused_rope_enabled(2048)


def _stub_rmsnorm(calls, name):
    """An RMSNorm object without a device: add_norm only records what it is given."""
    import torch
    from qorvix_b200.parts.rmsnorm import RMSNorm
    n = object.__new__(RMSNorm)
    n.size, n.eps, n.weight = 8, 1e-5, torch.ones(8)

    def add_norm(residual, delta, rows=None):
        calls.append((name, "add_norm", type(delta).__name__))
        return torch.zeros(residual.shape[0], 8)
    n.add_norm = add_norm
    return n


def test_pre_norm_block_hands_a_prepared_norm_input_only_to_parts_that_take_it(monkeypatch):
    """The routing of PreNormed between the parts of a block, with stub parts (no kernels run)."""
    import torch
    from qorvix_b200.parts.base import PreNormed
    from qorvix_b200.parts.block import PreNormBlock
    monkeypatch.delenv("QORVIX_FOLDED_NORM", raising=False)
    calls = []
    n1, n2, n_after = _stub_rmsnorm(calls, "n1"), _stub_rmsnorm(calls, "n2"), _stub_rmsnorm(calls, "after")

    class FoldingMixer:
        folds_norms = True

        def forward(self, x, ctx, cache, residual=None, next_norm=None):
            calls.append(("mixer", type(x).__name__, next_norm))
            return PreNormed(scaled=torch.zeros(2, 8), stats=torch.zeros(1, 64), norm=next_norm, residual=residual)

    class FoldingFfn:
        folds_norms = True

        def forward(self, x, ctx, residual=None, next_norm=None):
            calls.append(("ffn", type(x).__name__, next_norm))
            return PreNormed(scaled=torch.zeros(2, 8), stats=torch.zeros(1, 64), norm=next_norm, residual=residual)

    class PlainFfn:
        def forward(self, x, ctx):
            calls.append(("plain_ffn", type(x).__name__, None))
            return torch.zeros(2, 8)

    class Ctx:
        next_norm = None

    def block(mixer, ffn):
        b = object.__new__(PreNormBlock)
        b.mixer_norm, b.mixer, b.ffn_norm, b.feed_forward = n1, mixer, n2, ffn
        return b

    residual = torch.zeros(2, 8)
    ctx = Ctx()
    ctx.next_norm = n_after
    # both parts fold: the mixer prepares the ffn norm's input, the ffn takes it as it is and prepares the next block's
    _, pending = block(FoldingMixer(), FoldingFfn()).forward(residual, None, ctx, None)
    assert calls == [("n1", "add_norm", "NoneType"), ("mixer", "Tensor", n2), ("ffn", "PreNormed", n_after)]
    assert isinstance(pending, PreNormed) and pending.norm is n_after
    # a block that gets a PreNormed made for its first norm hands it to a folding mixer without running the norm
    calls.clear()
    block(FoldingMixer(), FoldingFfn()).forward(residual, PreNormed(torch.zeros(2, 8), torch.zeros(1, 64), n1, residual), ctx, None)
    assert calls[0] == ("mixer", "PreNormed", n2)
    # a feed-forward that does not fold gets normed rows: its norm is run on the PreNormed (the stream is complete)
    calls.clear()
    _, pending = block(FoldingMixer(), PlainFfn()).forward(residual, None, ctx, None)
    assert calls == [("n1", "add_norm", "NoneType"), ("mixer", "Tensor", n2), ("n2", "add_norm", "PreNormed"),
                     ("plain_ffn", "Tensor", None)]
    assert isinstance(pending, torch.Tensor)
    # many tokens: nothing is folded, the parts are called the plain way (no keywords)
    calls.clear()
    big = torch.zeros(100, 8)

    class CountingMixer:
        folds_norms = True

        def forward(self, x, ctx, cache, **kw):
            calls.append(("mixer_kw", sorted(kw)))
            return torch.zeros(100, 8)

    block(CountingMixer(), PlainFfn()).forward(big, None, ctx, None)
    assert ("mixer_kw", []) in calls
    # no folding norm after the block (another kind of norm, or the final norm): the last part is told so
    calls.clear()
    ctx.next_norm = object()
    block(FoldingMixer(), FoldingFfn()).forward(residual, None, ctx, None)
    assert calls[-1] == ("ffn", "PreNormed", None)
    # a norm class the package has never seen opts in by declaring the capability, nothing else
    class ForeignNorm:
        folds_into_products = True
        size, eps = 8, 1e-6

        def scale_weight(self):
            return torch.ones(8)

    calls.clear()
    ctx.next_norm = ForeignNorm()
    block(FoldingMixer(), FoldingFfn()).forward(residual, None, ctx, None)
    assert calls[-1] == ("ffn", "PreNormed", ctx.next_norm)
