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
