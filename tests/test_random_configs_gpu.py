"""Randomly drawn configurations (seeded): head counts and groups, head sizes in steps of 8 and 16 up to
256, widths and vocabularies that are no power of two, with and without llama3 scaling and tied output:
whole prompts and prompts in random portions against the plain implementation, in both precisions.
Sizes the tensor-core kernels refuse must come out right through the general kernels, never wrong."""
import random

import pytest
import torch

from helpers import PlainModel, assert_close_logits, make_model_dir, random_tokens
from qorvix_b200 import LlamaConfig, ModelRunner, StepEntry
from qorvix_b200.config import RopeScaling
from qorvix_b200.csrc import ops

pytestmark = pytest.mark.gpu


def draw(rng):
    heads = rng.choice([1, 2, 3, 4, 5, 8, 12])
    kv = rng.choice([k for k in (1, 2, 3, 4, 5, 8, 12) if heads % k == 0])
    sc = RopeScaling("llama3", rng.choice([2.0, 8.0]), 1.0, rng.choice([2.0, 4.0]), rng.choice([32, 64])) if rng.random() < 0.5 else None
    return LlamaConfig(architecture="LlamaForCausalLM", vocab_size=rng.choice([17, 100, 331, 1000]),
                       hidden_size=rng.choice([48, 72, 100, 130, 256, 200]), intermediate_size=rng.choice([33, 64, 100, 172, 512, 48]),
                       num_hidden_layers=rng.choice([1, 2, 3]), num_attention_heads=heads, num_key_value_heads=kv,
                       head_dim=rng.choice([8, 16, 24, 32, 40, 64, 80, 96, 128, 256]), max_position_embeddings=512,
                       rms_norm_eps=rng.choice([1e-5, 1e-6]), rope_theta=rng.choice([1e4, 5e5]), rope_scaling=sc,
                       tie_word_embeddings=rng.random() < 0.5)


@pytest.mark.parametrize("seed", range(8))
def test_random_configuration(seed):
    rng = random.Random(1000 + seed)
    cfg = draw(rng)
    sharpen = rng.choice([1.0, 4.0])
    d = make_model_dir(cfg, seed=seed, sharpen=sharpen)
    pm = PlainModel(d)
    n = rng.choice([5, 40, 97, 150])
    toks = random_tokens(cfg.vocab_size, n, seed)
    ref = pm.logits(toks)
    for dtype in ("float32", "bfloat16"):
        r = ModelRunner(d, dtype=dtype, max_tokens=256, max_requests=3)
        whole = r.step([StepEntry("w", toks, list(range(n)))], end=["w"])
        outs, i = [], 0
        while i < n:
            c = min(n - i, rng.choice([1, 1, 2, 7, 16, 33, 64]))
            outs.append(r.step([StepEntry("p", toks[i:i + c], list(range(c)))]))
            i += c
        r.step([], end=["p"])
        torch.cuda.synchronize()
        ops.check_kernel_errors()
        assert_close_logits(whole, ref, dtype, f"{cfg} {dtype}: whole prompt", sharp=sharpen > 1)
        assert_close_logits(torch.cat(outs), ref, dtype, f"{cfg} {dtype}: portions", sharp=sharpen > 1)
        r.cache.check_invariants()
