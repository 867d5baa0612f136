"""Configuration, registry and weight loading (no GPU)."""
import json

import pytest
import torch

from helpers import TINY_A, TINY_B, make_model_dir
from qorvix_b200.config import (ConfigError, LlamaConfig, load_config, lookup_architecture,
                                register_architecture, registered_architectures, unregister_architecture)
from qorvix_b200.weights import (Checkpoint, TensorSource, WeightError, random_tensors, storage_dtype,
                                 write_random_model, write_safetensors)
import plain_llama as plain


def test_llama_config_from_own_keys(tmp_path):
    raw = TINY_B.to_dict()
    (tmp_path / "config.json").write_text(json.dumps(raw))
    cfg = load_config(tmp_path)
    assert cfg == TINY_B
    assert cfg.rope_scaling.factor == 8.0 and cfg.rope_scaling.original_max_position_embeddings == 64
    assert cfg.tie_word_embeddings and cfg.head_dim == 32


def test_config_defaults_and_head_dim_rule():
    raw = dict(architectures=["LlamaForCausalLM"], vocab_size=100, hidden_size=96, intermediate_size=64,
               num_hidden_layers=1, num_attention_heads=4)
    cfg = LlamaConfig.from_dict(raw)
    assert cfg.num_key_value_heads == 4 and cfg.head_dim == 24            # MHA default, hidden / heads
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 10000.0 and cfg.rope_scaling is None
    cfg = LlamaConfig.from_dict(dict(raw, head_dim=32))
    assert cfg.head_dim == 32                                             # head_dim is its own key


@pytest.mark.parametrize("change, word", [
    (dict(vocab_size=None), "vocab_size"), (dict(num_key_value_heads=3), "num_key_value_heads"),
    (dict(hidden_act="gelu"), "hidden_act"), (dict(head_dim=15), "head_dim"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 2.0}), "yarn"),
    (dict(rope_scaling={"rope_type": "llama3", "factor": 2.0}), "low_freq_factor"),
    (dict(num_hidden_layers=0), "num_hidden_layers")])
def test_config_errors_name_the_key(change, word):
    raw = dict(TINY_A.to_dict(), **change)
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(raw)
    assert word in str(e.value)


def test_registry_unknown_and_duplicate(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_A.to_dict(), architectures=["MysteryForCausalLM"])))
    with pytest.raises(ConfigError) as e:
        load_config(tmp_path)
    assert "MysteryForCausalLM" in str(e.value) and "LlamaForCausalLM" in str(e.value)
    with pytest.raises(ValueError):
        register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, lambda c: None)
    register_architecture("ToyArch", LlamaConfig.from_dict, lambda c: None)
    assert "ToyArch" in registered_architectures()
    unregister_architecture("ToyArch")
    assert "ToyArch" not in registered_architectures()


def test_random_model_folder_round_trip(tmp_path):
    d = write_random_model(tmp_path / "m", TINY_A, seed=3)
    cfg2 = load_config(d)
    assert cfg2 == TINY_A
    ck = Checkpoint(d)
    spec = lookup_architecture(cfg2.architecture).build_spec(cfg2)
    assert set(ck.names()) == set(spec.expected_shapes())
    assert ck.dtype("model.layers.0.mlp.gate_proj.weight") == torch.bfloat16
    # our reader and the plain reader see the same bytes
    _, pw = plain.read_model_dir(d)
    for n in ck.names():
        assert torch.equal(ck.tensor(n).float(), pw[n].float())
    # same seed, same tensors; another seed, other tensors; statistics as documented
    a = dict(random_tensors(TINY_A, 3))
    b = dict(random_tensors(TINY_A, 4))
    assert torch.equal(a["lm_head.weight"], ck.tensor("lm_head.weight"))
    assert not torch.equal(a["lm_head.weight"], b["lm_head.weight"])
    assert abs(float(a["model.embed_tokens.weight"].float().std()) - 0.02) < 2e-3
    assert abs(float(a["model.norm.weight"].float().mean()) - 1.0) < 0.05


def test_tied_model_has_no_head_tensor():
    names = set(n for n, _ in random_tensors(TINY_B, 1))
    assert "lm_head.weight" not in names and "model.embed_tokens.weight" in names


def test_storage_dtype_rule():
    assert storage_dtype(torch.bfloat16, torch.bfloat16) == torch.bfloat16
    assert storage_dtype(torch.float16, torch.bfloat16) == torch.bfloat16
    assert storage_dtype(torch.float32, torch.bfloat16) == torch.float32      # stored in 32-bit stays so
    assert storage_dtype(torch.bfloat16, torch.float32) == torch.float32
    assert storage_dtype(torch.int64, torch.bfloat16) == torch.int32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    spec = lookup_architecture(TINY_A.architecture).build_spec(TINY_A)
    tensors = dict(random_tensors(TINY_A, 2))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(32, 64, dtype=torch.bfloat16)
    (tmp_path / "config.json").write_text(json.dumps(TINY_A.to_dict()))
    write_safetensors(tmp_path / "model.safetensors", tensors.items())
    src = TensorSource(checkpoint=Checkpoint(tmp_path), device="cpu", where="model.safetensors")
    with pytest.raises(WeightError) as e:
        src.check(spec.expected_shapes(), spec.optional_tensors)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert [w[0] for w in err.wrong_shape] == ["model.layers.0.self_attn.k_proj.weight"]
    msg = str(err)
    for word in ("missing", "unexpected", "wrong shapes", "stored [32, 64], expected [64, 64]", "up_proj", "q_proj.bias"):
        assert word in msg


def test_missing_file_and_broken_file(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A.to_dict()))
    with pytest.raises(WeightError) as e:
        Checkpoint(tmp_path)
    assert "model.safetensors" in str(e.value)
    (tmp_path / "model.safetensors").write_bytes(b"\xff" * 16)
    with pytest.raises(WeightError):
        Checkpoint(tmp_path)


def test_untied_model_needs_its_head(tmp_path):
    tensors = dict(random_tensors(TINY_A, 2))
    del tensors["lm_head.weight"]
    spec = lookup_architecture(TINY_A.architecture).build_spec(TINY_A)
    with pytest.raises(WeightError) as e:
        TensorSource(tensors=tensors, device="cpu").check(spec.expected_shapes(), spec.optional_tensors)
    assert e.value.missing == ["lm_head.weight"]
    # a tied model may carry a copy of the head; it is tolerated
    tied = dict(random_tensors(TINY_B, 2))
    tied["lm_head.weight"] = tied["model.embed_tokens.weight"].clone()
    spec_b = lookup_architecture(TINY_B.architecture).build_spec(TINY_B)
    TensorSource(tensors=tied, device="cpu").check(spec_b.expected_shapes(), spec_b.optional_tensors)


def test_engine_refuses_to_run_without_cuda():
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from qorvix_b200 import ModelRunner
    with pytest.raises(RuntimeError) as e:
        ModelRunner(config=TINY_A, tensors=dict(random_tensors(TINY_A, 1)), dtype="float32")
    assert "no CPU path" in str(e.value)
