#!/usr/bin/env python3
"""Makes tests/golden/*.npz: logits of the reference's own CPU TextModel on tiny random models.

Run once, by hand, on a machine that has the reference sources:

    python tests/golden/make_golden.py /path/to/reference

It compiles the reference's unmodified CPU model (runtime/src/text_model.cpp and what it
needs) together with a small driver written here, feeds it weights drawn from
numpy.random.RandomState(seed) (a generator whose stream is frozen across numpy versions),
runs TextModel::forward(token, pos) position by position and stores tokens and logits.
`tests/test_plain_reference.py` regenerates the same weights from the seed and compares the
plain implementation with the stored logits.  Build products go to a temporary folder.

Two models, because the reference fixes head_dim = hidden/heads and has no rope scaling:
  golden_a: 2 layers, hidden 64, 4 heads, 4 kv heads, ffn 172, vocab 256, theta 1e4, eps 1e-5, untied
  golden_b: 3 layers, hidden 192, 6 heads, 2 kv heads, ffn 512, vocab 384, theta 5e5, eps 1e-6, tied
"""
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent

MODELS = {
    "golden_a": dict(seed=11, layers=2, hidden=64, heads=4, kv_heads=4, ffn=172, vocab=256,
                     theta=10000.0, eps=1e-5, tied=False, n_tokens=12),
    "golden_b": dict(seed=12, layers=3, hidden=192, heads=6, kv_heads=2, ffn=512, vocab=384,
                     theta=500000.0, eps=1e-6, tied=True, n_tokens=20),
}

DRIVER = r"""
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <vector>
#include "qorvix/runtime/text_model.hpp"
using namespace qorvix::runtime;
static std::vector<float> take(std::ifstream& f, size_t n) {
  std::vector<float> v(n);
  f.read(reinterpret_cast<char*>(v.data()), n * sizeof(float));
  if (!f) { std::cerr << "short weight file\n"; std::exit(2); }
  return v;
}
int main(int argc, char** argv) {
  // argv: weights.bin out.bin layers hidden heads kv_heads ffn vocab theta eps tied n_tokens tok...
  std::ifstream f(argv[1], std::ios::binary);
  ModelConfig c;
  c.architecture = "llama";
  c.blockCount = std::atoi(argv[3]);
  c.embeddingLength = std::atoi(argv[4]);
  c.headCount = std::atoi(argv[5]);
  c.headCountKv = std::atoi(argv[6]);
  c.feedForwardLength = std::atoi(argv[7]);
  c.vocabSize = std::atoi(argv[8]);
  c.ropeFreqBase = std::atof(argv[9]);
  c.normEpsilon = std::atof(argv[10]);
  const bool tied = std::atoi(argv[11]) != 0;
  const int n = std::atoi(argv[12]);
  c.contextLength = 512;
  const int d = c.embeddingLength, kv = c.kvDim(), ffn = c.feedForwardLength, V = c.vocabSize;
  Weights w;
  w.tokenEmbd = WeightMat::f32(take(f, (size_t)V * d), V, d);
  for (unsigned l = 0; l < c.blockCount; ++l) {
    LayerWeights L;
    L.attnNorm = take(f, d);
    L.wq = WeightMat::f32(take(f, (size_t)d * d), d, d);
    L.wk = WeightMat::f32(take(f, (size_t)kv * d), kv, d);
    L.wv = WeightMat::f32(take(f, (size_t)kv * d), kv, d);
    L.wo = WeightMat::f32(take(f, (size_t)d * d), d, d);
    L.ffnNorm = take(f, d);
    L.ffnGate = WeightMat::f32(take(f, (size_t)ffn * d), ffn, d);
    L.ffnUp = WeightMat::f32(take(f, (size_t)ffn * d), ffn, d);
    L.ffnDown = WeightMat::f32(take(f, (size_t)d * ffn), d, ffn);
    w.layers.push_back(std::move(L));
  }
  w.outputNorm = take(f, d);
  if (!tied) w.output = WeightMat::f32(take(f, (size_t)V * d), V, d);
  TextModel model(c, std::move(w), 512, 1);
  std::ofstream out(argv[2], std::ios::binary);
  for (int i = 0; i < n; ++i) {
    const auto& logits = model.forward(std::atoi(argv[13 + i]), i);
    out.write(reinterpret_cast<const char*>(logits.data()), logits.size() * sizeof(float));
  }
  return 0;
}
"""


def golden_weights(m: dict) -> dict:
    """HF-named fp32 weights, drawn in a fixed order from RandomState(seed)."""
    rs = np.random.RandomState(m["seed"])
    d, H, Hkv, f, V = m["hidden"], m["heads"], m["kv_heads"], m["ffn"], m["vocab"]
    hd = d // H

    def mat(r, c):
        return (rs.standard_normal((r, c)) * 0.08).astype(np.float32)

    def vec(n):
        return (1.0 + 0.1 * rs.standard_normal(n)).astype(np.float32)

    w = {"model.embed_tokens.weight": (rs.standard_normal((V, d))).astype(np.float32)}
    for l in range(m["layers"]):
        p = f"model.layers.{l}."
        w[p + "input_layernorm.weight"] = vec(d)
        w[p + "self_attn.q_proj.weight"] = mat(H * hd, d) * 4.0
        w[p + "self_attn.k_proj.weight"] = mat(Hkv * hd, d) * 4.0
        w[p + "self_attn.v_proj.weight"] = mat(Hkv * hd, d)
        w[p + "self_attn.o_proj.weight"] = mat(d, H * hd)
        w[p + "post_attention_layernorm.weight"] = vec(d)
        w[p + "mlp.gate_proj.weight"] = mat(f, d)
        w[p + "mlp.up_proj.weight"] = mat(f, d)
        w[p + "mlp.down_proj.weight"] = mat(d, f)
    w["model.norm.weight"] = vec(d)
    if not m["tied"]:
        w["lm_head.weight"] = mat(V, d)
    return w


def golden_tokens(m: dict) -> list:
    rs = np.random.RandomState(m["seed"] + 1000)
    return [int(t) for t in rs.randint(0, m["vocab"], size=m["n_tokens"])]


def golden_config(m: dict) -> dict:
    return {
        "architectures": ["LlamaForCausalLM"], "num_hidden_layers": m["layers"],
        "hidden_size": m["hidden"], "num_attention_heads": m["heads"],
        "num_key_value_heads": m["kv_heads"], "intermediate_size": m["ffn"],
        "vocab_size": m["vocab"], "rope_theta": m["theta"], "rms_norm_eps": m["eps"],
        "tie_word_embeddings": m["tied"], "max_position_embeddings": 512, "hidden_act": "silu",
    }


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/reference")
    ref = Path(sys.argv[1])
    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        (tmp / "driver.cpp").write_text(DRIVER)
        srcs = [ref / "runtime/src" / (n + ".cpp") for n in
                ("text_model", "ops", "weights", "model_config", "qmatmul", "dequant", "cpu_features")]
        srcs += [ref / "memory/src/kv_cache.cpp"]
        srcs += [ref / "gguf/src" / (n + ".cpp") for n in ("gguf_file", "gguf_types", "mapped_file")]
        exe = tmp / "ref_textmodel"
        cmd = ["g++", "-std=c++23", "-O1", f"-I{ref}/runtime/include", f"-I{ref}/memory/include",
               f"-I{ref}/gguf/include", f"-I{ref}/tokenizer/include", str(tmp / "driver.cpp"),
               *map(str, srcs), "-o", str(exe)]
        subprocess.run(cmd, check=True)
        for name, m in MODELS.items():
            w = golden_weights(m)
            with open(tmp / "w.bin", "wb") as fh:
                for t in w.values():  # insertion order = the driver's reading order
                    fh.write(np.ascontiguousarray(t, dtype=np.float32).tobytes())
            toks = golden_tokens(m)
            args = [str(exe), str(tmp / "w.bin"), str(tmp / "out.bin"), m["layers"], m["hidden"],
                    m["heads"], m["kv_heads"], m["ffn"], m["vocab"], m["theta"], m["eps"],
                    int(m["tied"]), len(toks), *toks]
            subprocess.run([str(a) for a in args], check=True)
            logits = np.fromfile(tmp / "out.bin", dtype=np.float32).reshape(len(toks), m["vocab"])
            np.savez_compressed(HERE / f"{name}.npz", tokens=np.array(toks, dtype=np.int32),
                                logits=logits)
            print(name, logits.shape, float(np.abs(logits).max()))


if __name__ == "__main__":
    main()
