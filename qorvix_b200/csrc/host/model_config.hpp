// The typed configuration of the native host code, read from the architecture's own config.json
// keys, and the registry from an architecture's name to what builds its model description.
// Same fields, defaults and rules as the Python side (config/model_config.py), which follow the
// reference's ModelConfig (runtime/include/qorvix/runtime/model_config.hpp:25-57; valid() :52-56);
// the reference maps an architecture string to a family the same way and rejects the others with
// a message that lists what it knows (runtime/src/model_config.cpp:20-38, 68-71).
#pragma once
#include <cmath>
#include <functional>
#include <map>
#include <string>
#include <vector>

#include "json.hpp"

namespace qv {

struct ConfigError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

struct RopeScaling {
  bool present = false;
  std::string rope_type;
  double factor = 1.0, low_freq_factor = 1.0, high_freq_factor = 4.0;
  long long original_max_position_embeddings = 0;
};

struct LlamaConfig {
  std::string architecture;
  long long vocab_size = 0, hidden_size = 0, intermediate_size = 0, num_hidden_layers = 0, num_attention_heads = 0,
            num_key_value_heads = 0, head_dim = 0, max_position_embeddings = 0;
  double rms_norm_eps = 1e-5, rope_theta = 10000.0;
  RopeScaling rope_scaling;
  bool tie_word_embeddings = false;
  std::string hidden_act = "silu";
  std::vector<long long> eos_token_ids;
};

namespace detail {
inline long long require_int(const Json& j, const char* key) {
  const Json* v = j.find(key);
  if (!v || v->is_null()) throw ConfigError(std::string("config.json: required key '") + key + "' is missing");
  if (v->kind != Json::Number || std::floor(v->num) != v->num)
    throw ConfigError(std::string("config.json: '") + key + "' must be an integer");
  return (long long)v->num;
}
inline double require_num(const Json& j, const char* key, const char* where) {
  const Json* v = j.find(key);
  if (!v || v->kind != Json::Number) throw ConfigError(std::string("config.json: ") + where + " needs a number '" + key + "'");
  return v->num;
}
inline double opt_num(const Json& j, const char* key, double def) {
  const Json* v = j.find(key);
  return (v && v->kind == Json::Number) ? v->num : def;
}
}  // namespace detail

inline std::string architecture_of(const Json& j) {
  const Json* a = j.find("architectures");
  if (!a || a->kind != Json::Array || a->arr.empty() || a->arr[0].kind != Json::String)
    throw ConfigError("config.json: 'architectures' must be a list that names the model's architecture");
  return a->arr[0].str;
}

inline LlamaConfig llama_config_from_json(const Json& j) {
  using namespace detail;
  LlamaConfig c;
  c.architecture = architecture_of(j);
  c.num_attention_heads = require_int(j, "num_attention_heads");
  c.hidden_size = require_int(j, "hidden_size");
  c.vocab_size = require_int(j, "vocab_size");
  c.intermediate_size = require_int(j, "intermediate_size");
  c.num_hidden_layers = require_int(j, "num_hidden_layers");
  c.num_key_value_heads = j.has("num_key_value_heads") ? require_int(j, "num_key_value_heads") : c.num_attention_heads;
  if (j.has("head_dim")) c.head_dim = require_int(j, "head_dim");
  else {
    if (c.num_attention_heads <= 0 || c.hidden_size % c.num_attention_heads)
      throw ConfigError("config.json: hidden_size " + std::to_string(c.hidden_size) + " is not divisible by num_attention_heads " +
                        std::to_string(c.num_attention_heads) + " and no 'head_dim' is given");
    c.head_dim = c.hidden_size / c.num_attention_heads;
  }
  const Json* ab = j.find("attention_bias");
  const Json* mb = j.find("mlp_bias");
  if ((ab && ab->kind == Json::Bool && ab->b) || (mb && mb->kind == Json::Bool && mb->b))
    throw ConfigError("config.json: attention_bias / mlp_bias are not supported by the Llama dense decoder here");
  c.max_position_embeddings = j.has("max_position_embeddings") ? require_int(j, "max_position_embeddings") : 0;
  c.rms_norm_eps = opt_num(j, "rms_norm_eps", 1e-5);
  c.rope_theta = opt_num(j, "rope_theta", 10000.0);
  if (const Json* rs = j.find("rope_scaling"); rs && rs->kind == Json::Object) {
    std::string kind;
    if (const Json* t = rs->find("rope_type"); t && t->kind == Json::String) kind = t->str;
    else if (const Json* t2 = rs->find("type"); t2 && t2->kind == Json::String) kind = t2->str;
    if (!kind.empty() && kind != "default") {
      if (kind != "llama3") throw ConfigError("config.json: rope_scaling type '" + kind + "' is not supported (known: llama3)");
      c.rope_scaling.present = true;
      c.rope_scaling.rope_type = kind;
      c.rope_scaling.factor = require_num(*rs, "factor", "rope_scaling");
      c.rope_scaling.low_freq_factor = require_num(*rs, "low_freq_factor", "rope_scaling");
      c.rope_scaling.high_freq_factor = require_num(*rs, "high_freq_factor", "rope_scaling");
      c.rope_scaling.original_max_position_embeddings = (long long)require_num(*rs, "original_max_position_embeddings", "rope_scaling");
    }
  }
  if (const Json* t = j.find("tie_word_embeddings"); t && t->kind == Json::Bool) c.tie_word_embeddings = t->b;
  if (const Json* a = j.find("hidden_act"); a && a->kind == Json::String) c.hidden_act = a->str;
  if (const Json* e = j.find("eos_token_id")) {
    if (e->kind == Json::Number) c.eos_token_ids.push_back((long long)e->num);
    else if (e->kind == Json::Array)
      for (const Json& x : e->arr)
        if (x.kind == Json::Number) c.eos_token_ids.push_back((long long)x.num);
  }
  // the reference's valid() (model_config.hpp:52-56) plus what the rotary pairs and the activation add
  const std::pair<const char*, long long> sizes[] = {{"vocab_size", c.vocab_size}, {"hidden_size", c.hidden_size},
      {"intermediate_size", c.intermediate_size}, {"num_hidden_layers", c.num_hidden_layers},
      {"num_attention_heads", c.num_attention_heads}, {"num_key_value_heads", c.num_key_value_heads}, {"head_dim", c.head_dim}};
  for (const auto& kv : sizes)
    if (kv.second <= 0) throw ConfigError(std::string("config.json: '") + kv.first + "' must be positive, got " + std::to_string(kv.second));
  if (c.num_attention_heads % c.num_key_value_heads)
    throw ConfigError("config.json: num_attention_heads " + std::to_string(c.num_attention_heads) +
                      " is not a multiple of num_key_value_heads " + std::to_string(c.num_key_value_heads));
  if (c.head_dim % 2) throw ConfigError("config.json: head_dim " + std::to_string(c.head_dim) + " must be even for rotary pairs");
  if (c.hidden_act != "silu") throw ConfigError("config.json: hidden_act '" + c.hidden_act + "' is not supported (known: silu)");
  if (c.rms_norm_eps < 0) throw ConfigError("config.json: rms_norm_eps must not be negative");
  return c;
}

// Rotary frequencies f_i = theta^(-2i/rotary_dim) (runtime/src/ops.cpp:132), with the llama3 rule
// when the configuration has it: wavelengths shorter than orig/high keep f, longer than orig/low
// use f/factor, those between blend linearly (the reference has no such rule; it only displays the
// keys, gguf/src/gguf_file.cpp:233-243).  Computed in double.
inline std::vector<double> inverse_frequencies(int rotary_dim, double theta, const RopeScaling& sc) {
  std::vector<double> f((size_t)rotary_dim / 2);
  for (int i = 0; i < rotary_dim / 2; ++i) f[(size_t)i] = std::exp(-(2.0 * i / rotary_dim) * std::log(theta));
  if (!sc.present) return f;
  const double orig = (double)sc.original_max_position_embeddings, pi = 3.14159265358979323846;
  for (double& fi : f) {
    const double wavelen = 2.0 * pi / fi;
    if (wavelen < orig / sc.high_freq_factor) continue;
    if (wavelen > orig / sc.low_freq_factor) { fi /= sc.factor; continue; }
    const double s = (orig / wavelen - sc.low_freq_factor) / (sc.high_freq_factor - sc.low_freq_factor);
    fi = (1.0 - s) * fi / sc.factor + s * fi;
  }
  return f;
}

// ------------------------------------------------------------------ model description
// What the loader and the engines need of a decoder, as data: tensor names and sizes layer by layer.
struct LayerDesc {
  std::string input_norm, q_proj, k_proj, v_proj, o_proj, post_norm, gate_proj, up_proj, down_proj;
};

struct ModelDesc {
  std::string architecture;
  long long vocab = 0, hidden = 0, ffn = 0, heads = 0, kv_heads = 0, head_dim = 0, max_position = 0;
  double eps = 1e-5, theta = 10000.0, attn_scale = 0.0;
  RopeScaling rope_scaling;
  std::string embedding, final_norm, lm_head;        // lm_head empty: the head is the embedding table
  std::vector<LayerDesc> layers;
  std::vector<long long> eos_token_ids;

  // name -> expected shape of every tensor the model reads
  std::map<std::string, std::vector<long long>> expected() const {
    std::map<std::string, std::vector<long long>> t;
    const long long q = heads * head_dim, kv = kv_heads * head_dim;
    t[embedding] = {vocab, hidden};
    for (const auto& L : layers) {
      t[L.input_norm] = {hidden}; t[L.post_norm] = {hidden};
      t[L.q_proj] = {q, hidden}; t[L.k_proj] = {kv, hidden}; t[L.v_proj] = {kv, hidden}; t[L.o_proj] = {hidden, q};
      t[L.gate_proj] = {ffn, hidden}; t[L.up_proj] = {ffn, hidden}; t[L.down_proj] = {hidden, ffn};
    }
    t[final_norm] = {hidden};
    if (!lm_head.empty()) t[lm_head] = {vocab, hidden};
    return t;
  }
};

// The Llama dense decoder as data (layer order and tensor roles: runtime/src/text_model.cpp:133-176,
// runtime/src/weights.cpp:27-47; names as a config.json + safetensors checkpoint has them).
inline ModelDesc llama_desc(const Json& j) {
  const LlamaConfig c = llama_config_from_json(j);
  ModelDesc m;
  m.architecture = c.architecture;
  m.vocab = c.vocab_size; m.hidden = c.hidden_size; m.ffn = c.intermediate_size; m.heads = c.num_attention_heads;
  m.kv_heads = c.num_key_value_heads; m.head_dim = c.head_dim; m.max_position = c.max_position_embeddings;
  m.eps = c.rms_norm_eps; m.theta = c.rope_theta; m.attn_scale = 1.0 / std::sqrt((double)c.head_dim);
  m.rope_scaling = c.rope_scaling;
  m.embedding = "model.embed_tokens.weight";
  m.final_norm = "model.norm.weight";
  m.lm_head = c.tie_word_embeddings ? "" : "lm_head.weight";
  m.eos_token_ids = c.eos_token_ids;
  for (long long i = 0; i < c.num_hidden_layers; ++i) {
    const std::string p = "model.layers." + std::to_string(i) + ".";
    LayerDesc L;
    L.input_norm = p + "input_layernorm.weight";
    L.q_proj = p + "self_attn.q_proj.weight"; L.k_proj = p + "self_attn.k_proj.weight";
    L.v_proj = p + "self_attn.v_proj.weight"; L.o_proj = p + "self_attn.o_proj.weight";
    L.post_norm = p + "post_attention_layernorm.weight";
    L.gate_proj = p + "mlp.gate_proj.weight"; L.up_proj = p + "mlp.up_proj.weight"; L.down_proj = p + "mlp.down_proj.weight";
    m.layers.push_back(L);
  }
  return m;
}

// architecture name -> builder of its description; unknown names are refused with the list of known ones
inline std::map<std::string, std::function<ModelDesc(const Json&)>>& architecture_registry() {
  static std::map<std::string, std::function<ModelDesc(const Json&)>> reg = {{"LlamaForCausalLM", llama_desc}};
  return reg;
}

inline ModelDesc model_desc_from_config(const Json& j) {
  const std::string arch = architecture_of(j);
  auto& reg = architecture_registry();
  auto it = reg.find(arch);
  if (it == reg.end()) {
    std::string known;
    for (const auto& kv : reg) known += (known.empty() ? "" : ", ") + kv.first;
    throw ConfigError("config.json: architecture '" + arch + "' is not registered (known: " + known + ")");
  }
  return it->second(j);
}

// One error for everything wrong between a checkpoint's tensors and a model's: missing and
// unexpected names, wrong shapes (the reference stops at the first missing tensor,
// runtime/include/qorvix/runtime/tensor_load.hpp:32-45).  `ignored` are name suffixes of buffers
// some checkpoints store beside the weights.  Empty string: all is well.
template <typename CheckpointT>
std::string check_tensors(const ModelDesc& m, const CheckpointT& ck, const std::string& where) {
  const auto want = m.expected();
  std::string missing, unexpected, wrong;
  int nm = 0, nu = 0, nw = 0;
  for (const auto& kv : want) {
    const auto* t = ck.find(kv.first);
    if (!t) { missing += (nm++ ? ", " : "") + kv.first; continue; }
    if (t->shape != kv.second) {
      auto fmt = [](const std::vector<long long>& s) { std::string o = "["; for (size_t i = 0; i < s.size(); ++i) o += (i ? ", " : "") + std::to_string(s[i]); return o + "]"; };
      wrong += std::string(nw++ ? "; " : "") + kv.first + ": stored " + fmt(t->shape) + ", expected " + fmt(kv.second);
    }
  }
  for (const auto& kv : ck.all()) {
    if (want.count(kv.first)) continue;
    if (kv.first == "lm_head.weight" && m.lm_head.empty()) continue;                     // a tied head's stored copy
    const std::string suffix = "self_attn.rotary_emb.inv_freq";
    if (kv.first.size() >= suffix.size() && kv.first.compare(kv.first.size() - suffix.size(), suffix.size(), suffix) == 0) continue;
    unexpected += (nu++ ? ", " : "") + kv.first;
  }
  if (!nm && !nu && !nw) return "";
  std::string msg = where + ": the checkpoint does not fit the model";
  if (nm) msg += "\n  missing tensors (" + std::to_string(nm) + "): " + missing;
  if (nu) msg += "\n  unexpected tensors (" + std::to_string(nu) + "): " + unexpected;
  if (nw) msg += "\n  wrong shapes (" + std::to_string(nw) + "): " + wrong;
  return msg;
}

}  // namespace qv
