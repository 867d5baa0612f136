// The whole decoder in plain C++ over a model folder, from the twins of ref_ops.hpp: whole
// sequences, no cache, one token row after the other (the reference's CPU model walks the same way,
// runtime/src/text_model.cpp:133-176).  Host only.  Behind a C interface so that the command line
// (`qorvix gpu-check`), the native tools and the tests can hold the engine's logits against it,
// and with one entry point per operation for the kernel tests.
#include <cstring>
#include <memory>
#include <string>

#include "../host/model_config.hpp"
#include "../host/safetensors.hpp"
#include "ref_ops.hpp"

namespace {

struct RefModel {
  qv::ModelDesc desc;
  std::map<std::string, std::vector<float>> w;
  std::vector<double> inv_freq;
  std::string error;
};

thread_local std::string g_error;

const std::vector<float>& W(const RefModel& m, const std::string& name) { return m.w.at(name); }

}  // namespace

extern "C" {

const char* qvr_last_error() { return g_error.c_str(); }

// Opens a model folder (config.json + safetensors); null on failure (qvr_last_error says why).
void* qvr_model_open(const char* dir) {
  try {
    auto m = std::make_unique<RefModel>();
    const std::string d(dir);
    m->desc = qv::model_desc_from_config(qv::parse_json(qv::read_text_file(d + "/config.json")));
    qv::Checkpoint ck(d);
    const std::string problems = qv::check_tensors(m->desc, ck, d + "/model.safetensors");
    if (!problems.empty()) throw std::runtime_error(problems);
    for (const auto& kv : m->desc.expected()) m->w[kv.first] = qv::to_float(*ck.find(kv.first));
    m->inv_freq = qv::inverse_frequencies((int)m->desc.head_dim, m->desc.theta, m->desc.rope_scaling);
    return m.release();
  } catch (const std::exception& e) {
    g_error = e.what();
    return nullptr;
  }
}

void qvr_model_close(void* h) { delete (RefModel*)h; }
int qvr_model_vocab(void* h) { return (int)((RefModel*)h)->desc.vocab; }

// logits [n, vocab] of one whole sequence of n tokens; 0 on success
int qvr_forward(void* h, const int* tokens, int n, float* logits) {
  const RefModel& m = *(RefModel*)h;
  const qv::ModelDesc& c = m.desc;
  const int d = (int)c.hidden, H = (int)c.heads, Hkv = (int)c.kv_heads, hd = (int)c.head_dim, f = (int)c.ffn, V = (int)c.vocab;
  const int qd = H * hd, kvd = Hkv * hd;
  for (int t = 0; t < n; ++t)
    if (tokens[t] < 0 || tokens[t] >= V) { g_error = "token id outside the vocabulary"; return -1; }
  std::vector<float> x((size_t)n * d);
  const std::vector<float>& emb = W(m, c.embedding);
  for (int t = 0; t < n; ++t) std::memcpy(&x[(size_t)t * d], &emb[(size_t)tokens[t] * d], (size_t)d * 4);   // no scaling (text_model.cpp:120)
  std::vector<float> xn((size_t)d), q((size_t)n * qd), k((size_t)n * kvd), v((size_t)n * kvd), att((size_t)qd), proj((size_t)d),
      g((size_t)f), u((size_t)f), a((size_t)f);
  for (const auto& L : c.layers) {
    for (int t = 0; t < n; ++t) {                                                         // text_model.cpp:146-154
      qvref::rmsnorm(xn.data(), &x[(size_t)t * d], W(m, L.input_norm).data(), d, c.eps);
      qvref::matvec(&q[(size_t)t * qd], W(m, L.q_proj).data(), xn.data(), qd, d);
      qvref::matvec(&k[(size_t)t * kvd], W(m, L.k_proj).data(), xn.data(), kvd, d);
      qvref::matvec(&v[(size_t)t * kvd], W(m, L.v_proj).data(), xn.data(), kvd, d);
      qvref::rope(&q[(size_t)t * qd], H, hd, hd, t, m.inv_freq.data());
      qvref::rope(&k[(size_t)t * kvd], Hkv, hd, hd, t, m.inv_freq.data());
    }
    for (int t = 0; t < n; ++t) {                                                         // text_model.cpp:78-116, 158-159
      for (int hh = 0; hh < H; ++hh) {
        const int kvh = hh / (H / Hkv);
        qvref::attention_row(&att[(size_t)hh * hd], &q[(size_t)t * qd + (size_t)hh * hd], hd, 0, t, c.attn_scale,
                             [&](int p) { return &k[(size_t)p * kvd + (size_t)kvh * hd]; },
                             [&](int p) { return &v[(size_t)p * kvd + (size_t)kvh * hd]; });
      }
      qvref::matvec(proj.data(), W(m, L.o_proj).data(), att.data(), d, qd);
      for (int i = 0; i < d; ++i) x[(size_t)t * d + i] += proj[(size_t)i];
    }
    for (int t = 0; t < n; ++t) {                                                         // text_model.cpp:162-168
      qvref::rmsnorm(xn.data(), &x[(size_t)t * d], W(m, L.post_norm).data(), d, c.eps);
      qvref::matvec(g.data(), W(m, L.gate_proj).data(), xn.data(), f, d);
      qvref::matvec(u.data(), W(m, L.up_proj).data(), xn.data(), f, d);
      qvref::swiglu(a.data(), g.data(), u.data(), f);
      qvref::matvec(proj.data(), W(m, L.down_proj).data(), a.data(), d, f);
      for (int i = 0; i < d; ++i) x[(size_t)t * d + i] += proj[(size_t)i];
    }
  }
  const std::vector<float>& head = c.lm_head.empty() ? emb : W(m, c.lm_head);             // weights.hpp:119
  for (int t = 0; t < n; ++t) {                                                           // text_model.cpp:172-173
    qvref::rmsnorm(xn.data(), &x[(size_t)t * d], W(m, c.final_norm).data(), d, c.eps);
    qvref::matvec(logits + (size_t)t * V, head.data(), xn.data(), V, d);
  }
  return 0;
}

// ------------------------------------------------------------------ one entry point per operation
void qvr_rmsnorm(float* out, const float* x, const float* w, int rows, int n, double eps) {
  for (int r = 0; r < rows; ++r) qvref::rmsnorm(out + (size_t)r * n, x + (size_t)r * n, w, n, eps);
}
void qvr_gemm(float* C, const float* A, const float* Wt, int M, int N, int K) { qvref::gemm(C, A, Wt, M, N, K); }
void qvr_rope(float* vec, int rows, const int* positions, int n_heads, int head_dim, int rotary_dim, const double* inv_freq) {
  for (int r = 0; r < rows; ++r) qvref::rope(vec + (size_t)r * n_heads * head_dim, n_heads, head_dim, rotary_dim, positions[r], inv_freq);
}
void qvr_inverse_frequencies(double* out, int rotary_dim, double theta, int scaled, double factor, double low, double high, long long orig) {
  qv::RopeScaling sc;
  sc.present = scaled != 0; sc.factor = factor; sc.low_freq_factor = low; sc.high_freq_factor = high; sc.original_max_position_embeddings = orig;
  const auto f = qv::inverse_frequencies(rotary_dim, theta, sc);
  std::copy(f.begin(), f.end(), out);
}
void qvr_attention_paged(float* out, int ld_out, const float* q, int ld_q, const float* cache, const int* tok_pos, const int* tok_seg,
                         const int* block_table, int max_blocks, int T, int H, int Hkv, int hd, int page, int window, double scale) {
  qvref::attention_paged(out, ld_out, q, ld_q, cache, tok_pos, tok_seg, block_table, max_blocks, T, H, Hkv, hd, page, window, scale);
}
void qvr_swiglu(float* out, const float* gate, const float* up, long long n) { qvref::swiglu(out, gate, up, (int)n); }
int qvr_argmax(const float* x, int n) { return qvref::argmax(x, n); }
// the candidate set after all filters; returns how many survive (ids and probs hold at most `cap`)
int qvr_candidates(const float* logits, int vocab, double temperature, int top_k, double top_p, double min_p, int* ids, double* probs, int cap) {
  qvref::SamplerParams p;
  p.temperature = temperature; p.top_k = top_k; p.top_p = top_p; p.min_p = min_p;
  std::vector<int> i;
  std::vector<double> pr;
  qvref::candidates(logits, vocab, p, &i, &pr);
  for (size_t k = 0; k < i.size() && (int)k < cap; ++k) { ids[k] = i[k]; probs[k] = pr[k]; }
  return (int)i.size();
}
int qvr_sample(float* logits, int vocab, double temperature, int top_k, double top_p, double min_p, double rep, double freq, double pres,
               int last_n, const int* recent, int n_recent, double u) {
  qvref::SamplerParams p;
  p.temperature = temperature; p.top_k = top_k; p.top_p = top_p; p.min_p = min_p;
  p.repetition_penalty = rep; p.frequency_penalty = freq; p.presence_penalty = pres; p.penalty_last_n = last_n;
  qvref::apply_penalties(logits, vocab, recent, n_recent, p);
  return qvref::sample_with_uniform(logits, vocab, p, u);
}

}  // extern "C"
