// Plain C++ twins of the CUDA kernels: one short function for each operation, host only, no
// tiling, no cache tricks, reductions accumulated in double.  They restate the reference's CPU
// operations (runtime/src/ops.cpp, runtime/src/text_model.cpp, runtime/src/sampler.cpp) for batches
// of tokens and a paged cache; `qorvix gpu-check` and the tests hold the kernels against them.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <numeric>
#include <vector>

namespace qvref {

// out_i = x_i * (1 / sqrt(sum(x^2)/n + eps)) * w_i, the sum in double (runtime/src/ops.cpp:8-13)
inline void rmsnorm(float* out, const float* x, const float* w, int n, double eps) {
  double ss = 0.0;
  for (int i = 0; i < n; ++i) ss += (double)x[i] * (double)x[i];
  const double scale = 1.0 / std::sqrt(ss / n + eps);
  for (int i = 0; i < n; ++i) out[i] = (float)((double)x[i] * scale * (double)w[i]);
}

// out[r] = dot(W[r, :], x) (runtime/src/ops.cpp:34-56), accumulated in double
inline void matvec(float* out, const float* W, const float* x, int rows, int cols) {
  for (int r = 0; r < rows; ++r) {
    const float* wr = W + (size_t)r * cols;
    double acc = 0.0;
    for (int c = 0; c < cols; ++c) acc += (double)wr[c] * (double)x[c];
    out[r] = (float)acc;
  }
}

// C[M, N] = A[M, K] W[N, K]^T, row by row
inline void gemm(float* C, const float* A, const float* W, int M, int N, int K) {
  for (int m = 0; m < M; ++m) matvec(C + (size_t)m * N, W, A + (size_t)m * K, N, K);
}

// Split-half rotation of the first rotary_dim dims of every head of vec[n_heads * head_dim]:
// pairs (i, i + rotary_dim/2), a' = a cos - b sin, b' = a sin + b cos, angle = pos * inv_freq[i]
// (runtime/src/ops.cpp:127-148 with the frequencies as a table)
inline void rope(float* vec, int n_heads, int head_dim, int rotary_dim, int pos, const double* inv_freq) {
  const int half = rotary_dim / 2;
  for (int h = 0; h < n_heads; ++h) {
    float* v = vec + (size_t)h * head_dim;
    for (int i = 0; i < half; ++i) {
      const double th = (double)pos * inv_freq[i], c = std::cos(th), s = std::sin(th);
      const double a = v[i], b = v[i + half];
      v[i] = (float)(a * c - b * s);
      v[i + half] = (float)(a * s + b * c);
    }
  }
}

// exp(s - max) / sum, the sum in double (runtime/src/ops.cpp:83-94)
inline void softmax(double* s, int n) {
  double mx = s[0];
  for (int i = 1; i < n; ++i) mx = std::max(mx, s[i]);
  double sum = 0.0;
  for (int i = 0; i < n; ++i) { s[i] = std::exp(s[i] - mx); sum += s[i]; }
  for (int i = 0; i < n; ++i) s[i] /= sum;
}

// One query row of causal grouped-query attention over keys/values given by a lookup
// (runtime/src/text_model.cpp:83-114): kvHead = h / (H / Hkv); score = (q.k) * scale for the keys
// lo..pos; softmax; weighted sum of values.  key(t) / value(t) return the head's hd floats of position t.
template <typename KeyFn, typename ValueFn>
inline void attention_row(float* out, const float* q, int hd, int lo, int pos, double scale, KeyFn key, ValueFn value) {
  const int n = pos - lo + 1;
  std::vector<double> s((size_t)n);
  for (int t = 0; t < n; ++t) {
    const float* k = key(lo + t);
    double acc = 0.0;
    for (int d = 0; d < hd; ++d) acc += (double)q[d] * (double)k[d];
    s[(size_t)t] = acc * scale;
  }
  softmax(s.data(), n);
  std::vector<double> o((size_t)hd, 0.0);
  for (int t = 0; t < n; ++t) {
    const float* v = value(lo + t);
    for (int d = 0; d < hd; ++d) o[(size_t)d] += s[(size_t)t] * (double)v[d];
  }
  for (int d = 0; d < hd; ++d) out[d] = (float)o[(size_t)d];
}

// Attention of a step's tokens over a paged cache: cache [pages][2][Hkv][page][hd] (float), token t at
// position tok_pos[t] of segment tok_seg[t], whose pages are block_table[seg][...]; window 0 = all keys.
inline void attention_paged(float* out, int ld_out, const float* q, int ld_q, const float* cache, const int* tok_pos, const int* tok_seg,
                            const int* block_table, int max_blocks, int T, int H, int Hkv, int hd, int page, int window, double scale) {
  const size_t page_stride = (size_t)2 * Hkv * page * hd;
  for (int t = 0; t < T; ++t) {
    const int pos = tok_pos[t];
    const int* bt = block_table + (size_t)tok_seg[t] * max_blocks;
    const int lo = window > 0 ? std::max(0, pos - window + 1) : 0;
    for (int h = 0; h < H; ++h) {
      const int kvh = h / (H / Hkv);
      auto at = [&](int which, int p) { return cache + (size_t)bt[p / page] * page_stride + ((size_t)(which * Hkv + kvh) * page + p % page) * hd; };
      attention_row(out + (size_t)t * ld_out + (size_t)h * hd, q + (size_t)t * ld_q + (size_t)h * hd, hd, lo, pos, scale,
                    [&](int p) { return at(0, p); }, [&](int p) { return at(1, p); });
    }
  }
}

// silu(gate) * up, silu(z) = z / (1 + e^-z) (runtime/src/ops.cpp:96-100)
inline void swiglu(float* out, const float* gate, const float* up, int n) {
  for (int i = 0; i < n; ++i) {
    const double g = gate[i];
    out[i] = (float)(g / (1.0 + std::exp(-g)) * (double)up[i]);
  }
}

// index of the first maximum (runtime/src/ops.cpp:150-156)
inline int argmax(const float* x, int n) {
  int best = 0;
  for (int i = 1; i < n; ++i)
    if (x[i] > x[best]) best = i;
  return best;
}

// ------------------------------------------------------------------ sampling (runtime/src/sampler.cpp)
struct SamplerParams {
  double temperature = 0.8, top_p = 0.95, min_p = 0.05, repetition_penalty = 1.1, frequency_penalty = 0.0, presence_penalty = 0.0;
  int top_k = 40, penalty_last_n = 64;
};

// penalties over the last penalty_last_n ids: l > 0 ? l / rep : l * rep, - count * freq, - presence (sampler.cpp:13-34)
inline void apply_penalties(float* logits, int vocab, const int* recent, int n_recent, const SamplerParams& p) {
  if (p.penalty_last_n == 0) return;
  if (p.repetition_penalty == 1.0 && p.frequency_penalty == 0.0 && p.presence_penalty == 0.0) return;
  const int first = n_recent > p.penalty_last_n ? n_recent - p.penalty_last_n : 0;
  std::vector<int> seen;
  for (int i = first; i < n_recent; ++i) {
    const int tok = recent[i];
    if (tok < 0 || tok >= vocab || std::find(seen.begin(), seen.end(), tok) != seen.end()) continue;
    seen.push_back(tok);
    const int count = (int)std::count(recent + first, recent + n_recent, tok);
    float l = logits[tok];
    if (p.repetition_penalty != 1.0) l = l > 0 ? (float)(l / p.repetition_penalty) : (float)(l * p.repetition_penalty);
    l -= (float)(count * p.frequency_penalty);
    l -= (float)p.presence_penalty;
    logits[tok] = l;
  }
}

// The ids and probabilities that survive temperature -> softmax -> sort (descending, lower id first on
// a tie) -> top-k -> top-p (shortest prefix whose cumulative un-renormalised probability reaches p)
// -> min-p (sampler.cpp:53-87)
inline void candidates(const float* logits, int vocab, const SamplerParams& p, std::vector<int>* ids, std::vector<double>* probs) {
  std::vector<double> pr((size_t)vocab);
  double mx = -INFINITY;
  for (int i = 0; i < vocab; ++i) mx = std::max(mx, (double)logits[i] / p.temperature);
  double sum = 0.0;
  for (int i = 0; i < vocab; ++i) { pr[(size_t)i] = std::exp((double)logits[i] / p.temperature - mx); sum += pr[(size_t)i]; }
  for (double& x : pr) x /= sum;
  std::vector<int> order((size_t)vocab);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return pr[(size_t)a] > pr[(size_t)b]; });
  size_t keep = order.size();
  if (p.top_k > 0 && (size_t)p.top_k < keep) keep = (size_t)p.top_k;
  if (p.top_p < 1.0) {
    double cum = 0.0;
    for (size_t i = 0; i < keep; ++i) {
      cum += pr[(size_t)order[i]];
      if (cum >= p.top_p) { keep = i + 1; break; }
    }
  }
  ids->clear(); probs->clear();
  const double thr = p.min_p > 0.0 ? p.min_p * pr[(size_t)order[0]] : -1.0;
  for (size_t i = 0; i < keep; ++i)
    if (pr[(size_t)order[i]] >= thr) { ids->push_back(order[i]); probs->push_back(pr[(size_t)order[i]]); }
}

// A draw with a given uniform number u in [0, 1): r = u * total, walk the survivors (sampler.cpp:92-100);
// temperature <= 0 is greedy (sampler.cpp:50)
inline int sample_with_uniform(const float* logits, int vocab, const SamplerParams& p, double u) {
  if (p.temperature <= 0.0) return argmax(logits, vocab);
  std::vector<int> ids;
  std::vector<double> probs;
  candidates(logits, vocab, p, &ids, &probs);
  if (ids.empty()) return argmax(logits, vocab);
  double r = u * std::accumulate(probs.begin(), probs.end(), 0.0);
  for (size_t i = 0; i < ids.size(); ++i) {
    r -= probs[i];
    if (r <= 0.0) return ids[i];
  }
  return ids.back();
}

}  // namespace qvref
