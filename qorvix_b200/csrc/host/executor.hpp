// The step executor for decoders made of pre-norm blocks (RMS norm, rotary grouped-query attention
// over the paged cache, SwiGLU feed-forward): given a step's integer arrays on the device and a
// table of weight and cache pointers, it issues every launch of the forward pass itself, with the
// same kernels and the same choices as the part objects of the Python side make one call at a
// time.  It is what the native command-line tools run, and what the Python step function hands a
// step to when every block of the model is of this kind (one call a step instead of a dozen a
// layer).  The reference's counterpart is GpuModelImpl::forwardEager
// (cuda/src/cuda_backend.cu:1407-1452): one token of one session, float32, a launch per operation.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "dispatch.hpp"
#include "kernels.hpp"

namespace qv {

struct LinearW {
  const void* rows = nullptr;      // [N, K] row-major in `dt`, or null when only the packed tiles are kept
  const void* packed = nullptr;    // bfloat16 tiles (qv_pack_weight_tiles), or null
  int N = 0, K = 0;
  int dt = DT_BF16;                // storage type of `rows`
};

struct LayerW {
  const float* norm1 = nullptr;    // the mixer's norm weight [d]
  const float* norm2 = nullptr;    // the feed-forward's norm weight [d]
  LinearW qkv, o, gate_up, down;
  int interleaved = 1;             // gate/up rows interleaved in groups of 16 (else [gate; up])
  void* cache = nullptr;           // this layer's pages [pages + 1][2][Hkv][page][hd] in the compute dtype
  long long cache_pages = 0;       // pages + 1
  int window = 0;
};

struct ModelW {
  int dt = DT_BF16;                // compute dtype
  int d = 0, H = 0, Hkv = 0, hd = 0, f = 0, V = 0, page = 16, rot = 0, table_rows = 0, sms = 148;
  float eps = 1e-5f, scale = 0.f;
  const float* cos_sin = nullptr;  // [table_rows][rot / 2][2]
  const void* embedding = nullptr;
  int emb_dt = DT_BF16;
  const float* final_norm = nullptr;
  LinearW head;
  std::vector<LayerW> layers;
};

// One step's integer arrays (device pointers) and what the host knows of its shape.
struct StepIO {
  int T = 0, S = 0, R = 0;
  int n1 = 0;                      // leading segments of one token
  int max_q_len = 0, max_ctx_len = 0, rest_max_q = 0;   // rest_max_q: longest segment after the first n1
  int portion_max_ctx = 0;                              // longest context among the segments of more than one token (0: not known)
  int captured = 0;                // the step is captured or replayed as a graph: choices must not depend on contexts
  const int* token_ids = nullptr;
  const int* tok_pos = nullptr;
  const int* tok_seg = nullptr;
  const int* seg_q_start = nullptr;
  const int* seg_pos0 = nullptr;
  const int* block_table = nullptr;   // [S][max_blocks]
  const int* want_rows = nullptr;
  int max_blocks = 0;
  float* logits = nullptr;         // [R][V] out
};

// A piece of device memory handed out front to back; reset every step.
struct Arena {
  uint8_t* base = nullptr;
  size_t size = 0, used = 0;
  void* take(size_t bytes) {
    const size_t at = (used + 255) & ~(size_t)255;
    if (at + bytes > size) throw std::runtime_error("the executor's workspace is too small for this step");
    used = at + bytes;
    return base + at;
  }
};

inline size_t dt_size(int dt) { return dt == DT_F32 ? 4 : 2; }

// Bytes of workspace a step of T tokens with R wanted rows may take, n_decode of them single tokens
// that lead the step (all of them in a decode-only step).
inline size_t workspace_bytes(const ModelW& m, int T, int R, int n_decode) {
  const size_t e = dt_size(m.dt), t = (size_t)T;
  const size_t qkv = (size_t)(m.H + 2 * m.Hkv) * m.hd;
  size_t b = t * m.d * 4                       // residual stream
             + 2 * t * m.d * e                 // normed rows, a part's output
             + 2 * t * m.d * e                 // a prepared norm input, twice (one being read, one being made)
             + 2 * (size_t)((m.d + 127) / 128) * 64 * 4
             + t * qkv * e + t * (size_t)m.H * m.hd * e
             + t * (size_t)m.f * e + 2 * t * (size_t)m.f * e
             + (size_t)n_decode * m.H * 16 * (m.hd + 2) * 4
             + (size_t)R * m.d * e;
  return b + 64 * 256;
}

// How often each kernel that a step's shape chooses between has served, process-wide (tests read
// these to prove which kernels ran).
enum Route { ROUTE_PREFILL_TC, ROUTE_QKV_ROPE, ROUTE_DECODE, ROUTE_PREFILL_MMA, ROUTE_GENERIC, ROUTE_FOLDED_NORM, ROUTE_COUNT };
inline long long* route_counts() {
  static long long counts[ROUTE_COUNT] = {0};
  return counts;
}

class Executor {
 public:
  Executor(const Kernels* k, const ModelW* m, int* err_word) : k_(k), m_(m), err_(err_word) {}

  long long launches = 0;

  void forward(const StepIO& io, Arena& ws, cudaStream_t st) {
    const ModelW& m = *m_;
    const int T = io.T, d = m.d;
    const size_t e = dt_size(m.dt);
    ws.used = 0;
    float* residual = (float*)ws.take((size_t)T * d * 4);
    void* xn = ws.take((size_t)T * d * e);
    void* part_out = ws.take((size_t)T * d * e);
    void* scaled[2] = {ws.take((size_t)T * d * e), ws.take((size_t)T * d * e)};
    const size_t stats_bytes = (size_t)((d + 127) / 128) * 64 * 4;
    float* stats[2] = {(float*)ws.take(stats_bytes), (float*)ws.take(stats_bytes)};
    const int qkv_n = (m.H + 2 * m.Hkv) * m.hd;
    void* qkv = ws.take((size_t)T * qkv_n * e);
    void* att = ws.take((size_t)T * m.H * m.hd * e);
    void* act = ws.take((size_t)T * m.f * e);
    check(k_->embed(residual, m.embedding, io.token_ids, T, d, m.V, m.emb_dt, st), "embed");

    const bool fold = m.dt == DT_BF16 && folded_norm_enabled(T);
    // what the stream still owes: nothing, a delta the next norm adds, or a norm input a product prepared
    enum { NONE, DELTA, PRENORMED } pending = NONE;
    int pre = 0;                                   // which of scaled[]/stats[] holds the prepared input
    const int L = (int)m.layers.size();
    const size_t layer_scratch = ws.used;          // what a layer takes beyond this (slices' partial results, an unfused gate/up) is the next layer's again
    for (int li = 0; li < L; ++li) {
      const LayerW& w = m.layers[(size_t)li];
      ws.used = layer_scratch;
      // ---- attention
      bool have_qkv = false;
      if (pending == PRENORMED) {
        // the norm's scale is applied to the projection's sums
        const int rc = k_->gemm_bf16_norm(qkv, scaled[pre], w.qkv.packed, T, qkv_n, d, d, qkv_n, m.dt, err_, 0, nullptr, 0, nullptr, nullptr,
                                          stats[pre], (d + 127) / 128, 1.0f / d, m.eps, st);
        if (rc == ERR_UNSUPPORTED) norm(xn, residual, nullptr, w.norm1, T, st);       // the stream is complete: norm it the plain way
        else { check(rc, "gemm_bf16_norm (qkv)"); ++route_counts()[ROUTE_FOLDED_NORM]; rope(qkv, qkv_n, w, io, st); have_qkv = true; }
      } else {
        norm(xn, residual, pending == DELTA ? part_out : nullptr, w.norm1, T, st);
      }
      pending = NONE;
      if (!have_qkv) {
        bool done = false;
        if (m.dt == DT_BF16 && w.qkv.packed && m.cos_sin && m.rot == m.hd && fused_rope_enabled(T)) {
          const int rc = k_->gemm_bf16_qkv_rope(qkv, xn, w.qkv.packed, T, d, d, qkv_n, err_, m.cos_sin, m.table_rows, io.tok_pos, io.tok_seg,
                                                io.block_table, io.max_blocks, w.cache, m.H, m.Hkv, m.hd, m.page, st);
          if (rc != ERR_UNSUPPORTED) { check(rc, "gemm_qkv_rope"); ++route_counts()[ROUTE_QKV_ROPE]; done = true; }
        }
        if (!done) {
          gemm(qkv, qkv_n, m.dt, xn, d, w.qkv, T, st);
          rope(qkv, qkv_n, w, io, st);
        }
      }
      attention(att, qkv, qkv_n, w, io, ws, st);
      // ---- output projection: into the stream with the next norm prepared (few tokens), else a delta
      bool to_stream = false;
      if (fold && w.o.packed && w.o.N == d) {
        const int nxt = pre ^ 1;
        const int rc = k_->gemm_bf16_norm(scaled[nxt], att, w.o.packed, T, d, w.o.K, w.o.K, d, DT_BF16, err_, 0, residual, d, w.norm2,
                                          stats[nxt], nullptr, 0, 0.f, 0.f, st);
        if (rc != ERR_UNSUPPORTED) { check(rc, "gemm_bf16_norm (o)"); ++route_counts()[ROUTE_FOLDED_NORM]; pre = nxt; to_stream = true; }
      }
      if (!to_stream) gemm(part_out, d, m.dt, att, w.o.K, w.o, T, st);
      // ---- feed-forward
      bool have_act = false;
      if (to_stream) {
        if (w.interleaved) {
          const int rc = k_->gemm_bf16_norm(act, scaled[pre], w.gate_up.packed, T, 2 * m.f, d, d, m.f, m.dt, err_, 1, nullptr, 0, nullptr,
                                            nullptr, stats[pre], (d + 127) / 128, 1.0f / d, m.eps, st);
          if (rc != ERR_UNSUPPORTED) { check(rc, "gemm_bf16_norm (gate/up)"); ++route_counts()[ROUTE_FOLDED_NORM]; have_act = true; }
        }
        if (!have_act) norm(xn, residual, nullptr, w.norm2, T, st);
      } else {
        norm(xn, residual, part_out, w.norm2, T, st);
      }
      if (!have_act) gate_up(act, xn, w, T, ws, st);
      // ---- down projection: the next block's first norm may be prepared (none after the last block)
      to_stream = false;
      if (fold && li + 1 < L && w.down.packed && w.down.N == d) {
        const int nxt = pre ^ 1;
        const int rc = k_->gemm_bf16_norm(scaled[nxt], act, w.down.packed, T, d, m.f, m.f, d, DT_BF16, err_, 0, residual, d,
                                          m.layers[(size_t)li + 1].norm1, stats[nxt], nullptr, 0, 0.f, 0.f, st);
        if (rc != ERR_UNSUPPORTED) { check(rc, "gemm_bf16_norm (down)"); ++route_counts()[ROUTE_FOLDED_NORM]; pre = nxt; to_stream = true; }
      }
      if (to_stream) pending = PRENORMED;
      else { gemm(part_out, d, m.dt, act, m.f, w.down, T, st); pending = DELTA; }
    }
    ws.used = layer_scratch;
    if (io.R <= 0) return;
    // final norm on the wanted rows only, then the output head in float32
    void* h = ws.take((size_t)io.R * d * e);
    check(k_->add_rmsnorm(h, residual, pending == DELTA ? part_out : nullptr, m.final_norm, io.want_rows, io.R, d, m.eps, 0, m.dt, m.dt, st),
          "add_rmsnorm (final)");
    gemm(io.logits, m.V, DT_F32, h, d, m.head, io.R, st);
  }

 private:
  const Kernels* k_;
  const ModelW* m_;
  int* err_;

  void check(int rc, const char* what) {
    ++launches;
    if (rc != 0) throw std::runtime_error(std::string(what) + ": " + (k_->error_string ? k_->error_string(rc) : "error") + " (code " + std::to_string(rc) + ")");
  }

  // residual (+= delta); out = rmsnorm(residual) * w
  void norm(void* out, float* residual, const void* delta, const float* w, int T, cudaStream_t st) {
    check(k_->add_rmsnorm(out, residual, delta, w, nullptr, T, m_->d, m_->eps, delta ? 1 : 0, m_->dt, m_->dt, st), "add_rmsnorm");
  }

  // out[M, N] (row stride ldc, type c_dt) = x[M, K] (compute dtype, row stride lda) W^T with the kernel that fits
  void gemm(void* out, int ldc, int c_dt, const void* x, int lda, const LinearW& w, int M, cudaStream_t st) {
    const int a_dt = m_->dt;
    if (a_dt == DT_BF16 && w.packed) {
      const int rc = k_->gemm_bf16_packed(out, x, w.packed, M, w.N, w.K, lda, ldc, c_dt, err_, 0, 0, st);
      if (rc != ERR_UNSUPPORTED) { check(rc, "gemm_bf16_packed"); return; }
    }
    if (!w.rows) throw std::runtime_error("the product's shape is one the tensor-core kernel refuses and the weight rows were not kept");
    if (a_dt == DT_BF16 && w.dt == DT_BF16) {
      const int rc = k_->gemm_bf16_tc(out, x, w.rows, M, w.N, w.K, lda, w.K, ldc, c_dt, err_, 0, 0, st);
      if (rc != ERR_UNSUPPORTED) { check(rc, "gemm_bf16_tc"); return; }
    }
    check(k_->gemm_simt(out, x, w.rows, M, w.N, w.K, lda, w.K, ldc, a_dt, w.dt, c_dt, 0, st), "gemm_simt");
  }

  // act[M, f] = silu(x Wg^T) * (x Wu^T)
  void gate_up(void* act, const void* xn, const LayerW& w, int T, Arena& ws, cudaStream_t st) {
    const ModelW& m = *m_;
    if (w.interleaved && m.dt == DT_BF16) {
      if (w.gate_up.packed) {
        const int rc = k_->gemm_bf16_packed(act, xn, w.gate_up.packed, T, 2 * m.f, m.d, m.d, m.f, DT_BF16, err_, 0, 1, st);
        if (rc != ERR_UNSUPPORTED) { check(rc, "gemm_bf16_packed (swiglu)"); return; }
      }
      if (w.gate_up.rows && w.gate_up.dt == DT_BF16) {
        const int rc = k_->gemm_bf16_tc(act, xn, w.gate_up.rows, T, 2 * m.f, m.d, m.d, m.d, m.f, DT_BF16, err_, 0, 1, st);
        if (rc != ERR_UNSUPPORTED) { check(rc, "gemm_bf16_tc (swiglu)"); return; }
      }
    }
    void* gu = ws.take((size_t)T * 2 * m.f * dt_size(m.dt));
    gemm(gu, 2 * m.f, m.dt, xn, m.d, w.gate_up, T, st);
    check(k_->swiglu(act, gu, T, m.f, w.interleaved ? 1 : 0, m.dt, st), "swiglu");
  }

  void rope(void* qkv, int ld, const LayerW& w, const StepIO& io, cudaStream_t st) {
    const ModelW& m = *m_;
    check(k_->rope_kv_write(qkv, ld, w.cache, m.cos_sin, m.cos_sin ? m.table_rows : 1, io.tok_pos, io.tok_seg, io.block_table, io.max_blocks,
                            io.T, m.H, m.Hkv, m.hd, m.cos_sin ? m.rot : 0, m.page, m.dt, st), "rope_kv_write");
  }

  bool decode(void* out, int ld_out, const void* q, int ld_q, const LayerW& w, const StepIO& io, int T, Arena& ws, cudaStream_t st) {
    const ModelW& m = *m_;
    const int variant = decode_variant(T, m.Hkv);
    const int splits = decode_splits(T, m.Hkv, io.max_ctx_len, !io.captured, variant, m.sms);
    float* partial = splits > 1 ? (float*)ws.take((size_t)T * m.H * splits * (m.hd + 2) * 4) : nullptr;
    k_->attn_set_decode_variant(variant);
    const int rc = k_->attn_decode_bf16(out, ld_out, q, ld_q, w.cache, io.tok_pos, io.tok_seg, io.block_table, io.max_blocks, T, m.H, m.Hkv,
                                        m.hd, m.page, w.window, m.scale, splits, partial, st);
    if (rc == ERR_UNSUPPORTED) return false;
    check(rc, "attention_decode_bf16");
    ++route_counts()[ROUTE_DECODE];
    if (splits > 1) ++launches;                    // the merge of the slices
    return true;
  }

  bool portions(void* out, int ld_out, const void* q, int ld_q, const LayerW& w, const StepIO& io, int first_seg, int max_q, cudaStream_t st) {
    const ModelW& m = *m_;
    const int S = io.S - first_seg;
    const int* qs = io.seg_q_start + first_seg;
    const int* p0 = io.seg_pos0 + first_seg;
    const int* bt = io.block_table + (size_t)first_seg * io.max_blocks;
    if (max_q >= 32) {
      const int rc = k_->attn_prefill_tc(out, ld_out, q, ld_q, io.T, w.cache, w.cache_pages, qs, p0, bt, io.max_blocks, S, max_q, io.portion_max_ctx, m.H, m.Hkv,
                                         m.hd, m.page, w.window, m.scale, err_, st);
      if (rc != ERR_UNSUPPORTED) { check(rc, "attention_prefill_tc"); ++route_counts()[ROUTE_PREFILL_TC]; return true; }
    }
    const int rc = k_->attn_prefill_bf16(out, ld_out, q, ld_q, w.cache, qs, p0, bt, io.max_blocks, S, max_q, m.H, m.Hkv, m.hd, m.page,
                                         w.window, m.scale, 0, st);
    if (rc == ERR_UNSUPPORTED) return false;
    check(rc, "attention_prefill_bf16");
    ++route_counts()[ROUTE_PREFILL_MMA];
    return true;
  }

  // Attention of every token of the step over its request's pages: the tensor-core kernels when they
  // take the sizes (split-KV for single tokens, flash attention for portions; a step whose
  // single-token segments come first is served by both, each on its part), else the CUDA-core kernel.
  void attention(void* out, const void* qkv, int ld_q, const LayerW& w, const StepIO& io, Arena& ws, cudaStream_t st) {
    const ModelW& m = *m_;
    const int ld_out = m.H * m.hd;
    if (m.dt == DT_BF16) {
      if (io.max_q_len == 1) {
        if (decode(out, ld_out, qkv, ld_q, w, io, io.T, ws, st)) return;
      } else if (io.n1 >= kMinLeadingDecodeTokens && io.n1 < io.S) {
        if (decode(out, ld_out, qkv, ld_q, w, io, io.n1, ws, st) && portions(out, ld_out, qkv, ld_q, w, io, io.n1, io.rest_max_q, st)) return;
      } else if (portions(out, ld_out, qkv, ld_q, w, io, 0, io.max_q_len, st)) {
        return;
      }
    }
    check(k_->attention_generic(out, ld_out, qkv, ld_q, w.cache, io.tok_pos, io.tok_seg, io.block_table, io.max_blocks, io.T, m.H, m.Hkv, m.hd,
                                m.page, w.window, m.scale, m.dt, st), "attention_generic");
    ++route_counts()[ROUTE_GENERIC];
  }
};

}  // namespace qv
