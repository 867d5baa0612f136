// The native engine: a model folder on one GPU, the paged cache, and the step function
//   step(entries, end) -> logits at the wanted places,
// with the same meaning as the Python ModelRunner.step (any mix of prompt portions and single
// tokens, run as one batch from the cache earlier steps left).  It owns its device memory
// (cudaMalloc), loads weights from safetensors by name, fuses and packs them as the Python loader
// does, keeps the cache's bookkeeping in csrc/host_runtime.cpp, runs steps through the Executor and
// replays decode-only steps as captured CUDA graphs.  The reference's counterpart is its
// GpuModel (cuda/include/qorvix/cuda/gpu_model.hpp:44-82) behind IInferenceEngine::forward
// (runtime/include/qorvix/runtime/inference_engine.hpp:36-66).
#pragma once
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "executor.hpp"
#include "model_config.hpp"
#include "safetensors.hpp"
#include "step_types.hpp"

extern "C" {
// csrc/host_runtime.cpp
void* qvh_create(int n_groups, const int* windows, int num_pages, int page_size, int max_requests);
void qvh_destroy(void* h);
int qvh_has(void* h, long long rid);
int qvh_length(void* h, long long rid);
int qvh_free_slots(void* h);
int qvh_free_pages(void* h, int group);
int qvh_admit(void* h, long long rid);
int qvh_can_reserve(void* h, int n, const long long* rids, const int* is_new, const int* n_new);
int qvh_reserve(void* h, long long rid, int n_new);
int qvh_commit(void* h, long long rid, int n_new);
int qvh_release(void* h, long long rid);
int qvh_one_more_token_fits(void* h, int n, const long long* rids);
int qvh_table_len(void* h, long long rid, int group);
int qvh_table_copy(void* h, long long rid, int group, int* out, int cap);
int qvh_youngest(void* h, int n, const long long* rids);
int qvh_check(void* h, char* msg, int cap);
int qvh_fill_decode(void* h, int n, const long long* rids, const int* tokens, int S, int width, int scratch_page, int scratch_slot,
                    int* host, long long* row_epoch, int* row_len);
}

namespace qv {

struct EngineError : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct OutOfPages : EngineError {
  using EngineError::EngineError;
};
struct OutOfSlots : EngineError {
  using EngineError::EngineError;
};

inline void cuda_check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw EngineError(std::string(what) + ": " + cudaGetErrorString(e));
}

struct EngineOptions {
  std::string dtype = "bfloat16";       // bfloat16: the kernels and precisions of serving; float32: everything in true 32-bit
  long long max_tokens = 4096;          // sizes the page pool
  int page_size = 16;
  int max_requests = 8;
  long long max_model_len = 0;          // 0: the smaller of the configuration's limit and the pool
  bool use_graphs = true;
  int max_graph_batch = 64;
  bool packed_weights = true;
};

class Engine {
 public:
  Engine(const std::string& model_dir, const EngineOptions& opt, const std::map<std::string, std::string>& kernel_libs) : opt_(opt) {
    if (opt.dtype == "bfloat16" || opt.dtype == "bf16") dt_ = DT_BF16;
    else if (opt.dtype == "float32" || opt.dtype == "fp32") dt_ = DT_F32;
    else throw EngineError("dtype must be bfloat16 or float32, not '" + opt.dtype + "'");
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) throw EngineError("no CUDA device is available; this engine has no CPU path");
    k_.load(kernel_libs);
    desc_ = model_desc_from_config(parse_json(read_text_file(model_dir + "/config.json")));
    cuda_check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate");
    cuda_check(cudaMalloc(&err_word_, sizeof(int)), "cudaMalloc");
    cuda_check(cudaMemsetAsync(err_word_, 0, sizeof(int), stream_), "cudaMemsetAsync");
    k_.attn_set_error_word(err_word_);
    const char* share = getenv("QORVIX_SHARE_TILES");
    if (dt_ == DT_BF16 && !(share && share[0] == '0')) {
      // where CTAs of the many-token product hand partial sums of a shared tile to its owner: a slot and a flag per SM
      int dev = 0, sms = 0;
      cuda_check(cudaGetDevice(&dev), "cudaGetDevice");
      cuda_check(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "cudaDeviceGetAttribute");
      cuda_check(cudaMalloc(&split_slots_, (size_t)sms * (size_t)k_.gemm_split_slot_bytes()), "cudaMalloc");
      cuda_check(cudaMalloc(&split_flags_, (size_t)sms * sizeof(int)), "cudaMalloc");
      cuda_check(cudaMemsetAsync(split_flags_, 0, (size_t)sms * sizeof(int), stream_), "cudaMemsetAsync");
      k_.gemm_set_split_workspace(split_slots_, split_flags_, sms);
    }
    page_ = opt.page_size;
    const long long pool_tokens = (opt.max_tokens + page_ - 1) / page_ * page_;
    const long long limit = desc_.max_position > 0 ? desc_.max_position : pool_tokens;
    max_model_len_ = opt.max_model_len > 0 ? opt.max_model_len : std::min(limit, pool_tokens);
    num_pages_ = (int)(pool_tokens / page_);
    load_weights(model_dir);
    build_rotary_table();
    allocate_cache();
    int window = 0;
    cache_ = qvh_create(1, &window, num_pages_, page_, opt.max_requests);
    if (!cache_) throw EngineError("the cache manager could not be made");
    exec_.reset(new Executor(&k_, &w_, err_word_));
    cuda_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  }

  ~Engine() {
    for (auto& g : graphs_) {
      if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
      if (g.second.graph) cudaGraphDestroy(g.second.graph);
      if (g.second.host) cudaFreeHost(g.second.host);
    }
    if (split_slots_) { k_.gemm_set_split_workspace(nullptr, nullptr, 0); cudaFree(split_slots_); cudaFree(split_flags_); }
    for (void* p : owned_) cudaFree(p);
    for (auto& b : bufs_) if (b.second.ptr) cudaFree(b.second.ptr);
    if (pinned_) cudaFreeHost(pinned_);
    if (cache_) qvh_destroy(cache_);
    if (stream_) cudaStreamDestroy(stream_);
  }
  Engine(const Engine&) = delete;
  Engine& operator=(const Engine&) = delete;

  const ModelDesc& desc() const { return desc_; }
  int vocab() const { return (int)desc_.vocab; }
  long long max_model_len() const { return max_model_len_; }
  int page_size() const { return page_; }
  int num_pages() const { return num_pages_; }
  cudaStream_t stream() const { return stream_; }
  const Kernels& kernels() const { return k_; }
  long long launches() const { return exec_->launches + graph_launches_; }
  long long h2d_bytes() const { return h2d_bytes_; }
  int compute_dtype() const { return dt_; }

  bool has(long long id) const { return qvh_has(cache_, id) != 0; }
  int length(long long id) const { return has(id) ? qvh_length(cache_, id) : 0; }
  int free_pages() const { return qvh_free_pages(cache_, 0); }
  int free_slots() const { return qvh_free_slots(cache_); }
  void release(long long id) { if (has(id)) qvh_release(cache_, id); }
  int one_more_token_fits(const std::vector<long long>& ids) const { return qvh_one_more_token_fits(cache_, (int)ids.size(), ids.data()); }
  long long youngest(const std::vector<long long>& ids) const {
    const int i = qvh_youngest(cache_, (int)ids.size(), ids.data());
    return i < 0 ? -1 : ids[(size_t)i];
  }
  void check_invariants() const {
    char msg[512] = {0};
    if (qvh_check(cache_, msg, sizeof(msg)) != 0) throw EngineError(std::string("cache manager: ") + msg);
  }
  bool can_run(const std::vector<StepEntry>& entries) const {
    std::vector<long long> ids;
    std::vector<int> is_new, n_new;
    for (const auto& e : entries) { ids.push_back(e.id); is_new.push_back(has(e.id) ? 0 : 1); n_new.push_back((int)e.tokens.size()); }
    return qvh_can_reserve(cache_, (int)ids.size(), ids.data(), is_new.data(), n_new.data()) != 0;
  }

  // Raises if a kernel gave up on a bounded wait since the last check (synchronises the stream).
  void check_kernel_errors() {
    int code = 0;
    cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    cuda_check(cudaMemcpyAsync(&code, err_word_, sizeof(int), cudaMemcpyDeviceToHost, stream_), "cudaMemcpyAsync");
    cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    if (code) {
      cudaMemsetAsync(err_word_, 0, sizeof(int), stream_);
      throw EngineError("a tensor-core kernel gave up waiting on a barrier (code " + std::to_string(code) + ")");
    }
  }

  // Runs one batch.  Returns the device pointer of float32 logits [rows, vocab], ordered by entry and
  // then by `want` (null when nothing is wanted; valid until the next step), and sets *rows.
  // Requests in `end` are finished after this step and what they hold is given back.  After a
  // decode-only step whose every row is wanted, greedy_ids() holds each row's argmax on the device.
  const float* step(std::vector<StepEntry> entries, const std::vector<long long>& end, int* rows) {
    *rows = 0;
    greedy_ids_ = nullptr;
    const float* logits = nullptr;
    if (!entries.empty()) {
      validate(entries);
      bool decode_only = opt_.use_graphs && (int)entries.size() <= opt_.max_graph_batch;
      for (const auto& e : entries) decode_only = decode_only && e.tokens.size() == 1;
      if (decode_only) logits = step_decode(entries, rows);
      else logits = step_general(entries, rows);
      ++steps_run;
    }
    for (long long id : end) release(id);
    return logits;
  }
  const int* greedy_ids() const { return greedy_ids_; }
  long long steps_run = 0, tokens_run = 0;

  // One token per row of `logits` (float32 [rows, vocab] on the device, as step() returned them;
  // rewritten in place by the penalties), in the order of runtime/src/sampler.cpp:43-101: penalties,
  // greedy if temperature <= 0, temperature, softmax, top-k, top-p, min-p, draw.  Rows that are plainly
  // greedy take the argmax (the captured decode step's own when it has one).
  std::vector<int> sample(const float* logits, const std::vector<SampleRow>& rows_spec) {
    const int rows = (int)rows_spec.size(), V = vocab();
    std::vector<int> host((size_t)rows);
    if (rows == 0) return host;
    int* out = (int*)buffer("sampled", (size_t)rows * 4);
    bool all_greedy = true;
    int width = 0;
    for (const auto& r : rows_spec) { all_greedy = all_greedy && r.plain_greedy(); width = std::max(width, (int)r.recent.size()); }
    if (all_greedy) {
      const int* ids = greedy_ids_;
      if (!ids) {
        if (k_.argmax(out, logits, rows, V, V, stream_) != 0) throw EngineError("argmax failed to launch");
        ids = out;
      }
      cuda_check(cudaMemcpyAsync(host.data(), ids, (size_t)rows * 4, cudaMemcpyDeviceToHost, stream_), "cudaMemcpyAsync");
      cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
      return host;
    }
    // per-row parameters: 7 float rows, then top_k and the recent tokens (-1: none) as integers
    std::vector<float> f((size_t)7 * rows);
    std::vector<int> iv((size_t)rows * (1 + width), -1);
    for (int i = 0; i < rows; ++i) {
      const SampleRow& r = rows_spec[(size_t)i];
      const float vals[7] = {r.temperature, r.top_p, r.min_p, r.uniform, r.repetition_penalty, r.frequency_penalty, r.presence_penalty};
      for (int k = 0; k < 7; ++k) f[(size_t)k * rows + i] = vals[k];
      iv[(size_t)i] = r.top_k;
      for (size_t k = 0; k < r.recent.size(); ++k) iv[(size_t)rows + (size_t)i * width + k] = r.recent[k];
    }
    float* df = (float*)buffer("sample_f", f.size() * 4);
    int* di = (int*)buffer("sample_i", iv.size() * 4);
    cuda_check(cudaMemcpyAsync(df, f.data(), f.size() * 4, cudaMemcpyHostToDevice, stream_), "cudaMemcpyAsync");
    cuda_check(cudaMemcpyAsync(di, iv.data(), iv.size() * 4, cudaMemcpyHostToDevice, stream_), "cudaMemcpyAsync");
    const int rc = k_.sample(out, (float*)logits, rows, V, V, df, di, df + rows, df + 2 * rows, df + 3 * rows, width ? di + rows : nullptr, width,
                             width ? df + 4 * rows : nullptr, width ? df + 5 * rows : nullptr, width ? df + 6 * rows : nullptr, stream_);
    if (rc != 0) throw EngineError("the sampling kernel failed to launch (code " + std::to_string(rc) + ")");
    cuda_check(cudaMemcpyAsync(host.data(), out, (size_t)rows * 4, cudaMemcpyDeviceToHost, stream_), "cudaMemcpyAsync");
    cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    return host;
  }

  // Copies `rows` logits rows to the host.
  std::vector<float> logits_to_host(const float* dev, int rows) {
    std::vector<float> out((size_t)rows * desc_.vocab);
    cuda_check(cudaMemcpyAsync(out.data(), dev, out.size() * 4, cudaMemcpyDeviceToHost, stream_), "cudaMemcpyAsync");
    cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    return out;
  }

  // A device buffer that lives as long as the engine, grown on demand (outside captured steps).
  void* buffer(const std::string& name, size_t bytes) {
    Buf& b = bufs_[name];
    if (b.bytes < bytes) {
      cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
      if (b.ptr) cudaFree(b.ptr);
      b.ptr = nullptr;
      cuda_check(cudaMalloc(&b.ptr, bytes), ("cudaMalloc of " + std::to_string(bytes) + " bytes (" + name + ")").c_str());
      b.bytes = bytes;
    }
    return b.ptr;
  }

 private:
  struct Buf { void* ptr = nullptr; size_t bytes = 0; };
  struct DecodeGraph {
    int S = 0, width = 0, n_dyn = 0;
    int* dev = nullptr;                 // [n_dyn dynamic][3 S + 1 constant] integers
    int* host = nullptr;                // pinned mirror of the dynamic part
    std::vector<long long> row_epoch;
    std::vector<int> row_len;
    float* logits = nullptr;
    int* next_ids = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    cudaEvent_t copied = nullptr;
    long long kernels = 0;
    StepIO io;
  };

  EngineOptions opt_;
  int dt_ = DT_BF16;
  Kernels k_;
  ModelDesc desc_;
  ModelW w_;
  cudaStream_t stream_ = nullptr;
  int* err_word_ = nullptr;
  float* split_slots_ = nullptr;
  int* split_flags_ = nullptr;
  int page_ = 16, num_pages_ = 0;
  long long max_model_len_ = 0;
  void* cache_ = nullptr;
  std::unique_ptr<Executor> exec_;
  std::vector<void*> owned_;
  std::map<std::string, Buf> bufs_;
  int* pinned_ = nullptr;
  size_t pinned_ints_ = 0;
  cudaEvent_t pinned_free_ = nullptr;
  std::map<int, DecodeGraph> graphs_;
  const int* greedy_ids_ = nullptr;
  long long graph_launches_ = 0, h2d_bytes_ = 0;

  void* dev_alloc(size_t bytes) {
    void* p = nullptr;
    cuda_check(cudaMalloc(&p, std::max<size_t>(bytes, 16)), ("cudaMalloc of " + std::to_string(bytes) + " bytes").c_str());
    owned_.push_back(p);
    return p;
  }
  void dev_free(void* p) {
    auto it = std::find(owned_.begin(), owned_.end(), p);
    if (it != owned_.end()) owned_.erase(it);
    cudaFree(p);
  }

  // ---------------------------------------------------------------- weights
  // Storage rule: floating tensors are bfloat16 on the bfloat16 path, except that a tensor stored in
  // 32-bit stays 32-bit; on the float32 path every floating tensor is float32.  Norm weights are
  // always float32 (exact from bfloat16).
  static int stored_dt(const StTensor& t) {
    if (t.dtype == "F32" || t.dtype == "F64") return DT_F32;
    if (t.dtype == "BF16" || t.dtype == "F16") return DT_BF16;
    throw EngineError("tensor type " + t.dtype + " is not a floating type");
  }
  static uint16_t to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7F800000u) == 0x7F800000u) return (uint16_t)((u >> 16) | ((u & 0xFFFF) ? 0x40 : 0));
    return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1)) >> 16);
  }
  // Host to device on the engine's own stream, and done when it returns.  (The stream does not wait
  // for the default stream, so every copy, fill and kernel of the engine goes through this stream;
  // a plain cudaMemcpy from pageable memory may return before its last bytes have landed.)
  void copy_in(void* dst, const void* src, size_t bytes) {
    cuda_check(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream_), "cudaMemcpyAsync");
    cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
  }
  // uploads `t` in type `want`
  void upload(void* dst, int want, const StTensor& t) {
    const size_t n = (size_t)t.numel();
    if (want == DT_F32) {
      if (t.dtype == "F32") { copy_in(dst, t.data, n * 4); return; }
      const std::vector<float> f = to_float(t);
      copy_in(dst, f.data(), n * 4);
    } else {
      if (t.dtype == "BF16") { copy_in(dst, t.data, n * 2); return; }
      const std::vector<float> f = to_float(t);
      std::vector<uint16_t> h(n);
      for (size_t i = 0; i < n; ++i) h[i] = to_bf16(f[i]);
      copy_in(dst, h.data(), n * 2);
    }
  }
  int storage_dt(const StTensor& t) const { return dt_ == DT_F32 ? DT_F32 : stored_dt(t); }

  const float* load_vector(const Checkpoint& ck, const std::string& name) {
    const StTensor& t = *ck.find(name);
    void* p = dev_alloc((size_t)t.numel() * 4);
    upload(p, DT_F32, t);
    return (const float*)p;
  }

  // One Linear from several stored matrices stacked by rows (in float32 if any of them is).
  LinearW load_linear(const Checkpoint& ck, const std::vector<std::string>& names, bool pack) {
    LinearW L;
    int dt = DT_BF16;
    for (const auto& n : names) {
      const StTensor& t = *ck.find(n);
      if (storage_dt(t) == DT_F32) dt = DT_F32;
      L.N += (int)t.shape[0];
      L.K = (int)t.shape[1];
    }
    L.dt = dt;
    const size_t es = dt_size(dt);
    uint8_t* rows = (uint8_t*)dev_alloc((size_t)L.N * L.K * es);
    size_t at = 0;
    for (const auto& n : names) {
      const StTensor& t = *ck.find(n);
      upload(rows + at, dt, t);
      at += (size_t)t.numel() * es;
    }
    L.rows = rows;
    if (pack) finish_linear(L);
    return L;
  }

  // A bfloat16 matrix is also stored as the 16 KB tiles the MMA consumes, and its rows dropped.
  void finish_linear(LinearW& L) {
    if (L.dt != DT_BF16 || dt_ != DT_BF16 || (L.K % 8) || !opt_.packed_weights) return;
    const long long bytes = k_.packed_weight_bytes(L.N, L.K);
    void* packed = dev_alloc((size_t)bytes);
    const int rc = k_.pack_weight_tiles(packed, L.rows, L.N, L.K, L.K, stream_);
    if (rc != 0) { dev_free(packed); return; }
    cuda_check(cudaStreamSynchronize(stream_), "pack_weight_tiles");
    L.packed = packed;
    dev_free((void*)L.rows);
    L.rows = nullptr;
  }

  void load_weights(const std::string& dir) {
    Checkpoint ck(dir);
    const std::string problems = check_tensors(desc_, ck, dir + "/model.safetensors");
    if (!problems.empty()) throw EngineError(problems);
    const ModelDesc& c = desc_;
    w_.dt = dt_;
    w_.d = (int)c.hidden; w_.H = (int)c.heads; w_.Hkv = (int)c.kv_heads; w_.hd = (int)c.head_dim; w_.f = (int)c.ffn; w_.V = (int)c.vocab;
    w_.page = page_; w_.eps = (float)c.eps; w_.scale = (float)c.attn_scale; w_.rot = (int)c.head_dim;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&w_.sms, cudaDevAttrMultiProcessorCount, dev);
    const StTensor& emb = *ck.find(c.embedding);
    w_.emb_dt = storage_dt(emb);
    void* e = dev_alloc((size_t)emb.numel() * dt_size(w_.emb_dt));
    upload(e, w_.emb_dt, emb);
    w_.embedding = e;
    w_.final_norm = load_vector(ck, c.final_norm);
    if (c.lm_head.empty()) {
      // a tied head is the embedding table; on the bfloat16 path it gets packed tiles of its own (the lookup reads rows)
      w_.head.rows = w_.embedding; w_.head.N = w_.V; w_.head.K = w_.d; w_.head.dt = w_.emb_dt;
      if (w_.emb_dt == DT_BF16 && dt_ == DT_BF16 && w_.d % 8 == 0 && opt_.packed_weights) {
        void* packed = dev_alloc((size_t)k_.packed_weight_bytes(w_.V, w_.d));
        if (k_.pack_weight_tiles(packed, w_.embedding, w_.V, w_.d, w_.d, stream_) == 0) {
          cuda_check(cudaStreamSynchronize(stream_), "pack_weight_tiles");
          w_.head.packed = packed;
        } else dev_free(packed);
      }
    } else {
      w_.head = load_linear(ck, {c.lm_head}, true);
    }
    for (const auto& L : c.layers) {
      LayerW lw;
      lw.norm1 = load_vector(ck, L.input_norm);
      lw.norm2 = load_vector(ck, L.post_norm);
      lw.qkv = load_linear(ck, {L.q_proj, L.k_proj, L.v_proj}, true);
      lw.o = load_linear(ck, {L.o_proj}, true);
      lw.down = load_linear(ck, {L.down_proj}, true);
      // gate and up rows interleaved in groups of 16 when the width allows, so that one tile of the
      // product holds both halves of a feature and the activation runs in the product's epilogue
      lw.interleaved = (c.ffn % 16 == 0) ? 1 : 0;
      LinearW gu = load_linear(ck, {L.gate_proj, L.up_proj}, false);
      if (lw.interleaved) {
        const size_t es = dt_size(gu.dt), row = (size_t)gu.K * es, grp = 16 * row;
        uint8_t* mixed = (uint8_t*)dev_alloc((size_t)gu.N * row);
        const uint8_t* src = (const uint8_t*)gu.rows;
        cuda_check(cudaMemcpy2DAsync(mixed, 2 * grp, src, grp, grp, (size_t)c.ffn / 16, cudaMemcpyDeviceToDevice, stream_), "cudaMemcpy2DAsync");
        cuda_check(cudaMemcpy2DAsync(mixed + grp, 2 * grp, src + (size_t)c.ffn * row, grp, grp, (size_t)c.ffn / 16, cudaMemcpyDeviceToDevice, stream_),
                   "cudaMemcpy2DAsync");
        cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
        dev_free((void*)gu.rows);
        gu.rows = mixed;
      }
      finish_linear(gu);
      lw.gate_up = gu;
      w_.layers.push_back(lw);
    }
  }

  // cos and sin of pos * f_i for every position the engine may see, angles formed in double
  void build_rotary_table() {
    const int half = w_.rot / 2;
    const std::vector<double> f = inverse_frequencies(w_.rot, desc_.theta, desc_.rope_scaling);
    std::vector<float> table((size_t)max_model_len_ * half * 2);
    for (long long p = 0; p < max_model_len_; ++p)
      for (int i = 0; i < half; ++i) {
        const double a = (double)p * f[(size_t)i];
        table[((size_t)p * half + i) * 2] = (float)std::cos(a);
        table[((size_t)p * half + i) * 2 + 1] = (float)std::sin(a);
      }
    void* d = dev_alloc(table.size() * 4);
    copy_in(d, table.data(), table.size() * 4);
    w_.cos_sin = (const float*)d;
    w_.table_rows = (int)max_model_len_;
  }

  // [layers][pages + 1][2][Hkv][page][hd]; the last page is scratch for the padded rows of a captured step
  void allocate_cache() {
    const size_t per_layer = (size_t)(num_pages_ + 1) * 2 * w_.Hkv * page_ * w_.hd * dt_size(dt_);
    uint8_t* base = (uint8_t*)dev_alloc(per_layer * w_.layers.size());
    cuda_check(cudaMemsetAsync(base, 0, per_layer * w_.layers.size(), stream_), "cudaMemsetAsync");
    cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    for (size_t l = 0; l < w_.layers.size(); ++l) {
      w_.layers[l].cache = base + l * per_layer;
      w_.layers[l].cache_pages = num_pages_ + 1;
    }
  }

  // ---------------------------------------------------------------- steps
  void validate(const std::vector<StepEntry>& entries) {
    for (size_t i = 0; i < entries.size(); ++i) {
      const StepEntry& e = entries[i];
      for (size_t j = 0; j < i; ++j)
        if (entries[j].id == e.id) throw EngineError("request " + std::to_string(e.id) + " appears twice in one step");
      if (e.tokens.empty()) throw EngineError("request " + std::to_string(e.id) + " brings no tokens");
      for (int t : e.tokens)
        if (t < 0 || t >= vocab())
          throw EngineError("request " + std::to_string(e.id) + ": token id " + std::to_string(t) + " is outside the vocabulary of " + std::to_string(vocab()));
      for (int wv : e.want)
        if (wv < 0 || wv >= (int)e.tokens.size()) throw EngineError("request " + std::to_string(e.id) + ": a wanted place is outside its tokens");
      if (length(e.id) + (long long)e.tokens.size() > max_model_len_)
        throw EngineError("request " + std::to_string(e.id) + " would hold " + std::to_string(length(e.id) + e.tokens.size()) +
                          " tokens, more than the engine's limit of " + std::to_string(max_model_len_));
    }
    if (!can_run(entries)) {
      int fresh = 0;
      for (const auto& e : entries) fresh += has(e.id) ? 0 : 1;
      if (fresh > free_slots()) throw OutOfSlots(std::to_string(fresh) + " new requests but only " + std::to_string(free_slots()) + " free request slots");
      throw OutOfPages("the step needs more pages than the " + std::to_string(free_pages()) + " that are free");
    }
  }

  void reserve(const std::vector<StepEntry>& entries) {
    for (const auto& e : entries) {
      if (!has(e.id)) qvh_admit(cache_, e.id);
      if (qvh_reserve(cache_, e.id, (int)e.tokens.size()) != 1) throw EngineError("reservation was checked for the whole step and failed all the same");
    }
  }

  int* pinned(size_t ints) {
    if (pinned_free_) cuda_check(cudaEventSynchronize(pinned_free_), "cudaEventSynchronize");   // the last copy has read the buffer
    if (pinned_ints_ < ints) {
      if (pinned_) cudaFreeHost(pinned_);
      pinned_ints_ = std::max<size_t>(1024, ints * 2);
      cuda_check(cudaMallocHost((void**)&pinned_, pinned_ints_ * 4), "cudaMallocHost");
    }
    return pinned_;
  }

  // Any mix of segments.  A mixed step runs its single-token entries first (the attention kernels then
  // serve the decoded tokens and the portions each with the kernel made for them); the logits come
  // back in the order the caller gave.
  const float* step_general(std::vector<StepEntry>& entries, int* rows) {
    const int S = (int)entries.size();
    std::vector<int> order((size_t)S);
    for (int i = 0; i < S; ++i) order[(size_t)i] = i;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return (entries[(size_t)a].tokens.size() != 1) < (entries[(size_t)b].tokens.size() != 1); });
    reserve(entries);
    int T = 0, R = 0, max_q = 0, max_ctx = 0, n1 = 0, rest_q = 0, width = 1;
    for (int i = 0; i < S; ++i) {
      const StepEntry& e = entries[(size_t)order[(size_t)i]];
      T += (int)e.tokens.size();
      R += (int)e.want.size();
      max_q = std::max(max_q, (int)e.tokens.size());
      max_ctx = std::max(max_ctx, length(e.id) + (int)e.tokens.size());
      width = std::max(width, qvh_table_len(cache_, e.id, 0));
    }
    while (n1 < S && entries[(size_t)order[(size_t)n1]].tokens.size() == 1) ++n1;
    for (int i = n1; i < S; ++i) rest_q = std::max(rest_q, (int)entries[(size_t)order[(size_t)i]].tokens.size());
    // layout: token ids, positions, segments [T each]; seg_q_start [S+1]; seg_pos0 [S]; want_rows [R]; block table [S][width]
    const size_t total = 3 * (size_t)T + (S + 1) + S + R + (size_t)S * width;
    int* h = pinned(total);
    int* tok = h; int* pos = h + T; int* seg = h + 2 * T;
    int* qstart = h + 3 * T; int* pos0 = qstart + S + 1; int* want = pos0 + S; int* table = want + R;
    std::vector<int> first_row((size_t)S);
    int row = 0, at = 0, wrow = 0, portion_ctx = 0;
    for (int i = 0; i < S; ++i) {
      const StepEntry& e = entries[(size_t)order[(size_t)i]];
      const int p0 = length(e.id), n = (int)e.tokens.size();
      qstart[i] = at; pos0[i] = p0;
      if (n > 1) portion_ctx = std::max(portion_ctx, p0 + n);
      for (int t = 0; t < n; ++t) { tok[at + t] = e.tokens[(size_t)t]; pos[at + t] = p0 + t; seg[at + t] = i; }
      first_row[(size_t)order[(size_t)i]] = wrow;
      for (int wv : e.want) want[wrow++] = at + wv;
      int* trow = table + (size_t)i * width;
      std::fill(trow, trow + width, num_pages_);               // the scratch page
      qvh_table_copy(cache_, e.id, 0, trow, width);
      for (int b = 0; b < width; ++b) if (trow[b] < 0) trow[b] = num_pages_;
      at += n;
      (void)row;
    }
    qstart[S] = T;
    int* dev = (int*)buffer("step_ints", total * 4);
    cuda_check(cudaMemcpyAsync(dev, h, total * 4, cudaMemcpyHostToDevice, stream_), "cudaMemcpyAsync");
    if (!pinned_free_) cuda_check(cudaEventCreateWithFlags(&pinned_free_, cudaEventDisableTiming), "cudaEventCreate");
    cuda_check(cudaEventRecord(pinned_free_, stream_), "cudaEventRecord");
    h2d_bytes_ += (long long)total * 4;
    StepIO io;
    io.T = T; io.S = S; io.R = R; io.n1 = n1; io.max_q_len = max_q; io.max_ctx_len = max_ctx; io.rest_max_q = rest_q; io.captured = 0;
    io.portion_max_ctx = portion_ctx;
    io.token_ids = dev; io.tok_pos = dev + T; io.tok_seg = dev + 2 * T; io.seg_q_start = dev + 3 * T; io.seg_pos0 = dev + 3 * T + S + 1;
    io.want_rows = dev + 3 * T + 2 * S + 1; io.block_table = dev + 3 * T + 2 * S + 1 + R; io.max_blocks = width;
    float* logits = R > 0 ? (float*)buffer("logits", (size_t)R * w_.V * 4) : nullptr;
    io.logits = logits;
    Arena ws;
    ws.size = workspace_bytes(w_, T, R, n1);
    ws.base = (uint8_t*)buffer("workspace", ws.size);
    exec_->forward(io, ws, stream_);
    for (const auto& e : entries) qvh_commit(cache_, e.id, (int)e.tokens.size());
    tokens_run += T;
    *rows = R;
    if (R == 0) return nullptr;
    // back into the caller's order when the step's own order differs
    bool same = true;
    for (int i = 0; i < S; ++i) same = same && order[(size_t)i] == i;
    if (same) return logits;
    float* sorted = (float*)buffer("logits_sorted", (size_t)R * w_.V * 4);
    int out_row = 0;
    for (int i = 0; i < S; ++i) {
      const int n = (int)entries[(size_t)i].want.size();
      if (n) cuda_check(cudaMemcpyAsync(sorted + (size_t)out_row * w_.V, logits + (size_t)first_row[(size_t)i] * w_.V, (size_t)n * w_.V * 4,
                                        cudaMemcpyDeviceToDevice, stream_), "cudaMemcpyAsync");
      out_row += n;
    }
    return sorted;
  }

  static int bucket(int n) {
    int b = 1;
    while (b < n) b *= 2;
    return b;
  }

  // The captured decode step that holds S requests (rows beyond the live ones are padding: token 0 at
  // position 0 of the scratch page).  It ends with a greedy argmax whose result is also written
  // into the token slots, so that a decode loop can run with its tokens never leaving the device.
  DecodeGraph& decode_graph(int n) {
    const int S = bucket(n);
    auto it = graphs_.find(S);
    if (it != graphs_.end()) return it->second;
    DecodeGraph& g = graphs_[S];
    g.S = S;
    g.width = (int)((max_model_len_ + page_ - 1) / page_);
    g.n_dyn = 4 * S + S * g.width;
    const size_t total = (size_t)g.n_dyn + 3 * S + 1;
    g.dev = (int*)dev_alloc(total * 4);
    cuda_check(cudaMallocHost((void**)&g.host, (size_t)g.n_dyn * 4), "cudaMallocHost");
    std::vector<int> init(total, 0);
    for (int i = 0; i < S; ++i) init[(size_t)3 * S + i] = opt_.max_requests;              // scratch slot
    for (int i = 4 * S; i < g.n_dyn; ++i) init[(size_t)i] = num_pages_;                   // scratch page
    const int o = g.n_dyn;
    for (int i = 0; i < S; ++i) { init[(size_t)o + i] = i; init[(size_t)o + 2 * S + 1 + i] = i; }     // tok_seg, want_rows
    for (int i = 0; i <= S; ++i) init[(size_t)o + S + i] = i;                             // seg_q_start
    std::memcpy(g.host, init.data(), (size_t)g.n_dyn * 4);
    copy_in(g.dev, init.data(), total * 4);
    g.row_epoch.assign((size_t)S, 0);
    g.row_len.assign((size_t)S, 0);
    g.logits = (float*)dev_alloc((size_t)S * w_.V * 4);
    g.next_ids = (int*)dev_alloc((size_t)S * 4);
    cuda_check(cudaEventCreateWithFlags(&g.copied, cudaEventDisableTiming), "cudaEventCreate");
    StepIO& io = g.io;
    io.T = S; io.S = S; io.R = S; io.n1 = S; io.max_q_len = 1; io.max_ctx_len = (int)max_model_len_; io.rest_max_q = 0; io.captured = 1;
    io.token_ids = g.dev; io.tok_pos = g.dev + S; io.seg_pos0 = g.dev + 2 * S; io.block_table = g.dev + 4 * S; io.max_blocks = g.width;
    io.tok_seg = g.dev + o; io.seg_q_start = g.dev + o + S; io.want_rows = g.dev + o + 2 * S + 1;
    io.logits = g.logits;
    Arena ws;
    ws.size = workspace_bytes(w_, S, S, S);
    ws.base = (uint8_t*)dev_alloc(ws.size);                    // a captured step keeps its own workspace
    auto run = [&]() {
      exec_->forward(io, ws, stream_);
      if (k_.argmax(g.next_ids, g.logits, S, w_.V, w_.V, stream_) != 0) throw EngineError("argmax failed to launch");
      cuda_check(cudaMemcpyAsync(g.dev, g.next_ids, (size_t)S * 4, cudaMemcpyDeviceToDevice, stream_), "cudaMemcpyAsync");
    };
    run();                                                      // sets function attributes, warms up
    cuda_check(cudaStreamSynchronize(stream_), "cudaStreamSynchronize");
    const long long before = exec_->launches;
    cuda_check(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
    try {
      run();
    } catch (...) {
      cudaGraph_t broken = nullptr;
      cudaStreamEndCapture(stream_, &broken);
      if (broken) cudaGraphDestroy(broken);
      throw;
    }
    cuda_check(cudaStreamEndCapture(stream_, &g.graph), "cudaStreamEndCapture");
    cuda_check(cudaGraphInstantiate(&g.exec, g.graph, 0), "cudaGraphInstantiate");
    g.kernels = exec_->launches - before + 1;
    exec_->launches = before;                                   // the capture itself launched nothing
    cuda_check(cudaMemsetAsync(g.dev, 0, (size_t)S * 4, stream_), "cudaMemsetAsync");
    return g;
  }

  const float* step_decode(const std::vector<StepEntry>& entries, int* rows) {
    const int n = (int)entries.size();
    for (const auto& e : entries) {
      if (!has(e.id)) qvh_admit(cache_, e.id);
      if (qvh_reserve(cache_, e.id, 1) != 1) throw EngineError("reservation was checked for the whole step and failed all the same");
    }
    DecodeGraph& g = decode_graph(n);
    std::vector<long long> ids;
    std::vector<int> toks;
    for (const auto& e : entries) { ids.push_back(e.id); toks.push_back(e.tokens[0]); }
    run_decode_graph(g, ids, device_tokens_ ? nullptr : toks.data());
    device_tokens_ = false;
    for (const auto& e : entries) qvh_commit(cache_, e.id, 1);
    tokens_run += n;
    int wanted = 0;
    for (const auto& e : entries) wanted += e.want.empty() ? 0 : 1;
    *rows = wanted;
    if (wanted == 0) return nullptr;
    if (wanted == n) { greedy_ids_ = g.next_ids; return g.logits; }
    float* some = (float*)buffer("logits_sorted", (size_t)wanted * w_.V * 4);
    int out_row = 0;
    for (int i = 0; i < n; ++i)
      if (!entries[(size_t)i].want.empty())
        cuda_check(cudaMemcpyAsync(some + (size_t)(out_row++) * w_.V, g.logits + (size_t)i * w_.V, (size_t)w_.V * 4, cudaMemcpyDeviceToDevice, stream_),
                   "cudaMemcpyAsync");
    return some;
  }

  bool device_tokens_ = false;

 public:
  // The next decode-only step feeds the ids the last replay of its graph left on the device (its
  // greedy argmax) instead of the entries' own tokens.
  void feed_device_tokens() { device_tokens_ = true; }

 private:
  void run_decode_graph(DecodeGraph& g, const std::vector<long long>& ids, const int* tokens) {
    cuda_check(cudaEventSynchronize(g.copied), "cudaEventSynchronize");       // the last copy has read the mirror
    if (qvh_fill_decode(cache_, (int)ids.size(), ids.data(), tokens, g.S, g.width, num_pages_, opt_.max_requests, g.host, g.row_epoch.data(),
                        g.row_len.data()) != 0)
      throw EngineError("a request of the decode step is not live");
    const int lo = tokens ? 0 : g.S;
    cuda_check(cudaMemcpyAsync(g.dev + lo, g.host + lo, (size_t)(g.n_dyn - lo) * 4, cudaMemcpyHostToDevice, stream_), "cudaMemcpyAsync");
    cuda_check(cudaEventRecord(g.copied, stream_), "cudaEventRecord");
    h2d_bytes_ += (long long)(g.n_dyn - lo) * 4;
    cuda_check(cudaGraphLaunch(g.exec, stream_), "cudaGraphLaunch");
    graph_launches_ += g.kernels;
  }
};

}  // namespace qv
