// C interface of the step executor (executor.hpp) for a host that keeps its tensors elsewhere: the
// Python step function builds one of these from the weight and cache tensors of its parts when
// every block of the model is a pre-norm block of RMS norm, rotary attention and SwiGLU, and then
// hands it whole steps (one call instead of a dozen launches' worth of calls a layer).
#include <cstring>
#include <memory>

#include "executor.hpp"

extern "C" {

struct QvxLinear {
  const void* rows;
  const void* packed;
  int N, K, dt, pad;
};

struct QvxLayer {
  const float* norm1;
  const float* norm2;
  QvxLinear qkv, o, gate_up, down;
  void* cache;
  long long cache_pages;
  int interleaved, window;
};

struct QvxModel {
  int dt, d, H, Hkv, hd, f, V, page, rot, table_rows, sms, emb_dt, n_layers, pad;
  float eps, scale;
  const float* cos_sin;
  const void* embedding;
  const float* final_norm;
  QvxLinear head;
  const QvxLayer* layers;
};

struct QvxStep {
  int T, S, R, n1, max_q_len, max_ctx_len, rest_max_q, captured, max_blocks, portion_max_ctx;
  const int* token_ids;
  const int* tok_pos;
  const int* tok_seg;
  const int* seg_q_start;
  const int* seg_pos0;
  const int* block_table;
  const int* want_rows;
  float* logits;
};

}  // extern "C"

namespace {

struct Handle {
  qv::Kernels kernels;
  qv::ModelW model;
  std::unique_ptr<qv::Executor> exec;
};

thread_local std::string g_error;

qv::LinearW linear(const QvxLinear& l) {
  qv::LinearW w;
  w.rows = l.rows; w.packed = l.packed; w.N = l.N; w.K = l.K; w.dt = l.dt;
  return w;
}

}  // namespace

extern "C" {

const char* qvx_last_error() { return g_error.c_str(); }

// `manifest`: "name=path" lines of the kernel libraries.  Null on failure (qvx_last_error says why).
void* qvx_create(const char* manifest, const QvxModel* m, int* err_word) {
  try {
    auto h = std::make_unique<Handle>();
    h->kernels.load(qv::read_manifest(manifest));
    qv::ModelW& w = h->model;
    w.dt = m->dt; w.d = m->d; w.H = m->H; w.Hkv = m->Hkv; w.hd = m->hd; w.f = m->f; w.V = m->V; w.page = m->page; w.rot = m->rot;
    w.table_rows = m->table_rows; w.sms = m->sms; w.eps = m->eps; w.scale = m->scale; w.cos_sin = m->cos_sin; w.embedding = m->embedding;
    w.emb_dt = m->emb_dt; w.final_norm = m->final_norm; w.head = linear(m->head);
    for (int i = 0; i < m->n_layers; ++i) {
      const QvxLayer& s = m->layers[i];
      qv::LayerW l;
      l.norm1 = s.norm1; l.norm2 = s.norm2; l.qkv = linear(s.qkv); l.o = linear(s.o); l.gate_up = linear(s.gate_up); l.down = linear(s.down);
      l.interleaved = s.interleaved; l.cache = s.cache; l.cache_pages = s.cache_pages; l.window = s.window;
      w.layers.push_back(l);
    }
    h->exec.reset(new qv::Executor(&h->kernels, &h->model, err_word));
    return h.release();
  } catch (const std::exception& e) {
    g_error = e.what();
    return nullptr;
  }
}

void qvx_destroy(void* h) { delete (Handle*)h; }

long long qvx_workspace_bytes(void* h, int T, int R, int n_decode) { return (long long)qv::workspace_bytes(((Handle*)h)->model, T, R, n_decode); }

// Runs the step's forward pass on `stream`; returns the number of kernels launched, or -1 (qvx_last_error says why).
long long qvx_forward(void* hv, const QvxStep* s, void* workspace, long long workspace_bytes, void* stream) {
  Handle* h = (Handle*)hv;
  try {
    qv::StepIO io;
    io.T = s->T; io.S = s->S; io.R = s->R; io.n1 = s->n1; io.max_q_len = s->max_q_len; io.max_ctx_len = s->max_ctx_len;
    io.rest_max_q = s->rest_max_q; io.captured = s->captured; io.max_blocks = s->max_blocks; io.portion_max_ctx = s->portion_max_ctx;
    io.token_ids = s->token_ids; io.tok_pos = s->tok_pos; io.tok_seg = s->tok_seg; io.seg_q_start = s->seg_q_start; io.seg_pos0 = s->seg_pos0;
    io.block_table = s->block_table; io.want_rows = s->want_rows; io.logits = s->logits;
    qv::Arena ws;
    ws.base = (uint8_t*)workspace; ws.size = (size_t)workspace_bytes;
    const long long before = h->exec->launches;
    h->exec->forward(io, ws, (cudaStream_t)stream);
    return h->exec->launches - before;
  } catch (const std::exception& e) {
    g_error = e.what();
    return -1;
  }
}

// how often the kernel of route `r` (enum qv::Route) has served since the library was loaded
long long qvx_route_count(int r) { return (r >= 0 && r < qv::ROUTE_COUNT) ? qv::route_counts()[r] : -1; }

}  // extern "C"
