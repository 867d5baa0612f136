// Times the UNMODIFIED reference CUDA backend (cuda/src/cuda_backend.cu of QorVix) through its
// own public API: createGpuModel + GpuModel::forward(session, token, pos)
// (cuda/include/qorvix/cuda/gpu_model.hpp:15-82).  Nothing of qorvix_b200 is linked or used.
//
// The reference's GPU model is float32, one token of one session per forward, with the logits
// copied to the host after every forward (cuda_backend.cu:1449, 1510).  A "decode step" of batch
// B is one forward per session for B sessions, which is what its forwardBatch default does
// (runtime/include/qorvix/runtime/inference_engine.hpp:61-66); a prefill of T tokens is T
// forwards (runtime/include/qorvix/runtime/benchmark.hpp:89).  The token stream is the
// reference's own hash stream (benchmark.hpp:75).  Weights are random float32 (one random layer's
// matrices are shared by every layer on the host side, so that the host holds 3 GB and not 32;
// each layer still gets its own copy in device memory, as the reference allocates it).
//
// Prints one JSON object on standard output.
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "qorvix/cuda/gpu_model.hpp"

namespace {

struct Args {
  int layers = 32, hidden = 4096, heads = 32, kv = 8, hd = 128, ffn = 14336, vocab = 128256;
  int batch = 8, ctx = 1024, steps = 16, warmup = 3, prefill = 2048, fill = 1;
  float eps = 1e-5f, theta = 500000.0f;
};

int intArg(int argc, char** argv, const char* flag, int def) {
  for (int i = 1; i + 1 < argc; ++i)
    if (!std::strcmp(argv[i], flag)) return std::atoi(argv[i + 1]);
  return def;
}
float floatArg(int argc, char** argv, const char* flag, float def) {
  for (int i = 1; i + 1 < argc; ++i)
    if (!std::strcmp(argv[i], flag)) return static_cast<float>(std::atof(argv[i + 1]));
  return def;
}

// About N(0, 0.02): the sum of four uniforms, centred and scaled (the values do not matter to the
// timing; they only have to keep the activations finite).
void fillRandom(std::vector<float>& v, std::uint64_t seed, float stddev) {
  std::uint64_t s = seed * 0x9E3779B97F4A7C15ull + 0x1234567ull;
  const float scale = stddev * 1.7320508f / 65536.0f;      // var of the sum of 4 U(0,65536) = 4 * 65536^2 / 12
  for (auto& x : v) {
    s ^= s << 13; s ^= s >> 7; s ^= s << 17;
    const std::uint32_t a = s & 0xFFFF, b = (s >> 16) & 0xFFFF, c = (s >> 32) & 0xFFFF, d = (s >> 48) & 0xFFFF;
    x = (static_cast<float>(a + b + c + d) - 131070.0f) * scale;
  }
}

double seconds(std::chrono::steady_clock::time_point a, std::chrono::steady_clock::time_point b) {
  return std::chrono::duration<double>(b - a).count();
}

}  // namespace

int main(int argc, char** argv) {
  using namespace qorvix::cuda;
  using clock = std::chrono::steady_clock;
  Args a;
  a.layers = intArg(argc, argv, "--layers", a.layers);
  a.hidden = intArg(argc, argv, "--hidden", a.hidden);
  a.heads = intArg(argc, argv, "--heads", a.heads);
  a.kv = intArg(argc, argv, "--kv-heads", a.kv);
  a.hd = intArg(argc, argv, "--head-dim", a.hd);
  a.ffn = intArg(argc, argv, "--ffn", a.ffn);
  a.vocab = intArg(argc, argv, "--vocab", a.vocab);
  a.batch = intArg(argc, argv, "--batch", a.batch);
  a.ctx = intArg(argc, argv, "--ctx", a.ctx);
  a.steps = intArg(argc, argv, "--steps", a.steps);
  a.warmup = intArg(argc, argv, "--warmup", a.warmup);
  a.prefill = intArg(argc, argv, "--prefill", a.prefill);
  a.fill = intArg(argc, argv, "--fill", a.fill);
  a.eps = floatArg(argc, argv, "--eps", a.eps);
  a.theta = floatArg(argc, argv, "--rope-theta", a.theta);
  if (a.heads * a.hd != a.hidden) {
    // the reference sizes q as [dModel] in places (runtime/src/weights.cpp:37); its GPU model takes headDim apart
    std::fprintf(stderr, "note: heads*head_dim != hidden; the reference's GPU model still runs (q is heads*head_dim wide)\n");
  }
  const int maxSeq = std::max(a.prefill, a.ctx + a.steps + a.warmup) + 8;

  const auto t0 = clock::now();
  const std::size_t d = a.hidden, kvDim = static_cast<std::size_t>(a.kv) * a.hd, qDim = static_cast<std::size_t>(a.heads) * a.hd;
  std::vector<float> emb(static_cast<std::size_t>(a.vocab) * d), norm(d, 1.0f);
  std::vector<float> wq(qDim * d), wk(kvDim * d), wv(kvDim * d), wo(d * qDim), wg(static_cast<std::size_t>(a.ffn) * d),
      wu(static_cast<std::size_t>(a.ffn) * d), wd(d * static_cast<std::size_t>(a.ffn));
  fillRandom(emb, 1, 0.02f);
  fillRandom(wq, 2, 0.02f); fillRandom(wk, 3, 0.02f); fillRandom(wv, 4, 0.02f); fillRandom(wo, 5, 0.02f);
  fillRandom(wg, 6, 0.02f); fillRandom(wu, 7, 0.02f); fillRandom(wd, 8, 0.02f);

  GpuModelConfig cfg;
  cfg.nLayers = a.layers; cfg.dModel = a.hidden; cfg.nHeads = a.heads; cfg.headDim = a.hd; cfg.nKv = a.kv;
  cfg.ffn = a.ffn; cfg.vocab = a.vocab; cfg.maxSeq = maxSeq; cfg.normEps = a.eps; cfg.ropeFreqBase = a.theta;
  auto W = [](const std::vector<float>& v, int rows, int cols) {
    GpuWeight w; w.host = v.data(); w.ggmlType = 0; w.rows = rows; w.cols = cols; return w;
  };
  std::vector<GpuLayer> layers(a.layers);
  for (auto& L : layers) {
    L.attnNorm = norm.data(); L.ffnNorm = norm.data();
    L.wq = W(wq, static_cast<int>(qDim), a.hidden); L.wk = W(wk, static_cast<int>(kvDim), a.hidden);
    L.wv = W(wv, static_cast<int>(kvDim), a.hidden); L.wo = W(wo, a.hidden, static_cast<int>(qDim));
    L.ffnGate = W(wg, a.ffn, a.hidden); L.ffnUp = W(wu, a.ffn, a.hidden); L.ffnDown = W(wd, a.hidden, a.ffn);
  }
  // an untied head of its own values would cost another 2 GB of host memory for nothing: the head reads the table's bytes
  const GpuWeight head = W(emb, a.vocab, a.hidden);
  std::string err;
  auto model = createGpuModel(cfg, emb.data(), norm.data(), head, layers, err, a.batch);
  if (!model) {
    std::printf("{\"error\": \"createGpuModel: %s\"}\n", err.c_str());
    return 1;
  }
  cudaDeviceSynchronize();
  const double loadSec = seconds(t0, clock::now());
  std::fprintf(stderr, "[ref_bench] model on the device after %.1f s\n", loadSec);

  const unsigned vocab = static_cast<unsigned>(a.vocab);
  auto tokenAt = [vocab](int i) { return static_cast<int>((static_cast<unsigned>(i) * 2654435761u) % vocab); };

  cudaEvent_t e0, e1;
  cudaEventCreate(&e0); cudaEventCreate(&e1);

  // ---- prefill: T forwards of one session (warm-up of a few tokens first: graph capture, clocks)
  std::vector<int> sessions;
  for (int b = 0; b < a.batch; ++b) sessions.push_back(model->openSession());
  for (int i = 0; i < 4; ++i) model->forward(sessions[0], tokenAt(i), i);
  double prefillMs = 0.0, prefillWall = 0.0;
  if (a.prefill > 0) {
    cudaDeviceSynchronize();
    const auto tp = clock::now();
    cudaEventRecord(e0, 0);
    for (int i = 0; i < a.prefill; ++i) model->forward(sessions[0], tokenAt(i), i);
    cudaEventRecord(e1, 0);
    cudaEventSynchronize(e1);
    prefillWall = seconds(tp, clock::now());
    float ms = 0; cudaEventElapsedTime(&ms, e0, e1); prefillMs = ms;
    std::fprintf(stderr, "[ref_bench] prefill of %d tokens: %.1f s\n", a.prefill, prefillWall);
  }

  // ---- contexts.  Session 0 keeps what the prefill wrote when that is enough.  --fill 1: every other
  // session gets its ctx-1 tokens through forward() too (minutes at the reference's speed);
  // --fill 0: the other sessions decode over cache slices nothing has written yet.  The time of a
  // decode step is the same either way: the reference's kernels read the same bytes and take no
  // decision from a cached value (cuda_backend.cu:347-395 walks positions 0..pos whatever they hold).
  const int have0 = a.prefill >= a.ctx - 1 ? a.ctx - 1 : 0;
  const auto tf = clock::now();
  for (int b = 0; b < (a.fill ? a.batch : 1); ++b)
    for (int i = (b == 0 ? have0 : 0); i < a.ctx - 1; ++i) model->forward(sessions[b], tokenAt(i + b), i);
  std::fprintf(stderr, "[ref_bench] contexts of %d tokens for %d sessions: %.1f s\n", a.ctx - 1, a.batch, seconds(tf, clock::now()));

  // ---- decode: a step is one forward for each session
  int pos = a.ctx - 1;
  for (int w = 0; w < a.warmup; ++w, ++pos)
    for (int b = 0; b < a.batch; ++b) model->forward(sessions[b], tokenAt(pos + b), pos);
  cudaDeviceSynchronize();
  const auto td = clock::now();
  cudaEventRecord(e0, 0);
  float sink = 0.0f;
  for (int s = 0; s < a.steps; ++s, ++pos)
    for (int b = 0; b < a.batch; ++b) sink += model->forward(sessions[b], tokenAt(pos + b), pos)[0];
  cudaEventRecord(e1, 0);
  cudaEventSynchronize(e1);
  const double decodeWall = seconds(td, clock::now());
  float decodeMs = 0; cudaEventElapsedTime(&decodeMs, e0, e1);
  cudaError_t ce = cudaGetLastError();
  if (ce != cudaSuccess) {
    std::printf("{\"error\": \"%s\"}\n", cudaGetErrorString(ce));
    return 1;
  }
  std::printf("{\"decode_ms_per_step\": %.4f, \"decode_wall_ms_per_step\": %.4f, \"prefill_ms\": %.3f, \"prefill_wall_ms\": %.3f, "
              "\"prefill_tokens\": %d, \"batch\": %d, \"ctx\": %d, \"steps\": %d, \"warmup\": %d, \"filled\": %d, \"load_s\": %.1f, "
              "\"d2h_bytes_per_step\": %zu, \"h2d_bytes_per_step\": %d, \"forwards_per_step\": %d, \"finite\": %d}\n",
              decodeMs / a.steps, decodeWall * 1e3 / a.steps, prefillMs, prefillWall * 1e3, a.prefill, a.batch, a.ctx, a.steps,
              a.warmup, a.fill, loadSec, static_cast<std::size_t>(a.batch) * a.vocab * 4, a.batch * 8, a.batch,
              (sink == sink) ? 1 : 0);
  return 0;
}
