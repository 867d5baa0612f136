// The native command line, in the reference's manner (core/src/main.cpp:4280-4324 dispatches on the
// first word; flags are `--flag value`, core/src/main.cpp:269-303):
//
//   qorvix-native generate <model_dir> --tokens 1,2,3 | --random-prompt N  [--max N] [--temp T] [--top-k K]
//                          [--top-p P] [--seed S] [--dtype bfloat16|float32]
//   qorvix-native bench <model_dir> [--prompt N] [--gen N] [--warmup N] [--runs N] [--batch B] [--dtype D] [--json]
//   qorvix-native replay --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N     (steps as JSON lines on stdin)
//   qorvix-native model-info <model_dir>
//   qorvix-native gpu-check <model_dir> [--tokens ... | --random-prompt N]
//
// `generate` keeps the reference's option names and defaults (--max 128, --temp 0.8, --top-k 40,
// --top-p 0.95, --seed 0; core/src/main.cpp:499-503) and its summary lines (core/src/main.cpp:433-444);
// prompts are token ids, since tokenizers are out of scope.  `bench` is the reference's
// (runtime/include/qorvix/runtime/benchmark.hpp:54-115): its hash token stream, warm-up runs discarded,
// medians reported.  `gpu-check` is core/src/main.cpp:3629-3680 with the plain C++ decoder of
// csrc/ref/ as the CPU side.  Everything runs through the native Engine and Scheduler (csrc/host/).
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <iostream>
#include <numeric>
#include <sstream>

#include "../host/engine.hpp"
#include "../host/scheduler.hpp"

extern "C" {
// csrc/ref/ref_model.cpp
const char* qvr_last_error();
void* qvr_model_open(const char* dir);
void qvr_model_close(void* h);
int qvr_forward(void* h, const int* tokens, int n, float* logits);
}

namespace {

using Args = std::vector<std::string>;

std::string flag(const Args& a, const std::string& name, const std::string& def) {
  for (size_t i = 0; i + 1 < a.size(); ++i)
    if (a[i] == name) return a[i + 1];
  return def;
}
bool has_flag(const Args& a, const std::string& name) { return std::find(a.begin(), a.end(), name) != a.end(); }

double now_s() { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); }

std::string exe_dir() {
  char buf[4096];
  const ssize_t n = readlink("/proc/self/exe", buf, sizeof(buf) - 1);
  if (n <= 0) return ".";
  std::string p(buf, (size_t)n);
  return p.substr(0, p.rfind('/'));
}

std::map<std::string, std::string> kernel_libs(const Args& a) {
  const char* env = std::getenv("QORVIX_KERNEL_MANIFEST");
  return qv::read_manifest(flag(a, "--kernels", env ? env : exe_dir() + "/kernels.manifest"));
}

// the reference's token stream (benchmark.hpp:75), shifted by a seed
int stream_token(long long i, unsigned seed, int vocab) { return (int)(((unsigned)(i + seed) * 2654435761u) % (unsigned)vocab); }

std::vector<int> prompt_from(const Args& a, int vocab) {
  std::vector<int> out;
  const std::string toks = flag(a, "--tokens", "");
  if (!toks.empty()) {
    std::stringstream ss(toks);
    std::string item;
    while (std::getline(ss, item, ','))
      if (!item.empty()) out.push_back(std::atoi(item.c_str()));
    return out;
  }
  const int n = std::atoi(flag(a, "--random-prompt", "0").c_str());
  const unsigned seed = (unsigned)std::strtoul(flag(a, "--seed", "0").c_str(), nullptr, 10);
  for (int i = 0; i < n; ++i) out.push_back(stream_token(i, seed, vocab));
  return out;
}

int cmd_generate(const Args& a) {
  if (a.size() < 2) {
    std::fprintf(stderr, "usage: qorvix-native generate <model_dir> --tokens 1,2,3 | --random-prompt N [--max N] [--temp T] [--top-k K] "
                         "[--top-p P] [--seed S] [--dtype bfloat16|float32]\n");
    return 1;
  }
  const std::string dir = a[1];
  const qv::ModelDesc desc = qv::model_desc_from_config(qv::parse_json(qv::read_text_file(dir + "/config.json")));
  const std::vector<int> prompt = prompt_from(a, (int)desc.vocab);
  if (prompt.empty()) {
    std::fprintf(stderr, "error: give the prompt as --tokens 1,2,3 or --random-prompt N\n");
    return 1;
  }
  qv::SamplingParams sp;
  sp.temperature = std::atof(flag(a, "--temp", "0.8").c_str());
  sp.top_k = std::atoi(flag(a, "--top-k", "40").c_str());
  sp.top_p = std::atof(flag(a, "--top-p", "0.95").c_str());
  sp.seed = std::strtoull(flag(a, "--seed", "0").c_str(), nullptr, 10);
  sp.max_new_tokens = std::atoi(flag(a, "--max", "128").c_str());
  const double t0 = now_s();
  const long long max_seq = (long long)prompt.size() + sp.max_new_tokens + 4;       // as the reference sizes its engine (main.cpp:566)
  qv::EngineOptions opt;
  opt.dtype = flag(a, "--dtype", "bfloat16");
  opt.max_tokens = max_seq + 64; opt.max_requests = 1; opt.max_model_len = max_seq;
  qv::Engine engine(dir, opt, kernel_libs(a));
  const double load_s = now_s() - t0;
  for (size_t i = 0; i < prompt.size(); ++i) std::printf("%s%d", i ? " " : "", prompt[i]);
  std::printf("\n");
  std::fflush(stdout);
  qv::SchedulerConfig sc;
  sc.max_concurrent = 1;
  qv::SchedulerT<qv::Engine> sched(&engine, sc, desc.eos_token_ids);
  const double t1 = now_s();
  sched.submit(prompt, sp, 0, [](long long, int tok) { std::printf("%d ", tok); std::fflush(stdout); });
  const auto results = sched.run_to_completion();
  cudaStreamSynchronize(engine.stream());
  const double secs = now_s() - t1;
  engine.check_kernel_errors();
  const qv::RequestResult& r = results.at(0);
  const size_t forwards = prompt.size() + r.tokens.size();
  std::printf("\n\n[cuda | %zu prompt tokens, %zu generated%s]\n", prompt.size(), r.tokens.size(), r.hit_eos ? ", eos" : "");
  std::printf("[load %.1fs | %zu forwards in %.2fs = %.2f tok/s]\n", load_s, forwards, secs, forwards / std::max(secs, 1e-9));
  return 0;
}

int cmd_model_info(const Args& a) {
  if (a.size() < 2) { std::fprintf(stderr, "usage: qorvix-native model-info <model_dir>\n"); return 1; }
  const qv::ModelDesc d = qv::model_desc_from_config(qv::parse_json(qv::read_text_file(a[1] + "/config.json")));
  long long params = 0;
  for (const auto& kv : d.expected()) {
    long long n = 1;
    for (long long s : kv.second) n *= s;
    params += n;
  }
  std::printf("{\"architecture\": \"%s\", \"vocab_size\": %lld, \"hidden_size\": %lld, \"intermediate_size\": %lld, \"num_hidden_layers\": %zu, "
              "\"num_attention_heads\": %lld, \"num_key_value_heads\": %lld, \"head_dim\": %lld, \"max_position_embeddings\": %lld, "
              "\"rms_norm_eps\": %g, \"rope_theta\": %g, \"rope_scaling\": %s, \"tie_word_embeddings\": %s, \"parameters\": %lld}\n",
              d.architecture.c_str(), d.vocab, d.hidden, d.ffn, d.layers.size(), d.heads, d.kv_heads, d.head_dim, d.max_position, d.eps, d.theta,
              d.rope_scaling.present ? "\"llama3\"" : "null", d.lm_head.empty() ? "true" : "false", params);
  return 0;
}

double median(std::vector<double> v) {
  std::sort(v.begin(), v.end());
  const size_t n = v.size();
  return n == 0 ? 0.0 : (n % 2 ? v[n / 2] : 0.5 * (v[n / 2 - 1] + v[n / 2]));
}

int cmd_bench(const Args& a) {
  if (a.size() < 2) {
    std::fprintf(stderr, "usage: qorvix-native bench <model_dir> [--prompt N] [--gen N] [--warmup N] [--runs N] [--batch B] [--dtype D] [--json]\n");
    return 1;
  }
  const int P = std::atoi(flag(a, "--prompt", "64").c_str()), G = std::atoi(flag(a, "--gen", "128").c_str());
  const int warm = std::atoi(flag(a, "--warmup", "1").c_str()), runs = std::atoi(flag(a, "--runs", "3").c_str());
  const int B = std::atoi(flag(a, "--batch", "1").c_str());
  const double t0 = now_s();
  qv::EngineOptions opt;
  opt.dtype = flag(a, "--dtype", "bfloat16");
  opt.max_tokens = (long long)B * (P + G + 64); opt.max_requests = B;
  qv::Engine engine(a[1], opt, kernel_libs(a));
  const double load_s = now_s() - t0;
  const int V = engine.vocab();
  std::vector<double> pre, dec;
  for (int it = 0; it < warm + runs; ++it) {
    std::vector<qv::StepEntry> entries;
    for (int b = 0; b < B; ++b) {
      qv::StepEntry e;
      e.id = b + 1;
      for (int i = 0; i < P; ++i) e.tokens.push_back(stream_token(i, 0, V));
      e.want = {P - 1};
      entries.push_back(std::move(e));
    }
    cudaStreamSynchronize(engine.stream());
    double t = now_s();
    int rows = 0;
    engine.step(entries, {}, &rows);
    cudaStreamSynchronize(engine.stream());
    const double t_pre = now_s() - t;
    t = now_s();
    for (int g = 0; g < G; ++g) {
      std::vector<qv::StepEntry> d;
      for (int b = 0; b < B; ++b) d.push_back({b + 1, {stream_token(P + g, 0, V)}, {0}});
      engine.step(d, {}, &rows);
    }
    cudaStreamSynchronize(engine.stream());
    const double t_dec = now_s() - t;
    for (int b = 0; b < B; ++b) engine.release(b + 1);
    if (it >= warm) { pre.push_back(B * P / t_pre); dec.push_back(t_dec / std::max(G, 1) * 1e3); }
  }
  engine.check_kernel_errors();
  const double dm = median(dec);
  if (has_flag(a, "--json")) {
    std::printf("{\"backend\": \"cuda\", \"prompt_tokens\": %d, \"gen_tokens\": %d, \"batch\": %d, \"timed_runs\": %d, \"load_sec\": %.3f, "
                "\"prefill_tok_per_sec\": %.2f, \"decode_tok_per_sec\": %.2f, \"decode_ms_per_tok_median\": %.4f, \"decode_ms_per_tok_min\": %.4f, "
                "\"decode_ms_per_tok_max\": %.4f}\n", P, G, B, runs, load_s, median(pre), B * 1e3 / dm, dm, *std::min_element(dec.begin(), dec.end()),
                *std::max_element(dec.begin(), dec.end()));
  } else {
    std::printf("\n==== qorvix bench: cuda ====\n  model          : %s\n  load           : %.2f s\n  prompt / gen   : %d / %d tokens (batch %d)\n"
                "  prefill        : %.1f tok/s\n  decode         : %.1f tok/s (%.2f ms/step, min %.2f max %.2f)\n  timed runs     : %d (median reported)\n",
                a[1].c_str(), load_s, P, G, B, median(pre), B * 1e3 / dm, dm, *std::min_element(dec.begin(), dec.end()),
                *std::max_element(dec.begin(), dec.end()), runs);
  }
  return 0;
}

// Trace replay: given token ids through the engine step by step, logits written; nothing sampled.
// One JSON object a line on standard input:
//   {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
// <out>/<step>.f32 holds the logits at the wanted places as little-endian float32 [wanted, vocab];
// after every step a line `done <step>` is printed and flushed.
int cmd_replay(const Args& a) {
  const std::string model = flag(a, "--model", ""), out_dir = flag(a, "--out", ""), dtype = flag(a, "--dtype", "");
  const long long max_tokens = std::atoll(flag(a, "--max-tokens", "0").c_str());
  if (model.empty() || out_dir.empty() || max_tokens <= 0 || (dtype != "bfloat16" && dtype != "float32")) {
    std::fprintf(stderr, "usage: qorvix-native replay --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--page-size 16] [--max-requests 8]\n");
    return 2;
  }
  qv::EngineOptions opt;
  opt.dtype = dtype; opt.max_tokens = max_tokens;
  opt.page_size = std::atoi(flag(a, "--page-size", "16").c_str());
  opt.max_requests = std::atoi(flag(a, "--max-requests", "8").c_str());
  if (opt.page_size <= 0 || 64 % opt.page_size) { std::fprintf(stderr, "replay: --page-size %d must divide 64\n", opt.page_size); return 2; }
  (void)!system(("mkdir -p '" + out_dir + "'").c_str());
  qv::Engine engine(model, opt, kernel_libs(a));
  std::map<std::string, long long> ids;                  // request names of the trace -> engine ids
  auto id_of = [&](const qv::Json& j) {
    const std::string key = j.kind == qv::Json::String ? j.str : std::to_string((long long)j.num);
    auto it = ids.find(key);
    if (it == ids.end()) it = ids.emplace(key, (long long)ids.size() + 1).first;
    return it->second;
  };
  std::string line;
  while (std::getline(std::cin, line)) {
    if (line.find_first_not_of(" \t\r\n") == std::string::npos) continue;
    const qv::Json rec = qv::parse_json(line);
    const long long step = rec.at("step").integer();
    std::vector<qv::StepEntry> entries;
    if (const qv::Json* es = rec.find("entries"))
      for (const qv::Json& e : es->arr) {
        qv::StepEntry en;
        en.id = id_of(e.at("id"));
        for (const qv::Json& t : e.at("tokens").arr) en.tokens.push_back((int)t.integer());
        if (const qv::Json* w = e.find("want")) for (const qv::Json& x : w->arr) en.want.push_back((int)x.integer());
        entries.push_back(std::move(en));
      }
    std::vector<long long> end;
    if (const qv::Json* en = rec.find("end")) for (const qv::Json& e : en->arr) end.push_back(id_of(e));
    int rows = 0;
    const float* logits = engine.step(entries, end, &rows);
    if (logits && rows > 0) {
      const std::vector<float> host = engine.logits_to_host(logits, rows);
      const std::string tmp = out_dir + "/." + std::to_string(step) + ".f32.tmp", fin = out_dir + "/" + std::to_string(step) + ".f32";
      FILE* f = std::fopen(tmp.c_str(), "wb");
      if (!f || std::fwrite(host.data(), 4, host.size(), f) != host.size()) { std::fprintf(stderr, "replay: cannot write %s\n", tmp.c_str()); return 1; }
      std::fclose(f);
      std::rename(tmp.c_str(), fin.c_str());
      engine.check_kernel_errors();                      // a kernel that gave up on a barrier must not pass silently
    }
    std::printf("done %lld\n", step);
    std::fflush(stdout);
  }
  return 0;
}

int cmd_gpu_check(const Args& a) {
  if (a.size() < 2) { std::fprintf(stderr, "usage: qorvix-native gpu-check <model_dir> [--tokens 1,2,3 | --random-prompt N]\n"); return 1; }
  const qv::ModelDesc desc = qv::model_desc_from_config(qv::parse_json(qv::read_text_file(a[1] + "/config.json")));
  std::vector<int> prompt = prompt_from(a, (int)desc.vocab);
  if (prompt.empty()) for (int i = 0; i < 32; ++i) prompt.push_back(stream_token(i, 0, (int)desc.vocab));
  const int n = (int)prompt.size(), V = (int)desc.vocab;
  void* cpu = qvr_model_open(a[1].c_str());
  if (!cpu) { std::fprintf(stderr, "error: %s\n", qvr_last_error()); return 1; }
  std::vector<float> want((size_t)n * V);
  qvr_forward(cpu, prompt.data(), n, want.data());
  qvr_model_close(cpu);
  double scale = 1e-30;
  for (float x : want) scale = std::max(scale, (double)std::fabs(x));
  bool all_ok = true;
  for (const char* dt : {"float32", "bfloat16"}) {
    qv::EngineOptions opt;
    opt.dtype = dt; opt.max_tokens = n + 64; opt.max_requests = 1;
    qv::Engine engine(a[1], opt, kernel_libs(a));
    qv::StepEntry e;
    e.id = 1; e.tokens = prompt;
    for (int i = 0; i < n; ++i) e.want.push_back(i);
    int rows = 0;
    const float* dev = engine.step({e}, {1}, &rows);
    const std::vector<float> got = engine.logits_to_host(dev, rows);
    engine.check_kernel_errors();
    double max_abs = 0.0;
    for (size_t i = 0; i < got.size(); ++i) max_abs = std::max(max_abs, (double)std::fabs(got[i] - want[i]));
    int same = 0, decisive = 0;
    bool argmax_ok = true;
    for (int t = 0; t < n; ++t) {
      const float* w = &want[(size_t)t * V];
      const float* g = &got[(size_t)t * V];
      int bw = 0, bg = 0;
      float second = -INFINITY;
      for (int i = 1; i < V; ++i) { if (w[i] > w[bw]) bw = i; if (g[i] > g[bg]) bg = i; }
      for (int i = 0; i < V; ++i) if (i != bw) second = std::max(second, w[i]);
      const bool must = std::string(dt) == "float32" || (double)(w[bw] - second) > 2 * max_abs;
      same += bw == bg;
      decisive += must;
      if (must && bw != bg) argmax_ok = false;
    }
    const double rel = max_abs / scale;
    const bool ok = rel < 5e-2 && argmax_ok;               // the reference's rule (core/src/main.cpp:3660-3678)
    all_ok = all_ok && ok;
    std::printf("gpu-check %s: %d positions | max abs err %.3e | rel err %.3e | argmax equal %d/%d (%d decisive) | %s\n", dt, n, max_abs, rel, same,
                n, decisive, ok ? "ok" : "MISMATCH");
  }
  std::printf("%s\n", all_ok ? "PASS" : "FAIL");
  return all_ok ? 0 : 1;
}

}  // namespace

int main(int argc, char** argv) {
  Args a(argv + 1, argv + argc);
  const char* usage =
      "qorvix-native generate <model_dir> --tokens 1,2,3 | --random-prompt N [--max N] [--temp T] [--top-k K] [--top-p P] [--seed S] [--dtype D]\n"
      "qorvix-native bench <model_dir> [--prompt N] [--gen N] [--warmup N] [--runs N] [--batch B] [--dtype D] [--json]\n"
      "qorvix-native replay --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N\n"
      "qorvix-native model-info <model_dir>\n"
      "qorvix-native gpu-check <model_dir> [--tokens ... | --random-prompt N]\n";
  if (a.empty() || a[0] == "-h" || a[0] == "--help" || a[0] == "help") {
    std::fputs(usage, stderr);
    return a.empty() ? 1 : 0;
  }
  try {
    if (a[0] == "generate") return cmd_generate(a);
    if (a[0] == "bench") return cmd_bench(a);
    if (a[0] == "replay") return cmd_replay(a);
    if (a[0] == "model-info") return cmd_model_info(a);
    if (a[0] == "gpu-check") return cmd_gpu_check(a);
    std::fputs(usage, stderr);
    return 1;
  } catch (const std::exception& e) {                      // the reference prints "error: ..." and returns 1
    std::fprintf(stderr, "error: %s\n", e.what());
    return 1;
  }
}
