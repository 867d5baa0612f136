// The native scheduler's decisions without a GPU: a fake engine on top of the real cache bookkeeping
// (csrc/host_runtime.cpp) whose "logits" make the next token (last token + 1) % VOCAB, so that generated
// tokens are a function of the sequence alone.  The counterpart of tests/test_scheduler.py for
// qorvix_b200/csrc/host/scheduler.hpp; prints "ok" and returns 0 when every check holds.
#include <cstdio>
#include <cstdlib>
#include <map>
#include <stdexcept>

#include "host/scheduler.hpp"

extern "C" {
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
int qvh_check(void* h, char* msg, int cap);
}

namespace {

constexpr int VOCAB = 50;

#define CHECK(cond)                                                                  \
  do {                                                                               \
    if (!(cond)) { std::fprintf(stderr, "%s:%d: check failed: %s\n", __FILE__, __LINE__, #cond); std::exit(1); } \
  } while (0)

struct Batch { long long id; int n; int at; };

struct FakeEngine {
  void* cache;
  int page = 16, pages;
  long long limit;
  std::vector<std::vector<Batch>> batches;
  FakeEngine(int tokens, int max_requests, long long max_model_len) : pages(tokens / 16), limit(max_model_len) {
    int window = 0;
    cache = qvh_create(1, &window, pages, page, max_requests);
  }
  ~FakeEngine() { qvh_destroy(cache); }
  long long max_model_len() const { return limit; }
  int page_size() const { return page; }
  bool has(long long id) const { return qvh_has(cache, id) != 0; }
  int length(long long id) const { return has(id) ? qvh_length(cache, id) : 0; }
  int free_pages() const { return qvh_free_pages(cache, 0); }
  int free_slots() const { return qvh_free_slots(cache); }
  void release(long long id) { if (has(id)) qvh_release(cache, id); }
  int one_more_token_fits(const std::vector<long long>& ids) const { return qvh_one_more_token_fits(cache, (int)ids.size(), ids.data()); }
  bool can_run(const std::vector<qv::StepEntry>& entries) const {
    std::vector<long long> ids; std::vector<int> is_new, n_new;
    for (const auto& e : entries) { ids.push_back(e.id); is_new.push_back(has(e.id) ? 0 : 1); n_new.push_back((int)e.tokens.size()); }
    return qvh_can_reserve(cache, (int)ids.size(), ids.data(), is_new.data(), n_new.data()) != 0;
  }
  std::vector<int> step(const std::vector<qv::StepEntry>& entries, const std::vector<long long>&, int* rows) {
    std::vector<int> next;
    std::vector<Batch> b;
    for (const auto& e : entries) {
      b.push_back({e.id, (int)e.tokens.size(), length(e.id)});
      if (!has(e.id)) qvh_admit(cache, e.id);
      CHECK(qvh_reserve(cache, e.id, (int)e.tokens.size()) == 1);        // the scheduler planned a step that fits
      qvh_commit(cache, e.id, (int)e.tokens.size());
      for (int w : e.want) next.push_back((e.tokens[(size_t)w] + 1) % VOCAB);
    }
    batches.push_back(b);
    char msg[256];
    CHECK(qvh_check(cache, msg, sizeof(msg)) == 0);
    *rows = (int)next.size();
    return next;
  }
  std::vector<int> sample(const std::vector<int>& logits, const std::vector<qv::SampleRow>& rows) {
    CHECK(logits.size() == rows.size());
    return logits;
  }
};

using Sched = qv::SchedulerT<FakeEngine>;

std::vector<int> expect(int last, int n) {
  std::vector<int> out;
  for (int i = 0; i < n; ++i) { last = (last + 1) % VOCAB; out.push_back(last); }
  return out;
}
std::map<long long, qv::RequestResult> by_id(const std::vector<qv::RequestResult>& v) {
  std::map<long long, qv::RequestResult> m;
  for (const auto& r : v) m[r.id] = r;
  return m;
}
qv::SamplingParams greedy(int n) { return qv::SamplingParams::greedy_params(n); }

void two_requests_run_to_completion() {
  FakeEngine e(256, 4, 200);
  Sched s(&e, qv::SchedulerConfig(), {});
  const long long a = s.submit({1, 2, 3}, greedy(5)), b = s.submit({7}, greedy(3));
  auto res = by_id(s.run_to_completion());
  CHECK(res[a].tokens == expect(3, 5) && res[b].tokens == expect(7, 3));
  CHECK(res[a].finish_reason == "max_new_tokens" && res[a].prompt_tokens == 3);
  CHECK(e.free_pages() == 16 && e.free_slots() == 4 && s.idle());
}

void five_requests_through_two_slots_in_priority_order() {
  FakeEngine e(256, 4, 200);
  qv::SchedulerConfig c;
  c.max_concurrent = 2;
  Sched s(&e, c, {});
  std::vector<long long> ids;
  const int prio[5] = {0, 0, 5, 0, 1};
  for (int i = 0; i < 5; ++i) ids.push_back(s.submit({i + 1}, greedy(2), prio[i]));
  s.run_to_completion();
  std::vector<long long> first;
  for (const auto& b : e.batches) for (const auto& x : b) if (x.at == 0) first.push_back(x.id);
  CHECK((first == std::vector<long long>{ids[2], ids[4], ids[0], ids[1], ids[3]}));      // priority first, then arrival
}

void token_budget_cuts_prompts_into_portions_beside_decodes() {
  FakeEngine e(512, 4, 400);
  qv::SchedulerConfig c;
  c.max_batch_tokens = 32; c.max_concurrent = 4;
  Sched s(&e, c, {});
  const long long a = s.submit({1, 2, 3, 4, 5, 6, 7, 8, 9, 10}, greedy(40));
  s.step();                                             // a: whole prompt
  const long long b = s.submit(std::vector<int>(100, 3), greedy(2));
  s.step();
  CHECK(e.batches.back().size() == 2 && e.batches.back()[0].id == a && e.batches.back()[0].n == 1 && e.batches.back()[0].at == 10);
  CHECK(e.batches.back()[1].id == b && e.batches.back()[1].n == 31 && e.batches.back()[1].at == 0);   // decode first, the rest of the budget to b
  int fed = 31;
  while (!s.idle()) {
    s.step();
    int total = 0;
    for (const auto& x : e.batches.back()) { total += x.n; if (x.id == b && x.n > 1) fed += x.n; }
    CHECK(total <= 32);
  }
  CHECK(fed == 100);
}

void max_chunk_limits_a_portion() {
  FakeEngine e(512, 4, 400);
  qv::SchedulerConfig c;
  c.max_batch_tokens = 64; c.max_chunk = 24;
  Sched s(&e, c, {});
  s.submit(std::vector<int>(50, 2), greedy(1));
  s.run_to_completion();
  std::vector<int> sizes;
  for (const auto& b : e.batches) for (const auto& x : b) sizes.push_back(x.n);
  CHECK((sizes == std::vector<int>{24, 24, 2}));
}

void eos_stop_length_and_rejection() {
  FakeEngine e(256, 4, 12);
  Sched s(&e, qv::SchedulerConfig(), {9});
  const long long a = s.submit({5}, greedy(20));                      // 6 7 8 then 9 = eos, not emitted
  qv::SamplingParams pb = greedy(20);
  pb.ignore_eos = true;
  const long long b = s.submit({5}, pb);                              // runs into the sequence limit
  qv::SamplingParams pc = greedy(20);
  pc.stop_token_ids = {23};
  const long long c = s.submit({20}, pc);
  const long long d = s.submit({}, greedy(3));                        // empty: rejected
  const long long f = s.submit(std::vector<int>(12, 1), greedy(3));   // as long as the limit: rejected
  auto res = by_id(s.run_to_completion());
  CHECK((res[a].tokens == std::vector<int>{6, 7, 8}) && res[a].hit_eos && res[a].finish_reason == "eos");
  CHECK(res[b].finish_reason == "length" && (int)res[b].tokens.size() == 11 && !res[b].hit_eos);
  CHECK((res[c].tokens == std::vector<int>{21, 22}) && res[c].finish_reason == "stop");
  CHECK(res[d].rejected && res[f].rejected && res[d].finish_reason == "rejected");
  CHECK(e.free_pages() == 16 && e.free_slots() == 4);
}

void out_of_pages_preempts_the_youngest_and_recomputes_to_the_same_tokens() {
  // 8 pages of 16 tokens; three requests of 20 prompt + 40 generated tokens need 12 pages at the end
  FakeEngine e(128, 3, 200);
  qv::SchedulerConfig c;
  c.max_concurrent = 3;
  Sched s(&e, c, {});
  std::vector<long long> ids;
  for (int i = 0; i < 3; ++i) ids.push_back(s.submit(std::vector<int>(20, 10 + i), greedy(40)));
  auto res = by_id(s.run_to_completion());
  CHECK(s.stats.preemptions >= 1);
  int preempted = 0;
  for (int i = 0; i < 3; ++i) {
    CHECK(res[ids[(size_t)i]].tokens == expect(10 + i, 40) && res[ids[(size_t)i]].finish_reason == "max_new_tokens");
    preempted += res[ids[(size_t)i]].preemptions;
  }
  CHECK(preempted >= 1 && res[ids[0]].preemptions == 0);              // the most recently admitted goes first, never the oldest here
  CHECK(e.free_pages() == 8 && e.free_slots() == 3);
}

void a_waiting_request_that_does_not_fit_stays_queued_and_a_lone_one_finishes_with_length() {
  FakeEngine e(64, 4, 400);                                            // 4 pages
  Sched s(&e, qv::SchedulerConfig(), {});
  const long long a = s.submit(std::vector<int>(40, 1), greedy(4));    // 3 pages
  const long long b = s.submit(std::vector<int>(30, 2), greedy(4));    // 2 pages: must wait for a
  s.step();
  CHECK(e.batches.back().size() == 1 && e.batches.back()[0].id == a);
  auto res = by_id(s.run_to_completion());
  CHECK(res[a].tokens == expect(1, 4) && res[b].tokens == expect(2, 4) && !res[b].rejected);
  const long long big = s.submit(std::vector<int>(100, 3), greedy(4)); // 7 pages in a pool of 4: alone and still too big
  auto res2 = by_id(s.run_to_completion());
  CHECK(res2[big].finish_reason == "length" && res2[big].tokens.empty());
  CHECK(e.free_pages() == 4);
}

void sampling_rows_carry_parameters_history_and_a_stream_per_request() {
  struct Spy : FakeEngine {
    using FakeEngine::FakeEngine;
    std::vector<std::vector<qv::SampleRow>> seen;
    std::vector<int> sample(const std::vector<int>& logits, const std::vector<qv::SampleRow>& rows) { seen.push_back(rows); return logits; }
  };
  auto run = [](unsigned long long seed) {
    Spy e(256, 4, 200);
    qv::SchedulerT<Spy> s(&e, qv::SchedulerConfig(), {});
    qv::SamplingParams p;                    // the reference's defaults: temperature 0.8, top-k 40, top-p 0.95, min-p 0.05, repetition 1.1
    p.seed = seed; p.max_new_tokens = 3;
    s.submit({4, 5, 6}, p);
    s.submit({9}, qv::SamplingParams::greedy_params(3));
    s.run_to_completion();
    return e.seen;
  };
  const auto x = run(7), y = run(7), z = run(8);
  CHECK(x.size() == 3 && x[0].size() == 2);
  const qv::SampleRow& r = x[0][0];
  CHECK(r.top_k == 40 && r.temperature > 0.79f && r.temperature < 0.81f && r.repetition_penalty > 1.09f);
  CHECK((r.recent == std::vector<int>{4, 5, 6}) && x[1][0].recent.size() == 4);       // prompt, then prompt + generated
  CHECK(x[0][1].plain_greedy() && x[0][1].uniform == 0.f);
  CHECK(r.uniform >= 0.f && r.uniform < 1.f && r.uniform == y[0][0].uniform && x[1][0].uniform == y[1][0].uniform);
  CHECK(r.uniform != x[1][0].uniform && r.uniform != z[0][0].uniform);                // a stream per request and seed
}

}  // namespace

int main() {
  two_requests_run_to_completion();
  five_requests_through_two_slots_in_priority_order();
  token_budget_cuts_prompts_into_portions_beside_decodes();
  max_chunk_limits_a_portion();
  eos_stop_length_and_rejection();
  out_of_pages_preempts_the_youngest_and_recomputes_to_the_same_tokens();
  a_waiting_request_that_does_not_fit_stays_queued_and_a_lone_one_finishes_with_length();
  sampling_rows_carry_parameters_history_and_a_stream_per_request();
  std::puts("ok");
  return 0;
}
