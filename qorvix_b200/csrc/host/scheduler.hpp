// Continuous batching above the native engine's step function, and sampling.
//
// The reference's scheduler (scheduler/src/scheduler.cpp:94-188) admits up to maxConcurrent requests
// by (priority, arrival), prefills each whole prompt token by token inside the admitting step, then
// decodes one token per active request per step, and retires on EOS, maxNewTokens or the sequence
// limit.  Kept: queue order, one decoded token per request per step, the three ways to finish,
// results per request, streaming callback.  New: a token budget per step, prompts cut into
// portions that run beside the decode tokens of other requests, admission only when the pages of the
// whole prompt can be reserved, and a decided answer to running out of pages:
//   * a waiting request that does not fit stays queued (it is not rejected);
//   * when a running request cannot get the page its next token needs, the most recently admitted
//     running request is preempted: its pages go back, and it re-enters the front of the queue with
//     prompt + generated tokens as its prompt (recomputed later);
//   * a request that is alone and still does not fit finishes with reason "length".
// The same decisions as the Python scheduler (engine/scheduler.py) takes, without its lookahead.
//
// Sampling follows runtime/src/sampler.cpp:43-101 (penalties, greedy if temperature <= 0, temperature,
// softmax, top-k, top-p, min-p, draw) on the device; the uniform number of each draw comes from one
// std::mt19937_64 per request seeded with the request's seed, as the reference seeds its own
// (scheduler/src/scheduler.cpp:69), so a request's tokens do not depend on what else is in the batch.
#pragma once
#include <functional>
#include <queue>
#include <random>
#include <set>

#include <algorithm>
#include <string>
#include <tuple>
#include <unordered_map>
#include <vector>

#include "step_types.hpp"

namespace qv {

// names, defaults and disabled values of runtime/include/qorvix/runtime/sampler.hpp:12-21
struct SamplingParams {
  double temperature = 0.8, top_p = 0.95, min_p = 0.05, repetition_penalty = 1.1, frequency_penalty = 0.0, presence_penalty = 0.0;
  int top_k = 40, penalty_last_n = 64;
  unsigned long long seed = 0;
  int max_new_tokens = 128;
  bool ignore_eos = false;
  std::vector<int> stop_token_ids;
  bool greedy() const { return temperature <= 0.0; }
  bool has_penalties() const {
    return penalty_last_n != 0 && (repetition_penalty != 1.0 || frequency_penalty != 0.0 || presence_penalty != 0.0);
  }
  static SamplingParams greedy_params(int max_new) {
    SamplingParams p;
    p.temperature = 0.0; p.top_k = 0; p.top_p = 1.0; p.min_p = 0.0; p.repetition_penalty = 1.0; p.max_new_tokens = max_new;
    return p;
  }
};

struct RequestResult {
  long long id = 0;
  std::vector<int> tokens;
  int prompt_tokens = 0;
  bool hit_eos = false, rejected = false;
  std::string finish_reason;            // "eos" | "stop" | "max_new_tokens" | "length" | "rejected"
  int preemptions = 0;
};

struct SchedulerConfig {
  int max_concurrent = 8;               // requests running at once (reference default, scheduler.hpp:47)
  int max_batch_tokens = 2048;          // token budget of one step
  int max_chunk = 0;                    // longest prompt portion; 0: the budget alone limits it
};

// EngineT: max_model_len(), page_size(), length(id), can_run(entries), one_more_token_fits(ids),
// release(id), step(entries, end, &rows) -> logits handle, sample(logits, rows) -> one id per row.
// (The native Engine of engine.hpp; a fake with the real page bookkeeping in the scheduler's CPU test.)
template <class EngineT>
class SchedulerT {
 public:
  using TokenCallback = std::function<void(long long, int)>;
  SchedulerT(EngineT* engine, const SchedulerConfig& cfg, const std::vector<long long>& eos) : e_(engine), cfg_(cfg) {
    for (long long t : eos) eos_.insert((int)t);
  }

  struct Stats { long long steps = 0, tokens = 0, preemptions = 0, admitted = 0; } stats;

  long long submit(const std::vector<int>& prompt, const SamplingParams& params, int priority = 0, TokenCallback on_token = nullptr) {
    const long long id = next_id_++;
    if (prompt.empty() || (long long)prompt.size() >= e_->max_model_len()) {
      RequestResult r;
      r.id = id; r.prompt_tokens = (int)prompt.size(); r.rejected = true; r.finish_reason = "rejected";
      early_.push_back(r);
      return id;
    }
    Request q;
    q.id = id; q.prompt = prompt; q.n_prompt = (int)prompt.size(); q.params = params; q.priority = priority; q.seq = next_seq_++;
    q.rng.seed(params.seed);
    q.on_token = std::move(on_token);
    requests_[id] = std::move(q);
    waiting_.insert({-priority, requests_[id].seq, id});
    return id;
  }

  bool idle() const { return waiting_.empty() && running_.empty() && early_.empty(); }
  bool decoding() const {
    if (!waiting_.empty() || running_.empty()) return false;
    for (long long id : running_) {
      const Request& r = requests_.at(id);
      if (r.computed < (int)r.prompt.size()) return false;
    }
    return true;
  }

  // One round: plan, run the batch, sample, finish and free.  Returns the requests that finished in it.
  std::vector<RequestResult> step() {
    std::vector<RequestResult> finished;
    finished.swap(early_);
    Plan plan = plan_step();
    for (long long id : plan.finished_for_length) { finished.push_back(result(requests_.at(id))); requests_.erase(id); }
    std::vector<StepEntry> entries;
    std::vector<long long> samplers;
    for (long long id : plan.decode) {
      Request& r = requests_.at(id);
      entries.push_back({id, {r.pending}, {0}});
      samplers.push_back(id);
    }
    for (const auto& pf : plan.prefill) {
      Request& r = requests_.at(pf.first);
      const bool last = r.computed + pf.second == (int)r.prompt.size();
      StepEntry en;
      en.id = pf.first;
      en.tokens.assign(r.prompt.begin() + r.computed, r.prompt.begin() + r.computed + pf.second);
      if (last) { en.want.push_back(pf.second - 1); samplers.push_back(pf.first); }
      entries.push_back(std::move(en));
    }
    if (entries.empty()) return finished;
    int rows = 0;
    const auto logits = e_->step(entries, {}, &rows);
    ++stats.steps;
    stats.tokens += (long long)plan.decode.size();
    for (long long id : plan.decode) { Request& r = requests_.at(id); r.computed += 1; r.has_pending = false; }
    for (const auto& pf : plan.prefill) { requests_.at(pf.first).computed += pf.second; stats.tokens += pf.second; }
    if (!samplers.empty()) {
      const std::vector<int> ids = e_->sample(logits, sample_rows(samplers));
      for (size_t i = 0; i < samplers.size(); ++i) accept(requests_.at(samplers[i]), ids[i]);
    }
    for (size_t i = 0; i < running_.size();) {
      Request& r = requests_.at(running_[i]);
      if (r.done) {
        e_->release(r.id);
        finished.push_back(result(r));
        requests_.erase(r.id);
        running_.erase(running_.begin() + (long)i);
      } else ++i;
    }
    return finished;
  }

  std::vector<RequestResult> run_to_completion() {
    std::vector<RequestResult> out;
    while (!idle()) {
      auto f = step();
      out.insert(out.end(), f.begin(), f.end());
    }
    return out;
  }

 private:
  struct Request {
    long long id = 0;
    std::vector<int> prompt;            // what must be in the cache before decoding (grows on preemption)
    int n_prompt = 0;
    SamplingParams params;
    int priority = 0;
    long long seq = 0;
    std::mt19937_64 rng;
    TokenCallback on_token;
    std::vector<int> generated;
    int computed = 0;
    int pending = 0;
    bool has_pending = false, done = false, hit_eos = false;
    std::string finish_reason;
    int preemptions = 0;
  };
  struct Plan {
    std::vector<long long> decode;
    std::vector<std::pair<long long, int>> prefill;
    std::vector<long long> finished_for_length;
  };
  struct Waiting {
    int neg_priority;
    long long seq, id;
    bool operator<(const Waiting& o) const { return std::tie(neg_priority, seq, id) < std::tie(o.neg_priority, o.seq, o.id); }
  };

  EngineT* e_;
  SchedulerConfig cfg_;
  std::set<int> eos_;
  long long next_id_ = 1, next_seq_ = 0, front_ = -1;
  std::set<Waiting> waiting_;
  std::unordered_map<long long, Request> requests_;
  std::vector<long long> running_;
  std::vector<RequestResult> early_;

  static std::vector<StepEntry> wants_with(const std::vector<std::pair<long long, int>>& wants, long long id, int n) {
    std::vector<StepEntry> v;
    for (const auto& w : wants) { StepEntry e; e.id = w.first; e.tokens.assign((size_t)w.second, 0); v.push_back(std::move(e)); }
    StepEntry e;
    e.id = id; e.tokens.assign((size_t)n, 0);
    v.push_back(std::move(e));
    return v;
  }

  // a shorter portion that ends on a page edge, or 0
  int shrink(long long id, int n) const {
    const int page = e_->page_size(), have = e_->length(id);
    const int shorter = ((have + n - 1) / page) * page - have;
    return (shorter > 0 && shorter < n) ? shorter : 0;
  }

  Plan plan_step() {
    Plan plan;
    int budget = 0;
    std::vector<std::pair<long long, int>> wants;
    while (true) {
      budget = cfg_.max_batch_tokens;
      wants.clear();
      plan.decode.clear();
      plan.prefill.clear();
      bool fits = true;
      std::vector<long long> ready;                       // decode tokens first
      for (long long id : running_)
        if (requests_.at(id).has_pending && (int)ready.size() < budget) ready.push_back(id);
      if (e_->one_more_token_fits(ready) < (int)ready.size()) fits = false;
      else {
        plan.decode = ready;
        for (long long id : ready) wants.push_back({id, 1});
        budget -= (int)ready.size();
      }
      if (fits) {
        for (long long id : running_) {                   // then portions of running prompts
          Request& r = requests_.at(id);
          if (r.has_pending || budget <= 0) continue;
          int n = std::min({(int)r.prompt.size() - r.computed, budget, cfg_.max_chunk ? cfg_.max_chunk : budget});
          while (n > 0 && !e_->can_run(wants_with(wants, id, n))) n = shrink(id, n);
          if (n <= 0) {
            if (plan.decode.empty() && plan.prefill.empty()) fits = false;        // nothing at all can move
            break;
          }
          wants.push_back({id, n});
          plan.prefill.push_back({id, n});
          budget -= n;
        }
      }
      if (fits) break;
      const long long victim = running_.back();           // most recently admitted
      if (running_.size() == 1) {
        running_.pop_back();
        finish(requests_.at(victim), "length");
        e_->release(victim);
        plan.finished_for_length.push_back(victim);
        return plan;
      }
      preempt(victim);
    }
    // admission: by priority then arrival, while a slot, budget and the pages of the whole prompt exist
    while (!waiting_.empty() && (int)running_.size() < cfg_.max_concurrent && budget > 0) {
      const Waiting w = *waiting_.begin();
      Request& r = requests_.at(w.id);
      const int left = (int)r.prompt.size() - r.computed;
      int n = std::min({left, budget, cfg_.max_chunk ? cfg_.max_chunk : budget});
      if (!e_->can_run(wants_with(wants, w.id, left))) n = 0;
      if (n <= 0) {
        if (running_.empty() && wants.empty()) {            // alone and still too big for the pool
          waiting_.erase(waiting_.begin());
          finish(r, "length");
          plan.finished_for_length.push_back(w.id);
          continue;
        }
        break;
      }
      waiting_.erase(waiting_.begin());
      running_.push_back(w.id);
      ++stats.admitted;
      wants.push_back({w.id, n});
      plan.prefill.push_back({w.id, n});
      budget -= n;
    }
    return plan;
  }

  void preempt(long long id) {
    Request& r = requests_.at(id);
    running_.erase(std::find(running_.begin(), running_.end(), id));
    e_->release(id);
    if (r.has_pending) {
      r.prompt.assign(r.prompt.begin(), r.prompt.begin() + r.n_prompt);
      r.prompt.insert(r.prompt.end(), r.generated.begin(), r.generated.end());   // generated includes the pending token
      r.has_pending = false;
    }
    r.computed = 0;
    ++r.preemptions;
    ++stats.preemptions;
    waiting_.insert({-r.priority, front_--, id});
  }

  // A sampled token: EOS ends the request and is not emitted (scheduler.cpp:149-156); else it is
  // emitted and becomes the next token to feed unless a limit is reached.
  void accept(Request& r, int tok) {
    const SamplingParams& p = r.params;
    if (!p.ignore_eos && eos_.count(tok)) { r.hit_eos = true; finish(r, "eos"); return; }
    if (std::find(p.stop_token_ids.begin(), p.stop_token_ids.end(), tok) != p.stop_token_ids.end()) { finish(r, "stop"); return; }
    r.generated.push_back(tok);
    if (r.on_token) r.on_token(r.id, tok);
    if ((int)r.generated.size() >= p.max_new_tokens) { finish(r, "max_new_tokens"); return; }
    if (r.n_prompt + (long long)r.generated.size() >= e_->max_model_len()) { finish(r, "length"); return; }
    r.pending = tok;
    r.has_pending = true;
  }
  void finish(Request& r, const char* reason) { r.done = true; r.finish_reason = reason; }
  RequestResult result(const Request& r) const {
    RequestResult o;
    o.id = r.id; o.tokens = r.generated; o.prompt_tokens = r.n_prompt; o.hit_eos = r.hit_eos; o.finish_reason = r.finish_reason;
    o.preemptions = r.preemptions;
    return o;
  }

  // what sampling needs of each row: the request's parameters, the next number of its own random
  // stream, and the tokens its penalties look at
  std::vector<SampleRow> sample_rows(const std::vector<long long>& ids) {
    std::vector<SampleRow> rows;
    for (long long id : ids) {
      Request& r = requests_.at(id);
      const SamplingParams& p = r.params;
      SampleRow row;
      row.temperature = (float)p.temperature; row.top_k = p.top_k; row.top_p = (float)p.top_p; row.min_p = (float)p.min_p;
      row.uniform = p.greedy() ? 0.f : (float)((double)(r.rng() >> 11) * (1.0 / 9007199254740992.0));
      if (p.has_penalties()) {
        row.repetition_penalty = (float)p.repetition_penalty; row.frequency_penalty = (float)p.frequency_penalty;
        row.presence_penalty = (float)p.presence_penalty;
        std::vector<int> hist(r.prompt.begin(), r.prompt.begin() + r.n_prompt);
        hist.insert(hist.end(), r.generated.begin(), r.generated.end());
        const size_t n = std::min(hist.size(), (size_t)p.penalty_last_n);
        row.recent.assign(hist.end() - (long)n, hist.end());
      }
      rows.push_back(std::move(row));
    }
    return rows;
  }
};

}  // namespace qv
