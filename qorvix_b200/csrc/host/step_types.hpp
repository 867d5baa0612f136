// What the scheduler and an engine say to each other: a step's entries, and what sampling needs to
// know of each row.  No CUDA in here, so that the scheduler can be compiled and tested without a GPU.
#pragma once
#include <vector>

namespace qv {

struct StepEntry {
  long long id = 0;
  std::vector<int> tokens;
  std::vector<int> want;                // places among these tokens whose logits are asked for
};

// One row of logits to be sampled: the request's parameters (runtime/include/qorvix/runtime/sampler.hpp:12-21),
// the uniform number of its draw, and the recent tokens its penalties look at (empty: no penalties).
struct SampleRow {
  float temperature = 0.f, top_p = 1.f, min_p = 0.f, uniform = 0.f, repetition_penalty = 1.f, frequency_penalty = 0.f, presence_penalty = 0.f;
  int top_k = 0;
  std::vector<int> recent;
  bool plain_greedy() const { return temperature <= 0.f && recent.empty(); }
};

}  // namespace qv
