// The rules by which a step's shape picks its kernels, in one place for every host that launches
// them (the Python step function through csrc/host_runtime.cpp's C entry points, the native
// executor directly).  Each is a function of the step's shape only, so that a captured step keeps
// its choice.  The figures in the comments were measured on a B200 (148 SMs).
#pragma once
#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace qv {

// Which decode-attention kernel a step of T single tokens takes: 0 reads keys and values through a
// ring in shared memory that bulk copies fill (the faster one when many (token, kv head) pairs
// stream long key ranges), 1 through per-thread loads (less set-up; better when there are few pairs).
inline int decode_variant(int T, int Hkv) { return T * Hkv >= 32 ? 0 : 1; }

// How many slices of the keys each (token, kv head) is cut into.  `variant` as above; `known`: max_ctx
// is the step's real longest context (else the most a captured step may be replayed at).
inline int decode_splits(int T, int Hkv, int max_ctx, bool known, int variant, int sms) {
  const int pairs = std::max(1, T * Hkv);
  if (variant == 0 && !known) {
    // a captured step is replayed at contexts from a few keys up to max_ctx: one wave of CTAs, no
    // more (more slices than that pay only at long contexts and cost up to a third at short ones)
    return std::max(1, std::min({16, (2 * sms) / pairs, max_ctx / 256}));
  }
  if (variant == 0) {
    // two CTAs per SM run at once; a CTA's time is its slice of the keys plus a fixed part worth about
    // 256 keys.  The count that needs the least time over all waves, the smaller one on a tie.
    const int resident = 2 * sms;
    int best = 1;
    long long best_cost = -1;
    for (int s = 1; s <= std::max(1, std::min(16, max_ctx / 256)); ++s) {
      const long long cost = (long long)((pairs * s + resident - 1) / resident) * ((max_ctx + s - 1) / s + 256);
      if (best_cost < 0 || cost < best_cost) { best = s; best_cost = cost; }
    }
    return best;
  }
  // per-thread loads: about three CTAs per SM
  return std::max(1, std::min({16, (3 * sms + pairs - 1) / pairs, (max_ctx + 63) / 64}));
}

inline const char* env_or(const char* name, const char* def) {
  const char* v = std::getenv(name);
  return v ? v : def;
}

// Whether the RMS norms of a step of `tokens` tokens ride in the epilogues of the products around
// them: up to 16 tokens (one chunk of the epilogue; at 64 tokens the longer epilogues cost more
// than the two launches they save: 11.0k against 11.9k tokens/s at batch 64), unless
// QORVIX_FOLDED_NORM=0 (never) or =64 (up to 64 tokens; for comparison).
inline bool folded_norm_enabled(int tokens) {
  const char* mode = env_or("QORVIX_FOLDED_NORM", "1");
  if (!std::strcmp(mode, "0")) return false;
  return tokens <= (!std::strcmp(mode, "64") ? 64 : 16);
}

// Whether the QKV projection of a step of `tokens` tokens takes the rotation and the cache write
// into its epilogue: above 64 tokens, unless QORVIX_FUSED_ROPE=0 (for comparison).
inline bool fused_rope_enabled(int tokens) { return tokens > 64 && std::strcmp(env_or("QORVIX_FUSED_ROPE", "1"), "0") != 0; }

// A mixed step whose single-token segments come first gives those to the split-KV kernel and the
// rest to the portion kernels when at least this many lead.
constexpr int kMinLeadingDecodeTokens = 4;

}  // namespace qv
