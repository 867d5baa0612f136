// Host-side bookkeeping of the cache manager in C++: free lists of pages, per-request block
// tables for several groups of layers, request slots, all-or-nothing reservation, early release of
// pages a window has passed, and the filling of the integer rows of a captured decode step.
// No CUDA in here; the device tensors live on the Python side, this library only decides which
// page and slot ids they are indexed with.
//
// The reference keeps the same bookkeeping in memory/src/kv_cache.cpp (a LIFO free stack that
// hands out low ids first, per-session page lists, a refused double free); this is its
// counterpart for pages shared by all layers of a group, several groups, and batched steps.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "host/dispatch.hpp"

namespace {

struct Pool {
  int num_pages = 0;
  std::vector<int> free_list;      // back() is handed out next: 0, 1, 2, ... at the start
  std::vector<uint8_t> held;

  explicit Pool(int n) : num_pages(n), held(n, 0) {
    free_list.reserve(n);
    for (int p = n - 1; p >= 0; --p) free_list.push_back(p);
  }
  int num_free() const { return (int)free_list.size(); }
  // n pages into out, or nothing at all
  bool alloc(int n, std::vector<int>* out) {
    if (n < 0 || n > num_free()) return false;
    for (int i = 0; i < n; ++i) {
      const int p = free_list.back();
      free_list.pop_back();
      held[p] = 1;
      out->push_back(p);
    }
    return true;
  }
  // 0 ok, -1 page not of this pool, -2 freed twice (nothing is changed on error)
  int release(const int* pages, int n) {
    for (int i = 0; i < n; ++i) {
      const int p = pages[i];
      if (p < 0 || p >= num_pages) return -1;
      if (!held[p]) return -2;
      for (int j = 0; j < i; ++j)
        if (pages[j] == p) return -2;
    }
    for (int i = 0; i < n; ++i) {
      held[pages[i]] = 0;
      free_list.push_back(pages[i]);
    }
    return 0;
  }
};

struct Request {
  int slot = 0;
  int length = 0;
  long long epoch = 0;
  std::vector<std::vector<int>> tables;   // per group: page id per block, -1 once given back
};

struct Manager {
  int page_size = 16;
  int max_requests = 0;
  std::vector<Pool> pools;
  std::vector<int> windows;
  std::vector<int> free_slots;            // back() is handed out next
  std::unordered_map<long long, Request> requests;
  long long clock = 0;
  std::string last_error;

  int blocks_for(int tokens) const { return (tokens + page_size - 1) / page_size; }
};

int needed(const Manager& m, const Request* r, int group, int n_new) {
  const int length = r ? r->length : 0;
  const int have = r ? (int)r->tables[group].size() : 0;
  const int want = m.blocks_for(length + n_new);
  return want > have ? want - have : 0;
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------ a single pool (also used on its own)
void* qvh_pool_create(int num_pages) { return num_pages > 0 ? new Pool(num_pages) : nullptr; }
void qvh_pool_destroy(void* p) { delete (Pool*)p; }
int qvh_pool_num_free(void* p) { return ((Pool*)p)->num_free(); }
int qvh_pool_alloc(void* p, int n, int* out) {
  std::vector<int> got;
  if (!((Pool*)p)->alloc(n, &got)) return 0;
  std::copy(got.begin(), got.end(), out);
  return 1;
}
int qvh_pool_free(void* p, const int* pages, int n) { return ((Pool*)p)->release(pages, n); }
int qvh_pool_is_held(void* p, int page) {
  Pool* pool = (Pool*)p;
  return page >= 0 && page < pool->num_pages && pool->held[page];
}

// ------------------------------------------------------------------ the manager
void* qvh_create(int n_groups, const int* windows, int num_pages, int page_size, int max_requests) {
  if (n_groups < 0 || num_pages <= 0 || page_size <= 0 || max_requests <= 0) return nullptr;
  Manager* m = new Manager();
  m->page_size = page_size;
  m->max_requests = max_requests;
  for (int g = 0; g < n_groups; ++g) {
    m->pools.emplace_back(num_pages);
    m->windows.push_back(windows[g]);
  }
  for (int s = max_requests - 1; s >= 0; --s) m->free_slots.push_back(s);
  return m;
}
void qvh_destroy(void* h) { delete (Manager*)h; }

int qvh_has(void* h, long long rid) { return ((Manager*)h)->requests.count(rid) ? 1 : 0; }
int qvh_length(void* h, long long rid) { return ((Manager*)h)->requests.at(rid).length; }
int qvh_slot(void* h, long long rid) { return ((Manager*)h)->requests.at(rid).slot; }
long long qvh_epoch(void* h, long long rid) { return ((Manager*)h)->requests.at(rid).epoch; }
int qvh_free_slots(void* h) { return (int)((Manager*)h)->free_slots.size(); }
int qvh_num_live(void* h) { return (int)((Manager*)h)->requests.size(); }
int qvh_free_pages(void* h, int group) {
  Manager* m = (Manager*)h;
  if (group >= 0) return m->pools[group].num_free();
  int best = -1;
  for (auto& p : m->pools) best = best < 0 ? p.num_free() : std::min(best, p.num_free());
  return best;
}
int qvh_held_pages(void* h, int group) {
  Manager* m = (Manager*)h;
  return m->pools[group].num_pages - m->pools[group].num_free();
}

// slot, or -1 when every slot is taken, -2 when the request is live already
int qvh_admit(void* h, long long rid) {
  Manager* m = (Manager*)h;
  if (m->requests.count(rid)) return -2;
  if (m->free_slots.empty()) return -1;
  Request r;
  r.slot = m->free_slots.back();
  m->free_slots.pop_back();
  r.epoch = ++m->clock;
  r.tables.resize(m->pools.size());
  m->requests.emplace(rid, std::move(r));
  return m->requests.at(rid).slot;
}

int qvh_pages_needed(void* h, long long rid, int has_rid, int n_new, int group) {
  Manager* m = (Manager*)h;
  const Request* r = nullptr;
  if (has_rid) {
    auto it = m->requests.find(rid);
    if (it != m->requests.end()) r = &it->second;
  }
  return needed(*m, r, group, n_new);
}

// whether all (request, new tokens) fit together; is_new[i] != 0: a request that is not live yet
int qvh_can_reserve(void* h, int n, const long long* rids, const int* is_new, const int* n_new) {
  Manager* m = (Manager*)h;
  int new_slots = 0;
  std::vector<int> total(m->pools.size(), 0);
  for (int i = 0; i < n; ++i) {
    const Request* r = nullptr;
    if (!is_new[i]) {
      auto it = m->requests.find(rids[i]);
      if (it != m->requests.end()) r = &it->second;
    }
    if (!r) ++new_slots;
    for (size_t g = 0; g < m->pools.size(); ++g) total[g] += needed(*m, r, (int)g, n_new[i]);
  }
  if (new_slots > (int)m->free_slots.size()) return 0;
  for (size_t g = 0; g < m->pools.size(); ++g)
    if (total[g] > m->pools[g].num_free()) return 0;
  return 1;
}

// pages for n_new more tokens in every group, or nothing: 1 done, 0 no room, -1 unknown request
int qvh_reserve(void* h, long long rid, int n_new) {
  Manager* m = (Manager*)h;
  auto it = m->requests.find(rid);
  if (it == m->requests.end()) return -1;
  Request& r = it->second;
  for (size_t g = 0; g < m->pools.size(); ++g)
    if (needed(*m, &r, (int)g, n_new) > m->pools[g].num_free()) return 0;
  for (size_t g = 0; g < m->pools.size(); ++g) m->pools[g].alloc(needed(*m, &r, (int)g, n_new), &r.tables[g]);
  return 1;
}

// the request holds n_new more tokens; pages wholly before a group's window go back.
// 0 ok, -1 unknown request, -3 more tokens than its pages hold
int qvh_commit(void* h, long long rid, int n_new) {
  Manager* m = (Manager*)h;
  auto it = m->requests.find(rid);
  if (it == m->requests.end()) return -1;
  Request& r = it->second;
  r.length += n_new;
  for (size_t g = 0; g < m->pools.size(); ++g) {
    std::vector<int>& table = r.tables[g];
    if ((int)table.size() * m->page_size < r.length) return -3;
    const int w = m->windows[g];
    if (w > 0) {
      const int first_needed = std::max(0, r.length - w + 1);     // the oldest key a later query reads
      const int dead = first_needed / m->page_size;
      for (int b = 0; b < dead; ++b)
        if (table[b] >= 0) {
          m->pools[g].release(&table[b], 1);
          table[b] = -1;
        }
    }
  }
  return 0;
}

// everything the request holds goes back: 0 ok, -1 unknown request
int qvh_release(void* h, long long rid) {
  Manager* m = (Manager*)h;
  auto it = m->requests.find(rid);
  if (it == m->requests.end()) return -1;
  Request& r = it->second;
  for (size_t g = 0; g < m->pools.size(); ++g)
    for (int p : r.tables[g])
      if (p >= 0) m->pools[g].release(&p, 1);
  m->free_slots.push_back(r.slot);
  m->requests.erase(it);
  return 0;
}

// how many of the given live requests, in order, can each take one more token with the free pages
int qvh_one_more_token_fits(void* h, int n, const long long* rids) {
  Manager* m = (Manager*)h;
  std::vector<int> free_now;
  for (auto& p : m->pools) free_now.push_back(p.num_free());
  for (int i = 0; i < n; ++i) {
    const Request& r = m->requests.at(rids[i]);
    const int blocks = r.length / m->page_size + 1;
    for (size_t g = 0; g < m->pools.size(); ++g)
      if ((int)r.tables[g].size() < blocks) {
        if (free_now[g] == 0) return i;
        --free_now[g];
      }
  }
  return n;
}

int qvh_table_len(void* h, long long rid, int group) { return (int)((Manager*)h)->requests.at(rid).tables[group].size(); }
int qvh_table_copy(void* h, long long rid, int group, int* out, int cap) {
  const std::vector<int>& t = ((Manager*)h)->requests.at(rid).tables[group];
  const int n = std::min((int)t.size(), cap);
  std::copy(t.begin(), t.begin() + n, out);
  return n;
}

// the most recently admitted among the given live requests (index into rids), or -1
int qvh_youngest(void* h, int n, const long long* rids) {
  Manager* m = (Manager*)h;
  int best = -1;
  long long best_epoch = -1;
  for (int i = 0; i < n; ++i) {
    auto it = m->requests.find(rids[i]);
    if (it != m->requests.end() && it->second.epoch > best_epoch) {
      best_epoch = it->second.epoch;
      best = i;
    }
  }
  return best;
}

// no page lost, held twice, or both free and held; no slot lost or held twice.  0 ok, else -1 and
// a description in msg.
int qvh_check(void* h, char* msg, int cap) {
  Manager* m = (Manager*)h;
  auto fail = [&](const std::string& s) {
    snprintf(msg, cap, "%s", s.c_str());
    return -1;
  };
  for (size_t g = 0; g < m->pools.size(); ++g) {
    Pool& pool = m->pools[g];
    std::vector<long long> owner(pool.num_pages, -1);
    int seen = 0;
    for (auto& kv : m->requests)
      for (int p : kv.second.tables[g]) {
        if (p < 0) continue;
        if (p >= pool.num_pages) return fail("group " + std::to_string(g) + ": page " + std::to_string(p) + " is out of range");
        if (owner[p] >= 0) return fail("group " + std::to_string(g) + ": page " + std::to_string(p) + " is held by two requests");
        if (!pool.held[p]) return fail("group " + std::to_string(g) + ": page " + std::to_string(p) + " of a request is on the free list");
        owner[p] = kv.first;
        ++seen;
      }
    if (seen != pool.num_pages - pool.num_free())
      return fail("group " + std::to_string(g) + ": " + std::to_string(pool.num_pages - pool.num_free()) + " pages are taken but requests hold " + std::to_string(seen));
    std::vector<uint8_t> on_list(pool.num_pages, 0);
    for (int p : pool.free_list) {
      if (on_list[p]) return fail("group " + std::to_string(g) + ": a page is on the free list twice");
      on_list[p] = 1;
    }
  }
  std::vector<uint8_t> slot_used(m->max_requests, 0);
  for (auto& kv : m->requests) {
    if (slot_used[kv.second.slot]) return fail("a request slot is held twice");
    slot_used[kv.second.slot] = 1;
  }
  for (int s : m->free_slots)
    if (slot_used[s]) return fail("a request slot is both free and held");
  if ((int)m->requests.size() + (int)m->free_slots.size() != m->max_requests) return fail("a request slot was lost");
  return 0;
}

// Integer rows of a decode-only step for the live requests rids[0..n), padded to S rows, written
// into `host` laid out as [token S][position S][position S][slot S][per group: S x width page ids].
// tokens == null leaves the token part alone.  row_epoch[g*S + i] / row_len[g*S + i] remember what row i
// of group g held after the last call, so that only new table entries are written; a row whose
// request changed (or a group with a window) is rewritten whole.  Pages given back (-1) and padding
// read as the scratch page.  Returns 0, or -1 for an unknown request.
int qvh_fill_decode(void* h, int n, const long long* rids, const int* tokens, int S, int width, int scratch_page,
                    int scratch_slot, int* host, long long* row_epoch, int* row_len) {
  Manager* m = (Manager*)h;
  const int G = (int)m->pools.size();
  for (int i = 0; i < S; ++i) {
    const Request* r = nullptr;
    if (i < n) {
      auto it = m->requests.find(rids[i]);
      if (it == m->requests.end()) return -1;
      r = &it->second;
    }
    if (tokens) host[i] = r ? tokens[i] : 0;
    host[S + i] = r ? r->length : 0;
    host[2 * S + i] = r ? r->length : 0;
    host[3 * S + i] = r ? r->slot : scratch_slot;
    for (int g = 0; g < G; ++g) {
      int* row = host + 4 * S + ((size_t)g * S + i) * width;
      long long& ep = row_epoch[(size_t)g * S + i];
      int& len = row_len[(size_t)g * S + i];
      if (!r) {
        if (ep != 0) std::fill(row, row + width, scratch_page);
        ep = 0;
        len = 0;
        continue;
      }
      const std::vector<int>& t = r->tables[g];
      const int tl = std::min((int)t.size(), width);
      int from = 0;
      if (ep == r->epoch && len <= tl && m->windows[g] == 0) {
        from = len;
      } else {
        std::fill(row, row + width, scratch_page);
      }
      for (int b = from; b < tl; ++b) row[b] = t[b] >= 0 ? t[b] : scratch_page;
      ep = r->epoch;
      len = tl;
    }
  }
  return 0;
}

// ------------------------------------------------------------------ kernel choice (host/dispatch.hpp)
int qvh_decode_variant(int T, int Hkv) { return qv::decode_variant(T, Hkv); }
int qvh_decode_splits(int T, int Hkv, int max_ctx, int known, int variant, int sms) {
  return qv::decode_splits(T, Hkv, max_ctx, known != 0, variant, sms);
}
int qvh_folded_norm_enabled(int tokens) { return qv::folded_norm_enabled(tokens) ? 1 : 0; }
int qvh_fused_rope_enabled(int tokens) { return qv::fused_rope_enabled(tokens) ? 1 : 0; }

}  // extern "C"
