// Host-side bookkeeping of the paged key/value cache: page pools with reference counts and
// generations, request slots with generation handles, block tables per request and layer
// group, all-or-nothing reservation, commit with window release, truncate, free, and a bulk
// routine that writes a whole decode step's integers in one call.  Plain C++17 with a C
// interface (loaded with ctypes); no CUDA, so it is tested without a GPU.
//
// The reference spreads these duties over base::BlockAllocator (block_allocator.cpp:205-230,
// 264-282), base::SequenceKVManager (sequence_kv_manager.cpp:204-299) and
// base::KVCacheManager (kv_cache_manager.cpp:44-59, 167-236, 756-784); see cache/manager.py
// for how this design differs (one page id for all layers of a group, windowed groups).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <string>
#include <vector>

namespace {
constexpr int kSlotBits = 20;
constexpr int64_t kSlotMask = (1 << kSlotBits) - 1;

enum Err : int {
  kOk = 0,
  kStale = -1,        // stale or malformed request handle
  kFreedTwice = -2,   // a page freed twice / outside the pool
  kBadArg = -3,
  kCorrupt = -4,
};

struct Pool {
  int num_pages = 0;
  bool lifo = false;
  std::deque<int> free_q;
  // The page directory: per page its reference count (the block table that holds it plus any
  // further holds taken with share()), how often it has been handed out, the request that it
  // was handed to (-1 while free) and how many further holds it has.  A page goes back to the
  // free queue when its count reaches zero, whoever lets go last.  The reference keeps the same
  // record in base::PageDirectory (page_directory.cpp:16-47) over BlockAllocator's counts
  // (block_allocator.cpp:232-262).
  std::vector<int> refs, generation, shares;
  std::vector<int64_t> owner;
  int64_t allocations = 0;
  int allocate(int64_t handle) {
    if (free_q.empty()) return -1;
    int page;
    if (lifo) { page = free_q.back(); free_q.pop_back(); }
    else { page = free_q.front(); free_q.pop_front(); }
    refs[page] = 1;
    owner[page] = handle;
    generation[page] += 1;
    allocations += 1;
    return page;
  }
  int release(int page) {
    if (page < 0 || page >= num_pages || refs[page] <= 0) return kFreedTwice;
    if (--refs[page] == 0) {
      owner[page] = -1;
      free_q.push_back(page);
    }
    return kOk;
  }
  int share(int page) {            // one more hold on a page that is held
    if (page < 0 || page >= num_pages || refs[page] <= 0) return kBadArg;
    refs[page] += 1;
    shares[page] += 1;
    return kOk;
  }
  int unshare(int page) {
    if (page < 0 || page >= num_pages || shares[page] <= 0) return kFreedTwice;
    shares[page] -= 1;
    return release(page);
  }
};

struct Request {
  bool live = false;
  int64_t generation = 0;
  int64_t reserved = 0, computed = 0;
  std::vector<std::vector<int>> tables;   // per group
  std::vector<int> first_live;
};

struct Manager {
  int page_tokens = 0, max_requests = 0;
  std::vector<int> windows;               // -1: keep every key
  std::vector<Pool> pools;
  std::vector<Request> slots;
  std::vector<int64_t> slot_generation;
  std::deque<int> free_slots;
  std::string last_error;

  Request* lookup(int64_t handle) {
    if (handle < 0) return nullptr;
    const int64_t slot = handle & kSlotMask, gen = handle >> kSlotBits;
    if (slot >= max_requests) return nullptr;
    Request& r = slots[slot];
    if (!r.live || r.generation != gen) return nullptr;
    return &r;
  }
  int64_t blocks_for(int64_t tokens) const { return (tokens + page_tokens - 1) / page_tokens; }
};
}  // namespace

#define API extern "C" __attribute__((visibility("default")))

API void* pbe_cm_new(int n_groups, const int* windows, int page_tokens, const int* num_pages, int max_requests,
                     int lifo) {
  if (n_groups < 0 || page_tokens <= 0 || max_requests <= 0 || max_requests > kSlotMask) return nullptr;
  for (int g = 0; g < n_groups; ++g)
    if (num_pages[g] <= 0) return nullptr;
  Manager* m = new Manager();
  m->page_tokens = page_tokens;
  m->max_requests = max_requests;
  m->windows.assign(windows, windows + n_groups);
  m->pools.resize(n_groups);
  for (int g = 0; g < n_groups; ++g) {
    Pool& p = m->pools[g];
    p.num_pages = num_pages[g];
    p.lifo = lifo != 0;
    p.refs.assign(p.num_pages, 0);
    p.generation.assign(p.num_pages, 0);
    p.shares.assign(p.num_pages, 0);
    p.owner.assign(p.num_pages, -1);
    for (int i = 0; i < p.num_pages; ++i) p.free_q.push_back(i);
  }
  m->slots.resize(max_requests);
  m->slot_generation.assign(max_requests, 0);
  for (int i = 0; i < max_requests; ++i) m->free_slots.push_back(i);
  return m;
}
API void pbe_cm_delete(void* h) { delete static_cast<Manager*>(h); }

API int64_t pbe_cm_add_request(void* h) {
  Manager* m = static_cast<Manager*>(h);
  if (m->free_slots.empty()) return -1;
  const int slot = m->free_slots.front();
  m->free_slots.pop_front();
  Request& r = m->slots[slot];
  r.live = true;
  r.generation = ++m->slot_generation[slot];
  r.reserved = r.computed = 0;
  r.tables.assign(m->pools.size(), {});
  r.first_live.assign(m->pools.size(), 0);
  return (r.generation << kSlotBits) | slot;
}
API int pbe_cm_is_live(void* h, int64_t handle) { return static_cast<Manager*>(h)->lookup(handle) != nullptr; }
API int pbe_cm_num_live(void* h) {
  Manager* m = static_cast<Manager*>(h);
  return m->max_requests - (int)m->free_slots.size();
}
API int64_t pbe_cm_context_len(void* h, int64_t handle) {
  Request* r = static_cast<Manager*>(h)->lookup(handle);
  return r ? r->computed : kStale;
}
API int64_t pbe_cm_reserved_len(void* h, int64_t handle) {
  Request* r = static_cast<Manager*>(h)->lookup(handle);
  return r ? r->reserved : kStale;
}
// The longest reserved length among n requests (one call a decode step instead of one per
// request): the context a step that fills its reservations will attend over.
API int64_t pbe_cm_max_reserved_len(void* h, const int64_t* handles, int n) {
  Manager* m = static_cast<Manager*>(h);
  int64_t longest = 0;
  for (int i = 0; i < n; ++i) {
    Request* r = m->lookup(handles[i]);
    if (!r) return kStale;
    if (r->reserved > longest) longest = r->reserved;
  }
  return longest;
}
API int pbe_cm_num_free_pages(void* h, int g) { return (int)static_cast<Manager*>(h)->pools[g].free_q.size(); }
API int pbe_cm_pool_num_pages(void* h, int g) { return static_cast<Manager*>(h)->pools[g].num_pages; }
API int64_t pbe_cm_pool_allocations(void* h, int g) { return static_cast<Manager*>(h)->pools[g].allocations; }
API int pbe_cm_page_generation(void* h, int g, int page) { return static_cast<Manager*>(h)->pools[g].generation[page]; }
API int pbe_cm_page_refcount(void* h, int g, int page) { return static_cast<Manager*>(h)->pools[g].refs[page]; }

// New pages per group that a reservation of n tokens would take; returns kStale for a bad handle.
API int pbe_cm_pages_needed(void* h, int64_t handle, int64_t n, int* out) {
  Manager* m = static_cast<Manager*>(h);
  Request* r = m->lookup(handle);
  if (!r) return kStale;
  const int64_t target = m->blocks_for(r->reserved + n);
  for (size_t g = 0; g < m->pools.size(); ++g)
    out[g] = (int)std::max<int64_t>(0, target - (int64_t)r->tables[g].size());
  return kOk;
}
API int64_t pbe_cm_max_appendable(void* h, int64_t handle) {
  Manager* m = static_cast<Manager*>(h);
  Request* r = m->lookup(handle);
  if (!r) return kStale;
  if (m->pools.empty()) return (int64_t)1 << 30;
  int64_t best = INT64_MAX;
  for (size_t g = 0; g < m->pools.size(); ++g) {
    const int64_t room = (int64_t)r->tables[g].size() * m->page_tokens - r->reserved +
                         (int64_t)m->pools[g].free_q.size() * m->page_tokens;
    best = std::min(best, room);
  }
  return std::max<int64_t>(0, best);
}
// 1: reserved; 0: not enough pages (nothing changed); <0: error
API int pbe_cm_reserve(void* h, int64_t handle, int64_t n) {
  Manager* m = static_cast<Manager*>(h);
  Request* r = m->lookup(handle);
  if (!r) return kStale;
  if (n < 0) return kBadArg;
  const int64_t target = m->blocks_for(r->reserved + n);
  for (size_t g = 0; g < m->pools.size(); ++g) {
    const int64_t need = target - (int64_t)r->tables[g].size();
    if (need > (int64_t)m->pools[g].free_q.size()) return 0;
  }
  for (size_t g = 0; g < m->pools.size(); ++g) {
    while ((int64_t)r->tables[g].size() < target) {
      const int page = m->pools[g].allocate(handle);
      if (page < 0) return kCorrupt;
      r->tables[g].push_back(page);
    }
  }
  r->reserved += n;
  return 1;
}
API int pbe_cm_commit(void* h, int64_t handle, int64_t n) {
  Manager* m = static_cast<Manager*>(h);
  Request* r = m->lookup(handle);
  if (!r) return kStale;
  if (n < 0 || r->computed + n > r->reserved) return kBadArg;
  r->computed += n;
  for (size_t g = 0; g < m->pools.size(); ++g) {
    const int w = m->windows[g];
    if (w < 0) continue;
    const int64_t first_needed = r->computed - w + 1;
    if (first_needed <= 0) continue;
    const int64_t dead = std::min<int64_t>(first_needed / m->page_tokens, (int64_t)r->tables[g].size());
    for (int64_t b = r->first_live[g]; b < dead; ++b) {
      int& page = r->tables[g][b];
      if (page >= 0) {
        if (m->pools[g].release(page) != kOk) return kFreedTwice;
        page = -1;
      }
    }
    r->first_live[g] = (int)std::max<int64_t>(r->first_live[g], dead);
  }
  return kOk;
}
API int pbe_cm_truncate(void* h, int64_t handle, int64_t n) {
  Manager* m = static_cast<Manager*>(h);
  Request* r = m->lookup(handle);
  if (!r) return kStale;
  if (n < 0 || n > r->reserved) return kBadArg;
  const int64_t keep = m->blocks_for(n);
  for (size_t g = 0; g < m->pools.size(); ++g)
    if (keep < r->first_live[g]) return kBadArg;
  for (size_t g = 0; g < m->pools.size(); ++g) {
    auto& t = r->tables[g];
    while ((int64_t)t.size() > keep) {
      const int page = t.back();
      t.pop_back();
      if (page >= 0 && m->pools[g].release(page) != kOk) return kFreedTwice;
    }
  }
  r->reserved = n;
  r->computed = std::min(r->computed, n);
  return kOk;
}
API int pbe_cm_free(void* h, int64_t handle) {
  Manager* m = static_cast<Manager*>(h);
  Request* r = m->lookup(handle);
  if (!r) return kStale;
  for (size_t g = 0; g < m->pools.size(); ++g) {
    for (int page : r->tables[g])
      if (page >= 0 && m->pools[g].release(page) != kOk) return kFreedTwice;
    r->tables[g].clear();
  }
  r->live = false;
  m->free_slots.push_back((int)(handle & kSlotMask));
  return kOk;
}
// Copies the request's block table of group g into out (capacity cap); returns its length.
API int pbe_cm_block_table(void* h, int64_t handle, int g, int* out, int cap) {
  Manager* m = static_cast<Manager*>(h);
  Request* r = m->lookup(handle);
  if (!r) return kStale;
  const auto& t = r->tables[g];
  const int n = (int)t.size();
  if (out != nullptr) std::memcpy(out, t.data(), sizeof(int) * std::min(n, cap));
  return n;
}
// Test hook: the order in which free pages will be handed out.
API int pbe_cm_set_free_order(void* h, int g, const int* pages, int n) {
  Pool& p = static_cast<Manager*>(h)->pools[g];
  if (n != (int)p.free_q.size()) return kBadArg;
  std::vector<char> seen(p.num_pages, 0);
  for (int i = 0; i < n; ++i) {
    if (pages[i] < 0 || pages[i] >= p.num_pages || p.refs[pages[i]] != 0 || seen[pages[i]]) return kBadArg;
    seen[pages[i]] = 1;
  }
  p.free_q.assign(pages, pages + n);
  return kOk;
}
// 0 when every page is held once or free once, nothing lost; else a message in buf.
API int pbe_cm_check(void* h, char* buf, int cap) {
  Manager* m = static_cast<Manager*>(h);
  std::string msg;
  for (size_t g = 0; g < m->pools.size() && msg.empty(); ++g) {
    Pool& p = m->pools[g];
    std::vector<int> held(p.num_pages, 0), freec(p.num_pages, 0);
    for (const Request& r : m->slots) {
      if (!r.live) continue;
      for (int page : r.tables[g])
        if (page >= 0) held[page] += 1;
    }
    for (int page : p.free_q) freec[page] += 1;
    for (int i = 0; i < p.num_pages && msg.empty(); ++i) {
      if (freec[i] > 1) msg = "group " + std::to_string(g) + ": page " + std::to_string(i) + " is in the free queue twice";
      else if (held[i] > 1) msg = "group " + std::to_string(g) + ": page " + std::to_string(i) + " is held by " + std::to_string(held[i]) + " block tables";
      else if (held[i] + p.shares[i] > 0 && freec[i] == 1) msg = "group " + std::to_string(g) + ": page " + std::to_string(i) + " is both held and free";
      else if (held[i] + p.shares[i] == 0 && freec[i] == 0) msg = "group " + std::to_string(g) + ": page " + std::to_string(i) + " is lost";
      else if (p.refs[i] != held[i] + p.shares[i]) msg = "group " + std::to_string(g) + ": page " + std::to_string(i) + " is held " + std::to_string(held[i] + p.shares[i]) + " times but its count is " + std::to_string(p.refs[i]);
      else if ((p.refs[i] == 0) != (p.owner[i] < 0)) msg = "group " + std::to_string(g) + ": page " + std::to_string(i) + " has an owner while free, or none while held";
    }
  }
  for (const Request& r : m->slots) {
    if (!r.live || !msg.empty()) continue;
    if (r.computed < 0 || r.computed > r.reserved) msg = "computed/reserved out of order";
    for (const auto& t : r.tables)
      if ((int64_t)t.size() != m->blocks_for(r.reserved)) msg = "a block table does not cover the reservation";
  }
  if (msg.empty()) return 0;
  if (buf != nullptr && cap > 0) {
    std::strncpy(buf, msg.c_str(), cap - 1);
    buf[cap - 1] = 0;
  }
  return 1;
}

// The page directory's further holds: share() pins a held page (its count goes up, it stays out
// of the free queue when its request lets go of it), unshare() lets go of one such hold.
API int pbe_cm_share_page(void* h, int group, int page) {
  Manager* m = static_cast<Manager*>(h);
  if (group < 0 || group >= (int)m->pools.size()) return kBadArg;
  return m->pools[group].share(page);
}
API int pbe_cm_unshare_page(void* h, int group, int page) {
  Manager* m = static_cast<Manager*>(h);
  if (group < 0 || group >= (int)m->pools.size()) return kBadArg;
  return m->pools[group].unshare(page);
}
// The handle of the request a page was handed to; -1 for a free page, kBadArg outside the pool.
API int64_t pbe_cm_page_owner(void* h, int group, int page) {
  Manager* m = static_cast<Manager*>(h);
  if (group < 0 || group >= (int)m->pools.size() || page < 0 || page >= m->pools[group].num_pages) return kBadArg;
  return m->pools[group].owner[page];
}
// Handles of all live requests into out[0..cap); returns how many there are.
API int pbe_cm_live_handles(void* h, int64_t* out, int cap) {
  Manager* m = static_cast<Manager*>(h);
  int n = 0;
  for (int slot = 0; slot < m->max_requests; ++slot) {
    const Request& r = m->slots[slot];
    if (!r.live) continue;
    if (n < cap) out[n] = (r.generation << kSlotBits) | slot;
    ++n;
  }
  return n;
}

// One decode step's integers for R requests, each bringing one token at its last reserved
// position (the context length when the step before it is committed; one more when that step
// is still in flight and this one was scheduled ahead of it): writes those positions, state slots, the block-table rows (only entries from
// known[r] on, unless the group is windowed or refresh is set) and the cache slots.
// bt[g] points at an int32 matrix with row stride bt_stride[g]; known is [n_groups][R].
// Returns 0, kStale, or kBadArg when a token's page is not held or a row does not fit.
API int pbe_cm_decode_fill(void* h, int R, const int64_t* handles, int64_t* ctx_before, int64_t* state_slots,
                           int32_t* const* bt, const int* bt_stride, int32_t* const* slots, int* known, int refresh) {
  Manager* m = static_cast<Manager*>(h);
  const int P = m->page_tokens;
  const int G = (int)m->pools.size();
  for (int r = 0; r < R; ++r) {
    Request* req = m->lookup(handles[r]);
    if (!req) return kStale;
    const int64_t pos = req->reserved - 1;
    if (pos < req->computed) return kBadArg;               // nothing reserved for this step
    ctx_before[r] = pos;
    state_slots[r] = handles[r] & kSlotMask;
    for (int g = 0; g < G; ++g) {
      const auto& t = req->tables[g];
      const int n = (int)t.size();
      if (n > bt_stride[g]) return kBadArg;
      int32_t* row = bt[g] + (size_t)r * bt_stride[g];
      int& k = known[g * R + r];
      const int lo = (refresh || m->windows[g] >= 0) ? 0 : std::min(k, n);
      for (int i = lo; i < n; ++i) row[i] = t[i];
      k = n;
      const int64_t blk = pos / P;
      if (blk >= n || t[blk] < 0) return kBadArg;
      slots[g][r] = (int32_t)((int64_t)t[blk] * P + pos % P);
    }
  }
  return kOk;
}

// reserve(handle, 1) for many requests at once; ok[r] = 1 / 0 / error code.
API void pbe_cm_reserve_many(void* h, int R, const int64_t* handles, int64_t n, int* ok) {
  for (int r = 0; r < R; ++r) ok[r] = pbe_cm_reserve(h, handles[r], n);
}

// The attention work list of a captured decode step: request r (one token, context
// ctx_before[r] + 1) has ns = ceil(seq / split_keys) - lo / split_keys key splits; work rows
// [r][s] = {r or -1 when s >= ns, 0, s, ns}; split_counts[r] = ns.  Rows of requests beyond R
// are idle.  Returns the largest ns, or kBadArg when one exceeds S.
API int pbe_decode_work_fill(int R, int B, int S, const int64_t* ctx_before, int window, int split_keys,
                             int32_t* work, int32_t* split_counts, int32_t* positions, int32_t* seq_len,
                             int32_t* tokens, const int64_t* token_values, int pad_from) {
  int worst = 0;
  for (int r = 0; r < R; ++r) {
    const int64_t ctx = ctx_before[r], seq = ctx + 1;
    const int64_t lo = window > 0 ? std::max<int64_t>(0, ctx - window + 1) : 0;
    const int ns = (int)((seq + split_keys - 1) / split_keys - lo / split_keys);
    if (ns > S) return kBadArg;
    worst = std::max(worst, ns);
    int32_t* w = work + (size_t)r * S * 4;
    for (int s = 0; s < S; ++s) {
      w[s * 4 + 0] = s < ns ? r : -1;
      w[s * 4 + 1] = 0;
      w[s * 4 + 2] = s;
      w[s * 4 + 3] = ns;
    }
    split_counts[r] = ns;
    if (positions) positions[r] = (int32_t)ctx;
    if (seq_len) seq_len[r] = (int32_t)seq;
    if (tokens) tokens[r] = (int32_t)token_values[r];
  }
  for (int r = std::max(R, pad_from); r < B; ++r) {      // idle rows (written when the batch changes)
    int32_t* w = work + (size_t)r * S * 4;
    for (int s = 0; s < S; ++s) {
      w[s * 4 + 0] = -1;
      w[s * 4 + 1] = 0;
      w[s * 4 + 2] = s;
      w[s * 4 + 3] = 0;
    }
    split_counts[r] = 0;
    if (positions) positions[r] = 0;
    if (seq_len) seq_len[r] = 0;
    if (tokens) tokens[r] = 0;
  }
  return worst;
}

// commit(handle, n[r]) for many requests; returns 0 or the first error.
API int pbe_cm_commit_many(void* h, int R, const int64_t* handles, const int64_t* n) {
  for (int r = 0; r < R; ++r) {
    const int rc = pbe_cm_commit(h, handles[r], n[r]);
    if (rc != kOk) return rc;
  }
  return kOk;
}
