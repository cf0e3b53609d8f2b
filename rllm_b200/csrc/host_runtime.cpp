// The host side of the cache manager, native: page pools, what every live request holds, and
// the writer of a decode step's metadata. No CUDA in this file; it is loaded by the Python
// package through ctypes like the kernel libraries (library "host").
//
// PagePool: a LIFO free list (a page given back is the next one handed out: reuse is
// immediate, as in the reference's KvPool, src/model/kv_cache.rs:779, 852-857) with the holder
// of every page recorded, so that a page can never be lost, held twice or freed twice; a
// violation is reported, never silently absorbed (the reference panics on a stale handle,
// src/model/kv_cache.rs:864-875).
// Cache: one pool per group of layers with equal needs; per live request a block table per
// group (page of positions [i * page_size, (i + 1) * page_size), or -1 once a window has passed
// it), its token count and its state slot. Parity: src/model/kv_cache.rs:725-947 (pool) and
// 949-1091 (per-sequence table) of the reference.
// fill_decode: the int32 vectors of a step in which every request brings one token, written
// straight into the pinned buffer that is copied to the device; a block-table row is rewritten
// only when another holding took the row or its pages changed other than by growing.
#include <cstdint>
#include <cstring>
#include <vector>

#define RLLM_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr long long NOBODY = INT64_MIN;

struct Pool {
  int num_pages;
  std::vector<int> free_list;            // back() is handed out next
  std::vector<long long> holder;         // NOBODY: free
  explicit Pool(int n) : num_pages(n), holder((size_t)n, NOBODY) {
    free_list.reserve((size_t)n);
    for (int p = n - 1; p >= 0; --p) free_list.push_back(p);      // pop yields 0, 1, 2, ...
  }
  int alloc(long long owner) {
    if (free_list.empty()) return -1;
    const int page = free_list.back();
    if (holder[(size_t)page] != NOBODY) return -2;                // on the free list while held
    free_list.pop_back();
    holder[(size_t)page] = owner;
    return page;
  }
  int release(int page, long long owner) {
    if (page < 0 || page >= num_pages) return -1;                 // no such page
    if (holder[(size_t)page] == NOBODY) return -2;                // freed twice
    if (holder[(size_t)page] != owner) return -3;                 // held by someone else
    holder[(size_t)page] = NOBODY;
    free_list.push_back(page);
    return 0;
  }
  int check() const {                                             // every page free or held, never both, never neither
    std::vector<char> on_list((size_t)num_pages, 0);
    for (int p : free_list) {
      if (p < 0 || p >= num_pages) return -1;
      if (on_list[(size_t)p]) return -2;                          // twice on the free list
      on_list[(size_t)p] = 1;
    }
    for (int p = 0; p < num_pages; ++p)
      if ((on_list[(size_t)p] != 0) == (holder[(size_t)p] != NOBODY)) return -3;
    return 0;
  }
};

struct Holding {
  bool live = false;
  long long rid = 0;
  int num_tokens = 0;
  long long serial = 0;      // tells two holdings apart even when a request id comes back
  int epoch = 0;             // changes to the tables other than appending a page
  std::vector<std::vector<int>> pages;   // per group
};

struct Cache {
  int page_size;
  std::vector<Pool> pools;           // per group
  std::vector<int> window;           // per group, < 0: every key is kept
  Pool slots;
  std::vector<Holding> held;         // by state slot
  long long serials = 0;
  Cache(int G, const int* num_pages, const int* windows, int ps, int max_requests)
      : page_size(ps), slots(max_requests), held((size_t)max_requests) {
    for (int g = 0; g < G; ++g) { pools.emplace_back(num_pages[g]); window.push_back(windows[g]); }
  }
  int pages_for(int tokens) const { return (tokens + page_size - 1) / page_size; }
};

// What the rows of one decode-graph slot's block tables hold (see fill_decode).
struct Rows {
  int S, G;
  std::vector<long long> serial;     // per row, -1: nothing yet
  std::vector<int> epoch;
  std::vector<int> count;            // [row][group] pages written
  Rows(int s, int g) : S(s), G(g), serial((size_t)s, -1), epoch((size_t)s, 0), count((size_t)s * g, 0) {}
};

inline Holding* holding(Cache* c, int h) {
  if (h < 0 || h >= (int)c->held.size() || !c->held[(size_t)h].live) return nullptr;
  return &c->held[(size_t)h];
}

}  // namespace

// ------------------------------------------------------------------------------------ pool
RLLM_API void* rllm_pool_new(int num_pages) { return num_pages < 0 ? nullptr : new Pool(num_pages); }
RLLM_API void rllm_pool_delete(void* p) { delete static_cast<Pool*>(p); }
RLLM_API int rllm_pool_alloc(void* p, long long owner) { return static_cast<Pool*>(p)->alloc(owner); }
RLLM_API int rllm_pool_release(void* p, int page, long long owner) { return static_cast<Pool*>(p)->release(page, owner); }
RLLM_API long long rllm_pool_holder(void* p, int page) {
  Pool* q = static_cast<Pool*>(p);
  return (page < 0 || page >= q->num_pages) ? NOBODY : q->holder[(size_t)page];
}
RLLM_API long long rllm_pool_nobody() { return NOBODY; }
RLLM_API int rllm_pool_num_free(void* p) { return (int)static_cast<Pool*>(p)->free_list.size(); }
RLLM_API int rllm_pool_num_pages(void* p) { return static_cast<Pool*>(p)->num_pages; }
RLLM_API int rllm_pool_check(void* p) { return static_cast<Pool*>(p)->check(); }

// ------------------------------------------------------------------------------------ cache
RLLM_API void* rllm_cache_new(int groups, const int* num_pages, const int* windows, int page_size, int max_requests) {
  if (groups < 0 || page_size <= 0 || max_requests < 0) return nullptr;
  return new Cache(groups, num_pages, windows, page_size, max_requests);
}
RLLM_API void rllm_cache_delete(void* c) { delete static_cast<Cache*>(c); }
RLLM_API void* rllm_cache_pool(void* c, int group) { return &static_cast<Cache*>(c)->pools[(size_t)group]; }
RLLM_API void* rllm_cache_slots(void* c) { return &static_cast<Cache*>(c)->slots; }

// A new holding for request `rid`: its state slot (>= 0, also the handle), or -1 when every slot is taken.
RLLM_API int rllm_cache_open(void* cv, long long rid) {
  Cache* c = static_cast<Cache*>(cv);
  const int slot = c->slots.alloc(rid);
  if (slot < 0) return slot;
  Holding& h = c->held[(size_t)slot];
  h.live = true; h.rid = rid; h.num_tokens = 0; h.serial = ++c->serials; h.epoch = 0;
  h.pages.assign(c->pools.size(), {});
  return slot;
}

// Pages for positions [num_tokens, new_total) in every group, or none at all.
// 0 fine | -1 out of pages (nothing changed) | -2 the request would shrink | -9 no such holding
RLLM_API int rllm_cache_reserve(void* cv, int handle, int new_total) {
  Cache* c = static_cast<Cache*>(cv);
  Holding* h = holding(c, handle);
  if (!h) return -9;
  if (new_total < h->num_tokens) return -2;
  const int total = c->pages_for(new_total);
  for (size_t g = 0; g < c->pools.size(); ++g) {
    const int need = total - (int)h->pages[g].size();
    if (need > (int)c->pools[g].free_list.size()) return -1;
  }
  for (size_t g = 0; g < c->pools.size(); ++g)
    while ((int)h->pages[g].size() < total) {
      const int page = c->pools[g].alloc(h->rid);
      if (page < 0) return -8;                                    // the count above said there was one
      h->pages[g].push_back(page);
    }
  return 0;
}

// Could `reserve(handle, new_total)` succeed now? handle < 0: a request that holds nothing yet.
RLLM_API int rllm_cache_can_reserve(void* cv, int handle, int new_total) {
  Cache* c = static_cast<Cache*>(cv);
  Holding* h = handle >= 0 ? holding(c, handle) : nullptr;
  const int total = c->pages_for(new_total);
  for (size_t g = 0; g < c->pools.size(); ++g) {
    const int have = h ? (int)h->pages[g].size() : 0;
    if (total - have > (int)c->pools[g].free_list.size()) return 0;
  }
  return 1;
}

// The step stored positions up to new_total; pages a window has passed are given back.
// 0 fine | -2 beyond the reserved pages | -9 no such holding | < -10: the pool refused a release
RLLM_API int rllm_cache_commit(void* cv, int handle, int new_total) {
  Cache* c = static_cast<Cache*>(cv);
  Holding* h = holding(c, handle);
  if (!h) return -9;
  const int total = c->pages_for(new_total);
  for (size_t g = 0; g < c->pools.size(); ++g)
    if (total > (int)h->pages[g].size()) return -2;
  h->num_tokens = new_total;
  for (size_t g = 0; g < c->pools.size(); ++g) {
    if (c->window[g] < 0) continue;
    const int first_key = new_total - c->window[g] + 1;           // oldest key the next query sees
    int last = first_key > 0 ? first_key / c->page_size : 0;
    if (last > (int)h->pages[g].size()) last = (int)h->pages[g].size();
    for (int i = 0; i < last; ++i) {
      int& page = h->pages[g][(size_t)i];
      if (page >= 0) {
        const int rc = c->pools[g].release(page, h->rid);
        if (rc) return -10 + rc;
        page = -1;
        ++h->epoch;
      }
    }
  }
  return 0;
}

// Give back pages reserved beyond what the stored positions need (a step that did not run).
RLLM_API int rllm_cache_trim(void* cv, int handle) {
  Cache* c = static_cast<Cache*>(cv);
  Holding* h = holding(c, handle);
  if (!h) return -9;
  const int keep = c->pages_for(h->num_tokens);
  for (size_t g = 0; g < c->pools.size(); ++g)
    while ((int)h->pages[g].size() > keep) {
      const int page = h->pages[g].back();
      h->pages[g].pop_back();
      ++h->epoch;
      if (page >= 0) {
        const int rc = c->pools[g].release(page, h->rid);
        if (rc) return -10 + rc;
      }
    }
  return 0;
}

RLLM_API int rllm_cache_close(void* cv, int handle) {
  Cache* c = static_cast<Cache*>(cv);
  Holding* h = holding(c, handle);
  if (!h) return -9;
  for (size_t g = 0; g < c->pools.size(); ++g) {
    for (int page : h->pages[g])
      if (page >= 0) {
        const int rc = c->pools[g].release(page, h->rid);
        if (rc) return -10 + rc;
      }
    h->pages[g].clear();
  }
  const int rc = c->slots.release(handle, h->rid);
  h->live = false;
  return rc ? -10 + rc : 0;
}

RLLM_API int rllm_cache_num_tokens(void* cv, int handle) { Holding* h = holding(static_cast<Cache*>(cv), handle); return h ? h->num_tokens : -9; }
RLLM_API long long rllm_cache_serial(void* cv, int handle) { Holding* h = holding(static_cast<Cache*>(cv), handle); return h ? h->serial : -9; }
RLLM_API int rllm_cache_epoch(void* cv, int handle) { Holding* h = holding(static_cast<Cache*>(cv), handle); return h ? h->epoch : -9; }
RLLM_API int rllm_cache_num_held(void* cv, int handle, int group) {
  Holding* h = holding(static_cast<Cache*>(cv), handle);
  return h ? (int)h->pages[(size_t)group].size() : -9;
}
// Copies the block table of (holding, group) into out[0 .. n): returns n.
RLLM_API int rllm_cache_pages(void* cv, int handle, int group, int* out, int cap) {
  Holding* h = holding(static_cast<Cache*>(cv), handle);
  if (!h) return -9;
  const std::vector<int>& p = h->pages[(size_t)group];
  const int n = (int)p.size() < cap ? (int)p.size() : cap;
  if (n > 0) std::memcpy(out, p.data(), (size_t)n * sizeof(int));
  return (int)p.size();
}

// No page lost, held twice or freed twice; the holders are live requests.
// 0 fine | 100 * (group + 1) + code
RLLM_API int rllm_cache_check(void* cv) {
  Cache* c = static_cast<Cache*>(cv);
  for (size_t g = 0; g < c->pools.size(); ++g) {
    const int rc = c->pools[g].check();
    if (rc) return 100 * ((int)g + 1) - rc;
    std::vector<char> seen((size_t)c->pools[g].num_pages, 0);
    int held = 0;
    for (const Holding& h : c->held) {
      if (!h.live) continue;
      for (int page : h.pages[g]) {
        if (page < 0) continue;
        if (page >= c->pools[g].num_pages) return 100 * ((int)g + 1) + 4;
        if (seen[(size_t)page]) return 100 * ((int)g + 1) + 5;              // in two tables
        seen[(size_t)page] = 1;
        if (c->pools[g].holder[(size_t)page] != h.rid) return 100 * ((int)g + 1) + 6;   // in a table, not held
        ++held;
      }
    }
    if (held + (int)c->pools[g].free_list.size() != c->pools[g].num_pages) return 100 * ((int)g + 1) + 7;   // lost
  }
  const int rc = c->slots.check();
  return rc ? 1000 - rc : 0;
}

// ------------------------------------------------------------------------------------ decode metadata
RLLM_API void* rllm_rows_new(int S, int G) { return new Rows(S, G); }
RLLM_API void rllm_rows_delete(void* r) { delete static_cast<Rows*>(r); }
// Rows `from` and up no longer hold what they were written with (the caller has put stand-in rows there).
RLLM_API void rllm_rows_forget(void* r, int from) {
  Rows* rows = static_cast<Rows*>(r);
  for (int s = from < 0 ? 0 : from; s < rows->S; ++s) {
    rows->serial[(size_t)s] = -1;
    for (int g = 0; g < rows->G; ++g) rows->count[(size_t)s * rows->G + g] = 0;
  }
}

// The metadata of a step in which each of S holdings brings one token, into the first S rows of
// `host` (int32; the buffer may have more rows than S, which this leaves alone):
//   offs[0] ids | offs[1] positions | offs[4] key counts | offs[5] state slots |
//   per group g: offs[7 + 2g] cache slot of the new token, offs[8 + 2g] block table [S, P].
// (Vectors 2, 3 and 6 do not change from step to step and are written when the buffer is made.)
// Returns 1 when a block-table row was touched, 0 when not, < 0 on a bad handle or a table wider than P.
RLLM_API int rllm_fill_decode(void* cv, void* rv, int S, const int* handles, const int* tokens, int P,
                              int* host, const long long* offs) {
  Cache* c = static_cast<Cache*>(cv);
  Rows* rows = static_cast<Rows*>(rv);
  const int G = (int)c->pools.size();
  if (S > rows->S || G != rows->G) return -3;
  const int ps = c->page_size;
  int dirty = 0;
  for (int s = 0; s < S; ++s) {
    Holding* h = holding(c, handles[s]);
    if (!h) return -9;
    const int n = h->num_tokens;
    host[offs[0] + s] = tokens[s];
    host[offs[1] + s] = n;
    host[offs[4] + s] = n + 1;
    host[offs[5] + s] = handles[s];
    const bool same = rows->serial[(size_t)s] == h->serial && rows->epoch[(size_t)s] == h->epoch;
    for (int g = 0; g < G; ++g) {
      const std::vector<int>& pages = h->pages[(size_t)g];
      const int held = (int)pages.size();
      if (n / ps >= held) return -2;                              // the new token has no page
      if (held > P) return -4;
      host[offs[7 + 2 * g] + s] = pages[(size_t)(n / ps)] * ps + n % ps;
      int* row = host + offs[8 + 2 * g] + (long long)s * P;
      int done = same ? rows->count[(size_t)s * G + g] : 0;
      if (done == held) continue;
      dirty = 1;
      if (done == 0 || done > held) { for (int i = 0; i < P; ++i) row[i] = -1; done = 0; }
      for (int i = done; i < held; ++i) row[i] = pages[(size_t)i];
      rows->count[(size_t)s * G + g] = held;
    }
    if (!same) { rows->serial[(size_t)s] = h->serial; rows->epoch[(size_t)s] = h->epoch; dirty = 1; }
  }
  return dirty;
}
