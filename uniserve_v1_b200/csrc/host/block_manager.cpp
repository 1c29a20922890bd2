// In-process paged KV block manager with a prefix cache.
//
// Pages are the unit of KV storage (page_size tokens of every layer).  Page 0 is
// the padding sentinel and is never handed out.  A full page can be committed
// under a chained content key (SHA-256 over the previous key and the page's
// token ids, rooted at a seed that names the weights and the isolation salt);
// committed pages whose reference count drops to zero stay resident and are
// evicted least-recently-used when an allocation needs room.
//
// The verbs follow the buffer-pool interface the reference's scheduler speaks
// (Attach/Allocate/Pin/Release/Commit/Evict; crates/storage/src/runtime.rs:349-497
// and crates/storage/src/key.rs:1-30, reference project paths), folded into one
// process: there is no Storage Server.
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <list>
#include <mutex>
#include <unordered_map>
#include <vector>

#define US_API extern "C" __attribute__((visibility("default")))

namespace {

// ------------------------------------------------------------------ SHA-256 --
struct Sha256 {
  uint32_t h[8];
  uint8_t buf[64];
  uint64_t len = 0;
  size_t fill = 0;
  static constexpr uint32_t K[64] = {
      0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4,
      0xab1c5ed5, 0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe,
      0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f,
      0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7,
      0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc,
      0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85, 0xa2bfe8a1, 0xa81a664b,
      0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116,
      0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
      0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7,
      0xc67178f2};
  Sha256() {
    static const uint32_t init[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a,
                                     0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    memcpy(h, init, sizeof(h));
  }
  static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
  void block(const uint8_t* p) {
    uint32_t w[64];
    for (int i = 0; i < 16; ++i)
      w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 |
             p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
      const uint32_t ch = (e & f) ^ (~e & g);
      const uint32_t t1 = hh + S1 + ch + K[i] + w[i];
      const uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
      const uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
      const uint32_t t2 = S0 + mj;
      hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
  }
  void update(const void* data, size_t n) {
    const uint8_t* p = (const uint8_t*)data;
    len += n;
    while (n) {
      const size_t take = (64 - fill) < n ? (64 - fill) : n;
      memcpy(buf + fill, p, take);
      fill += take; p += take; n -= take;
      if (fill == 64) { block(buf); fill = 0; }
    }
  }
  void finish(uint8_t out[32]) {
    const uint64_t bits = len * 8;
    const uint8_t one = 0x80, zero = 0;
    update(&one, 1);
    while (fill != 56) update(&zero, 1);
    uint8_t lb[8];
    for (int i = 0; i < 8; ++i) lb[i] = (uint8_t)(bits >> (56 - 8 * i));
    update(lb, 8);
    for (int i = 0; i < 8; ++i) {
      out[4 * i] = (uint8_t)(h[i] >> 24); out[4 * i + 1] = (uint8_t)(h[i] >> 16);
      out[4 * i + 2] = (uint8_t)(h[i] >> 8); out[4 * i + 3] = (uint8_t)h[i];
    }
  }
};
constexpr uint32_t Sha256::K[64];

struct Key {
  uint64_t a, b;
  bool operator==(const Key& o) const { return a == o.a && b == o.b; }
};
struct KeyHash {
  size_t operator()(const Key& k) const { return (size_t)(k.a ^ (k.b * 0x9E3779B97F4A7C15ull)); }
};

struct Pool {
  int num_pages, page_size;
  std::vector<int> ref;
  std::vector<uint8_t> has_key;
  std::vector<Key> key;
  std::vector<int> free_list;
  std::unordered_map<Key, int, KeyHash> cached;
  std::list<int> lru;  // committed pages with ref == 0, oldest first
  std::vector<std::list<int>::iterator> lru_pos;
  std::vector<uint8_t> in_lru;
  uint64_t hits = 0, lookups = 0, evictions = 0;
  // Host tier: content-keyed pages that fell out of the device pool keep living in
  // `host_slots` slots of pinned host memory, LRU-evicted among themselves.  The pool
  // only decides; the caller copies (device page -> host slot before the device page
  // is reused, host slot -> device page on a later hit).
  int host_slots = 0;
  std::vector<int> host_free;
  std::unordered_map<Key, int, KeyHash> host_cached;
  std::vector<Key> host_key;
  std::list<int> host_lru;
  std::vector<std::list<int>::iterator> host_pos;
  // A slot matched for a fetch is pinned (out of `host_lru`) until its host -> device copy
  // has been handed to the caller: an offload decided in between must not recycle it.
  std::vector<int> host_pins;
  std::vector<std::pair<int, int>> offloads;   // (device page, host slot) decided by alloc
  uint64_t host_hits = 0, host_offloads = 0, host_dropped = 0;
  std::mutex mu;
};

// Called with the lock held when a keyed device page is about to be reused.
void offload_page(Pool* p, int page) {
  if (p->host_slots == 0) return;
  const Key k = p->key[page];
  if (p->host_cached.count(k)) return;   // the host already holds this content
  int slot;
  if (!p->host_free.empty()) {
    slot = p->host_free.back();
    p->host_free.pop_back();
  } else if (!p->host_lru.empty()) {
    slot = p->host_lru.front();
    p->host_lru.pop_front();
    p->host_cached.erase(p->host_key[slot]);
  } else {
    p->host_dropped++;                   // every slot is pinned by a pending fetch
    return;
  }
  p->host_key[slot] = k;
  p->host_cached[k] = slot;
  p->host_lru.push_back(slot);
  p->host_pos[slot] = std::prev(p->host_lru.end());
  p->offloads.emplace_back(page, slot);
  p->host_offloads++;
}

}  // namespace

US_API void* us_bm_create(int num_pages, int page_size) {
  if (num_pages < 2 || page_size < 1) return nullptr;
  Pool* p = new Pool();
  p->num_pages = num_pages;
  p->page_size = page_size;
  p->ref.assign(num_pages, 0);
  p->has_key.assign(num_pages, 0);
  p->key.resize(num_pages);
  p->lru_pos.resize(num_pages);
  p->in_lru.assign(num_pages, 0);
  for (int i = num_pages - 1; i >= 1; --i) p->free_list.push_back(i);  // page 0 = sentinel
  return p;
}

US_API void us_bm_destroy(void* h) { delete (Pool*)h; }

US_API int us_bm_num_free(void* h) {
  Pool* p = (Pool*)h;
  std::lock_guard<std::mutex> g(p->mu);
  return (int)(p->free_list.size() + p->lru.size());
}

US_API int us_bm_num_cached(void* h) {
  Pool* p = (Pool*)h;
  std::lock_guard<std::mutex> g(p->mu);
  return (int)p->cached.size();
}

// Takes n pages with reference count 1; evicts cached pages LRU-first when the
// free list runs dry.  Returns 0, or -1 (nothing taken) when n do not fit.
US_API int us_bm_alloc(void* h, int n, int* out) {
  Pool* p = (Pool*)h;
  std::lock_guard<std::mutex> g(p->mu);
  if ((size_t)n > p->free_list.size() + p->lru.size()) return -1;
  for (int i = 0; i < n; ++i) {
    int page;
    if (!p->free_list.empty()) {
      page = p->free_list.back();
      p->free_list.pop_back();
    } else {
      page = p->lru.front();
      p->lru.pop_front();
      p->in_lru[page] = 0;
      offload_page(p, page);
      p->cached.erase(p->key[page]);
      p->has_key[page] = 0;
      p->evictions++;
    }
    p->ref[page] = 1;
    out[i] = page;
  }
  return 0;
}

US_API void us_bm_release(void* h, const int* pages, int n) {
  Pool* p = (Pool*)h;
  std::lock_guard<std::mutex> g(p->mu);
  for (int i = 0; i < n; ++i) {
    const int page = pages[i];
    if (page <= 0 || page >= p->num_pages || p->ref[page] <= 0) continue;
    if (--p->ref[page] == 0) {
      if (p->has_key[page]) {
        p->lru.push_back(page);
        p->lru_pos[page] = std::prev(p->lru.end());
        p->in_lru[page] = 1;
      } else {
        p->free_list.push_back(page);
      }
    }
  }
}

// Chained page keys: state_i = SHA256(state_{i-1} || tokens of page i); the key
// is the first 16 bytes of the state.  `seed32` is the 32-byte root (weights
// identity + isolation salt).  Writes 2 x uint64 per full page; returns the count.
US_API int us_bm_hash_chain(const uint8_t* seed32, const int* tokens, int n_tokens, int page_size,
                            uint64_t* out_keys) {
  uint8_t state[32];
  memcpy(state, seed32, 32);
  const int full = n_tokens / page_size;
  for (int i = 0; i < full; ++i) {
    Sha256 s;
    s.update(state, 32);
    s.update(tokens + (size_t)i * page_size, sizeof(int) * (size_t)page_size);
    s.finish(state);
    memcpy(&out_keys[2 * i], state, 16);
  }
  return full;
}

US_API void us_sha256(const void* data, size_t n, uint8_t out[32]) {
  Sha256 s;
  s.update(data, n);
  s.finish(out);
}

// Pins the longest run of leading keys present in the cache; returns its length.
US_API int us_bm_match_prefix(void* h, const uint64_t* keys, int n, int* out_pages) {
  Pool* p = (Pool*)h;
  std::lock_guard<std::mutex> g(p->mu);
  int m = 0;
  p->lookups += (uint64_t)n;
  for (; m < n; ++m) {
    auto it = p->cached.find(Key{keys[2 * m], keys[2 * m + 1]});
    if (it == p->cached.end()) break;
    const int page = it->second;
    if (p->ref[page] == 0 && p->in_lru[page]) {
      p->lru.erase(p->lru_pos[page]);
      p->in_lru[page] = 0;
    }
    p->ref[page]++;
    out_pages[m] = page;
  }
  p->hits += (uint64_t)m;
  return m;
}

// Registers a full page under its key.  Returns the page that now owns the key
// (an earlier page when the same content was committed before).
US_API int us_bm_commit(void* h, int page, uint64_t ka, uint64_t kb) {
  Pool* p = (Pool*)h;
  std::lock_guard<std::mutex> g(p->mu);
  if (page <= 0 || page >= p->num_pages) return -1;
  const Key k{ka, kb};
  auto it = p->cached.find(k);
  if (it != p->cached.end()) return it->second;
  if (p->has_key[page]) p->cached.erase(p->key[page]);
  p->key[page] = k;
  p->has_key[page] = 1;
  p->cached[k] = page;
  return page;
}

// Committed (content-keyed) device pages, most recently released last: keys_out [cap][2],
// pages_out [cap].  Pages in use come first (they have no place in the LRU order).  Returns
// the number written (at most cap).
US_API int us_bm_enumerate(void* h, uint64_t* keys_out, int* pages_out, int cap) {
  Pool* p = (Pool*)h;
  std::lock_guard<std::mutex> g(p->mu);
  int n = 0;
  for (int page = 1; page < p->num_pages && n < cap; ++page) {
    if (p->has_key[page] && !p->in_lru[page]) {
      keys_out[2 * n] = p->key[page].a;
      keys_out[2 * n + 1] = p->key[page].b;
      pages_out[n++] = page;
    }
  }
  for (int page : p->lru) {
    if (n >= cap) break;
    if (!p->has_key[page]) continue;
    keys_out[2 * n] = p->key[page].a;
    keys_out[2 * n + 1] = p->key[page].b;
    pages_out[n++] = page;
  }
  return n;
}

US_API void us_bm_stats(void* h, uint64_t* hits, uint64_t* lookups, uint64_t* evictions) {
  Pool* p = (Pool*)h;
  std::lock_guard<std::mutex> g(p->mu);
  *hits = p->hits;
  *lookups = p->lookups;
  *evictions = p->evictions;
}

US_API int us_bm_refcount(void* h, int page) {
  Pool* p = (Pool*)h;
  std::lock_guard<std::mutex> g(p->mu);
  return (page >= 0 && page < p->num_pages) ? p->ref[page] : -1;
}

// Drops every cached page that is not referenced (Evict-all / flush).
US_API int us_bm_flush(void* h) {
  Pool* p = (Pool*)h;
  std::lock_guard<std::mutex> g(p->mu);
  int n = 0;
  while (!p->lru.empty()) {
    const int page = p->lru.front();
    p->lru.pop_front();
    p->in_lru[page] = 0;
    p->cached.erase(p->key[page]);
    p->has_key[page] = 0;
    p->free_list.push_back(page);
    ++n;
  }
  return n;
}

// ---------------------------------------------------------------- host tier --
US_API int us_bm_enable_host(void* h, int host_slots) {
  Pool* p = (Pool*)h;
  std::lock_guard<std::mutex> g(p->mu);
  if (host_slots < 0 || p->host_slots != 0) return -1;
  p->host_slots = host_slots;
  p->host_key.resize(host_slots);
  p->host_pos.resize(host_slots);
  p->host_pins.assign(host_slots, 0);
  for (int i = host_slots - 1; i >= 0; --i) p->host_free.push_back(i);
  return 0;
}

// Moves the (device page, host slot) copies decided since the last call into
// out[2 * i], out[2 * i + 1]; returns how many (at most `cap`; the rest stay queued).
US_API int us_bm_take_offloads(void* h, int* out, int cap) {
  Pool* p = (Pool*)h;
  std::lock_guard<std::mutex> g(p->mu);
  const int n = (int)std::min((size_t)cap, p->offloads.size());
  for (int i = 0; i < n; ++i) {
    out[2 * i] = p->offloads[i].first;
    out[2 * i + 1] = p->offloads[i].second;
  }
  p->offloads.erase(p->offloads.begin(), p->offloads.begin() + n);
  return n;
}

// Host slots of the leading run of `keys` that the host tier holds; returns the length of
// the run.  Every returned slot is pinned (taken out of the LRU list, so no offload can
// recycle it) until `us_bm_unpin_host` gives it back.
US_API int us_bm_match_host(void* h, const uint64_t* keys, int n, int* out_slots) {
  Pool* p = (Pool*)h;
  std::lock_guard<std::mutex> g(p->mu);
  int m = 0;
  for (; m < n; ++m) {
    auto it = p->host_cached.find(Key{keys[2 * m], keys[2 * m + 1]});
    if (it == p->host_cached.end()) break;
    const int slot = it->second;
    if (p->host_pins[slot]++ == 0) p->host_lru.erase(p->host_pos[slot]);
    out_slots[m] = slot;
  }
  p->host_hits += (uint64_t)m;
  return m;
}

// Ends the pins `us_bm_match_host` took (once the copies are issued, or for slots the
// caller did not use); an unpinned slot re-enters the LRU list as most recently used.
US_API void us_bm_unpin_host(void* h, const int* slots, int n) {
  Pool* p = (Pool*)h;
  std::lock_guard<std::mutex> g(p->mu);
  for (int i = 0; i < n; ++i) {
    const int slot = slots[i];
    if (slot < 0 || slot >= p->host_slots || p->host_pins[slot] <= 0) continue;
    if (--p->host_pins[slot] == 0) {
      p->host_lru.push_back(slot);
      p->host_pos[slot] = std::prev(p->host_lru.end());
    }
  }
}

US_API void us_bm_host_stats(void* h, uint64_t* hits, uint64_t* offloads, int* used) {
  Pool* p = (Pool*)h;
  std::lock_guard<std::mutex> g(p->mu);
  *hits = p->host_hits;
  *offloads = p->host_offloads;
  *used = (int)p->host_cached.size();
}
