// Paged KV bookkeeping on the host: reference-counted block pool and the automatic prefix cache.
//
// Behaviour follows the reference driver (crates/poot-llm/src/driver/block_table.rs:18-303 and
// crates/poot-llm/src/driver/prefix_cache.rs:15-250):
//   * blocks of 16 token positions, reference counted; a block returns to the free list at count 0;
//   * the prefix cache is keyed by (FNV-1a chain hash of the full prefix blocks, weights identity);
//     a hit is accepted only when the entry's tokens and its parent hash equal the probe's (a hash
//     collision is a miss, never shared K/V); the partial tail block is never cached; the cache
//     holds one reference per cached block and drops it in evict_unused() when it is the only holder.
// Exposed as a C ABI over opaque handles; Python drives it through ctypes.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <unordered_map>
#include <vector>

#define HOST_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int kBlock = 16;
constexpr uint64_t kChainRoot = 0xcbf29ce484222325ull;

inline uint64_t chain_hash(uint64_t prev, const uint32_t* block) {
  uint64_t h = prev ^ (0x100000001b3ull * 0x517cc1b727220a95ull);
  for (int i = 0; i < kBlock; ++i) {
    h ^= (uint64_t)block[i];
    h *= 0x100000001b3ull;
  }
  return h;
}

struct Pool {
  std::vector<int32_t> refs;
  std::vector<int32_t> free_list;  // LIFO
  explicit Pool(int n) : refs(n, 0) {
    free_list.reserve(n);
    for (int i = n - 1; i >= 0; --i) free_list.push_back(i);
  }
};

struct Key {
  uint64_t hash, identity;
  bool operator==(const Key& o) const { return hash == o.hash && identity == o.identity; }
};
struct KeyHash {
  size_t operator()(const Key& k) const { return (size_t)(k.hash ^ (k.identity * 0x9E3779B97F4A7C15ull)); }
};
struct Entry {
  uint64_t parent;
  uint32_t tokens[kBlock];
  int32_t block;
  uint64_t last_use;
};

struct PrefixCache {
  std::unordered_map<Key, Entry, KeyHash> cached;
  uint64_t clock = 0;
  uint64_t hit_tokens = 0, query_tokens = 0;
  bool force_collisions = false;  // tests: every block hashes to the same value
  uint64_t hash(uint64_t prev, const uint32_t* b) const { return force_collisions ? 42ull : chain_hash(prev, b); }
};

}  // namespace

// ---------------------------------------------------------------- pool
HOST_API void* poot_pool_new(int num_blocks) { return new Pool(num_blocks); }
HOST_API void poot_pool_free(void* p) { delete (Pool*)p; }
HOST_API int poot_pool_available(void* p) { return (int)((Pool*)p)->free_list.size(); }
HOST_API int poot_pool_total(void* p) { return (int)((Pool*)p)->refs.size(); }
HOST_API int poot_pool_refcount(void* p, int b) { return ((Pool*)p)->refs[b]; }

// Allocate n blocks into out; returns n on success, -1 (nothing allocated) when fewer are free.
HOST_API int poot_pool_alloc(void* p, int n, int32_t* out) {
  Pool* pool = (Pool*)p;
  if ((int)pool->free_list.size() < n) return -1;
  for (int i = 0; i < n; ++i) {
    int32_t b = pool->free_list.back();
    pool->free_list.pop_back();
    pool->refs[b] = 1;
    out[i] = b;
  }
  return n;
}
HOST_API void poot_pool_retain(void* p, int b) { ((Pool*)p)->refs[b] += 1; }
// Returns the remaining count; the block goes back to the free list at 0.  -1 on a double free.
HOST_API int poot_pool_release(void* p, int b) {
  Pool* pool = (Pool*)p;
  if (b < 0 || b >= (int)pool->refs.size() || pool->refs[b] <= 0) return -1;
  int r = --pool->refs[b];
  if (r == 0) pool->free_list.push_back(b);
  return r;
}

// ---------------------------------------------------------------- prefix cache
HOST_API void* poot_prefix_new() { return new PrefixCache(); }
HOST_API void poot_prefix_free(void* c) { delete (PrefixCache*)c; }
HOST_API void poot_prefix_force_collisions(void* c, int on) { ((PrefixCache*)c)->force_collisions = on != 0; }
HOST_API int poot_prefix_len(void* c) { return (int)((PrefixCache*)c)->cached.size(); }
HOST_API uint64_t poot_prefix_hit_tokens(void* c) { return ((PrefixCache*)c)->hit_tokens; }
HOST_API uint64_t poot_prefix_query_tokens(void* c) { return ((PrefixCache*)c)->query_tokens; }
HOST_API uint64_t poot_chain_hash(uint64_t prev, const uint32_t* block) { return chain_hash(prev, block); }
HOST_API uint64_t poot_chain_root() { return kChainRoot; }

// Longest cached prefix of `tokens` (n_tokens) in whole blocks.  Each matched block is retained for the caller
// and written to out_blocks.  At most max_blocks are matched.  Returns the number of matched blocks.
HOST_API int poot_prefix_match(void* c, void* p, uint64_t identity, const uint32_t* tokens, int n_tokens,
                               int max_blocks, int32_t* out_blocks) {
  PrefixCache* pc = (PrefixCache*)c;
  Pool* pool = (Pool*)p;
  int full = n_tokens / kBlock;
  if (full > max_blocks) full = max_blocks;
  uint64_t parent = kChainRoot;
  int matched = 0;
  pc->query_tokens += (uint64_t)n_tokens;
  for (int i = 0; i < full; ++i) {
    const uint32_t* blk = tokens + (size_t)i * kBlock;
    uint64_t h = pc->hash(parent, blk);
    auto it = pc->cached.find(Key{h, identity});
    if (it == pc->cached.end()) break;
    Entry& e = it->second;
    if (e.parent != parent || std::memcmp(e.tokens, blk, sizeof(e.tokens)) != 0) break;  // collision = miss
    e.last_use = ++pc->clock;
    pool->refs[e.block] += 1;
    out_blocks[matched++] = e.block;
    parent = h;
  }
  pc->hit_tokens += (uint64_t)matched * kBlock;
  return matched;
}

// Register the full blocks of a finished prompt: block i of the sequence holds tokens [16i, 16i+16).
// Blocks already cached under the same key are left alone.  Returns prompt tokens covered by cached blocks.
HOST_API int poot_prefix_register(void* c, void* p, uint64_t identity, const uint32_t* tokens, int n_tokens,
                                  const int32_t* seq_blocks, int n_seq_blocks) {
  PrefixCache* pc = (PrefixCache*)c;
  Pool* pool = (Pool*)p;
  int full = n_tokens / kBlock;
  if (full > n_seq_blocks) full = n_seq_blocks;
  uint64_t parent = kChainRoot;
  int covered = 0;
  for (int i = 0; i < full; ++i) {
    const uint32_t* blk = tokens + (size_t)i * kBlock;
    uint64_t h = pc->hash(parent, blk);
    Key key{h, identity};
    auto it = pc->cached.find(key);
    if (it == pc->cached.end()) {
      Entry e;
      e.parent = parent;
      std::memcpy(e.tokens, blk, sizeof(e.tokens));
      e.block = seq_blocks[i];
      e.last_use = ++pc->clock;
      pool->refs[e.block] += 1;  // the cache's own reference
      pc->cached.emplace(key, e);
    } else if (it->second.parent != parent || std::memcmp(it->second.tokens, blk, sizeof(it->second.tokens)) != 0) {
      break;  // a colliding entry owns the key: stop, later blocks could never be matched through it
    }
    covered += kBlock;
    parent = h;
  }
  return covered;
}

// Drop entries whose block only the cache still references until `want` blocks were freed (want <= 0: all of them).
// Order: leaves of the prefix chains first, least recently used first among them.  A match stamps a chain's blocks in
// prefix order, so a parent always carries an older stamp than its children; evicting by stamp alone would take the
// parent and leave children that can never be matched again (the match stops at the missing parent) yet still hold
// blocks.  An entry becomes evictable when no cached entry names it as parent.  Returns the blocks returned to the pool.
HOST_API int poot_prefix_evict_unused(void* c, void* p, int want) {
  PrefixCache* pc = (PrefixCache*)c;
  Pool* pool = (Pool*)p;
  std::unordered_map<Key, int, KeyHash> children;
  for (auto& kv : pc->cached) children[Key{kv.second.parent, kv.first.identity}] += 1;  // the root key names no entry
  using Cand = std::pair<uint64_t, Key>;
  auto later = [](const Cand& a, const Cand& b) { return a.first > b.first; };
  std::vector<Cand> heap;
  auto evictable = [&](const Key& k, const Entry& e) {
    auto ch = children.find(k);
    return pool->refs[e.block] == 1 && (ch == children.end() || ch->second <= 0);
  };
  for (auto& kv : pc->cached)
    if (evictable(kv.first, kv.second)) heap.push_back({kv.second.last_use, kv.first});
  std::make_heap(heap.begin(), heap.end(), later);
  int freed = 0;
  while (!heap.empty() && !(want > 0 && freed >= want)) {
    std::pop_heap(heap.begin(), heap.end(), later);
    Key k = heap.back().second;
    heap.pop_back();
    auto it = pc->cached.find(k);
    if (it == pc->cached.end()) continue;
    const Key parent{it->second.parent, k.identity};
    const int b = it->second.block;
    pc->cached.erase(it);
    if (--pool->refs[b] == 0) pool->free_list.push_back(b);
    ++freed;
    auto ch = children.find(parent);
    if (ch != children.end() && --ch->second <= 0) {
      auto pit = pc->cached.find(parent);
      if (pit != pc->cached.end() && !(pit->first == k) && evictable(pit->first, pit->second)) {
        heap.push_back({pit->second.last_use, pit->first});
        std::push_heap(heap.begin(), heap.end(), later);
      }
    }
  }
  return freed;
}

// Number of cached blocks that only the cache references: what evict_unused() could return to the pool.
HOST_API int poot_prefix_count_unused(void* c, void* p) {
  PrefixCache* pc = (PrefixCache*)c;
  Pool* pool = (Pool*)p;
  int n = 0;
  for (auto& kv : pc->cached)
    if (pool->refs[kv.second.block] == 1) ++n;
  return n;
}

// Remove every entry of one weights identity (an adapter that was unloaded).
HOST_API int poot_prefix_drop_identity(void* c, void* p, uint64_t identity) {
  PrefixCache* pc = (PrefixCache*)c;
  Pool* pool = (Pool*)p;
  int n = 0;
  for (auto it = pc->cached.begin(); it != pc->cached.end();) {
    if (it->first.identity == identity) {
      int b = it->second.block;
      if (--pool->refs[b] == 0) pool->free_list.push_back(b);
      it = pc->cached.erase(it);
      ++n;
    } else {
      ++it;
    }
  }
  return n;
}
