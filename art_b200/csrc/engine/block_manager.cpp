// Paged-KV block manager with reference counting and hash-chained prefix cache.
//
// The KV cache of the rollout engine is a pool of fixed-size blocks.  A sequence owns a
// list of block ids (its block table).  Full blocks whose content is known are registered
// under a chain hash  h_i = H(h_{i-1}, tokens of block i, salt)  so that a later request
// with the same prefix (same adapter salt) re-uses them instead of recomputing the
// prefill.  Blocks with refcount 0 that still hold registered content sit in an LRU list
// and are evicted only when the free list is empty.
//
// This is the host-side half of what the reference gets from its third-party engine's
// block manager / prefix cache (enable_prefix_caching, src/art/dev/model.py:33;
// reset_prefix_cache before training, src/art/local/state.py:146-171).
#include <cstdint>
#include <cstring>
#include <list>
#include <mutex>
#include <unordered_map>
#include <vector>

#define ARTB_API extern "C" __attribute__((visibility("default")))

namespace {

struct Block {
  int ref = 0;
  uint64_t hash = 0;  // 0 = content not registered
  std::list<int>::iterator lru_it;
  bool in_lru = false;
};

struct BlockManager {
  int num_blocks, block_size;
  bool prefix_cache;
  std::vector<Block> blocks;
  std::vector<int> free_list;            // blocks with no registered content
  std::list<int> lru;                    // refcount-0 blocks with registered content (front = oldest)
  std::unordered_map<uint64_t, int> by_hash;
  std::mutex mu;
  uint64_t hits = 0, queries = 0;

  BlockManager(int n, int bs, bool pc) : num_blocks(n), block_size(bs), prefix_cache(pc), blocks(n) {
    free_list.reserve(n);
    for (int i = n - 1; i >= 0; --i) free_list.push_back(i);
  }
  int num_free() const { return static_cast<int>(free_list.size() + lru.size()); }

  int take_one() {
    if (!free_list.empty()) {
      int b = free_list.back();
      free_list.pop_back();
      return b;
    }
    if (lru.empty()) return -1;
    int b = lru.front();
    lru.pop_front();
    Block& blk = blocks[b];
    blk.in_lru = false;
    if (blk.hash) {
      auto it = by_hash.find(blk.hash);
      if (it != by_hash.end() && it->second == b) by_hash.erase(it);
      blk.hash = 0;
    }
    return b;
  }
};

inline uint64_t mix(uint64_t h, uint64_t v) {
  h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
  h *= 0xff51afd7ed558ccdull;
  h ^= h >> 33;
  return h;
}

uint64_t chain_hash(uint64_t prev, const int32_t* tok, int n, uint64_t salt) {
  uint64_t h = mix(prev ^ 0x1234567ull, salt);
  for (int i = 0; i < n; ++i) h = mix(h, static_cast<uint32_t>(tok[i]));
  return h ? h : 1;
}

}  // namespace

ARTB_API void* artb_bm_create(int num_blocks, int block_size, int enable_prefix_cache) {
  if (num_blocks <= 0 || block_size <= 0) return nullptr;
  return new BlockManager(num_blocks, block_size, enable_prefix_cache != 0);
}
ARTB_API void artb_bm_destroy(void* h) { delete static_cast<BlockManager*>(h); }
ARTB_API int artb_bm_num_free(void* h) {
  auto* bm = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> g(bm->mu);
  return bm->num_free();
}
ARTB_API int artb_bm_num_blocks(void* h) { return static_cast<BlockManager*>(h)->num_blocks; }

// Allocate n fresh blocks (refcount 1).  Returns 0, or -1 (nothing allocated) if fewer than n are free.
ARTB_API int artb_bm_alloc(void* h, int n, int* out) {
  auto* bm = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> g(bm->mu);
  if (bm->num_free() < n) return -1;
  for (int i = 0; i < n; ++i) {
    int b = bm->take_one();
    bm->blocks[b].ref = 1;
    out[i] = b;
  }
  return 0;
}

// Drop one reference on each block.  Registered blocks that reach 0 become evictable (LRU).
ARTB_API void artb_bm_free(void* h, const int* ids, int n) {
  auto* bm = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> g(bm->mu);
  for (int i = 0; i < n; ++i) {
    int b = ids[i];
    if (b < 0 || b >= bm->num_blocks) continue;
    Block& blk = bm->blocks[b];
    if (blk.ref <= 0) continue;
    if (--blk.ref == 0) {
      if (blk.hash && bm->prefix_cache) {
        bm->lru.push_back(b);
        blk.lru_it = std::prev(bm->lru.end());
        blk.in_lru = true;
      } else {
        blk.hash = 0;
        bm->free_list.push_back(b);
      }
    }
  }
}

// Longest cached prefix of `tokens` in whole blocks.  Matched blocks get one more reference
// and are written to out (at most max_out).  Returns the number of matched blocks.
ARTB_API int artb_bm_match_prefix(void* h, const int32_t* tokens, int n_tokens, uint64_t salt, int* out, int max_out) {
  auto* bm = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> g(bm->mu);
  bm->queries++;
  if (!bm->prefix_cache) return 0;
  int matched = 0;
  uint64_t prev = 0;
  const int bs = bm->block_size;
  for (int off = 0; off + bs <= n_tokens && matched < max_out; off += bs) {
    uint64_t hh = chain_hash(prev, tokens + off, bs, salt);
    auto it = bm->by_hash.find(hh);
    if (it == bm->by_hash.end()) break;
    int b = it->second;
    Block& blk = bm->blocks[b];
    if (blk.in_lru) {
      bm->lru.erase(blk.lru_it);
      blk.in_lru = false;
    }
    blk.ref++;
    out[matched++] = b;
    prev = hh;
  }
  if (matched) bm->hits++;
  return matched;
}

// Register the content of the first n_tokens/block_size blocks of a sequence so later
// requests can match them.  Blocks already registered (or duplicated by another block
// with the same hash) are left as they are.
ARTB_API void artb_bm_commit(void* h, const int* block_ids, int n_blocks, const int32_t* tokens, int n_tokens,
                             uint64_t salt) {
  auto* bm = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> g(bm->mu);
  if (!bm->prefix_cache) return;
  uint64_t prev = 0;
  const int bs = bm->block_size;
  for (int i = 0; i < n_blocks && (i + 1) * bs <= n_tokens; ++i) {
    uint64_t hh = chain_hash(prev, tokens + i * bs, bs, salt);
    prev = hh;
    int b = block_ids[i];
    if (b < 0 || b >= bm->num_blocks) break;
    Block& blk = bm->blocks[b];
    if (blk.hash == hh) continue;
    if (blk.hash != 0) continue;                       // holds other registered content
    if (bm->by_hash.find(hh) != bm->by_hash.end()) continue;  // another block already serves this prefix
    blk.hash = hh;
    bm->by_hash[hh] = b;
  }
}

// Forget every registered prefix (used when the adapter that produced the KV changes).
ARTB_API void artb_bm_reset_cache(void* h) {
  auto* bm = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> g(bm->mu);
  bm->by_hash.clear();
  for (int b : bm->lru) {
    bm->blocks[b].hash = 0;
    bm->blocks[b].in_lru = false;
    bm->free_list.push_back(b);
  }
  bm->lru.clear();
  for (auto& blk : bm->blocks) blk.hash = 0;
}

ARTB_API void artb_bm_stats(void* h, uint64_t* out4) {
  auto* bm = static_cast<BlockManager*>(h);
  std::lock_guard<std::mutex> g(bm->mu);
  out4[0] = bm->queries;
  out4[1] = bm->hits;
  out4[2] = bm->free_list.size();
  out4[3] = bm->lru.size();
}

// ---------------------------------------------------------------------------- packer
// First-fit-in-order row assignment used by the trainer-side packer: given the length each
// result would add to a row (full length, or completion-only length when its prompt id is
// already present in that row), assign results to rows of capacity seq_len.
//   lens_full[i], lens_tail[i], prompt_id[i]  ->  row_of[i], shared[i]; returns number of rows.
ARTB_API int artb_pack_assign(const int* lens_full, const int* lens_tail, const int64_t* prompt_id, int n, int seq_len,
                              int* row_of, uint8_t* shared) {
  int row = 0, used = 0;
  std::vector<int64_t> in_row;
  for (int i = 0; i < n; ++i) {
    bool sh = false;
    for (int64_t p : in_row)
      if (p == prompt_id[i]) { sh = true; break; }
    int add = sh ? lens_tail[i] : lens_full[i];
    if (used + add > seq_len) {
      ++row;
      used = 0;
      in_row.clear();
      sh = false;
      add = lens_full[i];
    }
    row_of[i] = row;
    shared[i] = sh ? 1 : 0;
    used += add;
    if (used > seq_len) used = seq_len;  // truncated row
    if (!sh) in_row.push_back(prompt_id[i]);
  }
  return n ? row + 1 : 0;
}
