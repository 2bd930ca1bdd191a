// Native host path of an engine step (no GPU work in this file): the KV-block pool with chained-hash prefix
// caching and the per-step attention metadata, in C++ behind the C ABI.
//
// The reference keeps this in Python: BlockManager (engine/block_manager.py:8-157) with a deque whose
// remove() is linear in the pool size (:67) and one xxhash + numpy round trip per block (:45-57), and
// ModelRunner.prepare_prefill / prepare_decode (engine/model_runner.py:202-278) with list.extend(range())
// per block.  Here the pool is an intrusive doubly linked free list (take the oldest, take a particular
// block, return a block: all O(1)), the hash chain is computed in place, and the metadata builders write
// straight into caller-owned (pinned) arrays.
//
// Behaviour is the engine's default mode: reference counts start at 1, so a block is released when its
// last user finishes; a released block keeps its contents and can be revived by a later prefix hit; a
// prefix hit never covers a whole prompt (the block that ends a fully cached prompt is recomputed, so the
// prefill step has a query token); allocation order is the reference's (oldest free block first, FIFO).
#include <string.h>

#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace b200 {
namespace {

struct Pool {
  int32_t num_blocks, block_size;
  std::vector<int32_t> ref;         // reference count, 0 = free
  std::vector<uint8_t> has_hash;    // the block is sealed: `hash` and `tokens` are meaningful
  std::vector<uint64_t> hash;
  std::vector<int32_t> tokens;      // [num_blocks][block_size] contents of sealed blocks
  std::vector<int32_t> prev, next;  // free list links; head = oldest
  int32_t head = -1, tail = -1;
  int64_t num_free = 0;
  std::unordered_map<uint64_t, int32_t> by_hash;

  Pool(int32_t n, int32_t bs)
      : num_blocks(n), block_size(bs), ref(n, 0), has_hash(n, 0), hash(n, 0),
        tokens(static_cast<size_t>(n) * bs, 0), prev(n, -1), next(n, -1) {
    for (int32_t i = 0; i < n; ++i) push_back(i);
    by_hash.reserve(static_cast<size_t>(n) * 2);
  }
  void push_back(int32_t b) {
    prev[b] = tail;
    next[b] = -1;
    if (tail >= 0) next[tail] = b; else head = b;
    tail = b;
    ++num_free;
  }
  void unlink(int32_t b) {
    const int32_t p = prev[b], q = next[b];
    if (p >= 0) next[p] = q; else head = q;
    if (q >= 0) prev[q] = p; else tail = p;
    prev[b] = next[b] = -1;
    --num_free;
  }
  // a free block becomes a fresh one: its stale hash entry (if it still points here) is dropped
  int32_t take_oldest_fresh() {
    const int32_t b = head;
    if (b < 0) return -1;
    unlink(b);
    if (has_hash[b]) {
      auto it = by_hash.find(hash[b]);
      if (it != by_hash.end() && it->second == b) by_hash.erase(it);
      has_hash[b] = 0;
    }
    ref[b] = 1;
    return b;
  }
  void seal(int32_t b, uint64_t h, const int32_t* toks) {
    has_hash[b] = 1;
    hash[b] = h;
    memcpy(&tokens[static_cast<size_t>(b) * block_size], toks, sizeof(int32_t) * block_size);
    by_hash[h] = b;
  }
  bool same_tokens(int32_t b, const int32_t* toks) const {
    return memcmp(&tokens[static_cast<size_t>(b) * block_size], toks, sizeof(int32_t) * block_size) == 0;
  }
};

inline bool valid_block(const Pool* p, int64_t b) { return b >= 0 && b < p->num_blocks; }

}  // namespace
}  // namespace b200

using b200::Pool;

extern "C" void* b200_pool_create(int64_t num_blocks, int32_t block_size) {
  if (num_blocks <= 0 || num_blocks > 2147483647LL || block_size <= 0) return nullptr;
  return new (std::nothrow) Pool(static_cast<int32_t>(num_blocks), block_size);
}

extern "C" void b200_pool_destroy(void* pool) { delete static_cast<Pool*>(pool); }

extern "C" int64_t b200_pool_num_free(const void* pool) {
  return pool ? static_cast<const Pool*>(pool)->num_free : -1;
}

extern "C" int64_t b200_pool_allocate(void* pool, const int32_t* token_ids, int64_t num_tokens, int32_t* table_out,
                                      int64_t* num_cached_out) {
  Pool* p = static_cast<Pool*>(pool);
  if (!p || num_tokens < 0 || (num_tokens > 0 && (!token_ids || !table_out)) || !num_cached_out) return B200_ERR_ARG;
  const int bs = p->block_size;
  const int64_t nblk = (num_tokens + bs - 1) / bs;
  int64_t cached = 0;
  uint64_t h = 0;
  bool chain = false;                                    // h holds the hash of the previous (full) block
  for (int64_t i = 0; i < nblk; ++i) {
    const int32_t* toks = token_ids + i * bs;
    const bool full = (i + 1) * bs <= num_tokens;
    int32_t b = -1;
    if (full) {
      h = b200_block_hash(toks, bs, chain ? h : 0, chain ? 1 : 0);
      chain = true;
      auto it = p->by_hash.find(h);
      // a hit on the block that ends the prompt would leave no token to run through the model
      if (it != p->by_hash.end() && p->has_hash[it->second] && p->hash[it->second] == h &&
          p->same_tokens(it->second, toks) && cached + bs < num_tokens)
        b = it->second;
    }
    if (b >= 0) {
      cached += bs;
      if (p->ref[b] > 0) {
        ++p->ref[b];
      } else {                      // a free block whose contents are still what this prompt needs
        p->unlink(b);
        p->ref[b] = 1;
      }
    } else {
      b = p->take_oldest_fresh();
      if (b < 0) return B200_ERR_TOO_LARGE;
      if (full) p->seal(b, h, toks);
    }
    table_out[i] = b;
  }
  *num_cached_out = cached;
  return nblk;
}

extern "C" int b200_pool_deallocate(void* pool, const int32_t* table, int64_t num_blocks) {
  Pool* p = static_cast<Pool*>(pool);
  if (!p || num_blocks < 0 || (num_blocks > 0 && !table)) return B200_ERR_ARG;
  for (int64_t i = num_blocks - 1; i >= 0; --i) {        // last block first, so that the free list hands a
    const int32_t b = table[i];                          // prompt's blocks back in reverse and prefixes live longest
    if (!b200::valid_block(p, b) || p->ref[b] <= 0) return B200_ERR_ARG;
    if (--p->ref[b] == 0) p->push_back(b);
  }
  return B200_OK;
}

// Decode-time growth for a sequence that has just reached `num_tokens` tokens (the call the scheduler makes
// before each decode step), given the last block of its table and the one before it (-1: none): at
// num_tokens % block_size == 1 a fresh block is opened and returned (>= 0); at == 0 the now full last block is
// sealed with its chained hash (`last_block_tokens` = its block_size tokens); otherwise nothing happens.
// Returns the opened block id, -1 when none was opened, or an error code < -1 (B200_ERR_* - 1).
extern "C" int64_t b200_pool_append(void* pool, int32_t last_block, int32_t prev_block, int64_t num_tokens,
                                    const int32_t* last_block_tokens) {
  Pool* p = static_cast<Pool*>(pool);
  if (!p || num_tokens <= 0 || !b200::valid_block(p, last_block)) return B200_ERR_ARG - 1;
  const int64_t rem = num_tokens % p->block_size;
  if (rem == 0) {
    if (!last_block_tokens) return B200_ERR_ARG - 1;
    const bool has_prev = b200::valid_block(p, prev_block) && p->has_hash[prev_block];
    const uint64_t h = b200_block_hash(last_block_tokens, p->block_size, has_prev ? p->hash[prev_block] : 0, has_prev);
    p->seal(last_block, h, last_block_tokens);
    return -1;
  }
  if (rem == 1) {
    const int32_t b = p->take_oldest_fresh();
    return b >= 0 ? b : B200_ERR_TOO_LARGE - 1;
  }
  return -1;
}

// Opens a block ahead of time (a window of decode steps); seals a block afterwards (prev_block: the block
// before it in its sequence's table, -1 for the first).
extern "C" int64_t b200_pool_open_block(void* pool) {
  Pool* p = static_cast<Pool*>(pool);
  if (!p) return B200_ERR_ARG - 1;
  const int32_t b = p->take_oldest_fresh();
  return b >= 0 ? b : B200_ERR_TOO_LARGE - 1;
}

extern "C" int b200_pool_seal_block(void* pool, int32_t block, int32_t prev_block, const int32_t* block_tokens) {
  Pool* p = static_cast<Pool*>(pool);
  if (!p || !block_tokens || !b200::valid_block(p, block)) return B200_ERR_ARG;
  const bool has_prev = b200::valid_block(p, prev_block) && p->has_hash[prev_block];
  const uint64_t h = b200_block_hash(block_tokens, p->block_size, has_prev ? p->hash[prev_block] : 0, has_prev);
  p->seal(block, h, block_tokens);
  return B200_OK;
}

// The block a hash currently resolves to, or -1.
extern "C" int64_t b200_pool_lookup(const void* pool, uint64_t hash) {
  const Pool* p = static_cast<const Pool*>(pool);
  if (!p) return -1;
  auto it = p->by_hash.find(hash);
  return it == p->by_hash.end() ? -1 : it->second;
}

// State for inspection: free block ids oldest first (returns their number), and per block its reference
// count, whether it is sealed, and its hash.  Any output may be NULL.
extern "C" int64_t b200_pool_snapshot(const void* pool, int32_t* free_order, int32_t* ref_counts, uint8_t* sealed,
                                      uint64_t* hashes) {
  const Pool* p = static_cast<const Pool*>(pool);
  if (!p) return -1;
  if (free_order) {
    int64_t i = 0;
    for (int32_t b = p->head; b >= 0; b = p->next[b]) free_order[i++] = b;
  }
  for (int32_t b = 0; b < p->num_blocks; ++b) {
    if (ref_counts) ref_counts[b] = p->ref[b];
    if (sealed) sealed[b] = p->has_hash[b];
    if (hashes) hashes[b] = p->hash[b];
  }
  return p->num_free;
}

// ---------------------------------------------------------------------------------------------
// Step metadata (ModelRunner.prepare_prefill / prepare_decode, engine/model_runner.py:202-278).  Block tables
// arrive as one flat int32 array with offsets (sequence i owns tables[offsets[i] : offsets[i+1]]).
// ---------------------------------------------------------------------------------------------

// Prefill: the non-cached suffix of every sequence.  Writes cu_seqlens_q/k [n+1], positions [T] (RoPE position of
// packed token j of a sequence = num_cached + j) and slot_mapping [T] (slots of blocks num_cached/bs .. end, the
// last one ragged); max_seqlens[0..1] = longest q / k.  Returns T, or a negative code (capacity too small,
// a table too short for its sequence).
extern "C" int64_t b200_prepare_prefill(int32_t num_seqs, const int64_t* num_tokens, const int64_t* num_cached,
                                        const int64_t* table_offsets, const int32_t* tables, int32_t block_size,
                                        int32_t* cu_seqlens_q, int32_t* cu_seqlens_k, int64_t* positions,
                                        int64_t* slot_mapping, int64_t capacity, int32_t* max_seqlens) {
  if (num_seqs < 0 || block_size <= 0 || !cu_seqlens_q || !cu_seqlens_k || !max_seqlens) return B200_ERR_ARG;
  if (num_seqs > 0 && (!num_tokens || !num_cached || !table_offsets || !tables || !positions || !slot_mapping))
    return B200_ERR_ARG;
  int64_t t = 0, tk = 0;
  int32_t mq = 0, mk = 0;
  cu_seqlens_q[0] = cu_seqlens_k[0] = 0;
  for (int32_t i = 0; i < num_seqs; ++i) {
    const int64_t n = num_tokens[i], c = num_cached[i];
    if (c < 0 || c > n) return B200_ERR_ARG;
    const int64_t fresh = n - c;
    if (t + fresh > capacity) return B200_ERR_WORKSPACE;
    const int32_t* tab = tables + table_offsets[i];
    const int64_t tab_len = table_offsets[i + 1] - table_offsets[i];
    if (fresh > 0 && (n + block_size - 1) / block_size > tab_len) return B200_ERR_ARG;
    for (int64_t pos = c; pos < n; ++pos, ++t) {
      positions[t] = pos;
      slot_mapping[t] = static_cast<int64_t>(tab[pos / block_size]) * block_size + pos % block_size;
    }
    tk += n;
    if (t > 2147483647LL || tk > 2147483647LL) return B200_ERR_TOO_LARGE;
    cu_seqlens_q[i + 1] = static_cast<int32_t>(t);
    cu_seqlens_k[i + 1] = static_cast<int32_t>(tk);
    if (fresh > mq) mq = static_cast<int32_t>(fresh);
    if (n > mk) mk = static_cast<int32_t>(n);
  }
  max_seqlens[0] = mq;
  max_seqlens[1] = mk;
  return t;
}

// Decode: one token per running sequence.  context_lens [n] = num_tokens, slot_mapping [n] = slot of the last
// token (in the block that holds position num_tokens - 1), block_tables [n, width] padded with -1.
extern "C" int b200_prepare_decode(int32_t num_seqs, const int64_t* num_tokens, const int64_t* table_offsets,
                                   const int32_t* tables, int32_t block_size, int64_t* context_lens,
                                   int64_t* slot_mapping, int32_t* block_tables, int64_t width) {
  if (num_seqs < 0 || block_size <= 0 || width < 0) return B200_ERR_ARG;
  if (num_seqs > 0 && (!num_tokens || !table_offsets || !tables || !context_lens || !slot_mapping || !block_tables))
    return B200_ERR_ARG;
  for (int32_t i = 0; i < num_seqs; ++i) {
    const int64_t n = num_tokens[i];
    const int32_t* tab = tables + table_offsets[i];
    const int64_t tab_len = table_offsets[i + 1] - table_offsets[i];
    if (n <= 0 || tab_len > width || (n - 1) / block_size >= tab_len) return B200_ERR_ARG;
    context_lens[i] = n;
    slot_mapping[i] = static_cast<int64_t>(tab[(n - 1) / block_size]) * block_size + (n - 1) % block_size;
    int32_t* row = block_tables + static_cast<int64_t>(i) * width;
    memcpy(row, tab, sizeof(int32_t) * tab_len);
    for (int64_t j = tab_len; j < width; ++j) row[j] = -1;
  }
  return B200_OK;
}
