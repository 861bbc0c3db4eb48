// Paged KV-cache block manager of the rollout engine (host side, C++).
//
// Keeps a free list of physical blocks, per-sequence block tables, reference counts for blocks
// shared between sequences (n samples forked from one prompt, multi-turn re-submission) and a
// content-hash index of *full* blocks for prefix caching: a block's key is the hash of
// (parent block key, the block_size token ids it holds), so equal prefixes map to equal chains.
// Cached blocks whose refcount dropped to zero stay in the index on an LRU list and are evicted
// only when the free list runs dry.
//
// Counterpart in the reference: the block manager / prefix cache inside the external rollout
// engine it drives (docs/zh/features/vLLM_prefix_cache.md:5-24).  Exposed as a C API (ctypes).
#include <cstdint>
#include <cstring>
#include <list>
#include <mutex>
#include <unordered_map>
#include <vector>

#define API extern "C" __attribute__((visibility("default")))

namespace {

struct Block {
  int ref = 0;
  uint64_t key = 0;      // content hash when cached (0 = not in the prefix index)
  bool cached = false;
  std::list<int>::iterator lru_it;
  bool in_lru = false;
};

struct Seq {
  std::vector<int> blocks;
  int64_t num_tokens = 0;      // tokens that have a slot
  int64_t num_cached_tokens = 0;  // leading tokens whose KV was found in the prefix cache
  uint64_t last_key = 0;       // hash chain value of the last full block registered
  int64_t hashed_blocks = 0;   // number of leading blocks already registered in the index
};

struct Manager {
  int num_blocks, block_size;
  bool prefix_caching;
  std::vector<Block> blocks;
  std::vector<int> free_list;
  std::list<int> lru;  // evictable cached blocks, front = oldest
  std::unordered_map<uint64_t, int> index;  // content key -> block
  std::unordered_map<int64_t, Seq> seqs;
  std::mutex mu;
  int64_t hits = 0, queries = 0;
};

inline uint64_t mix(uint64_t h, uint64_t v) {
  h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
  h *= 0xff51afd7ed558ccdull;
  h ^= h >> 33;
  return h;
}

uint64_t block_key(uint64_t parent, const int32_t* toks, int n) {
  uint64_t h = mix(0x1234567ull, parent);
  for (int i = 0; i < n; ++i) h = mix(h, (uint64_t)(uint32_t)toks[i] + 1);
  return h ? h : 1;
}

int num_free(Manager* m) { return (int)m->free_list.size() + (int)m->lru.size(); }

int take_block(Manager* m) {
  if (!m->free_list.empty()) {
    int b = m->free_list.back();
    m->free_list.pop_back();
    return b;
  }
  if (!m->lru.empty()) {  // evict the oldest unreferenced cached block
    int b = m->lru.front();
    m->lru.pop_front();
    Block& B = m->blocks[b];
    B.in_lru = false;
    if (B.cached) {
      auto it = m->index.find(B.key);
      if (it != m->index.end() && it->second == b) m->index.erase(it);
      B.cached = false;
      B.key = 0;
    }
    return b;
  }
  return -1;
}

void release_block(Manager* m, int b) {
  Block& B = m->blocks[b];
  if (--B.ref > 0) return;
  B.ref = 0;
  if (B.cached && m->prefix_caching) {
    m->lru.push_back(b);
    B.lru_it = std::prev(m->lru.end());
    B.in_lru = true;
  } else {
    B.cached = false;
    B.key = 0;
    m->free_list.push_back(b);
  }
}

void ref_block(Manager* m, int b) {
  Block& B = m->blocks[b];
  if (B.ref == 0 && B.in_lru) {
    m->lru.erase(B.lru_it);
    B.in_lru = false;
  }
  ++B.ref;
}

}  // namespace

API void* msrl_bm_create(int num_blocks, int block_size, int prefix_caching) {
  Manager* m = new Manager();
  m->num_blocks = num_blocks;
  m->block_size = block_size;
  m->prefix_caching = prefix_caching != 0;
  m->blocks.resize(num_blocks);
  m->free_list.reserve(num_blocks);
  for (int b = num_blocks - 1; b >= 0; --b) m->free_list.push_back(b);
  return m;
}

API void msrl_bm_destroy(void* h) { delete (Manager*)h; }

API int msrl_bm_num_free(void* h) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  return num_free(m);
}

API int msrl_bm_blocks_needed(void* h, int64_t seq_id, int64_t new_total_tokens) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  auto it = m->seqs.find(seq_id);
  int64_t have = it == m->seqs.end() ? 0 : (int64_t)it->second.blocks.size();
  int64_t need = (new_total_tokens + m->block_size - 1) / m->block_size;
  return (int)(need > have ? need - have : 0);
}

// Create a sequence for a prompt. With prefix caching, leading full blocks whose content is in
// the index are shared instead of allocated. Returns the number of prompt tokens whose KV is
// already cached (a multiple of block_size, < n_tokens so that at least one token is computed),
// or -1 when there are not enough blocks (nothing is changed then).
API int64_t msrl_bm_allocate(void* h, int64_t seq_id, const int32_t* tokens, int64_t n_tokens) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  if (m->seqs.count(seq_id)) return -2;
  const int bs = m->block_size;
  const int64_t need = (n_tokens + bs - 1) / bs;
  std::vector<int> shared;
  uint64_t key = 0;
  if (m->prefix_caching) {
    const int64_t full = (n_tokens - 1) / bs;  // keep >= 1 token to compute
    for (int64_t i = 0; i < full; ++i) {
      uint64_t k = block_key(key, tokens + i * bs, bs);
      ++m->queries;
      auto it = m->index.find(k);
      if (it == m->index.end()) break;
      ++m->hits;
      shared.push_back(it->second);
      key = k;
    }
  }
  int evictable_shared = 0;
  for (int b : shared)
    if (m->blocks[b].ref == 0) ++evictable_shared;
  if (need - (int64_t)shared.size() > num_free(m) - evictable_shared) return -1;
  Seq s;
  for (int b : shared) {
    ref_block(m, b);
    s.blocks.push_back(b);
  }
  for (int64_t i = (int64_t)shared.size(); i < need; ++i) {
    int b = take_block(m);
    m->blocks[b].ref = 1;
    s.blocks.push_back(b);
  }
  s.num_tokens = n_tokens;
  s.num_cached_tokens = (int64_t)shared.size() * bs;
  s.last_key = key;
  s.hashed_blocks = (int64_t)shared.size();
  m->seqs.emplace(seq_id, std::move(s));
  return (int64_t)shared.size() * bs;
}

// Make room for `n_new` more tokens. Returns 0, or -1 when out of blocks (nothing changed).
API int msrl_bm_append(void* h, int64_t seq_id, int64_t n_new) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  auto it = m->seqs.find(seq_id);
  if (it == m->seqs.end()) return -2;
  Seq& s = it->second;
  const int bs = m->block_size;
  const int64_t need = (s.num_tokens + n_new + bs - 1) / bs - (int64_t)s.blocks.size();
  if (need > num_free(m)) return -1;
  for (int64_t i = 0; i < need; ++i) {
    int b = take_block(m);
    m->blocks[b].ref = 1;
    s.blocks.push_back(b);
  }
  s.num_tokens += n_new;
  return 0;
}

// Register the full blocks of a sequence in the prefix index once their KV has been written.
// `tokens` are the sequence's token ids; only blocks fully covered by `n_computed` are hashed.
API void msrl_bm_commit(void* h, int64_t seq_id, const int32_t* tokens, int64_t n_computed) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  if (!m->prefix_caching) return;
  auto it = m->seqs.find(seq_id);
  if (it == m->seqs.end()) return;
  Seq& s = it->second;
  const int bs = m->block_size;
  const int64_t full = n_computed / bs;
  for (int64_t i = s.hashed_blocks; i < full && i < (int64_t)s.blocks.size(); ++i) {
    uint64_t k = block_key(s.last_key, tokens + i * bs, bs);
    int b = s.blocks[i];
    Block& B = m->blocks[b];
    if (!B.cached && !m->index.count(k)) {
      B.cached = true;
      B.key = k;
      m->index[k] = b;
    }
    s.last_key = k;
    s.hashed_blocks = i + 1;
  }
}

// Fork: the child shares every *full* block of the parent (refcount++) and gets a private copy
// slot for the trailing partial block. Writes (src_block, dst_block) of the partial block to
// copy_pair (or -1,-1 when the parent ends on a block boundary). Returns 0 / -1 (out of blocks).
API int msrl_bm_fork(void* h, int64_t parent_id, int64_t child_id, int32_t* copy_pair) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  auto it = m->seqs.find(parent_id);
  if (it == m->seqs.end() || m->seqs.count(child_id)) return -2;
  const Seq& p = it->second;
  const int bs = m->block_size;
  const int64_t full = p.num_tokens / bs;
  const bool partial = (p.num_tokens % bs) != 0;
  if (partial && num_free(m) < 1) return -1;
  Seq c;
  for (int64_t i = 0; i < full; ++i) {
    ref_block(m, p.blocks[i]);
    c.blocks.push_back(p.blocks[i]);
  }
  copy_pair[0] = copy_pair[1] = -1;
  if (partial) {
    int b = take_block(m);
    m->blocks[b].ref = 1;
    c.blocks.push_back(b);
    copy_pair[0] = p.blocks[full];
    copy_pair[1] = b;
  }
  c.num_tokens = p.num_tokens;
  c.num_cached_tokens = p.num_cached_tokens;
  c.last_key = p.last_key;
  c.hashed_blocks = p.hashed_blocks < full ? p.hashed_blocks : full;
  m->seqs.emplace(child_id, std::move(c));
  return 0;
}

API void msrl_bm_free(void* h, int64_t seq_id) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  auto it = m->seqs.find(seq_id);
  if (it == m->seqs.end()) return;
  for (int b : it->second.blocks) release_block(m, b);
  m->seqs.erase(it);
}

API int msrl_bm_num_blocks(void* h, int64_t seq_id) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  auto it = m->seqs.find(seq_id);
  return it == m->seqs.end() ? -1 : (int)it->second.blocks.size();
}

// Copy the block table of a sequence into out[0..max); returns the number of blocks.
API int msrl_bm_block_table(void* h, int64_t seq_id, int32_t* out, int max) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  auto it = m->seqs.find(seq_id);
  if (it == m->seqs.end()) return -1;
  const auto& b = it->second.blocks;
  const int n = (int)b.size() < max ? (int)b.size() : max;
  std::memcpy(out, b.data(), sizeof(int32_t) * n);
  return (int)b.size();
}

// Fill block tables for a batch: out is [n, max_blocks] row-major, padded with 0.
API int msrl_bm_block_tables(void* h, const int64_t* seq_ids, int n, int32_t* out, int max_blocks) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  for (int i = 0; i < n; ++i) {
    auto it = m->seqs.find(seq_ids[i]);
    if (it == m->seqs.end()) return -1;
    const auto& b = it->second.blocks;
    if ((int)b.size() > max_blocks) return -3;
    std::memcpy(out + (int64_t)i * max_blocks, b.data(), sizeof(int32_t) * b.size());
    for (int j = (int)b.size(); j < max_blocks; ++j) out[(int64_t)i * max_blocks + j] = 0;
  }
  return 0;
}

// Slot ids (block*block_size+offset) of token positions [start, start+count) of a sequence.
API int msrl_bm_slots(void* h, int64_t seq_id, int64_t start, int64_t count, int64_t* out) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  auto it = m->seqs.find(seq_id);
  if (it == m->seqs.end()) return -1;
  const auto& b = it->second.blocks;
  const int bs = m->block_size;
  for (int64_t i = 0; i < count; ++i) {
    const int64_t pos = start + i;
    const int64_t bi = pos / bs;
    if (bi >= (int64_t)b.size()) return -3;
    out[i] = (int64_t)b[bi] * bs + pos % bs;
  }
  return 0;
}

API void msrl_bm_stats(void* h, int64_t* out4) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  out4[0] = num_free(m);
  out4[1] = (int64_t)m->seqs.size();
  out4[2] = m->hits;
  out4[3] = m->queries;
}
