// Host-side paged-KV bookkeeping, bit-exact with the reference's BlockManager
// (src/scheduler/block_manager.rs), BlockAllocator (:46-102), PrefixCache
// (src/scheduler/prefix_cache.rs:53-131) and the Sequence block arithmetic
// (src/scheduler/sequence.rs:80-92).  "Bit-exact" means: for the same sequence of
// calls the block ids in every table, the free counts and the copy-on-write / swap
// pairs are identical.  Groups hold one sequence (the worker never builds larger ones,
// src/worker/mod.rs:316-331).
#include <deque>
#include <unordered_map>
#include <vector>

#include "common.h"

namespace hb {

uint64_t fnv1a_block(const uint32_t* tokens, int64_t n) {
  // hash_block: xor the whole u32 then multiply (prefix_cache.rs:40-50)
  uint64_t h = 0xcbf29ce484222325ull;
  for (int64_t i = 0; i < n; ++i) {
    h ^= (uint64_t)tokens[i];
    h *= 0x100000001b3ull;
  }
  return h;
}

class FifoAllocator {  // BlockAllocator
 public:
  explicit FifoAllocator(int64_t n) {
    for (int64_t i = 0; i < n; ++i) free_.push_back(i);
  }
  bool allocate(int64_t* id) {
    if (free_.empty()) return false;
    *id = free_.front();
    free_.pop_front();
    refs_[*id] = 1;
    return true;
  }
  void release(int64_t id) {
    auto it = refs_.find(id);
    if (it == refs_.end()) return;
    if (--it->second == 0) {
      refs_.erase(it);
      free_.push_back(id);
    }
  }
  int64_t num_free() const { return (int64_t)free_.size(); }
  int64_t ref_count(int64_t id) const {
    auto it = refs_.find(id);
    return it == refs_.end() ? 0 : it->second;
  }
  void increment_ref(int64_t id) {
    auto it = refs_.find(id);
    if (it != refs_.end()) ++it->second;
  }

 private:
  std::deque<int64_t> free_;
  std::unordered_map<int64_t, int64_t> refs_;
};

class PrefixCacheFifo {  // PrefixCache
 public:
  explicit PrefixCacheFifo(size_t cap) : cap_(cap) {}
  bool lookup(uint64_t h, int64_t* id) const {
    auto it = entries_.find(h);
    if (it == entries_.end()) return false;
    *id = it->second;
    return true;
  }
  void insert(uint64_t h, int64_t id) {
    auto it = entries_.find(h);
    if (it != entries_.end()) {
      if (it->second != id) block_to_hash_.erase(it->second);
      it->second = id;
      block_to_hash_[id] = h;
      return;
    }
    if (entries_.size() >= cap_ && !order_.empty()) {
      const uint64_t victim = order_.front();
      order_.pop_front();
      auto v = entries_.find(victim);
      if (v != entries_.end()) {
        block_to_hash_.erase(v->second);
        entries_.erase(v);
      }
    }
    entries_[h] = id;
    order_.push_back(h);
    block_to_hash_[id] = h;
  }
  size_t size() const { return entries_.size(); }

 private:
  size_t cap_;
  std::unordered_map<uint64_t, int64_t> entries_;
  std::deque<uint64_t> order_;
  std::unordered_map<int64_t, uint64_t> block_to_hash_;
};

}  // namespace hb

struct hb_block_manager {
  hb::FifoAllocator gpu, cpu;
  hb::PrefixCacheFifo prefix{128};  // PREFIX_CACHE_CAPACITY (block_manager.rs:115)
  std::unordered_map<uint64_t, std::vector<int64_t>> tables;
  std::unordered_map<int64_t, uint64_t> block_hashes;
  hb_block_manager(int64_t g, int64_t c) : gpu(g), cpu(c) {}
};

extern "C" {

int64_t hb_num_logical_blocks(int64_t len, int64_t block_size) {
  if (block_size <= 0 || len < 0) return -1;
  return (len + block_size - 1) / block_size;
}

int64_t hb_last_block_num_filled(int64_t len, int64_t block_size) {
  if (block_size <= 0 || len < 0) return -1;
  const int64_t rem = len % block_size;
  return (rem == 0 && len != 0) ? block_size : rem;
}

uint64_t hb_hash_block(const uint32_t* tokens, int64_t n) { return hb::fnv1a_block(tokens, n); }

int64_t hb_slot_for_position(const int64_t* table, int64_t table_len, int64_t pos) {
  if (!table || pos < 0 || pos / HB_BLOCK_SIZE >= table_len) return -1;
  return table[pos / HB_BLOCK_SIZE] * HB_BLOCK_SIZE + pos % HB_BLOCK_SIZE;
}

int hb_bm_create(int64_t num_gpu_blocks, int64_t num_cpu_blocks, hb_block_manager** out) {
  HB_CHECK_ARG(out && num_gpu_blocks >= 0 && num_cpu_blocks >= 0, "hb_bm_create: bad arguments");
  *out = new hb_block_manager(num_gpu_blocks, num_cpu_blocks);
  return HB_OK;
}

int hb_bm_free_manager(hb_block_manager* bm) {
  delete bm;
  return HB_OK;
}

int64_t hb_bm_num_free_gpu_blocks(const hb_block_manager* bm) { return bm ? bm->gpu.num_free() : -1; }
int64_t hb_bm_num_free_cpu_blocks(const hb_block_manager* bm) { return bm ? bm->cpu.num_free() : -1; }
int64_t hb_bm_num_prefix_cached_blocks(const hb_block_manager* bm) {
  return bm ? (int64_t)bm->prefix.size() : -1;
}

int hb_bm_can_allocate(const hb_block_manager* bm, int64_t total_len) {
  if (!bm) return 0;
  return hb_num_logical_blocks(total_len, HB_BLOCK_SIZE) <= bm->gpu.num_free() ? 1 : 0;
}

// BlockManager::allocate (block_manager.rs:194-253)
int hb_bm_allocate(hb_block_manager* bm, uint64_t seq_id, const uint32_t* prompt_ids,
                   int64_t prompt_len, int64_t output_len, int64_t* hit_blocks) {
  HB_CHECK_ARG(bm && prompt_len >= 0 && output_len >= 0 && (prompt_ids || prompt_len == 0),
               "hb_bm_allocate: bad arguments");
  const int64_t needed = hb_num_logical_blocks(prompt_len + output_len, HB_BLOCK_SIZE);
  if (needed > bm->gpu.num_free() + (int64_t)bm->prefix.size())
    return hb::fail(HB_ERR_OOM_BLOCKS, "not enough GPU blocks: need %lld, have %lld free + %zu cached",
                    (long long)needed, (long long)bm->gpu.num_free(), bm->prefix.size());
  std::vector<int64_t> table;
  int64_t hits = 0;
  const int64_t complete = prompt_len / HB_BLOCK_SIZE;
  for (int64_t b = 0; b < complete; ++b) {
    const uint64_t h = hb::fnv1a_block(prompt_ids + b * HB_BLOCK_SIZE, HB_BLOCK_SIZE);
    int64_t id;
    if (bm->prefix.lookup(h, &id)) {
      bm->gpu.increment_ref(id);
      table.push_back(id);
      ++hits;
    } else {
      if (!bm->gpu.allocate(&id))
        return hb::fail(HB_ERR_OOM_BLOCKS, "no free GPU blocks for allocation");
      table.push_back(id);
      bm->block_hashes[id] = h;
    }
  }
  for (int64_t r = 0; r < needed - complete; ++r) {
    int64_t id;
    if (!bm->gpu.allocate(&id)) return hb::fail(HB_ERR_OOM_BLOCKS, "no free GPU blocks for allocation");
    table.push_back(id);
  }
  bm->tables[seq_id] = std::move(table);
  if (hit_blocks) *hit_blocks = hits;
  return HB_OK;
}

// BlockManager::free (block_manager.rs:264-276)
int hb_bm_free_seq(hb_block_manager* bm, uint64_t seq_id) {
  HB_CHECK_ARG(bm, "hb_bm_free_seq: null manager");
  auto it = bm->tables.find(seq_id);
  if (it == bm->tables.end()) return HB_OK;
  std::vector<int64_t> table = std::move(it->second);
  bm->tables.erase(it);
  for (int64_t id : table) {
    auto h = bm->block_hashes.find(id);
    if (h != bm->block_hashes.end()) bm->prefix.insert(h->second, id);
    bm->gpu.release(id);
  }
  return HB_OK;
}

// BlockManager::can_append_slot (block_manager.rs:284-308)
int hb_bm_can_append_slot(const hb_block_manager* bm, uint64_t seq_id, int64_t total_len) {
  if (!bm) return 0;
  auto it = bm->tables.find(seq_id);
  if (it == bm->tables.end()) return 0;
  const int64_t filled = hb_last_block_num_filled(total_len, HB_BLOCK_SIZE);
  if (filled == HB_BLOCK_SIZE && bm->gpu.num_free() == 0) return 0;
  if (!it->second.empty() && bm->gpu.ref_count(it->second.back()) > 1 && bm->gpu.num_free() == 0)
    return 0;
  return 1;
}

// BlockManager::append_slot (block_manager.rs:314-351)
int hb_bm_append_slot(hb_block_manager* bm, uint64_t seq_id, int64_t total_len,
                      int64_t cow_pair[2]) {
  HB_CHECK_ARG(bm && total_len >= 0, "hb_bm_append_slot: bad arguments");
  if (cow_pair) cow_pair[0] = cow_pair[1] = -1;
  auto it = bm->tables.find(seq_id);
  if (it == bm->tables.end())
    return hb::fail(HB_ERR_INVALID_ARG, "no block table for seq %llu", (unsigned long long)seq_id);
  std::vector<int64_t>& table = it->second;
  const int64_t filled = hb_last_block_num_filled(total_len, HB_BLOCK_SIZE);
  if (filled == HB_BLOCK_SIZE || table.empty()) {
    int64_t id;
    if (!bm->gpu.allocate(&id)) return hb::fail(HB_ERR_OOM_BLOCKS, "no free GPU blocks for append");
    table.push_back(id);
  } else {
    const int64_t last = table.back();
    if (bm->gpu.ref_count(last) > 1) {
      int64_t id;
      if (!bm->gpu.allocate(&id)) return hb::fail(HB_ERR_OOM_BLOCKS, "no free GPU blocks for CoW");
      bm->gpu.release(last);
      table.back() = id;
      if (cow_pair) { cow_pair[0] = last; cow_pair[1] = id; }
    }
  }
  return HB_OK;
}

static int swap_impl(hb_block_manager* bm, uint64_t seq_id, bool out, int64_t* mapping,
                     int64_t* n_pairs) {
  HB_CHECK_ARG(bm && n_pairs, "swap: bad arguments");
  auto it = bm->tables.find(seq_id);
  if (it == bm->tables.end())
    return hb::fail(HB_ERR_INVALID_ARG, "no block table for seq %llu", (unsigned long long)seq_id);
  hb::FifoAllocator& from = out ? bm->gpu : bm->cpu;
  hb::FifoAllocator& to = out ? bm->cpu : bm->gpu;
  int64_t n = 0;
  for (int64_t& id : it->second) {
    int64_t nid;
    if (!to.allocate(&nid))
      return hb::fail(HB_ERR_OOM_BLOCKS, out ? "no free CPU blocks for swap_out" : "no free GPU blocks for swap_in");
    if (mapping) { mapping[2 * n] = id; mapping[2 * n + 1] = nid; }
    from.release(id);
    id = nid;
    ++n;
  }
  *n_pairs = n;
  return HB_OK;
}

int hb_bm_swap_out(hb_block_manager* bm, uint64_t seq_id, int64_t* mapping_out, int64_t* n_pairs) {
  return swap_impl(bm, seq_id, true, mapping_out, n_pairs);
}
int hb_bm_swap_in(hb_block_manager* bm, uint64_t seq_id, int64_t* mapping_out, int64_t* n_pairs) {
  return swap_impl(bm, seq_id, false, mapping_out, n_pairs);
}

int64_t hb_bm_block_table(const hb_block_manager* bm, uint64_t seq_id, int64_t* out, int64_t cap) {
  if (!bm) return HB_ERR_INVALID_ARG;
  auto it = bm->tables.find(seq_id);
  if (it == bm->tables.end()) return HB_ERR_INVALID_ARG;
  const int64_t n = (int64_t)it->second.size();
  for (int64_t i = 0; i < n && i < cap && out; ++i) out[i] = it->second[i];
  return n;
}

}  // extern "C"
