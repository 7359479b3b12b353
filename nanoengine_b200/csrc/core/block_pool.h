// Paged-KV block pool with a hash-chained prefix cache, and a slot pool.
//
// Parity: reference rust/src/cache/table/block/pool.rs:50-402 (Empty/Pending/
// Ready block states, refcounts, LRU eviction of unreferenced cached blocks,
// cached tokens capped at tokens-1), rust/src/cache/table/block/prefix.rs
// (block hash chained on the previous block's hash),
// rust/src/cache/table/slot/pool.rs (slot pools).
#pragma once
#include <cstdint>
#include <list>
#include <stdexcept>
#include <unordered_map>
#include <vector>

namespace ne {

enum BlockState : uint8_t { BLOCK_EMPTY = 0, BLOCK_PENDING = 1, BLOCK_READY = 2 };

inline uint64_t mix64(uint64_t x) {
  x ^= x >> 32; x *= 0xd6e8feb86659fd93ull; x ^= x >> 32; x *= 0xd6e8feb86659fd93ull; x ^= x >> 32;
  return x;
}

// Hash of one full block of tokens, seeded with the hash of the block before it.
inline uint64_t chain_hash(uint64_t prev, const int32_t* tok, int n) {
  uint64_t h = mix64(prev ^ 0x9e3779b97f4a7c15ull) + (uint64_t)n;
  for (int i = 0; i < n; i++) h = mix64(h ^ ((uint64_t)(uint32_t)tok[i] + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2)));
  return h ? h : 1;  // 0 is reserved for "no hash"
}

class BlockPool {
 public:
  BlockPool() = default;
  BlockPool(int num_blocks, int block_size, bool prefix_cache)
      : block_size_(block_size), prefix_cache_(prefix_cache) { resize(num_blocks); }

  void resize(int num_blocks) {
    if ((int)blocks_.size() > num_blocks && num_used() > 0)
      throw std::runtime_error("BlockPool: cannot shrink a pool with live blocks");
    blocks_.assign(num_blocks, Block{});
    free_.clear(); lru_.clear(); by_hash_.clear();
    for (int i = num_blocks - 1; i >= 0; i--) free_.push_back(i);  // pop_back hands out low ids first
  }

  int num_blocks() const { return (int)blocks_.size(); }
  int block_size() const { return block_size_; }
  int num_free() const { return (int)free_.size() + (int)lru_.size(); }  // allocatable right now
  int num_cached() const { return (int)by_hash_.size(); }
  int num_used() const { return num_blocks() - (int)free_.size() - (int)lru_.size(); }
  int refcount(int b) const { return blocks_.at(b).ref; }
  int state(int b) const { return blocks_.at(b).state; }
  uint64_t lookups() const { return lookups_; }
  uint64_t hit_tokens() const { return hit_tokens_; }
  uint64_t lookup_tokens() const { return lookup_tokens_; }

  // Longest cached prefix of `tok`.  Takes a reference on every matched block.
  // At most n-1 tokens count as cached, so the caller always computes one token.
  std::vector<int32_t> match_prefix(const int32_t* tok, int n, uint64_t* last_hash) {
    std::vector<int32_t> out;
    *last_hash = 0;
    lookups_++; lookup_tokens_ += (uint64_t)n;
    if (!prefix_cache_) return out;
    uint64_t h = 0;
    int max_blocks = (n - 1) / block_size_;
    for (int b = 0; b < max_blocks; b++) {
      uint64_t nh = chain_hash(h, tok + (size_t)b * block_size_, block_size_);
      auto it = by_hash_.find(nh);
      if (it == by_hash_.end()) break;
      int id = it->second;
      if (blocks_[id].state != BLOCK_READY) break;
      acquire(id);
      out.push_back(id);
      h = nh;
    }
    *last_hash = h;
    hit_tokens_ += (uint64_t)out.size() * block_size_;
    return out;
  }

  bool can_allocate(int n) const { return num_free() >= n; }

  // Allocate n blocks (state Pending, ref 1).  Evicts least-recently-released
  // cached blocks when the free list runs dry.  Returns false and changes nothing
  // if fewer than n are available.
  bool allocate(int n, std::vector<int32_t>* out, std::vector<int32_t>* evicted = nullptr) {
    if (!can_allocate(n)) return false;
    for (int i = 0; i < n; i++) {
      int id;
      if (!free_.empty()) { id = free_.back(); free_.pop_back(); }
      else {
        id = lru_.front(); lru_.pop_front();
        Block& b = blocks_[id];
        b.in_lru = false;
        if (b.hash) { by_hash_.erase(b.hash); if (evicted) evicted->push_back(id); evictions_++; }
        b.hash = 0;
      }
      Block& b = blocks_[id];
      b.ref = 1; b.state = BLOCK_PENDING; b.hash = 0;
      out->push_back(id);
    }
    return true;
  }

  // Publish a filled block under its chained hash.  If another block already holds
  // that hash the new one stays private (it is freed on release).
  void commit(int id, uint64_t hash) {
    Block& b = blocks_.at(id);
    b.state = BLOCK_READY;
    if (!prefix_cache_ || b.hash) return;
    if (by_hash_.emplace(hash, id).second) { b.hash = hash; if (log_commits_) commit_log_.emplace_back(hash, id); }
  }

  // ---- third-tier hooks ---------------------------------------------------------------
  // With the log on, every newly published (hash, block) pair is remembered until take_committed() drains it, so
  // a lower tier can persist fresh blocks.
  void set_commit_log(bool on) { log_commits_ = on; if (!on) commit_log_.clear(); }
  std::vector<std::pair<uint64_t, int32_t>> take_committed() { auto out = std::move(commit_log_); commit_log_.clear(); return out; }
  bool has_hash(uint64_t h) const { return by_hash_.count(h) != 0; }

  // Reserve one block per hash that is not cached yet (in order; stops when the pool runs dry).  Entry i of the result is
  // the reserved block id, or -1 when hashes[i] is already cached.  The caller fills the blocks and hands the same two
  // lists to finish_import(), which publishes them as cached, unreferenced blocks.
  std::vector<int32_t> begin_import(const std::vector<uint64_t>& hashes) {
    std::vector<int32_t> out;
    for (uint64_t h : hashes) {
      auto it = by_hash_.find(h);
      if (it != by_hash_.end()) {
        // already cached: hold it until finish_import, or a later allocation of this same import could evict the block the
        // chain being imported hangs on
        acquire(it->second);
        import_held_.push_back(it->second);
        out.push_back(-1);
        continue;
      }
      std::vector<int32_t> one;
      if (!allocate(1, &one)) break;
      out.push_back(one[0]);
    }
    return out;
  }
  void finish_import(const std::vector<uint64_t>& hashes, const std::vector<int32_t>& ids, bool ok) {
    const bool was = log_commits_;
    log_commits_ = false;                       // imported blocks came from the lower tier: nothing to persist again
    for (size_t i = 0; i < ids.size() && i < hashes.size(); i++) {
      if (ids[i] < 0) continue;
      if (ok) commit(ids[i], hashes[i]);
      release_one(ids[i]);
    }
    log_commits_ = was;
    for (int32_t id : import_held_) release_one(id);
    import_held_.clear();
  }

  void mark_ready(int id) { blocks_.at(id).state = BLOCK_READY; }

  void release(const std::vector<int32_t>& ids) {
    // release in reverse so the tail of a sequence is evicted before its head
    for (auto it = ids.rbegin(); it != ids.rend(); ++it) release_one(*it);
  }

  void release_one(int id) {
    Block& b = blocks_.at(id);
    if (b.ref <= 0) throw std::runtime_error("BlockPool: release of an unreferenced block");
    if (--b.ref > 0) return;
    if (b.hash && b.state == BLOCK_READY) { lru_.push_back(id); b.lru_it = std::prev(lru_.end()); b.in_lru = true; }
    else { b.state = BLOCK_EMPTY; b.hash = 0; free_.push_back(id); }
  }

  uint64_t evictions() const { return evictions_; }

  // Forget every cached prefix (the KV it describes is stale, e.g. after a weight update).  Blocks in use stay allocated
  // but lose their hash, so they return to the free list when released.
  void clear_cache() {
    for (int id : lru_) { Block& b = blocks_[id]; b.in_lru = false; b.hash = 0; b.state = BLOCK_EMPTY; free_.push_back(id); }
    lru_.clear();
    for (auto& b : blocks_) b.hash = 0;
    by_hash_.clear();
  }

 private:
  struct Block {
    int32_t ref = 0;
    uint8_t state = BLOCK_EMPTY;
    bool in_lru = false;
    uint64_t hash = 0;
    std::list<int32_t>::iterator lru_it;
  };
  void acquire(int id) {
    Block& b = blocks_[id];
    if (b.ref == 0 && b.in_lru) { lru_.erase(b.lru_it); b.in_lru = false; }
    b.ref++;
  }
  std::vector<int32_t> import_held_;          // cached blocks referenced by the import in progress
  int block_size_ = 64;
  bool prefix_cache_ = true;
  std::vector<Block> blocks_;
  std::vector<int32_t> free_;
  std::list<int32_t> lru_;
  std::unordered_map<uint64_t, int32_t> by_hash_;
  uint64_t lookups_ = 0, hit_tokens_ = 0, lookup_tokens_ = 0, evictions_ = 0;
  bool log_commits_ = false;
  std::vector<std::pair<uint64_t, int32_t>> commit_log_;
};

// Fixed set of integer slots (recurrent state rows, MTP hand-off rows, HiSparse hot buffers).
class SlotPool {
 public:
  SlotPool() = default;
  explicit SlotPool(int n) { for (int i = n - 1; i >= 0; i--) free_.push_back(i); total_ = n; }
  int acquire() { if (free_.empty()) return -1; int s = free_.back(); free_.pop_back(); return s; }
  void release(int s) { if (s >= 0) free_.push_back(s); }
  int num_free() const { return (int)free_.size(); }
  int total() const { return total_; }
 private:
  std::vector<int32_t> free_;
  int total_ = 0;
};

// Index of KV blocks persisted to a third (file-backed) tier, keyed by chained block hash.
// Parity: reference rust/src/l3.rs:1-497 (block index of the 3FS tier).
class L3Index {
 public:
  explicit L3Index(size_t capacity = 0) : capacity_(capacity) {}
  bool contains(uint64_t h) const { return map_.count(h) != 0; }
  // Returns the evicted hash (0 if none) so the caller can delete the backing file.
  uint64_t insert(uint64_t h, uint64_t file_id) {
    auto it = map_.find(h);
    if (it != map_.end()) { touch(it); it->second.file_id = file_id; return 0; }
    uint64_t ev = 0;
    if (capacity_ && map_.size() >= capacity_) { ev = order_.front(); order_.pop_front(); map_.erase(ev); }
    order_.push_back(h);
    map_[h] = Entry{file_id, std::prev(order_.end())};
    return ev;
  }
  int64_t lookup(uint64_t h) {
    auto it = map_.find(h);
    if (it == map_.end()) return -1;
    touch(it);
    return (int64_t)it->second.file_id;
  }
  // Longest run of consecutive block hashes present, starting at index 0.
  int match(const std::vector<uint64_t>& hashes) {
    int n = 0;
    for (auto h : hashes) { if (lookup(h) < 0) break; n++; }
    return n;
  }
  bool erase(uint64_t h) {
    auto it = map_.find(h); if (it == map_.end()) return false;
    order_.erase(it->second.it); map_.erase(it); return true;
  }
  size_t size() const { return map_.size(); }
 private:
  struct Entry { uint64_t file_id; std::list<uint64_t>::iterator it; };
  void touch(std::unordered_map<uint64_t, Entry>::iterator it) {
    order_.erase(it->second.it); order_.push_back(it->first); it->second.it = std::prev(order_.end());
  }
  size_t capacity_;
  std::list<uint64_t> order_;
  std::unordered_map<uint64_t, Entry> map_;
};

}  // namespace ne
