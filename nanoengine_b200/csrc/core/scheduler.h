// Continuous-batching scheduler, one instance per engine, one queue set per
// attention-DP rank.
//
// Parity: reference rust/src/scheduler/mod.rs:24-47 (queues), api.rs:19-478
// (entry points; prefill before decode :115-131), schedule.rs:15-135 (prefill with
// token budget and chunking), :137-178 (decode), :261-397 (admission: prefix
// lookup, allocate all blocks up front incl. speculative look-ahead),
// lifecycle.rs:7-56 (preemption of the least-recently-scheduled sequence),
// :72-260 (post-processing, bundle truncation at EOS / max_tokens /
// max_model_len, prefill-mode hand-over), :275-321 (abort), router.rs:42-80
// (routing strategies, 3-step affinity wait), cache_flow.rs (+N / +2N KV reservation).
#pragma once
#include <algorithm>
#include <deque>
#include <map>
#include <memory>
#include <set>
#include <unordered_map>

#include "block_pool.h"
#include "metrics.h"
#include "types.h"
#include "wire.h"

namespace ne {

struct ScheduleResult {
  bool has_work = false;
  bool is_prefill = false;
  int64_t step = 0;
  std::vector<Batch> batches;             // one per DP rank (dummy where idle) when has_work
  std::vector<MigrateBatch> migrations;   // KV pulls/pushes to complete before the sequences can run
  std::vector<uint64_t> preempted;
  int32_t num_tokens = 0, num_seqs = 0, prefix_hit_tokens = 0;
};

class Scheduler {
 public:
  explicit Scheduler(const SchedulerConfig& cfg) : cfg_(cfg) {
    if (cfg_.attention_dp < 1) throw std::invalid_argument("attention_dp must be >= 1");
    if (cfg_.block_size < 1) throw std::invalid_argument("block_size must be >= 1");
    int dp = cfg_.attention_dp;
    running_.resize(dp); prefilling_.resize(dp);
    for (int i = 0; i < dp; i++) {
      pools_.emplace_back(cfg_.num_blocks, cfg_.block_size, cfg_.prefix_cache_effective());
      host_pools_.emplace_back(cfg_.num_host_blocks, cfg_.block_size, false);
      state_slots_.emplace_back(cfg_.num_state_slots);
      handoff_slots_.emplace_back(cfg_.num_handoff_slots);
      hisparse_slots_.emplace_back(cfg_.num_hisparse_slots);
    }
  }

  const SchedulerConfig& config() const { return cfg_; }
  Metrics& metrics() { return metrics_; }

  void update_num_blocks(int n) {
    cfg_.num_blocks = n;
    for (auto& p : pools_) p.resize(n);
  }

  // ---- admission -------------------------------------------------------------------------
  uint64_t add_request(const RequestIn& r) {
    if (r.prompt_token_ids.empty()) throw std::invalid_argument("empty prompt");
    if (seqs_.count(r.seq_id)) throw std::invalid_argument("duplicate seq_id");
    if ((int)r.prompt_token_ids.size() >= cfg_.max_model_len) throw std::invalid_argument("prompt exceeds max_model_len");
    auto s = std::make_unique<Sequence>();
    s->seq_id = r.seq_id; s->tokens = r.prompt_token_ids; s->prompt_len = (int)r.prompt_token_ids.size();
    s->sampling = r.sampling_params; s->affinity_key = r.affinity_key; s->vision_slots = r.vision_slots;
    s->t_arrival = now_seconds();
    seqs_[r.seq_id] = std::move(s);
    waiting_.push_back(r.seq_id);
    metrics_.on_request();
    return r.seq_id;
  }

  uint64_t add_migration(const RequestMigrate& m) {
    if (seqs_.count(m.seq_id)) throw std::invalid_argument("duplicate seq_id");
    if (m.block_size != cfg_.block_size) throw std::invalid_argument("migration block_size mismatch");
    if (m.token_ids.empty() || m.prompt_len <= 0 || m.prompt_len > (int)m.token_ids.size())
      throw std::invalid_argument("malformed migration request");
    auto s = std::make_unique<Sequence>();
    s->seq_id = m.seq_id; s->tokens = m.token_ids; s->prompt_len = m.prompt_len; s->num_computed = m.num_computed;
    s->sampling = m.sampling_params; s->logprobs = m.logprobs; s->affinity_key = m.affinity_key;
    s->pending_migration = false; s->remote_block_table = m.migrate_block_table; s->remote_dp_idx = m.migrate_dp_idx;
    s->remote_handoff_slot = m.migrate_handoff_slot; s->remote_engine_id = m.migrate_engine_id;
    s->remote_state_slot = m.migrate_state_slot;
    s->t_arrival = now_seconds(); s->t_first_token = s->t_arrival; s->t_last_token = s->t_arrival;
    seqs_[m.seq_id] = std::move(s);
    waiting_migration_.push_back(m.seq_id);
    metrics_.on_request();
    return m.seq_id;
  }

  uint64_t add_request_bytes(const std::string& b) {
    uint8_t tag = peek_tag(b);
    if (tag == TAG_REQUEST_IN) return add_request(RequestIn::from_bytes(b));
    if (tag == TAG_REQUEST_MIGRATE) return add_migration(RequestMigrate::from_bytes(b));
    throw WireError("add_request_bytes: not a request packet");
  }

  // Third KV tier: see BlockPool::begin_import / finish_import / take_committed.
  void set_commit_log(bool on) { for (auto& p : pools_) p.set_commit_log(on); }
  std::vector<std::pair<uint64_t, int32_t>> take_committed(int dp) { return pools_.at(dp).take_committed(); }
  std::vector<int32_t> begin_import(int dp, const std::vector<uint64_t>& hashes) { return pools_.at(dp).begin_import(hashes); }
  void finish_import(int dp, const std::vector<uint64_t>& hashes, const std::vector<int32_t>& ids, bool ok) {
    pools_.at(dp).finish_import(hashes, ids, ok);
  }
  bool has_cached_hash(int dp, uint64_t h) const { return pools_.at(dp).has_hash(h); }

  void reset_prefix_cache() {
    for (auto& p : pools_) p.clear_cache();
    // Live sequences hold KV that is stale in part: they publish nothing from now on.  (Moving the cursor past the blocks
    // held now would not do: a later block would be hashed from the old chain value, skipping the tokens in between, and a
    // different prompt could reproduce that hash.)  A preempted sequence starts over at cursor 0 and publishes again.
    for (auto& kv : seqs_) kv.second->commit_cursor = INT32_MAX;
  }

  // ---- scheduling ------------------------------------------------------------------------
  const ScheduleResult& schedule() {
    step_++;
    last_ = ScheduleResult{};
    last_.step = step_;
    int dp = cfg_.attention_dp;
    std::vector<Batch> batches(dp);
    for (int i = 0; i < dp; i++) { batches[i].dp_idx = i; batches[i].step = step_; batches[i].block_offsets.push_back(0); }

    admit_migrations();

    // -- prefill first
    std::vector<int> budget(dp, cfg_.max_num_batched_tokens);
    int prefill_tokens = 0;
    {
      for (int d = 0; d < dp; d++) {
        for (uint64_t id : prefilling_[d]) {
          Sequence& s = *seqs_.at(id);
          int chunk = std::min(budget[d], (int)s.tokens.size() - s.num_computed);
          if (chunk <= 0) { s.chunk_len = 0; continue; }
          s.chunk_len = chunk; budget[d] -= chunk; prefill_tokens += chunk;
        }
      }
    }
    while (!waiting_.empty()) {
      uint64_t id = waiting_.front();
      Sequence& s = *seqs_.at(id);
      bool placed = false;
      if (!s.host_blocks.empty()) {
        placed = try_swap_in(s, batches);
      } else {
        for (int d : route_candidates(s)) {
          if ((int)(running_[d].size() + prefilling_[d].size()) >= cfg_.max_num_seqs) continue;
          if (budget[d] <= 0) continue;
          int remaining_hint = (int)s.tokens.size();
          if (!cfg_.enable_chunked_prefill && remaining_hint > budget[d] && budget[d] < cfg_.max_num_batched_tokens) continue;
          if (!try_allocate_prefill(s, d)) continue;
          int chunk = (int)s.tokens.size() - s.num_computed;
          if (cfg_.enable_chunked_prefill) chunk = std::min(chunk, budget[d]);
          s.chunk_len = chunk; budget[d] -= chunk; prefill_tokens += chunk;
          s.dp_idx = d; s.status = PREFILLING;
          if (s.t_first_scheduled == 0) s.t_first_scheduled = now_seconds();
          prefilling_[d].push_back(id);
          if (s.affinity_key) affinity_[s.affinity_key] = d;
          last_.prefix_hit_tokens += s.num_cached_prefix;
          placed = true;
          break;
        }
      }
      if (!placed) break;  // FIFO: the head blocks the queue
      affinity_wait_.erase(id);
      waiting_.pop_front();
    }

    if (prefill_tokens > 0) {
      last_.is_prefill = true; last_.has_work = true;
      for (int d = 0; d < dp; d++) {
        Batch& b = batches[d]; b.is_prefill = true;
        for (uint64_t id : prefilling_[d]) {
          Sequence& s = *seqs_.at(id);
          if (s.chunk_len <= 0) continue;
          int start = s.num_computed, end = start + s.chunk_len;
          b.seq_ids.push_back(id);
          for (int t = start; t < end; t++) { b.input_ids.push_back(s.tokens[t]); b.positions.push_back(t); }
          b.q_lens.push_back(s.chunk_len); b.seq_lens.push_back(end);
          push_common(b, s);
          b.sample_mask.push_back(end == (int)s.tokens.size() ? 1 : 0);
          s.last_scheduled_step = step_;
          last_.num_tokens += s.chunk_len; last_.num_seqs++;
        }
      }
    } else {
      // -- decode
      for (int d = 0; d < dp; d++) {
        Batch& b = batches[d];
        std::vector<uint64_t> order(running_[d].begin(), running_[d].end());
        for (uint64_t id : order) {
          auto it = seqs_.find(id);
          if (it == seqs_.end()) continue;
          Sequence& s = *it->second;
          if (s.status != RUNNING) continue;  // preempted earlier in this loop
          if (!ensure_decode_blocks(s, d, b)) continue;  // s itself was preempted
          int n = (int)s.tokens.size();
          b.seq_ids.push_back(id);
          b.input_ids.push_back(s.tokens[n - 1]); b.positions.push_back(n - 1);
          b.q_lens.push_back(1); b.seq_lens.push_back(n);
          push_common(b, s);
          b.sample_mask.push_back(1);
          s.last_scheduled_step = step_;
          last_.num_tokens += 1; last_.num_seqs++;
        }
        if (!b.seq_ids.empty()) last_.has_work = true;
      }
    }
    if (last_.has_work) {
      for (int d = 0; d < dp; d++) if (batches[d].seq_ids.empty()) { batches[d].is_dummy = true; batches[d].is_prefill = last_.is_prefill; }
      last_.batches = std::move(batches);
    } else {
      // swap / migration side effects may still need to reach the workers
      bool side = false;
      for (auto& b : batches) side = side || !b.swap_in_src.empty() || !b.swap_out_src.empty();
      if (side) { for (auto& b : batches) b.is_dummy = true; last_.batches = std::move(batches); last_.has_work = true; }
    }
    t_schedule_ = now_seconds();
    return last_;
  }

  std::vector<std::string> serialize_run_batches() const {
    std::vector<std::string> out;
    for (auto& b : last_.batches) out.push_back(b.to_bytes());
    return out;
  }
  std::vector<std::string> serialize_migrate_batches() const {
    std::vector<std::string> out;
    for (auto& m : last_.migrations) out.push_back(m.to_bytes());
    return out;
  }
  const ScheduleResult& last() const { return last_; }

  // Mark migrated sequences runnable (ok) or drop them (failed transfer).
  void complete_migration(const std::vector<uint64_t>& ids, bool ok) {
    for (uint64_t id : ids) {
      auto it = seqs_.find(id); if (it == seqs_.end()) continue;
      Sequence& s = *it->second;
      if (!s.pending_migration) continue;
      s.pending_migration = false;
      if (ok) { s.status = RUNNING; running_[s.dp_idx].push_back(id); }
      else { release_resources(s); metrics_.on_abort(); seqs_.erase(it); }
    }
  }

  // ---- post-processing -------------------------------------------------------------------
  std::vector<StepOut> postprocess(const std::vector<RunResult>& results, double latency_ms = -1.0) {
    std::vector<StepOut> outs;
    std::unordered_map<uint64_t, std::pair<const RunResult*, size_t>> by_seq;
    for (auto& r : results) for (size_t i = 0; i < r.seq_ids.size(); i++) by_seq[r.seq_ids[i]] = {&r, i};
    double now = now_seconds();
    uint64_t gen = 0, prompt = 0;
    for (auto& b : last_.batches) {
      for (size_t i = 0; i < b.seq_ids.size(); i++) {
        uint64_t id = b.seq_ids[i];
        auto sit = seqs_.find(id); if (sit == seqs_.end()) continue;  // aborted while in flight
        Sequence& s = *sit->second;
        StepOut so; so.seq_id = id;
        if (b.is_prefill) {
          s.num_computed += s.chunk_len; prompt += (uint64_t)s.chunk_len; s.chunk_len = 0; s.prefill_chunks++;
          commit_full_blocks(s);
          if (s.num_computed < (int)s.tokens.size()) { s.status = PREFILLING; so.status = PREFILLING; outs.push_back(std::move(so)); continue; }
          remove_from(prefilling_[s.dp_idx], id);
          s.status = RUNNING; running_[s.dp_idx].push_back(id);
        }
        auto rit = by_seq.find(id);
        if (rit == by_seq.end()) throw std::runtime_error("postprocess: missing result for sequence " + std::to_string(id));
        const RunResult& r = *rit->second.first; size_t k = rit->second.second;
        int lo = r.token_offsets[k], hi = r.token_offsets[k + 1];
        bool finished = false;
        for (int t = lo; t < hi && !finished; t++) {
          int32_t tok = r.token_ids[t];
          s.tokens.push_back(tok); so.token_ids.push_back(tok); gen++;
          if (s.sampling.return_completion_logprobs && (size_t)t < r.logprobs.size()) { s.logprobs.push_back(r.logprobs[t]); so.logprobs.push_back(r.logprobs[t]); }
          if (s.t_first_token == 0) s.t_first_token = now; else itl_[id].push_back(now - s.t_last_token);
          s.t_last_token = now;
          if (!s.sampling.ignore_eos && is_eos(tok)) finished = true;
          if (s.num_output_tokens() >= s.sampling.max_tokens) finished = true;
          if ((int)s.tokens.size() >= cfg_.max_model_len) finished = true;
        }
        s.num_computed = (int)s.tokens.size() - 1;
        commit_full_blocks(s);
        if (finished) { finish(s); so.status = FINISHED; }
        else if (cfg_.mode == MODE_PREFILL) {
          remove_from(running_[s.dp_idx], id);
          s.status = TO_BE_MIGRATED; to_be_migrated_.insert(id); so.status = TO_BE_MIGRATED;
        } else so.status = RUNNING;
        outs.push_back(std::move(so));
        if (finished) seqs_.erase(id);
      }
    }
    metrics_.on_tokens(prompt, gen);
    StepRecord rec; rec.step = step_; rec.is_prefill = last_.is_prefill; rec.num_seqs = last_.num_seqs;
    rec.num_tokens = last_.is_prefill ? last_.num_tokens : (int)gen; rec.prefix_hit_tokens = last_.prefix_hit_tokens;
    rec.preempted = (int)last_.preempted.size();
    rec.latency_ms = latency_ms >= 0 ? latency_ms : (now - t_schedule_) * 1e3;
    metrics_.on_step(rec);
    last_.batches.clear();
    return outs;
  }

  std::vector<StepOut> postprocess_bytes(const std::vector<std::string>& blobs, double latency_ms = -1.0) {
    std::vector<RunResult> rs; rs.reserve(blobs.size());
    for (auto& b : blobs) rs.push_back(RunResult::from_bytes(b));
    return postprocess(rs, latency_ms);
  }

  // ---- control ---------------------------------------------------------------------------
  bool abort(uint64_t id) {
    auto it = seqs_.find(id); if (it == seqs_.end()) return false;
    Sequence& s = *it->second;
    remove_from_deque(waiting_, id); remove_from_deque(waiting_migration_, id);
    if (s.dp_idx >= 0) { remove_from(running_[s.dp_idx], id); remove_from(prefilling_[s.dp_idx], id); }
    to_be_migrated_.erase(id);
    release_resources(s);
    itl_.erase(id); affinity_wait_.erase(id);
    metrics_.on_abort();
    seqs_.erase(it);
    return true;
  }

  // Prefill side of PD: blobs describing sequences whose prompt is done and whose KV waits for pick-up.
  std::vector<RequestMigrate> export_to_be_migrated() {
    std::vector<RequestMigrate> out;
    for (uint64_t id : to_be_migrated_) {
      if (exported_.count(id)) continue;
      Sequence& s = *seqs_.at(id);
      RequestMigrate m; m.seq_id = id; m.token_ids = s.tokens; m.prompt_len = s.prompt_len; m.num_computed = s.num_computed;
      m.sampling_params = s.sampling; m.logprobs = s.logprobs; m.affinity_key = s.affinity_key;
      m.migrate_block_table = s.block_table; m.migrate_dp_idx = s.dp_idx; m.migrate_state_slot = s.state_slot;
      m.migrate_handoff_slot = s.handoff_slot; m.migrate_hisparse_slot = s.hisparse_slot; m.migrate_engine_id = cfg_.engine_id;
      m.migrate_num_kvcache_blocks = cfg_.num_blocks; m.block_size = cfg_.block_size;
      out.push_back(std::move(m)); exported_.insert(id);
    }
    return out;
  }

  int free_to_be_migrated(const std::vector<uint64_t>& ids) {
    int n = 0;
    for (uint64_t id : ids) {
      if (!to_be_migrated_.erase(id)) continue;
      exported_.erase(id);
      auto it = seqs_.find(id); if (it == seqs_.end()) continue;
      finish_metrics(*it->second); release_resources(*it->second); itl_.erase(id); seqs_.erase(it); n++;
    }
    return n;
  }

  bool is_finished() const {
    if (!waiting_.empty() || !waiting_migration_.empty()) return false;
    for (auto& v : running_) if (!v.empty()) return false;
    for (auto& v : prefilling_) if (!v.empty()) return false;
    for (auto& kv : seqs_) if (kv.second->pending_migration) return false;
    return true;
  }

  // ---- introspection ---------------------------------------------------------------------
  const Sequence* get(uint64_t id) const { auto it = seqs_.find(id); return it == seqs_.end() ? nullptr : it->second.get(); }
  int num_waiting() const { return (int)waiting_.size(); }
  int num_waiting_migration() const { return (int)waiting_migration_.size(); }
  int num_running(int dp) const { return (int)running_.at(dp).size(); }
  int num_prefilling(int dp) const { return (int)prefilling_.at(dp).size(); }
  int num_to_be_migrated() const { return (int)to_be_migrated_.size(); }
  int num_free_blocks(int dp) const { return pools_.at(dp).num_free(); }
  int num_cached_blocks(int dp) const { return pools_.at(dp).num_cached(); }
  int num_free_host_blocks(int dp) const { return host_pools_.at(dp).num_free(); }
  int num_free_state_slots(int dp) const { return state_slots_.at(dp).num_free(); }
  int num_free_handoff_slots(int dp) const { return handoff_slots_.at(dp).num_free(); }
  int64_t step() const { return step_; }
  BlockPool& pool(int dp) { return pools_.at(dp); }

  std::string metrics_prometheus() const { return metrics_.prometheus(gauges()); }
  std::string status_line(const std::string& mode) const { return metrics_.status_line(gauges(), cfg_.engine_id, mode); }

  Metrics::Gauges gauges() const {
    Metrics::Gauges g; g.waiting = (int)waiting_.size() + (int)waiting_migration_.size();
    uint64_t hit = 0, look = 0;
    for (int d = 0; d < cfg_.attention_dp; d++) {
      g.running_per_dp.push_back((int)(running_[d].size() + prefilling_[d].size()));
      g.used_blocks_per_dp.push_back(pools_[d].num_used()); g.total_blocks_per_dp.push_back(pools_[d].num_blocks());
      g.waiting_blocks_per_dp.push_back(waiting_blocks());
      double r = pools_[d].lookup_tokens() ? (double)pools_[d].hit_tokens() / (double)pools_[d].lookup_tokens() : 0.0;
      g.prefix_hit_rate_per_dp.push_back(r);
      hit += pools_[d].hit_tokens(); look += pools_[d].lookup_tokens();
    }
    g.prefix_hit_rate = look ? (double)hit / (double)look : 0.0;
    g.waiting_migration = (int)waiting_migration_.size();
    g.total_host_blocks_per_dp = (int)cfg_.num_host_blocks;
    for (size_t d = 0; d < host_pools_.size(); d++) g.used_host_blocks_per_dp.push_back((int)cfg_.num_host_blocks - host_pools_[d].num_free());
    for (auto& sp : hisparse_slots_) { g.total_hisparse_slots += sp.total(); g.used_hisparse_slots += sp.total() - sp.num_free(); }
    return g;
  }

 private:
  int spec() const { return cfg_.num_speculative_tokens; }
  int blocks_for(int tokens) const { return (tokens + cfg_.block_size - 1) / cfg_.block_size; }
  bool is_eos(int32_t t) const { return std::find(cfg_.eos_token_ids.begin(), cfg_.eos_token_ids.end(), t) != cfg_.eos_token_ids.end(); }
  int waiting_blocks() const {
    int n = 0;
    for (uint64_t id : waiting_) n += blocks_for((int)seqs_.at(id)->tokens.size());
    return n;
  }
  static void remove_from(std::vector<uint64_t>& v, uint64_t id) { v.erase(std::remove(v.begin(), v.end(), id), v.end()); }
  static void remove_from_deque(std::deque<uint64_t>& v, uint64_t id) { v.erase(std::remove(v.begin(), v.end(), id), v.end()); }

  void push_common(Batch& b, const Sequence& s) {
    b.block_tables.insert(b.block_tables.end(), s.block_table.begin(), s.block_table.end());
    b.block_offsets.push_back((int)b.block_tables.size());
    b.temperatures.push_back(s.sampling.temperature);
    b.state_slots.push_back(s.state_slot); b.handoff_slots.push_back(s.handoff_slot); b.hisparse_slots.push_back(s.hisparse_slot);
    if (s.sampling.return_completion_logprobs) b.any_return_logprobs = true;
  }

  int dp_tokens(int d) const {
    int n = 0;
    for (uint64_t id : running_[d]) n += (int)seqs_.at(id)->tokens.size();
    for (uint64_t id : prefilling_[d]) n += (int)seqs_.at(id)->tokens.size();
    return n;
  }

  std::vector<int> route_candidates(Sequence& s) {
    int dp = cfg_.attention_dp;
    std::vector<int> order(dp);
    for (int i = 0; i < dp; i++) order[i] = i;
    switch (cfg_.routing) {
      case ROUND_ROBIN: {
        int start = rr_cursor_ % dp; rr_cursor_ = (rr_cursor_ + 1) % dp;
        std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return (a + dp - start) % dp < (b + dp - start) % dp; });
        break;
      }
      case LEAST_BATCH:
        std::stable_sort(order.begin(), order.end(), [&](int a, int b) {
          return running_[a].size() + prefilling_[a].size() < running_[b].size() + prefilling_[b].size(); });
        break;
      case LEAST_CACHE:
      case AFFINITY: {
        std::vector<int> tok(dp);
        for (int i = 0; i < dp; i++) tok[i] = dp_tokens(i);
        std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return tok[a] < tok[b]; });
        if (cfg_.routing == AFFINITY && s.affinity_key) {
          auto it = affinity_.find(s.affinity_key);
          if (it != affinity_.end()) {
            int pref = std::min(it->second, dp - 1);
            int& waited = affinity_wait_[s.seq_id];
            if (waited < 3) { waited++; return {pref}; }  // hold out for the rank that has this session's prefix
            order.erase(std::remove(order.begin(), order.end(), pref), order.end());
            order.insert(order.begin(), pref);
          }
        }
        break;
      }
      default: break;
    }
    return order;
  }

  bool acquire_slots(Sequence& s, int d) {
    bool need_state = cfg_.needs_state_slots();
    bool need_handoff = spec() > 0 && cfg_.num_handoff_slots > 0;
    bool need_hs = (cfg_.cache_plan & PLAN_HISPARSE) && cfg_.num_hisparse_slots > 0;
    if (need_state && s.state_slot < 0 && state_slots_[d].num_free() == 0) return false;
    if (need_handoff && s.handoff_slot < 0 && handoff_slots_[d].num_free() == 0) return false;
    if (need_hs && s.hisparse_slot < 0 && hisparse_slots_[d].num_free() == 0) return false;
    if (need_state && s.state_slot < 0) s.state_slot = state_slots_[d].acquire();
    if (need_handoff && s.handoff_slot < 0) s.handoff_slot = handoff_slots_[d].acquire();
    if (need_hs && s.hisparse_slot < 0) s.hisparse_slot = hisparse_slots_[d].acquire();
    return true;
  }

  // Admission: prefix lookup, then every block the sequence needs (plus speculative look-ahead) up front.
  bool try_allocate_prefill(Sequence& s, int d) {
    BlockPool& pool = pools_[d];
    int n = (int)s.tokens.size();
    uint64_t h = 0;
    std::vector<int32_t> matched = pool.match_prefix(s.tokens.data(), n, &h);
    int need = blocks_for(n + spec()) - (int)matched.size();
    std::vector<int32_t> fresh;
    if (need < 0) need = 0;
    if (!pool.allocate(need, &fresh) || !acquire_slots(s, d)) {
      if (!fresh.empty()) pool.release(fresh);
      pool.release(matched);
      return false;
    }
    s.block_table = matched;
    s.block_table.insert(s.block_table.end(), fresh.begin(), fresh.end());
    s.num_cached_prefix = (int)matched.size() * cfg_.block_size;
    s.num_computed = s.num_cached_prefix;
    s.commit_cursor = (int)matched.size(); s.last_block_hash = h;
    return true;
  }

  // Decode growth: one more token (+ verify and next-draft windows with MTP).  Preempts on shortage.
  bool ensure_decode_blocks(Sequence& s, int d, Batch& b) {
    int reserve = spec() > 0 ? 2 * spec() : 0;
    int need = blocks_for((int)s.tokens.size() + reserve) - (int)s.block_table.size();
    while (need > 0) {
      std::vector<int32_t> fresh;
      if (pools_[d].allocate(need, &fresh)) { s.block_table.insert(s.block_table.end(), fresh.begin(), fresh.end()); break; }
      uint64_t victim = 0;
      if (!pick_victim(d, &victim)) return false;
      Sequence& v = *seqs_.at(victim);
      bool self = (&v == &s);
      preempt(v, b);
      if (self) return false;
    }
    return true;
  }

  bool pick_victim(int d, uint64_t* out) const {
    uint64_t best = 0; int64_t best_step = INT64_MAX; bool found = false;
    // least recently scheduled; ties broken towards the youngest arrival so old requests finish
    for (auto it = running_[d].rbegin(); it != running_[d].rend(); ++it) {
      const Sequence& s = *seqs_.at(*it);
      if (s.status != RUNNING) continue;
      if (!found || s.last_scheduled_step < best_step) { best = *it; best_step = s.last_scheduled_step; found = true; }
    }
    *out = best;
    return found;
  }

  void preempt(Sequence& s, Batch& b) {
    int d = s.dp_idx;
    remove_from(running_[d], s.seq_id);
    bool swapped = false;
    if (cfg_.num_host_blocks > 0) {
      int used = blocks_for(s.num_computed);
      std::vector<int32_t> host;
      if (used > 0 && host_pools_[d].allocate(used, &host)) {
        for (int i = 0; i < used; i++) { b.swap_out_src.push_back(s.block_table[i]); b.swap_out_dst.push_back(host[i]); }
        s.host_blocks = host; s.num_checkpointed = s.num_computed; s.swapped_at_step = step_; swapped = true;
      }
    }
    pools_[d].release(s.block_table); s.block_table.clear();
    if (!swapped) { s.num_computed = 0; s.num_checkpointed = 0; release_slots(s); }
    s.commit_cursor = 0; s.last_block_hash = 0; s.num_cached_prefix = 0;
    s.status = WAITING; s.num_preemptions++;
    if (swapped) waiting_.push_back(s.seq_id); else waiting_.push_front(s.seq_id);
    last_.preempted.push_back(s.seq_id);
  }

  // A swapped-out sequence returns to its DP rank without recomputation once the cooldown has passed.
  bool try_swap_in(Sequence& s, std::vector<Batch>& batches) {
    int d = s.dp_idx;
    if (step_ - s.swapped_at_step < cfg_.swap_cooldown_steps) return false;
    if ((int)(running_[d].size() + prefilling_[d].size()) >= cfg_.max_num_seqs) return false;
    int reserve = spec() > 0 ? 2 * spec() : 0;
    int need = std::max((int)s.host_blocks.size(), blocks_for((int)s.tokens.size() + reserve));
    std::vector<int32_t> fresh;
    if (!pools_[d].allocate(need, &fresh)) return false;
    Batch& b = batches[d];
    for (size_t i = 0; i < s.host_blocks.size(); i++) { b.swap_in_src.push_back(s.host_blocks[i]); b.swap_in_dst.push_back(fresh[i]); }
    host_pools_[d].release(s.host_blocks); s.host_blocks.clear();
    s.block_table = fresh; s.num_computed = s.num_checkpointed; s.status = RUNNING;
    for (int i = 0; i < blocks_for(s.num_computed) && i < (int)fresh.size(); i++) pools_[d].mark_ready(fresh[i]);
    running_[d].push_back(s.seq_id);
    return true;
  }

  void admit_migrations() {
    if (waiting_migration_.empty()) return;
    std::map<int, MigrateBatch> per_dp;
    while (!waiting_migration_.empty()) {
      uint64_t id = waiting_migration_.front();
      Sequence& s = *seqs_.at(id);
      bool placed = false;
      for (int d : route_candidates(s)) {
        if ((int)(running_[d].size() + prefilling_[d].size() + pending_on(d)) >= cfg_.max_num_seqs) continue;
        int need = blocks_for((int)s.tokens.size() + (spec() > 0 ? 2 * spec() : 0));
        std::vector<int32_t> fresh;
        if (!pools_[d].allocate(need, &fresh)) continue;
        if (!acquire_slots(s, d)) { pools_[d].release(fresh); continue; }
        s.block_table = fresh; s.dp_idx = d; s.pending_migration = true;
        MigrateBatch& m = per_dp[d]; m.dp_idx = d;
        if (m.block_offsets.empty()) m.block_offsets.push_back(0);
        m.seq_ids.push_back(id);
        int nb = std::min((int)s.remote_block_table.size(), blocks_for(s.num_computed));
        for (int i = 0; i < nb; i++) { m.local_blocks.push_back(fresh[i]); m.remote_blocks.push_back(s.remote_block_table[i]); }
        m.block_offsets.push_back((int)m.local_blocks.size());
        m.remote_dp_idx.push_back(s.remote_dp_idx); m.local_handoff_slots.push_back(s.handoff_slot);
        m.remote_handoff_slots.push_back(s.remote_handoff_slot); m.remote_engine_ids.push_back(s.remote_engine_id);
        m.local_state_slots.push_back(s.state_slot); m.remote_state_slots.push_back(s.remote_state_slot);
        placed = true; break;
      }
      if (!placed) break;
      waiting_migration_.pop_front();
    }
    for (auto& kv : per_dp) last_.migrations.push_back(std::move(kv.second));
  }

  int pending_on(int d) const {
    int n = 0;
    for (auto& kv : seqs_) if (kv.second->pending_migration && kv.second->dp_idx == d) n++;
    return n;
  }

  void commit_full_blocks(Sequence& s) {
    if (s.dp_idx < 0) return;
    BlockPool& pool = pools_[s.dp_idx];
    int full = s.num_computed / cfg_.block_size;
    while (s.commit_cursor < full && s.commit_cursor < (int)s.block_table.size()) {
      uint64_t h = chain_hash(s.last_block_hash, s.tokens.data() + (size_t)s.commit_cursor * cfg_.block_size, cfg_.block_size);
      pool.commit(s.block_table[s.commit_cursor], h);
      s.last_block_hash = h; s.commit_cursor++;
    }
  }

  void release_slots(Sequence& s) {
    if (s.dp_idx < 0) return;
    state_slots_[s.dp_idx].release(s.state_slot); s.state_slot = -1;
    handoff_slots_[s.dp_idx].release(s.handoff_slot); s.handoff_slot = -1;
    hisparse_slots_[s.dp_idx].release(s.hisparse_slot); s.hisparse_slot = -1;
  }
  void release_resources(Sequence& s) {
    if (s.dp_idx >= 0) {
      if (!s.block_table.empty()) pools_[s.dp_idx].release(s.block_table);
      if (!s.host_blocks.empty()) host_pools_[s.dp_idx].release(s.host_blocks);
    }
    s.block_table.clear(); s.host_blocks.clear();
    release_slots(s);
  }
  void finish_metrics(Sequence& s) {
    int n_out = s.num_output_tokens();
    double ttft = s.t_first_token > 0 ? s.t_first_token - s.t_arrival : 0;
    double tpot = n_out > 1 ? (s.t_last_token - s.t_first_token) / (double)(n_out - 1) : 0;
    auto it = itl_.find(s.seq_id);
    metrics_.on_finish(ttft, tpot, n_out, it == itl_.end() ? std::vector<double>{} : it->second);
    itl_.erase(s.seq_id);
  }
  void finish(Sequence& s) {
    s.status = FINISHED;
    if (s.dp_idx >= 0) { remove_from(running_[s.dp_idx], s.seq_id); remove_from(prefilling_[s.dp_idx], s.seq_id); }
    finish_metrics(s);
    release_resources(s);
  }

  SchedulerConfig cfg_;
  std::unordered_map<uint64_t, std::unique_ptr<Sequence>> seqs_;
  std::deque<uint64_t> waiting_, waiting_migration_;
  std::vector<std::vector<uint64_t>> running_, prefilling_;
  std::set<uint64_t> to_be_migrated_, exported_;
  std::vector<BlockPool> pools_, host_pools_;
  std::vector<SlotPool> state_slots_, handoff_slots_, hisparse_slots_;
  std::unordered_map<uint64_t, int> affinity_;
  std::unordered_map<uint64_t, int> affinity_wait_;
  std::unordered_map<uint64_t, std::vector<double>> itl_;
  int rr_cursor_ = 0;
  int64_t step_ = 0;
  double t_schedule_ = 0;
  ScheduleResult last_;
  Metrics metrics_;
};

}  // namespace ne
