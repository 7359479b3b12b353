// Core value types of the native control plane: sampling parameters, sequence
// state, cache-plan flags and the scheduler configuration.
//
// Parity: reference rust/src/sampling.rs:3-45 (SamplingParams defaults),
// rust/src/sequence.rs:21-57 (status codes 0..4), rust/src/config/mod.rs and
// rust/src/scheduler/types.rs:33-65 (CachePlan bits, SchedulerConfig).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace ne {

struct SamplingParams {
  float temperature = 1.0f;
  int32_t max_tokens = 256;
  bool ignore_eos = false;
  bool return_completion_logprobs = false;
};

enum SeqStatus : int32_t {
  WAITING = 0,
  RUNNING = 1,
  FINISHED = 2,
  TO_BE_MIGRATED = 3,
  PREFILLING = 4,
};

// Which cache families a model needs; one bit each (a model may combine them).
enum CachePlanBits : uint32_t {
  PLAN_GQA = 1u << 0,
  PLAN_MLA = 1u << 1,
  PLAN_GDN = 1u << 2,      // recurrent-state layers: needs a state slot, disables prefix caching
  PLAN_HCA = 1u << 3,      // DeepSeek-V4 shared-row pages (window rows)
  PLAN_CSA = 1u << 4,      // DeepSeek-V4 pooled-row pages + compressor carry: needs a state slot, disables prefix caching
  PLAN_INDEXER = 1u << 5,  // DSA lightning-indexer key pages share the main page table
  PLAN_HISPARSE = 1u << 6, // hot/cold tiering: needs a hot-buffer slot per sequence
};

enum RoutingStrategy : int32_t {
  ROUND_ROBIN = 0,
  LEAST_BATCH = 1,
  LEAST_CACHE = 2,
  AFFINITY = 3,
};

enum EngineMode : int32_t { MODE_HYBRID = 0, MODE_PREFILL = 1, MODE_DECODE = 2 };

struct SchedulerConfig {
  int32_t num_blocks = 0;          // device KV blocks per attention-DP rank
  int32_t num_host_blocks = 0;     // host swap tier per DP rank (0 = off)
  int32_t block_size = 64;
  int32_t max_num_seqs = 16;       // per DP rank
  int32_t max_num_batched_tokens = 16384;  // per DP rank and step
  int32_t max_model_len = 1 << 20;
  int32_t attention_dp = 1;
  int32_t mode = MODE_HYBRID;
  int32_t num_speculative_tokens = 0;
  bool enable_prefix_caching = true;
  bool enable_chunked_prefill = true;
  int32_t routing = ROUND_ROBIN;
  uint32_t cache_plan = PLAN_MLA;
  int32_t num_state_slots = 0;     // per DP rank, for GDN / recurrent MTP state
  int32_t num_handoff_slots = 0;   // per DP rank, MTP hand-off rows
  int32_t num_hisparse_slots = 0;  // per DP rank
  int32_t swap_cooldown_steps = 2; // steps a swapped-out sequence waits before restore
  std::vector<int32_t> eos_token_ids;
  std::string engine_id;

  bool prefix_cache_effective() const {
    // plans with per-sequence state cannot reuse KV prefixes (state is not per block)
    // (PLAN_GDN: recurrent state; PLAN_CSA: the compressor's unfinished block)
    return enable_prefix_caching && !(cache_plan & (PLAN_GDN | PLAN_CSA));
  }
  bool needs_state_slots() const { return (cache_plan & (PLAN_GDN | PLAN_CSA)) && num_state_slots > 0; }
};

struct Sequence {
  uint64_t seq_id = 0;
  std::vector<int32_t> tokens;       // prompt + generated
  int32_t prompt_len = 0;
  int32_t num_computed = 0;          // tokens whose KV already sits in the cache
  int32_t num_cached_prefix = 0;     // of which came from a prefix-cache hit (last admission)
  int32_t num_checkpointed = 0;      // tokens preserved across a preemption (host tier)
  int32_t chunk_len = 0;             // tokens scheduled in the current prefill step
  SamplingParams sampling;
  uint64_t affinity_key = 0;
  int32_t status = WAITING;
  int32_t dp_idx = -1;
  std::vector<int32_t> block_table;  // device blocks
  std::vector<int32_t> host_blocks;  // host tier blocks while swapped out
  int32_t state_slot = -1;
  int32_t handoff_slot = -1;
  int32_t hisparse_slot = -1;
  int64_t last_scheduled_step = -1;
  int64_t swapped_at_step = -1;
  int32_t num_preemptions = 0;
  int32_t prefill_chunks = 0;
  int32_t commit_cursor = 0;         // blocks already published to the prefix cache
  uint64_t last_block_hash = 0;      // chained hash up to commit_cursor
  std::vector<float> logprobs;
  std::vector<int32_t> vision_slots;
  // PD migration bookkeeping (decode side)
  bool pending_migration = false;
  std::vector<int32_t> remote_block_table;
  int32_t remote_dp_idx = 0;
  int32_t remote_handoff_slot = -1;
  int32_t remote_state_slot = -1;    // the prefill engine's state slot of a migrated sequence
  std::string remote_engine_id;
  // timing (seconds, steady clock)
  double t_arrival = 0, t_first_token = 0, t_last_token = 0, t_first_scheduled = 0;
  int32_t num_output_tokens() const { return (int32_t)tokens.size() - prompt_len; }
};

}  // namespace ne
