// Stand-alone exerciser of the control plane for sanitizer builds (-fsanitize=address,undefined or thread): it drives the
// scheduler, the block pool, the slot pools, the L3 index and the wire codec through their busy paths - admission with prefix
// hits, chunked prefill, decode growth with preemption and host swap, speculative bundles, aborts, imports from a lower tier,
// corrupted packets - and checks a few invariants on the way.  Exit code 0 = every check held; the sanitizer aborts on its own.
//
// The reference has no sanitizer configuration; its scheduler scenarios live in rust/src/scheduler/tests.rs:254-852.
#include <cstdio>
#include <cstdlib>
#include <random>
#include <thread>

#include "scheduler.h"

using namespace ne;

#define CHECK(c) do { if (!(c)) { std::fprintf(stderr, "selftest: check failed at %s:%d: %s\n", __FILE__, __LINE__, #c); std::exit(1); } } while (0)

static SchedulerConfig make_cfg(int blocks, int bs) {
  SchedulerConfig c;
  c.num_blocks = blocks; c.block_size = bs; c.max_num_seqs = 8; c.max_num_batched_tokens = 48; c.max_model_len = 4096;
  c.eos_token_ids = {2};
  return c;
}

static void add(Scheduler& s, uint64_t id, std::vector<int32_t> toks, int max_tokens, bool ignore_eos = false) {
  RequestIn r; r.seq_id = id; r.prompt_token_ids = std::move(toks);
  r.sampling_params.temperature = 0.f; r.sampling_params.max_tokens = max_tokens; r.sampling_params.ignore_eos = ignore_eos;
  s.add_request_bytes(r.to_bytes());
}

// one engine step with a fake runner that emits `per` tokens per sampled sequence
static std::vector<StepOut> step(Scheduler& s, std::mt19937& rng, int per = 1) {
  const ScheduleResult& r = s.schedule();
  if (!r.has_work) return {};
  for (const std::string& b : s.serialize_run_batches()) (void)Batch::from_bytes(b);      // the wire form of every batch parses back
  std::vector<RunResult> outs;
  for (const Batch& b : r.batches) {
    RunResult o; o.token_offsets.push_back(0);
    for (size_t i = 0; i < b.seq_ids.size(); i++) {
      if (!b.sample_mask[i]) continue;
      o.seq_ids.push_back(b.seq_ids[i]);
      for (int j = 0; j < per; j++) o.token_ids.push_back(3 + (int)(rng() % 50));
      o.token_offsets.push_back((int32_t)o.token_ids.size());
    }
    outs.push_back(std::move(o));
  }
  return s.postprocess(outs, 1.0);
}

static void run_until_done(Scheduler& s, std::mt19937& rng, int per = 1) {
  for (int i = 0; i < 100000 && !s.is_finished(); i++) step(s, rng, per);
  CHECK(s.is_finished());
}

static void scenario_prefix_chunks_preemption() {
  std::mt19937 rng(1);
  SchedulerConfig c = make_cfg(24, 4);
  c.num_host_blocks = 8; c.swap_cooldown_steps = 1;
  Scheduler s(c);
  std::vector<int32_t> shared(30);
  for (int i = 0; i < 30; i++) shared[i] = 100 + i;
  for (uint64_t id = 1; id <= 6; id++) {
    std::vector<int32_t> p = shared;
    for (int i = 0; i < (int)id * 7; i++) p.push_back(200 + (int)(rng() % 90));      // longer than the token budget: chunked
    add(s, id, p, 20, true);
  }
  run_until_done(s, rng);
  CHECK(s.num_free_blocks(0) + s.num_cached_blocks(0) >= 0);
  add(s, 7, shared, 3, true);                                                         // a prefix hit on what the others left
  const ScheduleResult& r = s.schedule();
  CHECK(r.has_work && r.prefix_hit_tokens > 0);
  std::vector<RunResult> outs(1);
  outs[0].seq_ids = {7}; outs[0].token_ids = {9}; outs[0].token_offsets = {0, 1};
  s.postprocess(outs, 1.0);
  CHECK(s.abort(7));
  CHECK(!s.abort(7));
  s.reset_prefix_cache();
  CHECK(s.num_cached_blocks(0) == 0);
  (void)s.metrics_prometheus();
}

static void scenario_speculative_and_slots() {
  std::mt19937 rng(2);
  SchedulerConfig c = make_cfg(64, 4);
  c.num_speculative_tokens = 2; c.num_handoff_slots = 2; c.attention_dp = 2;
  Scheduler s(c);
  for (uint64_t id = 1; id <= 5; id++) add(s, id, std::vector<int32_t>(5 + id, 4), 9);
  run_until_done(s, rng, 3);                                                          // bundles of 3, truncated at the limits
  CHECK(s.num_free_handoff_slots(0) == 2 && s.num_free_handoff_slots(1) == 2);
}

static void scenario_pool_and_import() {
  BlockPool p(6, 4, true);
  std::vector<int32_t> ids;
  CHECK(p.allocate(3, &ids));
  int32_t t0[] = {1, 2, 3, 4}, t1[] = {5, 6, 7, 8}, t2[] = {9, 9, 9, 9};
  uint64_t h0 = chain_hash(0, t0, 4), h1 = chain_hash(h0, t1, 4), h2 = chain_hash(h1, t2, 4);
  p.commit(ids[0], h0);
  p.release(ids);
  std::vector<int32_t> got = p.begin_import({h0, h1, h2});
  CHECK(got.size() == 3 && got[0] == -1 && got[1] >= 0 && got[2] >= 0);
  p.finish_import({h0, h1, h2}, got, true);
  uint64_t last = 0;
  int32_t toks[] = {1, 2, 3, 4, 5, 6, 7, 8, 9, 9, 9, 9, 0};
  std::vector<int32_t> m = p.match_prefix(toks, 13, &last);
  CHECK(m.size() == 3 && last == h2);
  p.release(m);
  p.clear_cache();
  CHECK(p.num_cached() == 0);
  L3Index l3(2);
  CHECK(l3.insert(1, 10) == 0 && l3.insert(2, 20) == 0 && l3.insert(3, 30) == 1);
  SlotPool sp(2);
  int a = sp.acquire(), b = sp.acquire();
  CHECK(a >= 0 && b >= 0 && sp.acquire() < 0);
  sp.release(a); sp.release(b);
}

static void scenario_wire_corruption() {
  RequestIn r; r.seq_id = 5; r.prompt_token_ids = {1, 2, 3};
  std::string good = r.to_bytes();
  std::mt19937 rng(3);
  int rejected = 0;
  for (int i = 0; i < 2000; i++) {
    std::string bad = good;
    size_t cut = rng() % (bad.size() + 1);
    if (i % 2) bad.resize(cut); else bad[rng() % bad.size()] ^= (char)(1 + rng() % 255);
    try { (void)RequestIn::from_bytes(bad); } catch (const std::exception&) { rejected++; }
  }
  CHECK(rejected > 0);
  Packet pk; pk.action = ACT_ADD; pk.payload = good;
  CHECK(Packet::from_bytes(pk.to_bytes()).payload == good);
}

int main() {
  scenario_prefix_chunks_preemption();
  scenario_speculative_and_slots();
  scenario_pool_and_import();
  scenario_wire_corruption();
  // independent schedulers on their own threads (one per engine process in a deployment; here they share an address space,
  // which is what a thread sanitizer build wants to see: no hidden shared state between instances)
  {
    std::vector<std::thread> th;
    for (int t = 0; t < 3; t++)
      th.emplace_back([t] {
        std::mt19937 rng(10 + t);
        Scheduler s(make_cfg(64, 4));
        for (uint64_t id = 1; id <= 4; id++) add(s, id, std::vector<int32_t>(9 + t, 4), 30, true);
        run_until_done(s, rng);
        (void)s.metrics_prometheus();
      });
    for (auto& x : th) x.join();
  }
  std::puts("selftest ok");
  return 0;
}
