// pybind11 surface of the native control plane (module nanoengine_b200._native._core).
//
// Parity: the reference exposes its Rust crate as dlengine._engine and re-exports it
// from dlengine/_rust/{core,config,proto,wrapper}.py (Scheduler, ScheduleResult,
// SamplingParams, RequestIn, RequestMigrate, RunnerIn, RunnerOut, StepOut, CachePlan,
// SchedulerConfig).  Runner-input derivation mirrors rust/src/proto/prepare.rs:18-190
// (cu_seqlens, slot_mapping = block*block_size+offset, padded block tables).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "scheduler.h"

namespace py = pybind11;
using namespace ne;

template <class T>
static py::array_t<T> to_np(const std::vector<T>& v) {
  py::array_t<T> a((py::ssize_t)v.size());
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), v.size() * sizeof(T));
  return a;
}

// Device-side inputs of one forward step, derived from a Batch on the worker.
static py::dict prepare_runner_inputs(const Batch& b, int block_size, int pad_blocks_to) {
  size_t n = b.num_seqs();
  std::vector<int32_t> cu_q(n + 1, 0), cu_k(n + 1, 0), ctx(n), last_idx(n);
  std::vector<int64_t> slot(b.input_ids.size());
  int max_blocks = 1, max_q = 0, max_k = 0;
  for (size_t i = 0; i < n; i++) max_blocks = std::max(max_blocks, b.block_offsets[i + 1] - b.block_offsets[i]);
  if (pad_blocks_to > 0) max_blocks = (max_blocks + pad_blocks_to - 1) / pad_blocks_to * pad_blocks_to;
  std::vector<int32_t> table(n * (size_t)max_blocks, 0);
  size_t t = 0;
  for (size_t i = 0; i < n; i++) {
    int q = b.q_lens[i], k = b.seq_lens[i];
    cu_q[i + 1] = cu_q[i] + q; cu_k[i + 1] = cu_k[i] + k; ctx[i] = k;
    max_q = std::max(max_q, q); max_k = std::max(max_k, k);
    const int32_t* bt = b.block_tables.data() + b.block_offsets[i];
    int nb = b.block_offsets[i + 1] - b.block_offsets[i];
    for (int j = 0; j < nb; j++) table[i * max_blocks + j] = bt[j];
    for (int j = 0; j < q; j++, t++) {
      int pos = b.positions[t];
      int blk = pos / block_size;
      if (blk >= nb) throw std::runtime_error("prepare: position beyond the sequence's block table");
      slot[t] = (int64_t)bt[blk] * block_size + pos % block_size;
    }
    last_idx[i] = cu_q[i + 1] - 1;
  }
  py::dict d;
  d["cu_seqlens_q"] = to_np(cu_q); d["cu_seqlens_k"] = to_np(cu_k); d["context_lens"] = to_np(ctx);
  d["slot_mapping"] = to_np(slot); d["block_tables"] = to_np(table); d["max_blocks"] = max_blocks;
  d["max_seqlen_q"] = max_q; d["max_seqlen_k"] = max_k; d["last_token_indices"] = to_np(last_idx);
  d["input_ids"] = to_np(b.input_ids); d["positions"] = to_np(b.positions);
  return d;
}

PYBIND11_MODULE(_core, m) {
  m.doc() = "nanoengine_b200 native control plane: scheduler, block manager, wire codec, metrics";
  py::register_exception<WireError>(m, "WireError", PyExc_ValueError);

  m.attr("WAITING") = (int)WAITING; m.attr("RUNNING") = (int)RUNNING; m.attr("FINISHED") = (int)FINISHED;
  m.attr("TO_BE_MIGRATED") = (int)TO_BE_MIGRATED; m.attr("PREFILLING") = (int)PREFILLING;
  m.attr("PLAN_GQA") = (uint32_t)PLAN_GQA; m.attr("PLAN_MLA") = (uint32_t)PLAN_MLA; m.attr("PLAN_GDN") = (uint32_t)PLAN_GDN;
  m.attr("PLAN_HCA") = (uint32_t)PLAN_HCA; m.attr("PLAN_CSA") = (uint32_t)PLAN_CSA;
  m.attr("PLAN_INDEXER") = (uint32_t)PLAN_INDEXER; m.attr("PLAN_HISPARSE") = (uint32_t)PLAN_HISPARSE;
  m.attr("ROUND_ROBIN") = (int)ROUND_ROBIN; m.attr("LEAST_BATCH") = (int)LEAST_BATCH;
  m.attr("LEAST_CACHE") = (int)LEAST_CACHE; m.attr("AFFINITY") = (int)AFFINITY;
  m.attr("MODE_HYBRID") = (int)MODE_HYBRID; m.attr("MODE_PREFILL") = (int)MODE_PREFILL; m.attr("MODE_DECODE") = (int)MODE_DECODE;
  m.attr("ACT_ADD") = (int)ACT_ADD; m.attr("ACT_GET_INFO") = (int)ACT_GET_INFO; m.attr("ACT_FREE") = (int)ACT_FREE;
  m.attr("ACT_STEPOUT_BATCH") = (int)ACT_STEPOUT_BATCH; m.attr("ACT_ABORT") = (int)ACT_ABORT;
  m.attr("ACT_GET_METRICS") = (int)ACT_GET_METRICS; m.attr("ACT_START_PROFILER") = (int)ACT_START_PROFILER;
  m.attr("ACT_STOP_PROFILER") = (int)ACT_STOP_PROFILER;
  m.attr("ACT_PD_OPEN") = (int)ACT_PD_OPEN; m.attr("ACT_PD_PUSH") = (int)ACT_PD_PUSH;

  py::class_<SamplingParams>(m, "SamplingParams")
      .def(py::init([](float temperature, int max_tokens, bool ignore_eos, bool return_completion_logprobs) {
             if (temperature < 0) throw std::invalid_argument("temperature must be >= 0");
             if (max_tokens < 1) throw std::invalid_argument("max_tokens must be >= 1");
             return SamplingParams{temperature, max_tokens, ignore_eos, return_completion_logprobs};
           }),
           py::arg("temperature") = 1.0f, py::arg("max_tokens") = 256, py::arg("ignore_eos") = false,
           py::arg("return_completion_logprobs") = false)
      .def_readwrite("temperature", &SamplingParams::temperature)
      .def_readwrite("max_tokens", &SamplingParams::max_tokens)
      .def_readwrite("ignore_eos", &SamplingParams::ignore_eos)
      .def_readwrite("return_completion_logprobs", &SamplingParams::return_completion_logprobs)
      .def("__repr__", [](const SamplingParams& s) {
        return "SamplingParams(temperature=" + std::to_string(s.temperature) + ", max_tokens=" + std::to_string(s.max_tokens) +
               ", ignore_eos=" + (s.ignore_eos ? "True" : "False") + ")";
      });

  py::class_<RequestIn>(m, "RequestIn")
      .def(py::init([](uint64_t seq_id, std::vector<int32_t> prompt, SamplingParams sp, uint64_t affinity, py::object vision) {
             RequestIn r; r.seq_id = seq_id; r.prompt_token_ids = std::move(prompt); r.sampling_params = sp; r.affinity_key = affinity;
             if (!vision.is_none()) r.vision_slots = vision.cast<std::vector<int32_t>>();
             return r;
           }),
           py::arg("seq_id"), py::arg("prompt_token_ids"), py::arg("sampling_params") = SamplingParams{},
           py::arg("affinity_key") = 0, py::arg("vision_slots") = py::none())
      .def_readwrite("seq_id", &RequestIn::seq_id)
      .def_readwrite("prompt_token_ids", &RequestIn::prompt_token_ids)
      .def_readwrite("sampling_params", &RequestIn::sampling_params)
      .def_readwrite("affinity_key", &RequestIn::affinity_key)
      .def_readwrite("vision_slots", &RequestIn::vision_slots)
      .def("to_bytes", [](const RequestIn& r) { return py::bytes(r.to_bytes()); })
      .def_static("from_bytes", [](const std::string& b) { return RequestIn::from_bytes(b); });

  py::class_<RequestMigrate>(m, "RequestMigrate")
      .def(py::init<>())
      .def_readwrite("seq_id", &RequestMigrate::seq_id)
      .def_readwrite("token_ids", &RequestMigrate::token_ids)
      .def_readwrite("prompt_len", &RequestMigrate::prompt_len)
      .def_readwrite("num_computed", &RequestMigrate::num_computed)
      .def_readwrite("sampling_params", &RequestMigrate::sampling_params)
      .def_readwrite("logprobs", &RequestMigrate::logprobs)
      .def_readwrite("affinity_key", &RequestMigrate::affinity_key)
      .def_readwrite("migrate_block_table", &RequestMigrate::migrate_block_table)
      .def_readwrite("migrate_dp_idx", &RequestMigrate::migrate_dp_idx)
      .def_readwrite("migrate_state_slot", &RequestMigrate::migrate_state_slot)
      .def_readwrite("migrate_handoff_slot", &RequestMigrate::migrate_handoff_slot)
      .def_readwrite("migrate_hisparse_slot", &RequestMigrate::migrate_hisparse_slot)
      .def_readwrite("migrate_engine_id", &RequestMigrate::migrate_engine_id)
      .def_readwrite("migrate_num_kvcache_blocks", &RequestMigrate::migrate_num_kvcache_blocks)
      .def_readwrite("block_size", &RequestMigrate::block_size)
      .def_property_readonly("metadata", [](const RequestMigrate& r) { return py::make_tuple(r.seq_id, r.first_token()); })
      .def("to_bytes", [](const RequestMigrate& r) { return py::bytes(r.to_bytes()); })
      .def_static("from_bytes", [](const std::string& b) { return RequestMigrate::from_bytes(b); });

  py::class_<Batch>(m, "RunnerIn")
      .def(py::init<>())
      .def_readwrite("is_prefill", &Batch::is_prefill)
      .def_readwrite("is_dummy", &Batch::is_dummy)
      .def_readwrite("any_return_logprobs", &Batch::any_return_logprobs)
      .def_readwrite("dp_idx", &Batch::dp_idx)
      .def_readwrite("step", &Batch::step)
      .def_readwrite("seq_ids", &Batch::seq_ids)
      .def_readwrite("input_ids", &Batch::input_ids)
      .def_readwrite("positions", &Batch::positions)
      .def_readwrite("q_lens", &Batch::q_lens)
      .def_readwrite("seq_lens", &Batch::seq_lens)
      .def_readwrite("block_tables", &Batch::block_tables)
      .def_readwrite("block_offsets", &Batch::block_offsets)
      .def_readwrite("temperatures", &Batch::temperatures)
      .def_readwrite("sample_mask", &Batch::sample_mask)
      .def_readwrite("state_slots", &Batch::state_slots)
      .def_readwrite("handoff_slots", &Batch::handoff_slots)
      .def_readwrite("hisparse_slots", &Batch::hisparse_slots)
      .def_readwrite("swap_in_src", &Batch::swap_in_src)
      .def_readwrite("swap_in_dst", &Batch::swap_in_dst)
      .def_readwrite("swap_out_src", &Batch::swap_out_src)
      .def_readwrite("swap_out_dst", &Batch::swap_out_dst)
      .def_property_readonly("num_seqs", &Batch::num_seqs)
      .def("prepare", &prepare_runner_inputs, py::arg("block_size"), py::arg("pad_blocks_to") = 0)
      .def("to_bytes", [](const Batch& b) { return py::bytes(b.to_bytes()); })
      .def_static("from_bytes", [](const std::string& b) { return Batch::from_bytes(b); });

  py::class_<RunResult>(m, "RunnerOut")
      .def(py::init([](std::vector<uint64_t> seq_ids, std::vector<std::vector<int32_t>> tokens, py::object logprobs) {
             RunResult r; r.seq_ids = std::move(seq_ids); r.token_offsets.push_back(0);
             for (auto& t : tokens) { r.token_ids.insert(r.token_ids.end(), t.begin(), t.end()); r.token_offsets.push_back((int)r.token_ids.size()); }
             if (r.token_offsets.size() != r.seq_ids.size() + 1) throw std::invalid_argument("RunnerOut: one token list per sequence");
             if (!logprobs.is_none()) {
               for (auto& l : logprobs.cast<std::vector<std::vector<float>>>()) r.logprobs.insert(r.logprobs.end(), l.begin(), l.end());
             }
             return r;
           }),
           py::arg("seq_ids"), py::arg("token_ids"), py::arg("logprobs") = py::none())
      .def_readwrite("seq_ids", &RunResult::seq_ids)
      .def_readwrite("flat_token_ids", &RunResult::token_ids)
      .def_readwrite("token_offsets", &RunResult::token_offsets)
      .def_readwrite("flat_logprobs", &RunResult::logprobs)
      .def_property_readonly("token_ids", [](const RunResult& r) {
        std::vector<std::vector<int32_t>> out;
        for (size_t i = 0; i + 1 < r.token_offsets.size(); i++)
          out.emplace_back(r.token_ids.begin() + r.token_offsets[i], r.token_ids.begin() + r.token_offsets[i + 1]);
        return out;
      })
      .def("to_bytes", [](const RunResult& r) { return py::bytes(r.to_bytes()); })
      .def_static("from_bytes", [](const std::string& b) { return RunResult::from_bytes(b); });

  py::class_<StepOut>(m, "StepOut")
      .def(py::init<>())
      .def_readwrite("seq_id", &StepOut::seq_id)
      .def_readwrite("token_ids", &StepOut::token_ids)
      .def_readwrite("status", &StepOut::status)
      .def_readwrite("logprobs", &StepOut::logprobs)
      .def("to_bytes", [](const StepOut& r) { return py::bytes(r.to_bytes()); })
      .def_static("from_bytes", [](const std::string& b) { return StepOut::from_bytes(b); });

  py::class_<Packet>(m, "WirePacket")
      .def(py::init([](int action, const std::string& payload) { Packet p; p.action = action; p.payload = payload; return p; }),
           py::arg("action"), py::arg("payload") = std::string())
      .def_readwrite("action", &Packet::action)
      .def_property("payload", [](const Packet& p) { return py::bytes(p.payload); },
                    [](Packet& p, const std::string& s) { p.payload = s; })
      .def("to_bytes", [](const Packet& r) { return py::bytes(r.to_bytes()); })
      .def_static("from_bytes", [](const std::string& b) { return Packet::from_bytes(b); });

  py::class_<MigrateBatch>(m, "MigrationIn")
      .def(py::init<>())
      .def_readwrite("dp_idx", &MigrateBatch::dp_idx)
      .def_readwrite("seq_ids", &MigrateBatch::seq_ids)
      .def_readwrite("local_blocks", &MigrateBatch::local_blocks)
      .def_readwrite("remote_blocks", &MigrateBatch::remote_blocks)
      .def_readwrite("block_offsets", &MigrateBatch::block_offsets)
      .def_readwrite("remote_dp_idx", &MigrateBatch::remote_dp_idx)
      .def_readwrite("local_handoff_slots", &MigrateBatch::local_handoff_slots)
      .def_readwrite("remote_handoff_slots", &MigrateBatch::remote_handoff_slots)
      .def_readwrite("remote_engine_ids", &MigrateBatch::remote_engine_ids)
      .def_readwrite("local_state_slots", &MigrateBatch::local_state_slots)
      .def_readwrite("remote_state_slots", &MigrateBatch::remote_state_slots)
      .def("to_bytes", [](const MigrateBatch& r) { return py::bytes(r.to_bytes()); })
      .def_static("from_bytes", [](const std::string& b) { return MigrateBatch::from_bytes(b); });

  py::class_<SchedulerConfig>(m, "SchedulerConfig")
      .def(py::init<>())
      .def_readwrite("num_blocks", &SchedulerConfig::num_blocks)
      .def_readwrite("num_host_blocks", &SchedulerConfig::num_host_blocks)
      .def_readwrite("block_size", &SchedulerConfig::block_size)
      .def_readwrite("max_num_seqs", &SchedulerConfig::max_num_seqs)
      .def_readwrite("max_num_batched_tokens", &SchedulerConfig::max_num_batched_tokens)
      .def_readwrite("max_model_len", &SchedulerConfig::max_model_len)
      .def_readwrite("attention_dp", &SchedulerConfig::attention_dp)
      .def_readwrite("mode", &SchedulerConfig::mode)
      .def_readwrite("num_speculative_tokens", &SchedulerConfig::num_speculative_tokens)
      .def_readwrite("enable_prefix_caching", &SchedulerConfig::enable_prefix_caching)
      .def_readwrite("enable_chunked_prefill", &SchedulerConfig::enable_chunked_prefill)
      .def_readwrite("routing", &SchedulerConfig::routing)
      .def_readwrite("cache_plan", &SchedulerConfig::cache_plan)
      .def_readwrite("num_state_slots", &SchedulerConfig::num_state_slots)
      .def_readwrite("num_handoff_slots", &SchedulerConfig::num_handoff_slots)
      .def_readwrite("num_hisparse_slots", &SchedulerConfig::num_hisparse_slots)
      .def_readwrite("swap_cooldown_steps", &SchedulerConfig::swap_cooldown_steps)
      .def_readwrite("eos_token_ids", &SchedulerConfig::eos_token_ids)
      .def_readwrite("engine_id", &SchedulerConfig::engine_id)
      .def("prefix_cache_effective", &SchedulerConfig::prefix_cache_effective);

  py::class_<ScheduleResult>(m, "ScheduleResult")
      .def_readonly("has_work", &ScheduleResult::has_work)
      .def_readonly("is_prefill", &ScheduleResult::is_prefill)
      .def_readonly("step", &ScheduleResult::step)
      .def_readonly("batches", &ScheduleResult::batches)
      .def_readonly("migrations", &ScheduleResult::migrations)
      .def_readonly("preempted", &ScheduleResult::preempted)
      .def_readonly("num_tokens", &ScheduleResult::num_tokens)
      .def_readonly("num_seqs", &ScheduleResult::num_seqs)
      .def_readonly("prefix_hit_tokens", &ScheduleResult::prefix_hit_tokens);

  py::class_<Sequence>(m, "SequenceView")
      .def_readonly("seq_id", &Sequence::seq_id)
      .def_readonly("tokens", &Sequence::tokens)
      .def_readonly("prompt_len", &Sequence::prompt_len)
      .def_readonly("num_computed", &Sequence::num_computed)
      .def_readonly("num_cached_prefix", &Sequence::num_cached_prefix)
      .def_readonly("num_checkpointed", &Sequence::num_checkpointed)
      .def_readonly("status", &Sequence::status)
      .def_readonly("dp_idx", &Sequence::dp_idx)
      .def_readonly("block_table", &Sequence::block_table)
      .def_readonly("host_blocks", &Sequence::host_blocks)
      .def_readonly("state_slot", &Sequence::state_slot)
      .def_readonly("handoff_slot", &Sequence::handoff_slot)
      .def_readonly("hisparse_slot", &Sequence::hisparse_slot)
      .def_readonly("num_preemptions", &Sequence::num_preemptions)
      .def_readonly("prefill_chunks", &Sequence::prefill_chunks)
      .def_readonly("pending_migration", &Sequence::pending_migration)
      .def_readonly("logprobs", &Sequence::logprobs);

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<const SchedulerConfig&>())
      .def_property_readonly("config", &Scheduler::config)
      .def("update_num_blocks", &Scheduler::update_num_blocks)
      .def("reset_prefix_cache", &Scheduler::reset_prefix_cache)
      .def("set_commit_log", &Scheduler::set_commit_log)
      .def("take_committed", &Scheduler::take_committed, py::arg("dp") = 0)
      .def("begin_import", &Scheduler::begin_import, py::arg("dp"), py::arg("hashes"))
      .def("finish_import", &Scheduler::finish_import, py::arg("dp"), py::arg("hashes"), py::arg("ids"), py::arg("ok") = true)
      .def("has_cached_hash", &Scheduler::has_cached_hash, py::arg("dp"), py::arg("hash"))
      .def("add_request", &Scheduler::add_request)
      .def("add_migration", &Scheduler::add_migration)
      .def("add_request_bytes", [](Scheduler& s, const std::string& b) { return s.add_request_bytes(b); })
      .def("schedule", [](Scheduler& s) { return s.schedule(); })
      .def("serialize_run_batches", [](Scheduler& s) {
        py::list out; for (auto& b : s.serialize_run_batches()) out.append(py::bytes(b)); return out; })
      .def("serialize_migrate_batches", [](Scheduler& s) {
        py::list out; for (auto& b : s.serialize_migrate_batches()) out.append(py::bytes(b)); return out; })
      .def("complete_migration", &Scheduler::complete_migration, py::arg("seq_ids"), py::arg("ok") = true)
      .def("postprocess_runner_outs", &Scheduler::postprocess, py::arg("results"), py::arg("latency_ms") = -1.0)
      .def("postprocess_runner_out_bytes", [](Scheduler& s, const std::vector<std::string>& b, double ms) { return s.postprocess_bytes(b, ms); },
           py::arg("blobs"), py::arg("latency_ms") = -1.0)
      .def("abort", &Scheduler::abort)
      .def("export_to_be_migrated", &Scheduler::export_to_be_migrated)
      .def("free_to_be_migrated", &Scheduler::free_to_be_migrated)
      .def("is_finished", &Scheduler::is_finished)
      .def("get", [](Scheduler& s, uint64_t id) -> py::object {
        const Sequence* q = s.get(id); if (!q) return py::none(); return py::cast(*q); })
      .def("num_waiting", &Scheduler::num_waiting)
      .def("num_waiting_migration", &Scheduler::num_waiting_migration)
      .def("num_running", &Scheduler::num_running, py::arg("dp") = 0)
      .def("num_prefilling", &Scheduler::num_prefilling, py::arg("dp") = 0)
      .def("num_to_be_migrated", &Scheduler::num_to_be_migrated)
      .def("num_free_blocks", &Scheduler::num_free_blocks, py::arg("dp") = 0)
      .def("num_cached_blocks", &Scheduler::num_cached_blocks, py::arg("dp") = 0)
      .def("num_free_host_blocks", &Scheduler::num_free_host_blocks, py::arg("dp") = 0)
      .def("num_free_state_slots", &Scheduler::num_free_state_slots, py::arg("dp") = 0)
      .def("num_free_handoff_slots", &Scheduler::num_free_handoff_slots, py::arg("dp") = 0)
      .def_property_readonly("step", &Scheduler::step)
      .def("metrics_prometheus", &Scheduler::metrics_prometheus)
      .def("status_line", &Scheduler::status_line, py::arg("mode") = "hybrid")
      .def("metrics_summary", [](Scheduler& s) {
        auto v = s.metrics().summary(); py::dict d;
        d["ttft_p50"] = v[0]; d["ttft_p90"] = v[1]; d["ttft_p99"] = v[2]; d["tpot_p50"] = v[3]; d["tpot_p90"] = v[4];
        d["tpot_p99"] = v[5]; d["itl_p50"] = v[6]; d["itl_p99"] = v[7];
        d["requests_total"] = s.metrics().requests_total(); d["requests_finished"] = s.metrics().requests_finished();
        d["generated_tokens"] = s.metrics().generated_tokens(); d["prompt_tokens"] = s.metrics().prompt_tokens();
        d["steps"] = s.metrics().steps();
        return d; })
      .def("record_transfer", [](Scheduler& s, double ms, uint64_t bytes) { s.metrics().on_transfer(ms, bytes); })
      .def("record_forward_bytes", [](Scheduler& s, uint64_t b) { s.metrics().on_forward_bytes(b); });

  py::class_<BlockPool>(m, "BlockPool")
      .def(py::init<int, int, bool>(), py::arg("num_blocks"), py::arg("block_size"), py::arg("prefix_cache") = true)
      .def("num_free", &BlockPool::num_free)
      .def("num_cached", &BlockPool::num_cached)
      .def("num_used", &BlockPool::num_used)
      .def("refcount", &BlockPool::refcount)
      .def("state", &BlockPool::state)
      .def("evictions", &BlockPool::evictions)
      .def("match_prefix", [](BlockPool& p, const std::vector<int32_t>& tok) {
        uint64_t h = 0; auto v = p.match_prefix(tok.data(), (int)tok.size(), &h); return py::make_tuple(v, h); })
      .def("allocate", [](BlockPool& p, int n) -> py::object {
        std::vector<int32_t> out; if (!p.allocate(n, &out)) return py::none(); return py::cast(out); })
      .def("commit", &BlockPool::commit)
      .def("begin_import", &BlockPool::begin_import)
      .def("finish_import", &BlockPool::finish_import, py::arg("hashes"), py::arg("ids"), py::arg("ok") = true)
      .def("release", &BlockPool::release);
  m.def("chain_hash", [](uint64_t prev, const std::vector<int32_t>& tok) { return chain_hash(prev, tok.data(), (int)tok.size()); });

  py::class_<SlotPool>(m, "SlotPool")
      .def(py::init<int>())
      .def("acquire", &SlotPool::acquire)
      .def("release", &SlotPool::release)
      .def("num_free", &SlotPool::num_free);

  py::class_<L3Index>(m, "L3Index")
      .def(py::init<size_t>(), py::arg("capacity") = 0)
      .def("contains", &L3Index::contains)
      .def("insert", &L3Index::insert)
      .def("lookup", &L3Index::lookup)
      .def("match", &L3Index::match)
      .def("erase", &L3Index::erase)
      .def("__len__", &L3Index::size);
}
