// Wire protocol between controller, workers and servers.
//
// A little-endian, length-prefixed binary format (magic byte + message tag +
// fields).  It carries the same information as the reference's bincode
// structs (rust/src/proto/wire.rs:10-25 WireBatch, :58-64 WireRequestIn,
// :76-106 WireRequestMigrate, rust/src/proto/metadata.rs:452-500 WireStepOut,
// WirePacket{action,payload}); byte compatibility with bincode is not a goal.
#pragma once
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "types.h"

namespace ne {

constexpr uint8_t WIRE_MAGIC = 0xB2;
enum WireTag : uint8_t {
  TAG_REQUEST_IN = 1,
  TAG_REQUEST_MIGRATE = 2,
  TAG_BATCH = 3,
  TAG_RUN_RESULT = 4,
  TAG_STEP_OUT = 5,
  TAG_PACKET = 6,
  TAG_MIGRATE_BATCH = 7,
};

// Action codes of the engine-server IPC (reference server/engine_server.py:212-415).
enum WireAction : int32_t {
  ACT_ADD = 1, ACT_GET_INFO = 2, ACT_FREE = 3, ACT_STEPOUT_BATCH = 4, ACT_ABORT = 5,
  ACT_GET_METRICS = 6, ACT_START_PROFILER = 7, ACT_STOP_PROFILER = 8,
  ACT_PD_OPEN = 9,    // decode engine -> prefill engine: map my workers' KV pools (reply: the prefill engine's info)
  ACT_PD_PUSH = 10,   // decode engine -> prefill engine: push these pages into my pools (reply: bytes queued per request)
};

struct WireError : std::runtime_error { using std::runtime_error::runtime_error; };

class ByteWriter {
 public:
  std::string buf;
  template <class T> void pod(const T& v) { buf.append(reinterpret_cast<const char*>(&v), sizeof(T)); }
  void u8(uint8_t v) { pod(v); }
  void i32(int32_t v) { pod(v); }
  void u32(uint32_t v) { pod(v); }
  void u64(uint64_t v) { pod(v); }
  void i64(int64_t v) { pod(v); }
  void f32(float v) { pod(v); }
  void f64(double v) { pod(v); }
  void boolean(bool v) { u8(v ? 1 : 0); }
  void str(const std::string& s) { u32((uint32_t)s.size()); buf.append(s); }
  template <class T> void vec(const std::vector<T>& v) {
    u32((uint32_t)v.size());
    if (!v.empty()) buf.append(reinterpret_cast<const char*>(v.data()), v.size() * sizeof(T));
  }
  void header(uint8_t tag) { u8(WIRE_MAGIC); u8(tag); }
};

class ByteReader {
 public:
  ByteReader(const char* p, size_t n) : p_(p), end_(p + n) {}
  explicit ByteReader(const std::string& s) : ByteReader(s.data(), s.size()) {}
  template <class T> T pod() {
    need(sizeof(T));
    T v; std::memcpy(&v, p_, sizeof(T)); p_ += sizeof(T); return v;
  }
  uint8_t u8() { return pod<uint8_t>(); }
  int32_t i32() { return pod<int32_t>(); }
  uint32_t u32() { return pod<uint32_t>(); }
  uint64_t u64() { return pod<uint64_t>(); }
  int64_t i64() { return pod<int64_t>(); }
  float f32() { return pod<float>(); }
  double f64() { return pod<double>(); }
  bool boolean() { return u8() != 0; }
  std::string str() {
    uint32_t n = u32(); need(n);
    std::string s(p_, n); p_ += n; return s;
  }
  template <class T> std::vector<T> vec() {
    uint32_t n = u32();
    // guard against a corrupted length field before allocating
    if ((uint64_t)n * sizeof(T) > (uint64_t)(end_ - p_)) throw WireError("wire: vector length exceeds packet");
    std::vector<T> v(n);
    if (n) { std::memcpy(v.data(), p_, n * sizeof(T)); p_ += n * sizeof(T); }
    return v;
  }
  void header(uint8_t tag) {
    if (u8() != WIRE_MAGIC) throw WireError("wire: bad magic");
    uint8_t t = u8();
    if (t != tag) throw WireError("wire: unexpected tag " + std::to_string(t) + ", want " + std::to_string(tag));
  }
  bool done() const { return p_ == end_; }
  size_t remaining() const { return (size_t)(end_ - p_); }
 private:
  void need(size_t n) { if ((size_t)(end_ - p_) < n) throw WireError("wire: truncated packet"); }
  const char* p_; const char* end_;
};

inline uint8_t peek_tag(const std::string& s) {
  if (s.size() < 2 || (uint8_t)s[0] != WIRE_MAGIC) throw WireError("wire: bad magic");
  return (uint8_t)s[1];
}

inline void write_sampling(ByteWriter& w, const SamplingParams& s) {
  w.f32(s.temperature); w.i32(s.max_tokens); w.boolean(s.ignore_eos); w.boolean(s.return_completion_logprobs);
}
inline SamplingParams read_sampling(ByteReader& r) {
  SamplingParams s; s.temperature = r.f32(); s.max_tokens = r.i32(); s.ignore_eos = r.boolean();
  s.return_completion_logprobs = r.boolean(); return s;
}

struct RequestIn {
  uint64_t seq_id = 0;
  std::vector<int32_t> prompt_token_ids;
  SamplingParams sampling_params;
  uint64_t affinity_key = 0;
  std::vector<int32_t> vision_slots;
  std::string to_bytes() const {
    ByteWriter w; w.header(TAG_REQUEST_IN); w.u64(seq_id); w.vec(prompt_token_ids);
    write_sampling(w, sampling_params); w.u64(affinity_key); w.vec(vision_slots); return w.buf;
  }
  static RequestIn from_bytes(const std::string& s) {
    ByteReader r(s); r.header(TAG_REQUEST_IN); RequestIn q; q.seq_id = r.u64();
    q.prompt_token_ids = r.vec<int32_t>(); q.sampling_params = read_sampling(r);
    q.affinity_key = r.u64(); q.vision_slots = r.vec<int32_t>();
    if (!r.done()) throw WireError("wire: trailing bytes in RequestIn");
    return q;
  }
};

// A sequence handed from a prefill engine to a decode engine.
struct RequestMigrate {
  uint64_t seq_id = 0;
  std::vector<int32_t> token_ids;      // prompt + first token(s)
  int32_t prompt_len = 0;
  int32_t num_computed = 0;            // tokens whose KV exists on the prefill side
  SamplingParams sampling_params;
  std::vector<float> logprobs;
  uint64_t affinity_key = 0;
  // prefill-side ("migrate") placement
  std::vector<int32_t> migrate_block_table;
  int32_t migrate_dp_idx = 0;
  int32_t migrate_state_slot = -1;
  int32_t migrate_handoff_slot = -1;
  int32_t migrate_hisparse_slot = -1;
  std::string migrate_engine_id;
  int32_t migrate_num_kvcache_blocks = 0;
  int32_t block_size = 64;
  std::string to_bytes() const {
    ByteWriter w; w.header(TAG_REQUEST_MIGRATE); w.u64(seq_id); w.vec(token_ids); w.i32(prompt_len);
    w.i32(num_computed); write_sampling(w, sampling_params); w.vec(logprobs); w.u64(affinity_key);
    w.vec(migrate_block_table); w.i32(migrate_dp_idx); w.i32(migrate_state_slot); w.i32(migrate_handoff_slot);
    w.i32(migrate_hisparse_slot); w.str(migrate_engine_id); w.i32(migrate_num_kvcache_blocks); w.i32(block_size);
    return w.buf;
  }
  static RequestMigrate from_bytes(const std::string& s) {
    ByteReader r(s); r.header(TAG_REQUEST_MIGRATE); RequestMigrate m; m.seq_id = r.u64();
    m.token_ids = r.vec<int32_t>(); m.prompt_len = r.i32(); m.num_computed = r.i32();
    m.sampling_params = read_sampling(r); m.logprobs = r.vec<float>(); m.affinity_key = r.u64();
    m.migrate_block_table = r.vec<int32_t>(); m.migrate_dp_idx = r.i32(); m.migrate_state_slot = r.i32();
    m.migrate_handoff_slot = r.i32(); m.migrate_hisparse_slot = r.i32(); m.migrate_engine_id = r.str();
    m.migrate_num_kvcache_blocks = r.i32(); m.block_size = r.i32();
    if (!r.done()) throw WireError("wire: trailing bytes in RequestMigrate");
    return m;
  }
  uint64_t first_token() const { return token_ids.empty() ? 0 : (uint64_t)token_ids.back(); }
};

// One worker input: everything a DP rank needs for a forward step.
struct Batch {
  bool is_prefill = false;
  bool is_dummy = false;               // idle DP rank: run a 1-token pass to keep EP collectives matched
  bool any_return_logprobs = false;
  int32_t dp_idx = 0;
  int64_t step = 0;
  std::vector<uint64_t> seq_ids;
  std::vector<int32_t> input_ids;      // flat, sequence-major
  std::vector<int32_t> positions;      // flat, absolute
  std::vector<int32_t> q_lens;         // new tokens per sequence
  std::vector<int32_t> seq_lens;       // context length per sequence after this step
  std::vector<int32_t> block_tables;   // flat
  std::vector<int32_t> block_offsets;  // size n+1, offsets into block_tables
  std::vector<float> temperatures;
  std::vector<uint8_t> sample_mask;    // 0 for a non-final prefill chunk
  std::vector<int32_t> state_slots;
  std::vector<int32_t> handoff_slots;
  std::vector<int32_t> hisparse_slots;
  std::vector<int32_t> swap_in_src, swap_in_dst, swap_out_src, swap_out_dst;  // host<->device block copies before the step
  size_t num_seqs() const { return seq_ids.size(); }
  std::string to_bytes() const {
    ByteWriter w; w.header(TAG_BATCH); w.boolean(is_prefill); w.boolean(is_dummy); w.boolean(any_return_logprobs);
    w.i32(dp_idx); w.i64(step); w.vec(seq_ids); w.vec(input_ids); w.vec(positions); w.vec(q_lens); w.vec(seq_lens);
    w.vec(block_tables); w.vec(block_offsets); w.vec(temperatures); w.vec(sample_mask); w.vec(state_slots);
    w.vec(handoff_slots); w.vec(hisparse_slots); w.vec(swap_in_src); w.vec(swap_in_dst); w.vec(swap_out_src);
    w.vec(swap_out_dst); return w.buf;
  }
  static Batch from_bytes(const std::string& s) {
    ByteReader r(s); r.header(TAG_BATCH); Batch b; b.is_prefill = r.boolean(); b.is_dummy = r.boolean();
    b.any_return_logprobs = r.boolean(); b.dp_idx = r.i32(); b.step = r.i64(); b.seq_ids = r.vec<uint64_t>();
    b.input_ids = r.vec<int32_t>(); b.positions = r.vec<int32_t>(); b.q_lens = r.vec<int32_t>();
    b.seq_lens = r.vec<int32_t>(); b.block_tables = r.vec<int32_t>(); b.block_offsets = r.vec<int32_t>();
    b.temperatures = r.vec<float>(); b.sample_mask = r.vec<uint8_t>(); b.state_slots = r.vec<int32_t>();
    b.handoff_slots = r.vec<int32_t>(); b.hisparse_slots = r.vec<int32_t>(); b.swap_in_src = r.vec<int32_t>();
    b.swap_in_dst = r.vec<int32_t>(); b.swap_out_src = r.vec<int32_t>(); b.swap_out_dst = r.vec<int32_t>();
    if (!r.done()) throw WireError("wire: trailing bytes in Batch");
    size_t n = b.seq_ids.size();
    if (b.q_lens.size() != n || b.seq_lens.size() != n || b.block_offsets.size() != n + 1)
      throw WireError("wire: inconsistent Batch field sizes");
    return b;
  }
};

// One worker output: sampled tokens per sequence (1..N+1 with speculative decoding).
struct RunResult {
  std::vector<uint64_t> seq_ids;
  std::vector<int32_t> token_ids;     // flat
  std::vector<int32_t> token_offsets; // size n+1
  std::vector<float> logprobs;        // flat, aligned with token_ids (empty when not requested)
  std::string to_bytes() const {
    ByteWriter w; w.header(TAG_RUN_RESULT); w.vec(seq_ids); w.vec(token_ids); w.vec(token_offsets); w.vec(logprobs);
    return w.buf;
  }
  static RunResult from_bytes(const std::string& s) {
    ByteReader r(s); r.header(TAG_RUN_RESULT); RunResult o; o.seq_ids = r.vec<uint64_t>();
    o.token_ids = r.vec<int32_t>(); o.token_offsets = r.vec<int32_t>(); o.logprobs = r.vec<float>();
    if (!r.done()) throw WireError("wire: trailing bytes in RunResult");
    if (o.token_offsets.size() != o.seq_ids.size() + 1) throw WireError("wire: inconsistent RunResult");
    if (!o.token_offsets.empty() && (size_t)o.token_offsets.back() != o.token_ids.size())
      throw WireError("wire: RunResult offsets do not cover token_ids");
    return o;
  }
};

struct StepOut {
  uint64_t seq_id = 0;
  std::vector<int32_t> token_ids;  // tokens appended in this step
  int32_t status = RUNNING;
  std::vector<float> logprobs;
  std::string to_bytes() const {
    ByteWriter w; w.header(TAG_STEP_OUT); w.u64(seq_id); w.vec(token_ids); w.i32(status); w.vec(logprobs); return w.buf;
  }
  static StepOut from_bytes(const std::string& s) {
    ByteReader r(s); r.header(TAG_STEP_OUT); StepOut o; o.seq_id = r.u64(); o.token_ids = r.vec<int32_t>();
    o.status = r.i32(); o.logprobs = r.vec<float>();
    if (!r.done()) throw WireError("wire: trailing bytes in StepOut");
    return o;
  }
};

struct Packet {
  int32_t action = 0;
  std::string payload;
  std::string to_bytes() const { ByteWriter w; w.header(TAG_PACKET); w.i32(action); w.str(payload); return w.buf; }
  static Packet from_bytes(const std::string& s) {
    ByteReader r(s); r.header(TAG_PACKET); Packet p; p.action = r.i32(); p.payload = r.str();
    if (!r.done()) throw WireError("wire: trailing bytes in Packet");
    return p;
  }
};

// KV migration work for one DP rank of a decode engine: which remote blocks land in which local blocks.
struct MigrateBatch {
  int32_t dp_idx = 0;
  std::vector<uint64_t> seq_ids;
  std::vector<int32_t> local_blocks, remote_blocks;  // flat, paired
  std::vector<int32_t> block_offsets;                // size n+1
  std::vector<int32_t> remote_dp_idx;
  std::vector<int32_t> local_handoff_slots, remote_handoff_slots;
  std::vector<std::string> remote_engine_ids;
  std::vector<int32_t> local_state_slots, remote_state_slots;  // per-sequence state (recurrent state, compressor carry); -1 = none
  std::string to_bytes() const {
    ByteWriter w; w.header(TAG_MIGRATE_BATCH); w.i32(dp_idx); w.vec(seq_ids); w.vec(local_blocks); w.vec(remote_blocks);
    w.vec(block_offsets); w.vec(remote_dp_idx); w.vec(local_handoff_slots); w.vec(remote_handoff_slots);
    w.u32((uint32_t)remote_engine_ids.size()); for (auto& e : remote_engine_ids) w.str(e);
    w.vec(local_state_slots); w.vec(remote_state_slots); return w.buf;
  }
  static MigrateBatch from_bytes(const std::string& s) {
    ByteReader r(s); r.header(TAG_MIGRATE_BATCH); MigrateBatch m; m.dp_idx = r.i32(); m.seq_ids = r.vec<uint64_t>();
    m.local_blocks = r.vec<int32_t>(); m.remote_blocks = r.vec<int32_t>(); m.block_offsets = r.vec<int32_t>();
    m.remote_dp_idx = r.vec<int32_t>(); m.local_handoff_slots = r.vec<int32_t>();
    m.remote_handoff_slots = r.vec<int32_t>();
    uint32_t n = r.u32(); if (n > r.remaining()) throw WireError("wire: bad engine id count");
    for (uint32_t i = 0; i < n; i++) m.remote_engine_ids.push_back(r.str());
    m.local_state_slots = r.vec<int32_t>(); m.remote_state_slots = r.vec<int32_t>();
    if (!r.done()) throw WireError("wire: trailing bytes in MigrateBatch");
    return m;
  }
};

}  // namespace ne
