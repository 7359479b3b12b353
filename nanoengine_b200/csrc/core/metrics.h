// Engine metrics: per-sequence TTFT / TPOT / ITL, step records, Prometheus text.
//
// Parity: reference rust/src/metrics/manager.rs:610-830 (exposition with the
// `dlengine_*` metric names and TTFT/TPOT histograms), rust/src/metrics/sequence.rs,
// rust/src/scheduler/observability.rs:9-238 (step reports, percentiles).
// The metric names are kept so existing dashboards keep working.
#pragma once
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <deque>
#include <string>
#include <vector>

namespace ne {

inline double now_seconds() {
  using namespace std::chrono;
  return duration<double>(steady_clock::now().time_since_epoch()).count();
}

struct Histogram {
  std::vector<double> bounds;
  std::vector<uint64_t> counts;  // bounds.size()+1, last = +Inf
  double sum = 0; uint64_t n = 0;
  explicit Histogram(std::vector<double> b = {}) : bounds(std::move(b)), counts(bounds.size() + 1, 0) {}
  void observe(double v) {
    size_t i = std::lower_bound(bounds.begin(), bounds.end(), v) - bounds.begin();
    counts[i]++; sum += v; n++;
  }
  void render(std::string& out, const char* name) const {
    char buf[256]; uint64_t cum = 0;
    for (size_t i = 0; i < bounds.size(); i++) {
      cum += counts[i];
      snprintf(buf, sizeof buf, "%s_bucket{le=\"%g\"} %llu\n", name, bounds[i], (unsigned long long)cum); out += buf;
    }
    cum += counts.back();
    snprintf(buf, sizeof buf, "%s_bucket{le=\"+Inf\"} %llu\n%s_sum %.9g\n%s_count %llu\n", name,
             (unsigned long long)cum, name, sum, name, (unsigned long long)n);
    out += buf;
  }
};

inline double percentile(std::vector<double> v, double p) {
  if (v.empty()) return 0.0;
  std::sort(v.begin(), v.end());
  double idx = p * (double)(v.size() - 1);
  size_t lo = (size_t)idx; size_t hi = std::min(lo + 1, v.size() - 1);
  return v[lo] + (v[hi] - v[lo]) * (idx - (double)lo);
}

struct StepRecord {
  int64_t step = 0; bool is_prefill = false; int32_t num_seqs = 0; int32_t num_tokens = 0;
  double latency_ms = 0; int32_t prefix_hit_tokens = 0; int32_t preempted = 0;
};

class Metrics {
 public:
  Metrics()
      : ttft_({0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1, 2.5, 5, 10, 30, 60, 120, 300}),
        tpot_({0.002, 0.005, 0.01, 0.02, 0.03, 0.05, 0.075, 0.1, 0.2, 0.5, 1}) { t_start_ = now_seconds(); }

  void on_request() { requests_total_++; }
  void on_finish(double ttft, double tpot, int n_out, const std::vector<double>& itl) {
    requests_finished_++;
    if (ttft > 0) { ttft_.observe(ttft); ttft_last_ = ttft; keep(ttft_samples_, ttft); }
    if (n_out > 1 && tpot > 0) { tpot_.observe(tpot); tpot_last_ = tpot; keep(tpot_samples_, tpot); }
    for (double d : itl) keep(itl_samples_, d);
  }
  void on_abort() { requests_aborted_++; }
  void on_tokens(uint64_t prompt, uint64_t generated) { prompt_tokens_ += prompt; generated_tokens_ += generated; }
  void on_step(const StepRecord& r) {
    steps_++; step_latency_last_ = r.latency_ms; step_latency_sum_ += r.latency_ms;
    recent_.push_back(r); if (recent_.size() > 1024) recent_.pop_front();
    preemptions_ += (uint64_t)r.preempted;
  }
  void on_transfer(double ms, uint64_t bytes) { transfer_latency_ms_ = ms; transfer_bytes_ += bytes; }
  void on_forward_bytes(uint64_t b) { forward_bytes_ += b; }

  struct Gauges {
    std::vector<int32_t> running_per_dp, waiting_blocks_per_dp, used_blocks_per_dp, total_blocks_per_dp;
    std::vector<double> prefix_hit_rate_per_dp;
    std::vector<int32_t> used_host_blocks_per_dp;        // host tier of the prefix cache (empty when there is none)
    int32_t total_host_blocks_per_dp = 0;
    int32_t used_hisparse_slots = 0, total_hisparse_slots = 0;      // hot / cold cache tier: sequences holding a hot buffer
    int32_t waiting = 0, waiting_migration = 0; double prefix_hit_rate = 0;
  };

  std::string prometheus(const Gauges& g) const {
    std::string o; char buf[320];
    double up = now_seconds() - t_start_;
    auto line = [&](const char* name, const char* type, double v) {
      snprintf(buf, sizeof buf, "# TYPE %s %s\n%s %.9g\n", name, type, name, v); o += buf;
    };
    line("dlengine_up", "gauge", 1);
    line("dlengine_uptime_seconds", "gauge", up);
    o += "# TYPE dlengine_requests gauge\n";
    snprintf(buf, sizeof buf, "dlengine_requests{state=\"total\"} %llu\ndlengine_requests{state=\"finished\"} %llu\n"
             "dlengine_requests{state=\"aborted\"} %llu\ndlengine_requests{state=\"waiting\"} %d\n"
             "dlengine_requests{state=\"waiting_migration\"} %d\n",
             (unsigned long long)requests_total_, (unsigned long long)requests_finished_,
             (unsigned long long)requests_aborted_, g.waiting, g.waiting_migration); o += buf;
    o += "# TYPE dlengine_tokens counter\n";
    snprintf(buf, sizeof buf, "dlengine_tokens{kind=\"prompt\"} %llu\ndlengine_tokens{kind=\"generated\"} %llu\n",
             (unsigned long long)prompt_tokens_, (unsigned long long)generated_tokens_); o += buf;
    line("dlengine_throughput_tokens_per_second", "gauge", recent_throughput());
    line("dlengine_avg_throughput_tokens_per_second", "gauge", up > 0 ? (double)generated_tokens_ / up : 0);
    line("dlengine_step_latency_ms", "gauge", step_latency_last_);
    line("dlengine_step_count", "counter", (double)steps_);
    line("dlengine_forward_bytes", "counter", (double)forward_bytes_);
    line("dlengine_transfer_latency_ms", "gauge", transfer_latency_ms_);
    line("dlengine_preemptions", "counter", (double)preemptions_);
    line("dlengine_prefix_cache_hit_rate", "gauge", g.prefix_hit_rate);
    o += "# TYPE dlengine_prefix_cache_hit_rate_per_dp gauge\n";
    for (size_t i = 0; i < g.prefix_hit_rate_per_dp.size(); i++) {
      snprintf(buf, sizeof buf, "dlengine_prefix_cache_hit_rate_per_dp{dp=\"%zu\"} %.9g\n", i, g.prefix_hit_rate_per_dp[i]); o += buf;
    }
    o += "# TYPE dlengine_ttft_seconds histogram\n"; ttft_.render(o, "dlengine_ttft_seconds");
    line("dlengine_ttft_seconds_avg", "gauge", ttft_.n ? ttft_.sum / (double)ttft_.n : 0);
    line("dlengine_ttft_ms_last", "gauge", ttft_last_ * 1e3);
    o += "# TYPE dlengine_tpot_seconds histogram\n"; tpot_.render(o, "dlengine_tpot_seconds");
    line("dlengine_tpot_seconds_avg", "gauge", tpot_.n ? tpot_.sum / (double)tpot_.n : 0);
    line("dlengine_tpot_ms_last", "gauge", tpot_last_ * 1e3);
    o += "# TYPE dlengine_running_requests_per_dp gauge\n";
    for (size_t i = 0; i < g.running_per_dp.size(); i++) {
      snprintf(buf, sizeof buf, "dlengine_running_requests_per_dp{dp=\"%zu\"} %d\n", i, g.running_per_dp[i]); o += buf;
    }
    o += "# TYPE dlengine_waiting_blocks gauge\n";
    for (size_t i = 0; i < g.waiting_blocks_per_dp.size(); i++) {
      snprintf(buf, sizeof buf, "dlengine_waiting_blocks{dp=\"%zu\"} %d\n", i, g.waiting_blocks_per_dp[i]); o += buf;
    }
    o += "# TYPE dlengine_kv_blocks gauge\n";
    for (size_t i = 0; i < g.used_blocks_per_dp.size(); i++) {
      snprintf(buf, sizeof buf, "dlengine_kv_blocks{dp=\"%zu\",state=\"used\"} %d\ndlengine_kv_blocks{dp=\"%zu\",state=\"total\"} %d\n",
               i, g.used_blocks_per_dp[i], i, g.total_blocks_per_dp[i]); o += buf;
    }
    if (g.total_host_blocks_per_dp > 0) {
      o += "# TYPE dlengine_host_kv_blocks gauge\n";
      for (size_t i = 0; i < g.used_host_blocks_per_dp.size(); i++) {
        snprintf(buf, sizeof buf, "dlengine_host_kv_blocks{dp=\"%zu\",state=\"used\"} %d\ndlengine_host_kv_blocks{dp=\"%zu\",state=\"total\"} %d\n",
                 i, g.used_host_blocks_per_dp[i], i, g.total_host_blocks_per_dp); o += buf;
      }
    }
    if (g.total_hisparse_slots > 0) {
      o += "# TYPE dlengine_hisparse_slots gauge\n";
      snprintf(buf, sizeof buf, "dlengine_hisparse_slots{state=\"used\"} %d\ndlengine_hisparse_slots{state=\"total\"} %d\n",
               g.used_hisparse_slots, g.total_hisparse_slots); o += buf;
    }
    return o;
  }

  // One line for the engine's periodic log: running / waiting / migrating requests, cache occupancy per tier, recent prefill and
  // decode throughput, finished requests.  Parity: reference rust/src/metrics/manager.rs:500-610 (the periodic status line).
  std::string status_line(const Gauges& g, const std::string& engine_id, const std::string& mode) const {
    std::string run, kv, host;
    for (size_t i = 0; i < g.running_per_dp.size(); i++) run += (i ? "," : "") + std::to_string(g.running_per_dp[i]);
    for (size_t i = 0; i < g.used_blocks_per_dp.size(); i++)
      kv += (i ? "," : "") + std::to_string(g.used_blocks_per_dp[i]) + "/" + std::to_string(g.total_blocks_per_dp[i]);
    for (size_t i = 0; i < g.used_host_blocks_per_dp.size(); i++) host += (i ? "," : "") + std::to_string(g.used_host_blocks_per_dp[i]);
    double pf_ms = 0, pf_tok = 0, dc_ms = 0, dc_tok = 0;
    int k = 0;
    for (auto it = recent_.rbegin(); it != recent_.rend() && k < 256; ++it, ++k) {
      if (it->is_prefill) { pf_ms += it->latency_ms; pf_tok += it->num_tokens; } else { dc_ms += it->latency_ms; dc_tok += it->num_tokens; }
    }
    char buf[640];
    std::string o;
    snprintf(buf, sizeof buf, "[engine %s %s] run=%s wait=%d mig=%d | kv=%s blk", engine_id.c_str(), mode.c_str(), run.c_str(),
             g.waiting - g.waiting_migration, g.waiting_migration, kv.c_str());
    o = buf;
    if (g.total_host_blocks_per_dp > 0) { snprintf(buf, sizeof buf, " host=%s/%d blk", host.c_str(), g.total_host_blocks_per_dp); o += buf; }
    if (g.total_hisparse_slots > 0) { snprintf(buf, sizeof buf, " hisparse_hot=%d/%d slot", g.used_hisparse_slots, g.total_hisparse_slots); o += buf; }
    snprintf(buf, sizeof buf, " | tput pf=%.0f dec=%.0f tok/s (%.0fs) | prefix hit %.2f | done=%llu", pf_ms > 0 ? pf_tok / (pf_ms * 1e-3) : 0.0,
             dc_ms > 0 ? dc_tok / (dc_ms * 1e-3) : 0.0, now_seconds() - t_start_, g.prefix_hit_rate, (unsigned long long)requests_finished_);
    return o + buf;
  }

  // Percentile summary used by the final report and the serving benchmark.
  std::vector<double> summary() const {
    return {percentile(ttft_samples_, 0.5), percentile(ttft_samples_, 0.9), percentile(ttft_samples_, 0.99),
            percentile(tpot_samples_, 0.5), percentile(tpot_samples_, 0.9), percentile(tpot_samples_, 0.99),
            percentile(itl_samples_, 0.5), percentile(itl_samples_, 0.99)};
  }
  uint64_t requests_total() const { return requests_total_; }
  uint64_t requests_finished() const { return requests_finished_; }
  uint64_t generated_tokens() const { return generated_tokens_; }
  uint64_t prompt_tokens() const { return prompt_tokens_; }
  uint64_t steps() const { return steps_; }
  const std::deque<StepRecord>& recent() const { return recent_; }

 private:
  static void keep(std::vector<double>& v, double x) { if (v.size() < (1u << 20)) v.push_back(x); }
  double recent_throughput() const {
    double ms = 0; double tok = 0; int k = 0;
    for (auto it = recent_.rbegin(); it != recent_.rend() && k < 32; ++it, ++k) { ms += it->latency_ms; tok += it->num_tokens; }
    return ms > 0 ? tok / (ms * 1e-3) : 0;
  }
  Histogram ttft_, tpot_;
  double t_start_ = 0, ttft_last_ = 0, tpot_last_ = 0, step_latency_last_ = 0, step_latency_sum_ = 0, transfer_latency_ms_ = 0;
  uint64_t requests_total_ = 0, requests_finished_ = 0, requests_aborted_ = 0, prompt_tokens_ = 0, generated_tokens_ = 0;
  uint64_t steps_ = 0, forward_bytes_ = 0, transfer_bytes_ = 0, preemptions_ = 0;
  std::deque<StepRecord> recent_;
  std::vector<double> ttft_samples_, tpot_samples_, itl_samples_;
};

}  // namespace ne
