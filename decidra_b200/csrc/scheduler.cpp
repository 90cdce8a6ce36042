// State-once request scheduler: one worker thread that owns the engine, a bounded queue with a
// coalescing window, exact-state grouping, a two-tier state cache (device entries, pinned-host
// second level) with byte budgets, memory-headroom checks and one out-of-memory retry per phase.
//
// Host C++ twin of juanqui/decidra's BatchHandle (src/batch.rs:265-1071): same order of decisions,
// same counters (kept as plain integers instead of Prometheus series), same failure texts. It talks
// to the engine only through a table of operations, so the same code drives the CUDA engine of this
// library or a test double. No CUDA call is made from this file.
#include <algorithm>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/decidra_b200.h"

namespace {

using Clock = std::chrono::steady_clock;

// Reply slot of one request (the oneshot channel of src/batch.rs:47).
struct Reply {
  std::mutex m;
  std::condition_variable cv;
  bool done = false;
  bool closed = false;  // the client gave up: reply.is_closed()
  int status = DCD_OK;
  std::string error;
  std::vector<float> rows;  // [questions, readout_rows]
};

struct Job {
  std::vector<uint32_t> state;
  std::vector<std::vector<uint32_t>> questions;
  uint8_t digest[32];
  Clock::time_point submitted;
  std::shared_ptr<Reply> reply;
};

struct CachedState { std::vector<uint32_t> state; uint8_t digest[32]; void* cache; size_t bytes; };
struct HostCachedState { std::vector<uint32_t> state; uint8_t digest[32]; void* cache; size_t bytes; };

enum CacheResult { GpuHit = 0, HostHit = 1, Miss = 2, Unresolved = 3 };

// MIN_PASS_RESERVE / pass_reserve / state_cache_bytes_for, src/batch.rs:198-214
constexpr size_t MIN_PASS_RESERVE = (size_t)1536 * 1024 * 1024;
size_t sat_mul(size_t a, size_t b) { return b && a > SIZE_MAX / b ? SIZE_MAX : a * b; }
size_t sat_add(size_t a, size_t b) { return a > SIZE_MAX - b ? SIZE_MAX : a + b; }
size_t default_pass_reserve(size_t state_len) { return std::max(sat_add(sat_mul(state_len, 192 * 1024), (size_t)1024 * 1024 * 1024), MIN_PASS_RESERVE); }
size_t default_state_bytes(size_t state_len) { return state_len * 65536 + (size_t)160 * 1024 * 1024; }

bool same_identity(const std::vector<uint32_t>& a, const uint8_t* da, const std::vector<uint32_t>& b, const uint8_t* db) {
  return a == b && !memcmp(da, db, 32);
}

// The engine of this library behind the operation table.
int real_rebind(void* c) { return dcd_rebind_blas((dcd_engine*)c); }
int real_capture(void* c, const uint32_t* ids, size_t n, void** out) { return dcd_capture_state((dcd_engine*)c, ids, n, nullptr, (dcd_state**)out); }
int real_readout(void* c, const void* st, const uint32_t* const* q, const size_t* lens, size_t B, float* out) {
  return dcd_readout_state_once_batch((dcd_engine*)c, (const dcd_state*)st, q, lens, B, out);
}
int real_offload(void* c, const void* st, void** out) { return dcd_state_offload((dcd_engine*)c, (const dcd_state*)st, (dcd_host_state**)out); }
int real_restore(void* c, const void* hs, void** out) { return dcd_state_restore((dcd_engine*)c, (const dcd_host_state*)hs, (dcd_state**)out); }
void real_state_free(void* c, void* st) { dcd_state_free((dcd_engine*)c, (dcd_state*)st); }
void real_host_free(void*, void* hs) { dcd_host_state_free((dcd_host_state*)hs); }
int real_trim(void* c) { return dcd_trim_pools((dcd_engine*)c); }
int real_mem(void* c, size_t* f, size_t* t) { return dcd_mem_info((dcd_engine*)c, f, t); }
const char* real_err(void* c) { return dcd_last_error((dcd_engine*)c); }
size_t real_state_bytes_for(void* c, size_t n) { return dcd_state_bytes_for((const dcd_engine*)c, n); }
size_t real_pass_reserve(void* c, size_t n) { return dcd_pass_reserve_bytes((const dcd_engine*)c, n); }
int real_capture_readout(void* c, const uint32_t* ids, size_t n, const uint32_t* const* q, const size_t* lens, size_t B, void** st, float* out) {
  return dcd_capture_and_readout((dcd_engine*)c, ids, n, q, lens, B, (dcd_state**)st, out);
}
int real_readout_multi(void* c, const void* const* states, size_t n, const uint32_t* const* q, const size_t* lens, const uint32_t* state_of, size_t B,
                       float* out) {
  return dcd_readout_multi_state_batch((dcd_engine*)c, (const dcd_state* const*)states, n, q, lens, state_of, B, out);
}

thread_local std::string g_sched_error;

}  // namespace

struct Acquired;

struct dcd_ticket {
  std::shared_ptr<Reply> reply;
  size_t questions = 0;
};

struct dcd_scheduler {
  dcd_sched_engine_ops ops{};
  dcd_sched_options opt{};
  // queue (mpsc::sync_channel + the semaphore of queue slots)
  std::mutex qm;
  std::condition_variable q_nonempty, slot_free;
  std::deque<Job> queue;
  size_t slots_in_use = 0;
  bool closed = false;
  // state of the worker thread only
  std::vector<CachedState> cache;
  std::vector<HostCachedState> host_cache;
  std::thread worker;
  // counters
  mutable std::mutex sm;
  dcd_sched_stats st{};

  std::string engine_error() const { const char* s = ops.last_error ? ops.last_error(ops.ctx) : nullptr; return s ? s : ""; }
  template <typename F> void stat(F&& f) { std::lock_guard<std::mutex> g(sm); f(st); }

  size_t state_bytes_for(size_t n) const { return ops.state_bytes_for ? ops.state_bytes_for(ops.ctx, n) : default_state_bytes(n); }
  size_t pass_reserve(size_t n) const { return ops.pass_reserve ? ops.pass_reserve(ops.ctx, n) : default_pass_reserve(n); }

  void release_slot() {
    { std::lock_guard<std::mutex> g(qm); if (slots_in_use) --slots_in_use; }
    slot_free.notify_one();
  }
  void finish(Job& job, int status, const std::string& error, const float* rows, size_t n) {
    bool was_closed;
    {
      std::lock_guard<std::mutex> g(job.reply->m);
      was_closed = job.reply->closed;
      job.reply->status = status;
      job.reply->error = error;
      if (rows) job.reply->rows.assign(rows, rows + n);
      job.reply->done = true;
    }
    job.reply->cv.notify_all();
    if (status == DCD_OK && was_closed) stat([](dcd_sched_stats& s) { s.cancelled_at_reply += 1; });
    release_slot();
  }
  void fail_all(std::vector<Job>& jobs, const std::string& message) {
    size_t q = 0;
    for (Job& j : jobs) q += j.questions.size();
    stat([&](dcd_sched_stats& s) { s.questions_failed += q; });
    for (Job& j : jobs) finish(j, DCD_E_FAILED, message, nullptr, 0);
  }
  void refresh_gauges() {
    size_t gb = 0, hb = 0;
    for (auto& c : cache) gb += c.bytes;
    for (auto& c : host_cache) hb += c.bytes;
    stat([&](dcd_sched_stats& s) { s.gpu_entries = cache.size(); s.host_entries = host_cache.size(); s.gpu_bytes = gb; s.host_bytes = hb; });
  }

  struct GroupJobs { std::vector<uint32_t> state; uint8_t digest[32]; std::vector<Job> jobs; };
  void host_insert(CachedState entry, size_t bytes);
  bool acquire(const std::vector<uint32_t>& state, const uint8_t* digest, std::vector<Job>& jobs, struct Acquired* out, bool may_retry = false,
               int* retry = nullptr, bool count_lookup = true);
  void release(struct Acquired& a);
  bool pass_one(struct Acquired& a, std::vector<Job>& jobs);
  void run_groups_together(std::vector<GroupJobs>& groups);
  bool ensure_headroom(size_t need, const char* context, std::string* message);
  void run_group(const std::vector<uint32_t>& state, const uint8_t* digest, std::vector<Job>& jobs);
  CacheResult run_group_inner(const std::vector<uint32_t>& state, const uint8_t* digest, std::vector<Job>& jobs, bool* ok);
  void run_jobs(std::vector<Job>& jobs);
  void loop();
};

// host_insert, src/batch.rs:1026-1071: offload to pinned host memory, then evict the oldest host entries
// while the host tier is over its budget. The device copy is freed either way.
void dcd_scheduler::host_insert(CachedState entry, size_t bytes) {
  void* host = nullptr;
  const int rc = ops.offload(ops.ctx, entry.cache, &host);
  ops.state_free(ops.ctx, entry.cache);
  if (rc != DCD_OK) {
    stat([](dcd_sched_stats& s) { s.fail_state_offload += 1; s.evict_gpu_offload_failed += 1; });
    return;
  }
  stat([&](dcd_sched_stats& s) { s.offloads += 1; s.offload_bytes += bytes; });
  HostCachedState h;
  h.state = std::move(entry.state);
  memcpy(h.digest, entry.digest, 32);
  h.cache = host;
  h.bytes = bytes;
  host_cache.push_back(std::move(h));
  size_t total = 0;
  for (auto& c : host_cache) total += c.bytes;
  while (total > (size_t)opt.host_state_cache_bytes && !host_cache.empty()) {
    total -= std::min(total, host_cache.front().bytes);
    ops.host_free(ops.ctx, host_cache.front().cache);
    host_cache.erase(host_cache.begin());
    stat([](dcd_sched_stats& s) { s.evict_host_budget += 1; });
  }
}

// ensure_headroom, src/batch.rs:957-1024: trim the pools only when short, then move the oldest device entries
// to the host tier until `need` bytes are free.
bool dcd_scheduler::ensure_headroom(size_t need, const char* context, std::string* message) {
  size_t free_b = 0, total_b = 0;
  auto query = [&]() -> bool {
    if (ops.mem_info(ops.ctx, &free_b, &total_b) != DCD_OK) { *message = "failed to query GPU memory: " + engine_error(); return false; }
    stat([&](dcd_sched_stats& s) { s.gpu_free_bytes = free_b; });
    return true;
  };
  if (!query()) return false;
  if (free_b < need) {
    if (ops.trim_pools(ops.ctx) != DCD_OK) { *message = "failed to trim scratch pools: " + engine_error(); return false; }
    if (!query()) return false;
  }
  while (free_b < need && !cache.empty()) {
    CachedState entry = std::move(cache.front());
    cache.erase(cache.begin());
    const size_t bytes = entry.bytes;
    host_insert(std::move(entry), bytes);
    if (ops.trim_pools(ops.ctx) != DCD_OK) { *message = "failed to trim after state offload: " + engine_error(); return false; }
    if (!query()) return false;
  }
  if (free_b < need) {
    char buf[160];
    snprintf(buf, sizeof buf, "insufficient GPU memory for %s: %zu MiB free, %zu MiB required", context, free_b / (1024 * 1024), need / (1024 * 1024));
    *message = buf;
    return false;
  }
  return true;
}

// run_group_inner, src/batch.rs:571-955 (text states only: no vision encode), in three steps so that several groups can
// share one question pass: acquire (cache lookup, headroom, restore or capture), the pass, release (reply bookkeeping
// done by the caller; the state goes back to a cache tier).
struct Acquired {
  CachedState entry;
  CacheResult result = Unresolved;
  bool from_host = false;
  bool answered = false;  // a miss served by the one-pass call: the jobs have their rows already
  size_t entry_bytes = 0, pass_need = 0;
};

// may_retry: other groups' states are in hand (moved out of the device tier, so ensure_headroom cannot offload them). A memory
// failure then does not fail the requests: *retry is set and the caller runs and releases what it holds, then acquires again.
// (*retry = 2 when the lookup counters were already updated: the second attempt passes count_lookup = false.)
bool dcd_scheduler::acquire(const std::vector<uint32_t>& state, const uint8_t* digest, std::vector<Job>& jobs, Acquired* out, bool may_retry,
                            int* retry, bool count_lookup) {
  if (retry) *retry = 0;
  auto oom_text = [&]() { return engine_error().find("out of memory") != std::string::npos; };
  auto find_gpu = [&]() { for (size_t i = 0; i < cache.size(); ++i) if (same_identity(state, digest, cache[i].state, cache[i].digest)) return (int)i; return -1; };
  auto find_host = [&]() { for (size_t i = 0; i < host_cache.size(); ++i) if (same_identity(state, digest, host_cache[i].state, host_cache[i].digest)) return (int)i; return -1; };
  int cached = find_gpu();
  int host_cached = cached < 0 ? find_host() : -1;
  const size_t entry_bytes = state_bytes_for(state.size());
  out->entry_bytes = entry_bytes;
  if (!opt.pin_cache) {
    // keep the hit, evict older entries down to the limits the new entry will need
    CachedState preserved{};
    const bool have = cached >= 0;
    if (have) { preserved = std::move(cache[cached]); cache.erase(cache.begin() + cached); }
    const size_t max_len = (size_t)opt.state_cache_entries > (have ? 1u : 0u) ? (size_t)opt.state_cache_entries - (have ? 1 : 0) : 0;
    const size_t byte_budget = (size_t)opt.state_cache_bytes > entry_bytes ? (size_t)opt.state_cache_bytes - entry_bytes : 0;
    size_t bytes = 0;
    for (auto& c : cache) bytes += c.bytes;
    while (!cache.empty() && (cache.size() > max_len || bytes > byte_budget)) {
      const bool by_entries = cache.size() > max_len;
      bytes -= std::min(bytes, cache.front().bytes);
      ops.state_free(ops.ctx, cache.front().cache);
      cache.erase(cache.begin());
      stat([&](dcd_sched_stats& s) { (by_entries ? s.evict_gpu_entry_limit : s.evict_gpu_byte_limit) += 1; });
    }
    if (have) { cache.push_back(std::move(preserved)); cached = (int)cache.size() - 1; }
  }
  const size_t pass_need = pass_reserve(state.size());
  out->pass_need = pass_need;
  const size_t state_need = sat_add(entry_bytes, pass_need);
  std::string message;
  if (cached < 0) {
    if (!ensure_headroom(state_need, "state capture/restore", &message)) {
      if (may_retry) { *retry = 1; return false; }
      stat([](dcd_sched_stats& s) { s.fail_headroom += 1; });
      refresh_gauges();
      fail_all(jobs, message);
      out->result = Unresolved;
      return false;
    }
    if (host_cached >= 0) host_cached = find_host();  // offloading others may have evicted it from the host tier
    refresh_gauges();
  }
  const CacheResult result = cached >= 0 ? GpuHit : host_cached >= 0 ? HostHit : Miss;
  out->result = result;
  if (count_lookup) stat([&](dcd_sched_stats& s) {
    (result == GpuHit ? s.requests_gpu_hit : result == HostHit ? s.requests_host_hit : s.requests_miss) += jobs.size();
    if (result != Miss) s.reused_tokens += (uint64_t)state.size() * jobs.size();
  });
  out->from_host = host_cached >= 0;
  CachedState& entry = out->entry;
  if (cached >= 0) {
    entry = std::move(cache[cached]);
    cache.erase(cache.begin() + cached);
  } else if (host_cached >= 0) {
    void* restored = nullptr;
    if (ops.restore(ops.ctx, host_cache[host_cached].cache, &restored) != DCD_OK) {
      if (may_retry && oom_text()) { *retry = 2; return false; }
      stat([](dcd_sched_stats& s) { s.fail_state_restore += 1; });
      fail_all(jobs, "state restore failed: " + engine_error());
      return false;
    }
    stat([&](dcd_sched_stats& s) { s.restores += 1; s.restore_bytes += entry_bytes; });
    entry.state = state;
    memcpy(entry.digest, digest, 32);
    entry.cache = restored;
    entry.bytes = entry_bytes;
  } else {
    void* captured = nullptr;
    if (opt.cold_one_pass && ops.capture_readout && !may_retry) {
      // the state and its questions in one engine call (headroom for both was secured above); anything but success or a memory
      // failure that a retry cures leaves the group to the two steps below, whose failure texts are the reference's
      std::vector<const uint32_t*> qptr;
      std::vector<size_t> qlen;
      size_t question_tokens = 0;
      for (Job& j : jobs)
        for (auto& q : j.questions) { qptr.push_back(q.data()); qlen.push_back(q.size()); question_tokens += q.size(); }
      const size_t R = (size_t)ops.readout_rows;
      std::vector<float> rows(qptr.size() * R);
      int rc1 = ops.capture_readout(ops.ctx, state.data(), state.size(), qptr.data(), qlen.data(), qptr.size(), &captured, rows.data());
      if (rc1 != DCD_OK && oom_text()) {
        stat([](dcd_sched_stats& s) { s.oom_retry_capture += 1; });
        ops.trim_pools(ops.ctx);
        std::string ignored;
        ensure_headroom(state_need, "state capture retry", &ignored);
        captured = nullptr;
        rc1 = ops.capture_readout(ops.ctx, state.data(), state.size(), qptr.data(), qlen.data(), qptr.size(), &captured, rows.data());
      }
      if (rc1 == DCD_OK) {
        stat([&](dcd_sched_stats& s) {
          s.captures += 1; s.state_tokens += state.size(); s.question_tokens += question_tokens; s.questions_answered += qptr.size();
        });
        size_t at = 0;
        for (Job& j : jobs) {
          finish(j, DCD_OK, "", rows.data() + at * R, j.questions.size() * R);
          at += j.questions.size();
        }
        entry.state = state;
        memcpy(entry.digest, digest, 32);
        entry.cache = captured;
        entry.bytes = entry_bytes;
        out->answered = true;
        return true;
      }
      captured = nullptr;
    }
    int rc = ops.capture_state(ops.ctx, state.data(), state.size(), &captured);
    if (rc != DCD_OK && engine_error().find("out of memory") != std::string::npos) {
      // a long state can exceed the estimate: drop what can be dropped and retry once
      stat([](dcd_sched_stats& s) { s.oom_retry_capture += 1; });
      ops.trim_pools(ops.ctx);
      std::string ignored;
      ensure_headroom(state_need, "state capture retry", &ignored);
      rc = ops.capture_state(ops.ctx, state.data(), state.size(), &captured);
    }
    if (rc != DCD_OK) {
      if (may_retry && oom_text()) { *retry = 2; return false; }
      stat([](dcd_sched_stats& s) { s.fail_state_capture += 1; });
      fail_all(jobs, "state capture failed: " + engine_error());
      return false;
    }
    stat([&](dcd_sched_stats& s) { s.captures += 1; s.state_tokens += state.size(); });
    entry.state = state;
    memcpy(entry.digest, digest, 32);
    entry.cache = captured;
    entry.bytes = entry_bytes;
  }
  return true;
}

// The state goes back to the device tier if it has room, else (unless it came from there) to the host tier.
void dcd_scheduler::release(Acquired& a) {
  CachedState& entry = a.entry;
  bool kept = false;
  if (opt.state_cache_entries > 0) {
    size_t cached_bytes = 0;
    for (auto& c : cache) cached_bytes += c.bytes;
    const bool has_room = cache.size() < (size_t)opt.state_cache_entries && sat_add(cached_bytes, entry.bytes) <= (size_t)opt.state_cache_bytes;
    if (has_room) {
      if (a.from_host) {
        for (size_t i = 0; i < host_cache.size();) {
          if (same_identity(entry.state, entry.digest, host_cache[i].state, host_cache[i].digest)) { ops.host_free(ops.ctx, host_cache[i].cache); host_cache.erase(host_cache.begin() + i); }
          else ++i;
        }
      }
      cache.push_back(std::move(entry));
      kept = true;
    } else if (!a.from_host && opt.host_state_cache_bytes > 0) {
      host_insert(std::move(entry), a.entry_bytes);  // frees the device copy
      kept = true;
    }
  }
  if (!kept) ops.state_free(ops.ctx, entry.cache);
}

CacheResult dcd_scheduler::run_group_inner(const std::vector<uint32_t>& state, const uint8_t* digest, std::vector<Job>& jobs, bool* ok) {
  *ok = false;
  Acquired a;
  if (!acquire(state, digest, jobs, &a)) return a.result;
  if (a.answered) { release(a); *ok = true; }
  else *ok = pass_one(a, jobs);
  return a.result;
}

// The question pass of one group whose state is in hand, then the replies and the state's way back to a cache tier.
bool dcd_scheduler::pass_one(Acquired& a, std::vector<Job>& jobs) {
  std::vector<const uint32_t*> qptr;
  std::vector<size_t> qlen;
  std::vector<std::pair<size_t, size_t>> ranges;
  size_t question_tokens = 0;
  for (Job& j : jobs) {
    const size_t start = qptr.size();
    for (auto& q : j.questions) { qptr.push_back(q.data()); qlen.push_back(q.size()); question_tokens += q.size(); }
    ranges.emplace_back(start, qptr.size());
  }
  std::string message;
  if (!ensure_headroom(a.pass_need, "question pass", &message)) {
    stat([](dcd_sched_stats& s) { s.fail_headroom += 1; });
    ops.state_free(ops.ctx, a.entry.cache);
    refresh_gauges();
    fail_all(jobs, message);
    return false;
  }
  refresh_gauges();
  const size_t R = (size_t)ops.readout_rows;
  std::vector<float> rows(qptr.size() * R);
  int rc = ops.readout(ops.ctx, a.entry.cache, qptr.data(), qlen.data(), qptr.size(), rows.data());
  if (rc != DCD_OK && engine_error().find("out of memory") != std::string::npos) {
    stat([](dcd_sched_stats& s) { s.oom_retry_question += 1; });
    ops.trim_pools(ops.ctx);
    std::string ignored;
    ensure_headroom(a.pass_need, "question pass retry", &ignored);
    rc = ops.readout(ops.ctx, a.entry.cache, qptr.data(), qlen.data(), qptr.size(), rows.data());
  }
  if (rc != DCD_OK) {
    stat([](dcd_sched_stats& s) { s.fail_question_pass += 1; });
    const std::string msg = "state-once question pass failed: " + engine_error();
    ops.state_free(ops.ctx, a.entry.cache);
    fail_all(jobs, msg);
    return false;
  }
  stat([&](dcd_sched_stats& s) { s.question_tokens += question_tokens; s.questions_answered += qptr.size(); });
  for (size_t i = 0; i < jobs.size(); ++i)
    finish(jobs[i], DCD_OK, "", rows.data() + ranges[i].first * R, (ranges[i].second - ranges[i].first) * R);
  release(a);
  return true;
}

void dcd_scheduler::run_group(const std::vector<uint32_t>& state, const uint8_t* digest, std::vector<Job>& jobs) {
  size_t questions = 0;
  for (Job& j : jobs) questions += j.questions.size();
  const size_t n = jobs.size();
  stat([&](dcd_sched_stats& s) { s.waiting -= std::min<uint64_t>(s.waiting, n); s.running += n; s.group_requests += n; s.group_questions += questions; });
  bool ok = false;
  const CacheResult r = run_group_inner(state, digest, jobs, &ok);
  (void)r;
  stat([&](dcd_sched_stats& s) { s.running -= std::min<uint64_t>(s.running, n); (ok ? s.groups_success : s.groups_failed) += 1; });
  refresh_gauges();
}

// Several groups, one question pass (cross_state_pass; not in the reference, which lists it as future work): every group's
// state is acquired as above, then ONE pass answers all their questions. Groups whose state cannot be acquired fail alone.
// If the combined pass is refused or fails, the groups fall back to one pass each; if memory runs short while states are being
// collected, the groups in hand are served and released first and the group that did not fit is acquired again on its own. So a
// request never fares worse than in the reference's order of work.
void dcd_scheduler::run_groups_together(std::vector<GroupJobs>& groups) {
  struct Live { GroupJobs* g; Acquired a; };
  std::vector<Live> live;
  // The question pass(es) of the groups in hand, their replies, and their states' way back to the cache tiers.
  auto run_live = [&]() {
    if (live.empty()) return;
    std::vector<const void*> states;
    std::vector<const uint32_t*> qptr;
    std::vector<size_t> qlen;
    std::vector<uint32_t> state_of;
    size_t question_tokens = 0, pass_need = 0;
    for (size_t k = 0; k < live.size(); ++k) {
      states.push_back(live[k].a.entry.cache);
      pass_need = std::max(pass_need, live[k].a.pass_need);
      for (Job& j : live[k].g->jobs)
        for (auto& q : j.questions) { qptr.push_back(q.data()); qlen.push_back(q.size()); state_of.push_back((uint32_t)k); question_tokens += q.size(); }
    }
    const size_t R = (size_t)ops.readout_rows;
    std::vector<float> rows(qptr.size() * R);
    bool together = live.size() > 1;
    std::string message;
    if (together && !ensure_headroom(pass_need, "question pass", &message)) together = false;
    if (together && ops.readout_multi(ops.ctx, states.data(), states.size(), qptr.data(), qlen.data(), state_of.data(), qptr.size(), rows.data()) != DCD_OK)
      together = false;
    if (together) {
      stat([&](dcd_sched_stats& s) { s.cross_state_passes += 1; s.question_tokens += question_tokens; s.questions_answered += qptr.size(); });
      size_t at = 0;
      for (Live& l : live) {
        for (Job& j : l.g->jobs) {
          finish(j, DCD_OK, "", rows.data() + at * R, j.questions.size() * R);
          at += j.questions.size();
        }
        release(l.a);
        const size_t n = l.g->jobs.size();
        stat([&](dcd_sched_stats& s) { s.running -= std::min<uint64_t>(s.running, n); s.groups_success += 1; });
      }
    } else {
      // one pass per group, with the states already in hand
      for (Live& l : live) {
        const size_t n = l.g->jobs.size();
        if (live.size() > 1) stat([&](dcd_sched_stats& s) { s.requests_fallback += n; });
        const bool ok = pass_one(l.a, l.g->jobs);
        stat([&](dcd_sched_stats& s) { s.running -= std::min<uint64_t>(s.running, n); (ok ? s.groups_success : s.groups_failed) += 1; });
      }
    }
    live.clear();
  };
  for (GroupJobs& g : groups) {
    size_t questions = 0;
    for (Job& j : g.jobs) questions += j.questions.size();
    const size_t n = g.jobs.size();
    stat([&](dcd_sched_stats& s) { s.waiting -= std::min<uint64_t>(s.waiting, n); s.running += n; s.group_requests += n; s.group_questions += questions; });
    Live l{&g, {}};
    int retry = 0;
    bool got = acquire(g.state, g.digest, g.jobs, &l.a, !live.empty(), &retry);
    if (!got && retry) {
      // Memory ran short while other groups' states are in hand, where nothing can offload them: serve and release those first
      // (the reference's one-group-at-a-time order would have done exactly that), then acquire this group with the tiers intact.
      run_live();
      l.a = Acquired{};
      got = acquire(g.state, g.digest, g.jobs, &l.a, false, nullptr, retry != 2);
    }
    if (got) live.push_back(std::move(l));
    else stat([&](dcd_sched_stats& s) { s.running -= std::min<uint64_t>(s.running, n); s.groups_failed += 1; });
  }
  run_live();
  refresh_gauges();
}

// run_jobs, src/batch.rs:429-504: drop requests whose client left, group by exact state identity in first-seen
// order, optionally run the cheapest group first (groups older than 500 ms jump the queue).
void dcd_scheduler::run_jobs(std::vector<Job>& jobs) {
  std::vector<Job> live;
  for (Job& j : jobs) {
    bool closed;
    { std::lock_guard<std::mutex> g(j.reply->m); closed = j.reply->closed; }
    if (closed) {
      stat([&](dcd_sched_stats& s) { s.waiting -= std::min<uint64_t>(s.waiting, 1); s.cancelled_queued += 1; s.questions_cancelled += j.questions.size(); });
      { std::lock_guard<std::mutex> g(j.reply->m); j.reply->status = DCD_E_FAILED; j.reply->error = "cancelled"; j.reply->done = true; }
      j.reply->cv.notify_all();
      release_slot();
    } else {
      live.push_back(std::move(j));
    }
  }
  if (live.empty()) return;
  using Group = GroupJobs;
  std::vector<Group> groups;
  for (Job& j : live) {
    Group* hit = nullptr;
    for (Group& g : groups) if (same_identity(g.state, g.digest, j.state, j.digest)) { hit = &g; break; }
    if (!hit) { groups.emplace_back(); hit = &groups.back(); hit->state = j.state; memcpy(hit->digest, j.digest, 32); }
    hit->jobs.push_back(std::move(j));
  }
  if (opt.sched_priority) {
    const auto now = Clock::now();
    auto key = [&](const Group& g) -> size_t {
      size_t age_ms = 0, q = 0;
      for (const Job& j : g.jobs) {
        age_ms = std::max<size_t>(age_ms, (size_t)std::chrono::duration_cast<std::chrono::milliseconds>(now - j.submitted).count());
        for (auto& x : j.questions) q += x.size();
      }
      if (age_ms >= 500) return 0;
      bool cached = false;
      for (auto& c : cache) cached |= same_identity(g.state, g.digest, c.state, c.digest);
      return (cached ? 0 : g.state.size()) + q;
    };
    std::vector<std::pair<size_t, size_t>> order;
    for (size_t i = 0; i < groups.size(); ++i) order.emplace_back(key(groups[i]), i);
    std::stable_sort(order.begin(), order.end(), [](auto& a, auto& b) { return a.first < b.first; });
    std::vector<Group> sorted;
    for (auto& o : order) sorted.push_back(std::move(groups[o.second]));
    groups = std::move(sorted);
  }
  if (opt.cross_state_pass && ops.readout_multi && groups.size() > 1) { run_groups_together(groups); return; }
  for (Group& g : groups) run_group(g.state, g.digest, g.jobs);
}

// The worker loop of BatchHandle::spawn, src/batch.rs:289-353: block for the first request, then keep
// collecting until the request budget, the row budget (sum of questions) or the window is exhausted.
void dcd_scheduler::loop() {
  if (ops.rebind_blas) ops.rebind_blas(ops.ctx);
  for (;;) {
    std::vector<Job> jobs;
    bool stop = false;
    {
      std::unique_lock<std::mutex> g(qm);
      q_nonempty.wait(g, [&] { return closed || !queue.empty(); });
      if (queue.empty()) break;  // closed and drained
      jobs.push_back(std::move(queue.front()));
      queue.pop_front();
      size_t rows = std::max<size_t>(1, jobs[0].questions.size());
      const auto deadline = Clock::now() + std::chrono::microseconds(opt.batch_window_us);
      while (jobs.size() < (size_t)opt.batch_requests && rows < (size_t)opt.batch_rows) {
        if (Clock::now() >= deadline) break;  // checked first: a zero window takes exactly one request per pass
        if (queue.empty()) {
          if (closed) { stop = true; break; }
          if (!q_nonempty.wait_until(g, deadline, [&] { return closed || !queue.empty(); })) break;
          if (queue.empty()) { stop = true; break; }  // closed: flush what was collected, then stop
        }
        rows = sat_add(rows, std::max<size_t>(1, queue.front().questions.size()));
        jobs.push_back(std::move(queue.front()));
        queue.pop_front();
      }
      stat([&](dcd_sched_stats& s) { s.channel -= std::min<uint64_t>(s.channel, jobs.size()); });
    }
    run_jobs(jobs);
    if (stop) {
      std::lock_guard<std::mutex> g(qm);
      if (queue.empty()) break;
    }
  }
  for (auto& c : cache) ops.state_free(ops.ctx, c.cache);
  for (auto& c : host_cache) ops.host_free(ops.ctx, c.cache);
  cache.clear();
  host_cache.clear();
  stat([](dcd_sched_stats& s) { s.worker_alive = 0; s.waiting = s.running = s.channel = 0; });
  refresh_gauges();
}

extern "C" {

const char* dcd_scheduler_last_error(void) { return g_sched_error.c_str(); }

void dcd_sched_default_options(dcd_sched_options* o) {
  if (!o) return;
  memset(o, 0, sizeof *o);
  o->max_queue = 64;            // DEFAULT_MAX_QUEUE .. DEFAULT_HOST_STATE_CACHE_BYTES, src/config.rs:16-28
  o->batch_requests = 32;
  o->batch_rows = 32;
  o->batch_window_us = 2000;
  o->state_cache_entries = 16;
  o->state_cache_bytes = (int64_t)5 * 1024 * 1024 * 1024;
  o->host_state_cache_bytes = (int64_t)8 * 1024 * 1024 * 1024;
  o->pin_cache = 1;
  o->sched_priority = 0;
  o->submit_timeout_us = 0;
}

int dcd_scheduler_create_with_ops(const dcd_sched_engine_ops* ops, const dcd_sched_options* opt, dcd_scheduler** out) {
  if (!out) return DCD_E_INVALID;
  *out = nullptr;
  if (!ops || !ops->capture_state || !ops->readout || !ops->offload || !ops->restore || !ops->state_free || !ops->host_free || !ops->trim_pools ||
      !ops->mem_info || ops->readout_rows <= 0) {
    g_sched_error = "incomplete engine operation table";
    return DCD_E_INVALID;
  }
  dcd_sched_options o;
  if (opt) o = *opt; else dcd_sched_default_options(&o);
  // the checks of Config::from_env, src/config.rs:131-152
  if (o.max_queue <= 0) { g_sched_error = "max_queue must be at least 1"; return DCD_E_INVALID; }
  if (o.batch_requests <= 0) { g_sched_error = "batch_requests must be at least 1"; return DCD_E_INVALID; }
  if (o.batch_rows <= 0) { g_sched_error = "batch_rows must be at least 1"; return DCD_E_INVALID; }
  if (o.batch_window_us < 0 || o.batch_window_us > 50000) { g_sched_error = "batch_window_us must be at most 50000"; return DCD_E_INVALID; }
  if (o.state_cache_entries < 0 || o.state_cache_bytes < 0 || o.host_state_cache_bytes < 0) { g_sched_error = "negative cache limit"; return DCD_E_INVALID; }
  dcd_scheduler* s = new dcd_scheduler();
  s->ops = *ops;
  s->opt = o;
  s->st.worker_alive = 1;
  s->cache.reserve((size_t)o.state_cache_entries);
  s->host_cache.reserve((size_t)o.state_cache_entries);
  s->worker = std::thread([s] { s->loop(); });
  *out = s;
  return DCD_OK;
}

int dcd_scheduler_create(dcd_engine* e, const dcd_sched_options* opt, dcd_scheduler** out) {
  if (!out) return DCD_E_INVALID;
  *out = nullptr;
  if (!e) { g_sched_error = "null engine"; return DCD_E_INVALID; }
  dcd_info info;
  if (dcd_engine_info(e, &info) != DCD_OK) { g_sched_error = "engine info failed"; return DCD_E_INVALID; }
  dcd_sched_engine_ops ops{};
  ops.ctx = e;
  ops.readout_rows = info.readout_rows;
  ops.rebind_blas = real_rebind;
  ops.capture_state = real_capture;
  ops.readout = real_readout;
  ops.offload = real_offload;
  ops.restore = real_restore;
  ops.state_free = real_state_free;
  ops.host_free = real_host_free;
  ops.trim_pools = real_trim;
  ops.mem_info = real_mem;
  ops.last_error = real_err;
  ops.readout_multi = real_readout_multi;
  ops.state_bytes_for = real_state_bytes_for;
  ops.pass_reserve = real_pass_reserve;
  ops.capture_readout = real_capture_readout;
  return dcd_scheduler_create_with_ops(&ops, opt, out);
}

void dcd_scheduler_destroy(dcd_scheduler* s) {
  if (!s) return;
  { std::lock_guard<std::mutex> g(s->qm); s->closed = true; }
  s->q_nonempty.notify_all();
  s->slot_free.notify_all();
  if (s->worker.joinable()) s->worker.join();
  delete s;
}

int dcd_scheduler_submit(dcd_scheduler* s, const uint32_t* state, size_t n_state, const uint32_t* const* questions, const size_t* lens, size_t B,
                         const uint8_t* digest, dcd_ticket** out) {
  if (!out) return DCD_E_INVALID;
  *out = nullptr;
  if (!s || (!state && n_state) || (B && (!questions || !lens))) { g_sched_error = "bad argument"; return DCD_E_INVALID; }
  Job job;
  job.state.assign(state, state + n_state);
  job.questions.resize(B);
  for (size_t i = 0; i < B; ++i) job.questions[i].assign(questions[i], questions[i] + lens[i]);
  if (digest) memcpy(job.digest, digest, 32); else memset(job.digest, 0, 32);
  job.reply = std::make_shared<Reply>();
  {
    std::unique_lock<std::mutex> g(s->qm);
    auto can = [&] { return s->closed || s->slots_in_use < (size_t)s->opt.max_queue; };
    if (s->opt.submit_timeout_us > 0) {
      if (!s->slot_free.wait_for(g, std::chrono::microseconds(s->opt.submit_timeout_us), can)) {
        s->stat([](dcd_sched_stats& st) { st.reject_queue_full += 1; });
        g_sched_error = "d3-turbo queue is full; retry shortly";
        return DCD_E_OVERLOADED;
      }
    } else {
      s->slot_free.wait(g, can);
    }
    if (s->closed) {
      s->stat([](dcd_sched_stats& st) { st.reject_worker_stopped += 1; });
      g_sched_error = "d3-turbo CUDA worker stopped";
      return DCD_E_FAILED;
    }
    if (s->queue.size() >= (size_t)s->opt.max_queue) {
      s->stat([](dcd_sched_stats& st) { st.reject_queue_full += 1; });
      g_sched_error = "d3-turbo queue is full; retry shortly";
      return DCD_E_OVERLOADED;
    }
    ++s->slots_in_use;
    job.submitted = Clock::now();
    dcd_ticket* t = new dcd_ticket();
    t->reply = job.reply;
    t->questions = B;
    s->stat([](dcd_sched_stats& st) { st.waiting += 1; st.channel += 1; st.submitted += 1; });
    s->queue.push_back(std::move(job));
    *out = t;
  }
  s->q_nonempty.notify_one();
  return DCD_OK;
}

int dcd_ticket_wait(dcd_ticket* t, float* logits_out, size_t capacity) {
  if (!t) return DCD_E_INVALID;
  std::unique_lock<std::mutex> g(t->reply->m);
  t->reply->cv.wait(g, [&] { return t->reply->done; });
  if (t->reply->status != DCD_OK) return t->reply->status;
  if (t->reply->rows.size() > capacity || (!logits_out && !t->reply->rows.empty())) return DCD_E_INVALID;
  if (!t->reply->rows.empty()) memcpy(logits_out, t->reply->rows.data(), t->reply->rows.size() * sizeof(float));
  return DCD_OK;
}
int dcd_ticket_done(const dcd_ticket* t) {
  if (!t) return 0;
  std::lock_guard<std::mutex> g(t->reply->m);
  return t->reply->done ? 1 : 0;
}
const char* dcd_ticket_error(const dcd_ticket* t) { return t ? t->reply->error.c_str() : ""; }
void dcd_ticket_cancel(dcd_ticket* t) {
  if (!t) return;
  std::lock_guard<std::mutex> g(t->reply->m);
  t->reply->closed = true;
}
void dcd_ticket_free(dcd_ticket* t) {
  if (!t) return;
  { std::lock_guard<std::mutex> g(t->reply->m); t->reply->closed = true; }
  delete t;
}

int dcd_scheduler_stats(const dcd_scheduler* s, dcd_sched_stats* out) {
  if (!s || !out) return DCD_E_INVALID;
  std::lock_guard<std::mutex> g(s->sm);
  *out = s->st;
  return DCD_OK;
}

}  // extern "C"
