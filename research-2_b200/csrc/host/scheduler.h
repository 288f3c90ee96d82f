// The scheduler: admits requests, cuts prompts into portions under a token budget, gives every
// running request its next row, finishes requests and frees their pages.
//
// Policy, as the reference's core decides it (kelpie-core/src/scheduler.zig):
//   * two queues: running (admission order) and waiting (first in, first out; a preempted
//     request goes back to the FRONT)                                          :152-166,1304-1313
//   * per step a token budget and an entry cap; running first, then admission, and no
//     admission in a step that preempted anyone                                :413-452
//   * a portion that does not finish the history ends on a page boundary; one that finishes
//     it may end anywhere; a budget below one page yields no portion           :955-981
//   * admission takes the head of the waiting queue only, and only if its first portion's
//     pages plus a reserve for the runners are free                            :808-844
//   * when a runner's next row needs pages that are not free, the YOUNGEST runner not yet
//     planned gives up all its pages and is recomputed later from its whole history
//                                                                              :785-794,1304-1313
//   * a plan that schedules nothing, preempts nobody and still has work is a stall :454-467
//   * only an entry that reaches the end of its history keeps its sampled token :609-626
//   * `chunk_size` caps a portion that does not finish a history, whatever the token budget
//     has left (0: the budget alone decides); the reference reaches this only through its
//     token budget, which also caps the decoded tokens that share the step
//   * with several cache groups every count of pages is made group by group (each group has a
//     pool of its own), and portions end on a multiple of every group's page size
#pragma once

#include <cstdint>
#include <deque>
#include <string>
#include <vector>

#include "cache_manager.h"
#include "engine_abi.h"

namespace r2 {

constexpr int32_t MAX_STOP_TOKENS = 8;
constexpr float SAMPLING_EPS = 1e-6f;

enum RequestState : int32_t {
  REQ_FREE = 0,
  REQ_WAITING = 1,
  REQ_RUNNING = 2,
  REQ_FINISHED_EOS = 3,
  REQ_FINISHED_LENGTH = 4,
  REQ_CANCELLED = 5,
};

enum SchedStatus : int32_t {
  SCHED_OK = 0,
  SCHED_FULL = -1,             // no free request slot
  SCHED_TOO_LONG = -2,         // prompt + max_new_tokens > max_seq_len
  SCHED_BAD_ARGS = -3,         // empty prompt, bad temperature, too many stop tokens, bad token id
  SCHED_EXCEEDS_KV_POOL = -5,  // could never fit, even alone
  SCHED_BAD_TOP_K = -7,
  SCHED_BAD_ID = -8,
  SCHED_NO_PLAN = -9,          // commit without a plan, or plan while one is outstanding
  SCHED_BAD_COMMIT = -10,      // wrong count or a token id outside the vocabulary; nothing applied
};

enum EntryKind : int32_t { ENTRY_PREFILL = 0, ENTRY_DECODE = 1 };
enum Order : int32_t { ORDER_RUNNING_FIRST = 0, ORDER_WAITING_FIRST = 1 };

struct SchedulerConfig {
  int32_t max_requests;
  int32_t max_seq_len;
  int32_t max_batch_tokens;
  int32_t max_batch_reqs;
  int32_t order;
  float reserve_ratio;
  int32_t eos_token;  // -1: none
  int32_t vocab_size;
  int32_t chunk_size;  // 0: none; else the most rows of a portion that does not finish its history
};

struct Request {
  int32_t id = 0;
  int32_t state = REQ_FREE;
  std::vector<int32_t> tokens;  // prompt, then generated
  int32_t n_prompt = 0;
  int32_t n_computed = 0;
  int32_t max_new = 0;
  float temperature = 1.f;
  int32_t top_k = 1;
  uint32_t key0 = 0, key1 = 0;
  int32_t stops[MAX_STOP_TOKENS] = {};
  int32_t n_stops = 0;
  int32_t n_polled = 0;
  int32_t n_preempted = 0;
  int32_t n_chunks = 0;
  int32_t peak_pages = 0;  // the most pages it held at one time, summed over groups
  int64_t t_arrival_ns = 0, t_first_sched_ns = 0, t_first_token_ns = 0, t_last_token_ns = 0, t_finish_ns = 0;
  int64_t first_step = 0, last_step = 0;
  bool in_plan = false;
  bool cancel_pending = false;
  int32_t n_generated() const { return int32_t(tokens.size()) - n_prompt; }
};

struct Stall {
  int32_t stalled = 0;
  int32_t req_id = -1;
  int32_t n_work = 0;
  int32_t need_pages = 0;  // of the group that is shortest of pages
  int32_t free_pages = 0;
  int32_t group = 0;
};

// A request's life in numbers, complete once it has finished or was cancelled; times in
// nanoseconds of a monotonic clock (kelpie-core/src/events.zig:39-55).
struct RequestEvent {
  int64_t t_arrival_ns = 0, t_first_sched_ns = 0, t_first_token_ns = 0, t_last_token_ns = 0, t_finish_ns = 0;
  int64_t first_step = 0, last_step = 0;
  int32_t request_id = 0, n_prompt = 0, n_generated = 0, max_new = 0;
  int32_t n_preempted = 0, n_chunks = 0, state = 0, peak_pages = 0;
};

struct StepEvent {
  int64_t step = 0;
  int32_t n_entries = 0, n_tokens = 0, n_prefill_rows = 0, n_decode = 0;
  int32_t n_admitted = 0, n_preempted = 0, n_finished = 0;
  int32_t n_running = 0, n_waiting = 0, kv_free = 0;
  int64_t t_plan_ns = 0, t_commit_ns = 0;
};

struct Plan {
  std::vector<int32_t> req, start, rows, emits, kind;  // per entry; decode entries first
  std::vector<int32_t> input_ids;                       // per row
  std::vector<float> temperature;                       // per entry
  std::vector<int32_t> top_k, sample_pos;
  std::vector<uint32_t> key0, key1;
  int32_t n_tokens = 0;
  int32_t n_entries() const { return int32_t(req.size()); }
  void clear();
};

struct SchedEntry {
  int32_t req, start, rows, emits, kind;
};

class Scheduler {
 public:
  Scheduler(const SchedulerConfig& cfg, std::vector<GroupSpec> groups);

  int32_t submit(const int32_t* prompt, int32_t n, int32_t max_new, float temperature, int32_t top_k,
                 uint64_t seed, const int32_t* stops, int32_t n_stops);
  int32_t cancel(int32_t id);
  int32_t plan();    // SCHED_OK; the plan is read through current_plan()
  int32_t commit(const int32_t* tokens, int32_t n);
  // Copies tokens not yet polled. The first poll that reports a finished request frees its slot.
  int32_t poll(int32_t id, int32_t* out, int32_t cap, int32_t* finished, int32_t* state);

  const Plan& current_plan() const { return plan_; }
  // The outstanding plan written as a step batch into the caller's arrays (see R2StepBatch).
  int32_t fill_step_batch(const R2StepBatch& out) const;
  const Stall& stall() const { return stall_; }
  const StepEvent& last_event() const { return event_; }
  CacheManager& cache() { return cache_; }
  const CacheManager& cache() const { return cache_; }
  const SchedulerConfig& config() const { return cfg_; }
  int32_t n_running() const { return int32_t(running_.size()); }
  int32_t n_waiting() const { return int32_t(waiting_.size()); }
  bool has_work() const { return !running_.empty() || !waiting_.empty(); }
  const Request* request(int32_t id) const;
  // SCHED_OK and the record of a request that is queued, running, or finished and not yet polled away.
  int32_t request_event(int32_t id, RequestEvent* out) const;
  // Records of requests whose slots have been released (finished and polled to the end, or
  // cancelled), oldest first; at most the last 4096 are kept. Returns how many were copied out.
  int32_t drain_request_events(RequestEvent* out, int32_t cap);

  int32_t set_max_batch_tokens(int32_t v);
  int32_t set_max_batch_reqs(int32_t v);
  int32_t set_order(int32_t v);
  int32_t set_reserve_ratio(float v);
  int32_t set_chunk_size(int32_t v);
  // Portions end on multiples of this: the least common multiple of the groups' page sizes.
  int32_t grain() const { return grain_; }
  int32_t min_free() const;  // the free pages of the group that has fewest

 private:
  int32_t chunk_for(const Request& r, int32_t budget) const;
  int32_t reserve_pages(const Request& r) const;
  bool plan_running(int32_t& budget, size_t n_unplanned);
  void plan_waiting(int32_t& budget);
  void schedule(Request& r, int32_t n_work);
  void preempt(int32_t id);
  void finish(Request& r, int32_t state);
  void emit_plan();
  void detect_stall(bool preempted);
  void release_slot(Request& r);
  void note_pages(Request& r);

  SchedulerConfig cfg_;
  int32_t create_max_batch_tokens_, create_max_batch_reqs_;
  CacheManager cache_;
  int32_t grain_ = 1;
  std::vector<Request> reqs_;
  std::vector<int32_t> running_;
  std::deque<int32_t> waiting_;
  std::vector<SchedEntry> sched_;
  Plan plan_;
  bool outstanding_ = false;
  Stall stall_;
  StepEvent event_;
  std::deque<RequestEvent> done_events_;
  int64_t step_ = 0;
  size_t rr_ = 0;
};

}  // namespace r2
