#include "scheduler.h"

#include <algorithm>
#include <chrono>
#include <cmath>

namespace r2 {

static int64_t now_ns() {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(
             std::chrono::steady_clock::now().time_since_epoch())
      .count();
}

static inline int32_t ceil_div(int32_t a, int32_t b) { return (a + b - 1) / b; }
static int32_t gcd(int32_t a, int32_t b) { return b == 0 ? a : gcd(b, a % b); }

void Plan::clear() {
  req.clear(); start.clear(); rows.clear(); emits.clear(); kind.clear();
  input_ids.clear(); temperature.clear(); top_k.clear(); sample_pos.clear();
  key0.clear(); key1.clear();
  n_tokens = 0;
}

Scheduler::Scheduler(const SchedulerConfig& cfg, std::vector<GroupSpec> groups)
    : cfg_(cfg), create_max_batch_tokens_(cfg.max_batch_tokens), create_max_batch_reqs_(cfg.max_batch_reqs),
      cache_(std::move(groups), cfg.max_requests, cfg.max_seq_len), reqs_(size_t(cfg.max_requests)) {
  for (int32_t i = 0; i < cfg.max_requests; ++i) reqs_[i].id = i;
  for (int32_t g = 0; g < cache_.n_groups(); ++g) {
    int32_t ps = cache_.group(g).page_size;
    grain_ = grain_ / gcd(grain_, ps) * ps;
  }
}

int32_t Scheduler::min_free() const {
  int32_t least = cache_.n_free(0);
  for (int32_t g = 1; g < cache_.n_groups(); ++g) least = std::min(least, cache_.n_free(g));
  return least;
}

void Scheduler::note_pages(Request& r) {
  int32_t held = 0;
  for (int32_t g = 0; g < cache_.n_groups(); ++g) held += cache_.pages_held(r.id, g);
  r.peak_pages = std::max(r.peak_pages, held);
}

int32_t Scheduler::request_event(int32_t id, RequestEvent* out) const {
  const Request* r = request(id);
  if (r == nullptr) return SCHED_BAD_ID;
  *out = RequestEvent();
  out->t_arrival_ns = r->t_arrival_ns;
  out->t_first_sched_ns = r->t_first_sched_ns;
  out->t_first_token_ns = r->t_first_token_ns;
  out->t_last_token_ns = r->t_last_token_ns;
  out->t_finish_ns = r->t_finish_ns;
  out->first_step = r->first_step;
  out->last_step = r->last_step;
  out->request_id = r->id;
  out->n_prompt = r->n_prompt;
  out->n_generated = r->n_generated();
  out->max_new = r->max_new;
  out->n_preempted = r->n_preempted;
  out->n_chunks = r->n_chunks;
  out->state = r->state;
  out->peak_pages = r->peak_pages;
  return SCHED_OK;
}

const Request* Scheduler::request(int32_t id) const {
  if (id < 0 || id >= cfg_.max_requests || reqs_[id].state == REQ_FREE) return nullptr;
  return &reqs_[id];
}

int32_t Scheduler::submit(const int32_t* prompt, int32_t n, int32_t max_new, float temperature,
                          int32_t top_k, uint64_t seed, const int32_t* stops, int32_t n_stops) {
  if (top_k < 0 || top_k > cfg_.vocab_size) return SCHED_BAD_TOP_K;
  if (n <= 0 || max_new < 0 || !std::isfinite(temperature) || temperature < 0.f) return SCHED_BAD_ARGS;
  if (n_stops < 0 || n_stops > MAX_STOP_TOKENS) return SCHED_BAD_ARGS;
  for (int32_t i = 0; i < n; ++i) {
    if (prompt[i] < 0 || prompt[i] >= cfg_.vocab_size) return SCHED_BAD_ARGS;
  }
  const int32_t n_new = std::max(1, max_new);  // max_new_tokens 0 still yields one token
  if (int64_t(n) + n_new > cfg_.max_seq_len) return SCHED_TOO_LONG;
  for (int32_t g = 0; g < cache_.n_groups(); ++g) {
    // the largest portion under the knobs as they stand; one that is raised after this check can lead a
    // window group into a stall, which plan() then reports (kelpie-core/src/scheduler.zig:1040-1044)
    int32_t most = cfg_.max_batch_tokens;
    if (cfg_.chunk_size > 0) most = std::min(most, cfg_.chunk_size);
    if (cache_.worst_pages(g, n + n_new - 1, most, grain()) > cache_.group(g).num_pages) {
      return SCHED_EXCEEDS_KV_POOL;
    }
  }
  Request* slot = nullptr;
  for (Request& r : reqs_) {
    if (r.state == REQ_FREE) { slot = &r; break; }
  }
  if (slot == nullptr) return SCHED_FULL;
  Request& r = *slot;
  r.tokens.assign(prompt, prompt + n);
  r.n_prompt = n;
  r.n_computed = 0;
  r.max_new = max_new;
  if (temperature < SAMPLING_EPS) {  // the T=0 rule: greedy is (T=1, top_k=1)
    r.temperature = 1.f;
    r.top_k = 1;
  } else {
    r.temperature = temperature;
    r.top_k = top_k;
  }
  r.key0 = uint32_t(seed & 0xffffffffull);
  r.key1 = uint32_t(seed >> 32);
  r.n_stops = n_stops;
  for (int32_t i = 0; i < n_stops; ++i) r.stops[i] = stops[i];
  r.n_polled = 0;
  r.n_preempted = 0;
  r.n_chunks = 0;
  r.peak_pages = 0;
  r.t_arrival_ns = now_ns();
  r.t_first_sched_ns = r.t_first_token_ns = r.t_last_token_ns = r.t_finish_ns = 0;
  r.first_step = r.last_step = 0;
  r.in_plan = false;
  r.cancel_pending = false;
  r.state = REQ_WAITING;
  waiting_.push_back(r.id);
  return r.id;
}

int32_t Scheduler::drain_request_events(RequestEvent* out, int32_t cap) {
  int32_t n = 0;
  while (n < cap && !done_events_.empty()) {
    out[n++] = done_events_.front();
    done_events_.pop_front();
  }
  return n;
}

void Scheduler::release_slot(Request& r) {
  RequestEvent e;
  if (request_event(r.id, &e) == SCHED_OK) {
    if (e.t_finish_ns == 0) {  // cancelled: it ends now
      e.t_finish_ns = now_ns();
      e.state = REQ_CANCELLED;
    }
    if (done_events_.size() >= 4096) done_events_.pop_front();
    done_events_.push_back(e);
  }
  r.state = REQ_FREE;
  r.tokens.clear();
  r.in_plan = false;
  r.cancel_pending = false;
}

int32_t Scheduler::cancel(int32_t id) {
  if (id < 0 || id >= cfg_.max_requests) return SCHED_BAD_ID;
  Request& r = reqs_[id];
  switch (r.state) {
    case REQ_FREE:
      return SCHED_BAD_ID;
    case REQ_WAITING:
      waiting_.erase(std::find(waiting_.begin(), waiting_.end(), id));
      release_slot(r);
      return SCHED_OK;
    case REQ_RUNNING:
      if (outstanding_ && r.in_plan) {  // the plan in flight names it: commit lets it go
        r.cancel_pending = true;
        return SCHED_OK;
      }
      cache_.close(id);
      running_.erase(std::find(running_.begin(), running_.end(), id));
      release_slot(r);
      return SCHED_OK;
    default:  // finished and not yet polled
      release_slot(r);
      return SCHED_OK;
  }
}

int32_t Scheduler::chunk_for(const Request& r, int32_t budget) const {
  int32_t remaining = int32_t(r.tokens.size()) - r.n_computed;
  int32_t n_work = std::min(remaining, budget);
  if (cfg_.chunk_size > 0 && remaining > 1) n_work = std::min(n_work, cfg_.chunk_size);
  if (n_work < remaining) {  // does not finish the history: end on a page boundary
    int32_t g = grain();
    int32_t end = (r.n_computed + n_work) / g * g;
    n_work = end > r.n_computed ? end - r.n_computed : 0;
  }
  return n_work;
}

int32_t Scheduler::reserve_pages(const Request& r) const {
  if (cfg_.reserve_ratio <= 0.f) return 0;
  return int32_t(std::ceil(double(cfg_.reserve_ratio) * std::max(1, r.max_new)));  // in tokens; pages group by group
}

void Scheduler::schedule(Request& r, int32_t n_work) {
  cache_.reserve(r.id, r.n_computed, r.n_computed + n_work);
  SchedEntry e;
  e.req = r.id;
  e.start = r.n_computed;
  e.rows = n_work;
  e.emits = (r.n_computed + n_work == int32_t(r.tokens.size())) ? 1 : 0;
  bool newest = n_work == 1 && r.n_computed >= r.n_prompt && e.emits;
  e.kind = newest ? ENTRY_DECODE : ENTRY_PREFILL;
  sched_.push_back(e);
  r.in_plan = true;
  r.n_chunks += 1;
  r.last_step = step_;
  if (r.t_first_sched_ns == 0) {
    r.t_first_sched_ns = now_ns();
    r.first_step = step_;
  }
  note_pages(r);
}

void Scheduler::preempt(int32_t id) {
  Request& r = reqs_[id];
  cache_.close(id);
  r.n_computed = 0;
  r.state = REQ_WAITING;
  r.n_preempted += 1;
  running_.erase(std::find(running_.begin(), running_.end(), id));
  waiting_.push_front(id);
  event_.n_preempted += 1;
}

bool Scheduler::plan_running(int32_t& budget, size_t n_unplanned) {
  std::vector<int32_t> order(n_unplanned);
  size_t first = n_unplanned ? rr_ % n_unplanned : 0;
  for (size_t k = 0; k < n_unplanned; ++k) order[k] = running_[(first + k) % n_unplanned];
  rr_ = 0;
  size_t n_old = n_unplanned;
  bool preempted = false;
  for (size_t i = 0; i < n_old; ++i) {
    Request& r = reqs_[order[i]];
    if (budget == 0 || int32_t(sched_.size()) == cfg_.max_batch_reqs) {
      // No room in this batch: it keeps its pages and goes first next step.
      rr_ = size_t(std::find(running_.begin(), running_.end(), r.id) - running_.begin());
      return preempted;
    }
    cache_.slide(r.id, r.n_computed);
    int32_t n_work = chunk_for(r, budget);
    if (n_work == 0) continue;
    while (!cache_.can_reserve(r.id, r.n_computed, r.n_computed + n_work, 0)) {
      preempted = true;
      n_old -= 1;
      preempt(order[n_old]);  // the youngest runner not yet planned; at last the needy one itself
      if (n_old == i) return true;
    }
    schedule(r, n_work);
    budget -= n_work;
  }
  return preempted;
}

void Scheduler::plan_waiting(int32_t& budget) {
  while (!waiting_.empty() && budget > 0 && int32_t(running_.size()) < cfg_.max_batch_reqs &&
         int32_t(sched_.size()) < cfg_.max_batch_reqs) {
    Request& r = reqs_[waiting_.front()];
    int32_t n_work = chunk_for(r, budget);
    // The reserve keeps room for the runners' decoding; with nobody running there is no one
    // to keep it for, and submit has checked that the request fits alone.
    int32_t reserve = running_.empty() ? 0 : reserve_pages(r);  // tokens
    cache_.open(r.id);
    if (n_work == 0 || !cache_.can_reserve(r.id, 0, n_work, reserve)) {
      cache_.close(r.id);
      break;  // first in, first out: nobody overtakes the head
    }
    waiting_.pop_front();
    r.state = REQ_RUNNING;
    running_.push_back(r.id);
    event_.n_admitted += 1;
    schedule(r, n_work);
    budget -= n_work;
  }
}

void Scheduler::emit_plan() {
  plan_.clear();
  for (int pass = 0; pass < 2; ++pass) {  // decode entries first, each kind in scheduling order
    for (const SchedEntry& e : sched_) {
      if ((pass == 0) != (e.kind == ENTRY_DECODE)) continue;
      const Request& r = reqs_[e.req];
      plan_.req.push_back(e.req);
      plan_.start.push_back(e.start);
      plan_.rows.push_back(e.rows);
      plan_.emits.push_back(e.emits);
      plan_.kind.push_back(e.kind);
      plan_.temperature.push_back(r.temperature);
      plan_.top_k.push_back(r.top_k);
      plan_.key0.push_back(r.key0);
      plan_.key1.push_back(r.key1);
      plan_.sample_pos.push_back(e.start + e.rows);
      plan_.input_ids.insert(plan_.input_ids.end(), r.tokens.begin() + e.start,
                             r.tokens.begin() + e.start + e.rows);
      plan_.n_tokens += e.rows;
      if (e.kind == ENTRY_DECODE) event_.n_decode += 1; else event_.n_prefill_rows += e.rows;
    }
  }
}

void Scheduler::detect_stall(bool preempted) {
  stall_ = Stall();
  if (!sched_.empty() || preempted) return;
  if (running_.empty() && waiting_.empty()) return;
  int32_t id = !running_.empty() ? running_[0] : waiting_.front();
  const Request& r = reqs_[id];
  stall_.stalled = 1;
  stall_.req_id = id;
  stall_.n_work = chunk_for(r, cfg_.max_batch_tokens);
  // the group that is shortest of pages for this portion
  int32_t worst = 0, worst_gap = 0;
  for (int32_t g = 0; g < cache_.n_groups(); ++g) {
    int32_t need = ceil_div(r.n_computed + stall_.n_work, cache_.group(g).page_size) - cache_.first_needed_page(g, r.n_computed);
    if (cache_.is_open(id)) need = cache_.pages_to_take(id, g, r.n_computed, r.n_computed + stall_.n_work);
    if (stall_.n_work == 0) need = 0;
    int32_t gap = need - cache_.n_free(g);
    if (g == 0 || gap > worst_gap) {
      worst = g;
      worst_gap = gap;
      stall_.need_pages = need;
    }
  }
  stall_.group = worst;
  stall_.free_pages = cache_.n_free(worst);
}

int32_t Scheduler::plan() {
  if (outstanding_) return SCHED_NO_PLAN;
  int64_t t0 = now_ns();
  step_ += 1;
  event_ = StepEvent();
  event_.step = step_;
  sched_.clear();
  for (Request& r : reqs_) r.in_plan = false;
  int32_t budget = cfg_.max_batch_tokens;
  bool preempted = false;
  if (cfg_.order == ORDER_RUNNING_FIRST) {
    preempted = plan_running(budget, running_.size());
    if (!preempted) plan_waiting(budget);
  } else {
    size_t n_old = running_.size();
    plan_waiting(budget);
    preempted = plan_running(budget, n_old);
  }
  emit_plan();
  detect_stall(preempted);
  event_.n_entries = plan_.n_entries();
  event_.n_tokens = plan_.n_tokens;
  event_.n_running = n_running();
  event_.n_waiting = n_waiting();
  event_.kv_free = min_free();
  event_.t_plan_ns = now_ns() - t0;
  outstanding_ = true;
  return SCHED_OK;
}

void Scheduler::finish(Request& r, int32_t state) {
  cache_.close(r.id);
  running_.erase(std::find(running_.begin(), running_.end(), r.id));
  r.state = state;
  r.t_finish_ns = now_ns();
  event_.n_finished += 1;
}

int32_t Scheduler::commit(const int32_t* tokens, int32_t n) {
  if (!outstanding_) return SCHED_NO_PLAN;
  if (n != plan_.n_entries()) return SCHED_BAD_COMMIT;
  for (int32_t i = 0; i < n; ++i) {
    if (plan_.emits[i] && (tokens[i] < 0 || tokens[i] >= cfg_.vocab_size)) return SCHED_BAD_COMMIT;
  }
  int64_t t0 = now_ns();
  for (int32_t i = 0; i < n; ++i) {
    Request& r = reqs_[plan_.req[i]];
    r.in_plan = false;
    if (r.cancel_pending) {
      cache_.close(r.id);
      running_.erase(std::find(running_.begin(), running_.end(), r.id));
      release_slot(r);
      continue;
    }
    r.n_computed += plan_.rows[i];
    if (!plan_.emits[i]) continue;  // a portion inside the history: its token is dropped
    int32_t token = tokens[i];
    r.tokens.push_back(token);
    r.t_last_token_ns = t0;
    if (r.t_first_token_ns == 0) r.t_first_token_ns = t0;
    bool stop = token == cfg_.eos_token && cfg_.eos_token >= 0;
    for (int32_t s = 0; s < r.n_stops; ++s) stop = stop || token == r.stops[s];
    if (stop) {
      finish(r, REQ_FINISHED_EOS);  // the stop token is kept
    } else if (r.n_generated() >= std::max(1, r.max_new)) {
      finish(r, REQ_FINISHED_LENGTH);
    }
  }
  outstanding_ = false;
  event_.n_running = n_running();
  event_.n_waiting = n_waiting();
  event_.kv_free = min_free();
  event_.t_commit_ns = now_ns() - t0;
  return SCHED_OK;
}

int32_t Scheduler::poll(int32_t id, int32_t* out, int32_t cap, int32_t* finished, int32_t* state) {
  if (id < 0 || id >= cfg_.max_requests || reqs_[id].state == REQ_FREE) return SCHED_BAD_ID;
  Request& r = reqs_[id];
  int32_t avail = r.n_generated() - r.n_polled;
  int32_t n = std::min(avail, std::max(0, cap));
  for (int32_t i = 0; i < n; ++i) out[i] = r.tokens[size_t(r.n_prompt + r.n_polled + i)];
  r.n_polled += n;
  bool done = r.state == REQ_FINISHED_EOS || r.state == REQ_FINISHED_LENGTH;
  *state = r.state;
  *finished = (done && r.n_polled == r.n_generated()) ? 1 : 0;
  if (*finished) release_slot(r);
  return n;
}

int32_t Scheduler::set_max_batch_tokens(int32_t v) {
  if (v < 1 || v > create_max_batch_tokens_) return SCHED_BAD_ARGS;
  cfg_.max_batch_tokens = v;
  return SCHED_OK;
}

int32_t Scheduler::set_chunk_size(int32_t v) {
  if (v < 0 || v > create_max_batch_tokens_) return SCHED_BAD_ARGS;
  cfg_.chunk_size = v;
  return SCHED_OK;
}

int32_t Scheduler::set_max_batch_reqs(int32_t v) {
  if (v < 1 || v > create_max_batch_reqs_) return SCHED_BAD_ARGS;
  cfg_.max_batch_reqs = v;
  return SCHED_OK;
}

int32_t Scheduler::set_order(int32_t v) {
  if (v != ORDER_RUNNING_FIRST && v != ORDER_WAITING_FIRST) return SCHED_BAD_ARGS;
  cfg_.order = v;
  return SCHED_OK;
}

int32_t Scheduler::set_reserve_ratio(float v) {
  if (!(v >= 0.f && v <= 1.f)) return SCHED_BAD_ARGS;
  cfg_.reserve_ratio = v;
  return SCHED_OK;
}

int32_t Scheduler::fill_step_batch(const R2StepBatch& o) const {
  if (!outstanding_) return SCHED_NO_PLAN;
  const Plan& p = plan_;
  const int32_t n = p.n_entries(), t = p.n_tokens;
  if (n > o.r_cap || t > o.t_cap || n > o.w_cap) return SCHED_BAD_ARGS;
  if (n > 0) {
    int32_t status = cache_.fill_batch(n, p.req.data(), p.start.data(), p.rows.data(), o.t_cap, o.r_cap, o.positions,
                                       o.row_entry, o.q_start, o.seq_lens, o.state_slot, o.fresh, o.slot_mapping,
                                       o.block_tables);
    if (status != CACHE_OK) return status;
  } else {
    o.q_start[0] = 0;
  }
  std::copy(p.input_ids.begin(), p.input_ids.end(), o.input_ids);
  for (int32_t e = 0; e < n; ++e) {
    o.entry_req[e] = p.req[e];
    o.entry_start[e] = p.start[e];
    o.entry_rows[e] = p.rows[e];
    o.logit_rows[e] = o.q_start[e + 1] - 1;  // the entry's last row
    o.temperature[e] = p.temperature[e];
    o.top_k[e] = p.top_k[e];
    o.key0[e] = p.key0[e];
    o.key1[e] = p.key1[e];
    o.sample_pos[e] = p.sample_pos[e];
  }
  // everything beyond the counts is inert: rows of no entry that write to the null page, entries
  // of no rows, greedy logit rows on row 0
  for (int32_t i = t; i < o.t_cap; ++i) {
    o.input_ids[i] = 0;
    o.positions[i] = 0;
    o.row_entry[i] = -1;
  }
  for (int32_t g = 0; g < cache_.n_groups(); ++g) {
    std::fill(o.slot_mapping + size_t(g) * o.t_cap + t, o.slot_mapping + size_t(g + 1) * o.t_cap, 0);
  }
  for (int32_t e = n; e < o.r_cap; ++e) {
    o.q_start[e + 1] = t;
    o.seq_lens[e] = 0;
    o.state_slot[e] = 0;
    o.fresh[e] = 0;
  }
  size_t offset = 0;
  for (int32_t g = 0; g < cache_.n_groups(); ++g) {
    const size_t width = size_t(cache_.table_width(g));
    std::fill(o.block_tables + offset + size_t(n) * width, o.block_tables + offset + size_t(o.r_cap) * width, 0);
    offset += size_t(o.r_cap) * width;
  }
  for (int32_t e = n; e < o.w_cap; ++e) {
    o.logit_rows[e] = 0;
    o.temperature[e] = 1.f;
    o.top_k[e] = 1;
    o.key0[e] = 0;
    o.key1[e] = 0;
    o.sample_pos[e] = 0;
  }
  return n;
}

}  // namespace r2
