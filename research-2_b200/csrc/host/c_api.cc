#include <cstring>
#include <string>
#include <vector>

#include "cache_manager.h"
#include "engine_abi.h"
#include "scheduler.h"

using r2::CacheManager;
using r2::Scheduler;

static thread_local std::string g_error;

static_assert(sizeof(R2GroupSpec) == sizeof(r2::GroupSpec), "group spec layouts must agree");
static_assert(sizeof(R2SchedulerConfig) == sizeof(r2::SchedulerConfig), "config layouts must agree");
static_assert(sizeof(R2Stall) == sizeof(r2::Stall), "stall layouts must agree");
static_assert(sizeof(R2StepEvent) == sizeof(r2::StepEvent), "event layouts must agree");
static_assert(sizeof(R2RequestEvent) == sizeof(r2::RequestEvent), "request event layouts must agree");

static bool groups_ok(const R2GroupSpec* groups, int32_t n_groups, int32_t max_requests, int32_t max_seq_len) {
  if (groups == nullptr || n_groups < 1) { g_error = "at least one cache group is needed"; return false; }
  if (max_requests < 1) { g_error = "max_requests must be >= 1"; return false; }
  if (max_seq_len < 1) { g_error = "max_seq_len must be >= 1"; return false; }
  for (int32_t g = 0; g < n_groups; ++g) {
    if (groups[g].page_size < 1) { g_error = "group " + std::to_string(g) + ": page_size must be >= 1"; return false; }
    if (groups[g].window < 0) { g_error = "group " + std::to_string(g) + ": window must be >= 0"; return false; }
    if (groups[g].num_pages < 1) { g_error = "group " + std::to_string(g) + ": num_pages must be >= 1"; return false; }
  }
  return true;
}

static std::vector<r2::GroupSpec> to_groups(const R2GroupSpec* groups, int32_t n) {
  std::vector<r2::GroupSpec> out;
  for (int32_t g = 0; g < n; ++g) out.push_back({groups[g].page_size, groups[g].window, groups[g].num_pages});
  return out;
}

extern "C" {

int32_t r2_abi_version(void) { return R2_ABI_VERSION; }

int32_t r2_sizeof(int32_t which) {
  switch (which) {
    case 0: return sizeof(R2GroupSpec);
    case 1: return sizeof(R2SchedulerConfig);
    case 2: return sizeof(R2Plan);
    case 3: return sizeof(R2Stall);
    case 4: return sizeof(R2StepEvent);
    case 5: return sizeof(R2StepBatch);
    case 6: return sizeof(R2RequestEvent);
    default: return -1;
  }
}

const char* r2_last_error(void) { return g_error.c_str(); }

void* r2_cache_create(const R2GroupSpec* groups, int32_t n_groups, int32_t max_requests, int32_t max_seq_len) {
  if (!groups_ok(groups, n_groups, max_requests, max_seq_len)) return nullptr;
  return new CacheManager(to_groups(groups, n_groups), max_requests, max_seq_len);
}

void r2_cache_destroy(void* cache) { delete static_cast<CacheManager*>(cache); }

#define CM(p) (static_cast<CacheManager*>(p))
#define CCM(p) (static_cast<const CacheManager*>(p))

int32_t r2_cache_n_groups(const void* cache) { return CCM(cache)->n_groups(); }
int32_t r2_cache_table_width(const void* cache, int32_t g) {
  return (g < 0 || g >= CCM(cache)->n_groups()) ? r2::CACHE_BAD_ARG : CCM(cache)->table_width(g);
}
int32_t r2_cache_n_free(const void* cache, int32_t g) {
  return (g < 0 || g >= CCM(cache)->n_groups()) ? r2::CACHE_BAD_ARG : CCM(cache)->n_free(g);
}
int32_t r2_cache_open(void* cache, int32_t req) { return CM(cache)->open(req); }
int32_t r2_cache_close(void* cache, int32_t req) { return CM(cache)->close(req); }
int32_t r2_cache_is_open(const void* cache, int32_t req) { return CCM(cache)->is_open(req) ? 1 : 0; }
int32_t r2_cache_reserve(void* cache, int32_t req, int32_t n_computed, int32_t n_total) {
  return CM(cache)->reserve(req, n_computed, n_total);
}
int32_t r2_cache_can_reserve(const void* cache, int32_t req, int32_t n_computed, int32_t n_total, int32_t spare) {
  return CCM(cache)->can_reserve(req, n_computed, n_total, spare) ? 1 : 0;
}
int32_t r2_cache_slide(void* cache, int32_t req, int32_t n_computed) { return CM(cache)->slide(req, n_computed); }
int32_t r2_cache_pages_held(const void* cache, int32_t req, int32_t g) {
  if (!CCM(cache)->is_open(req) || g < 0 || g >= CCM(cache)->n_groups()) return r2::CACHE_BAD_REQUEST;
  return CCM(cache)->pages_held(req, g);
}
int32_t r2_cache_worst_pages(const void* cache, int32_t g, int32_t n_total, int32_t max_chunk, int32_t grain) {
  if (g < 0 || g >= CCM(cache)->n_groups()) return r2::CACHE_BAD_ARG;
  return CCM(cache)->worst_pages(g, n_total, max_chunk, grain);
}
int32_t r2_cache_table(const void* cache, int32_t req, int32_t g, int32_t* out, int32_t cap) {
  const CacheManager* c = CCM(cache);
  if (req < 0 || req >= c->max_requests() || g < 0 || g >= c->n_groups()) return r2::CACHE_BAD_REQUEST;
  int32_t n = c->table_width(g) < cap ? c->table_width(g) : cap;
  std::memcpy(out, c->table(req, g), size_t(n) * sizeof(int32_t));
  return n;
}
int32_t r2_cache_fill_batch(const void* cache, int32_t n_entries, const int32_t* req, const int32_t* start,
                            const int32_t* rows, int32_t t_stride, int32_t r_stride, int32_t* positions, int32_t* row_entry,
                            int32_t* q_start, int32_t* seq_lens, int32_t* state_slot, int32_t* fresh,
                            int32_t* slot_mapping, int32_t* block_tables) {
  return CCM(cache)->fill_batch(n_entries, req, start, rows, t_stride, r_stride, positions, row_entry, q_start, seq_lens,
                                state_slot, fresh, slot_mapping, block_tables);
}
int32_t r2_cache_check(const void* cache, char* out, int32_t cap) {
  std::string msg = CCM(cache)->check_invariants();
  if (cap > 0) {
    size_t n = msg.size() < size_t(cap - 1) ? msg.size() : size_t(cap - 1);
    std::memcpy(out, msg.data(), n);
    out[n] = 0;
  }
  return int32_t(msg.size());
}

/* ---- scheduler ---- */

void* r2_sched_create(const R2SchedulerConfig* cfg, const R2GroupSpec* groups, int32_t n_groups) {
  if (cfg == nullptr) { g_error = "no configuration"; return nullptr; }
  if (!groups_ok(groups, n_groups, cfg->max_requests, cfg->max_seq_len)) return nullptr;
  if (cfg->max_batch_tokens < 1 || cfg->max_batch_tokens > 8192) { g_error = "max_batch_tokens must be in [1, 8192]"; return nullptr; }
  if (cfg->max_batch_reqs < 1 || cfg->max_batch_reqs > 8192) { g_error = "max_batch_reqs must be in [1, 8192]"; return nullptr; }
  if (cfg->order != 0 && cfg->order != 1) { g_error = "order must be 0 (running first) or 1 (waiting first)"; return nullptr; }
  if (!(cfg->reserve_ratio >= 0.f && cfg->reserve_ratio <= 1.f)) { g_error = "reserve_ratio must be in [0, 1]"; return nullptr; }
  if (cfg->vocab_size < 1) { g_error = "vocab_size must be >= 1"; return nullptr; }
  if (cfg->eos_token < -1 || cfg->eos_token >= cfg->vocab_size) { g_error = "eos_token must be -1 or a token id"; return nullptr; }
  if (cfg->chunk_size < 0 || cfg->chunk_size > cfg->max_batch_tokens) { g_error = "chunk_size must be 0 or in [1, max_batch_tokens]"; return nullptr; }
  r2::SchedulerConfig c{cfg->max_requests, cfg->max_seq_len, cfg->max_batch_tokens, cfg->max_batch_reqs,
                        cfg->order, cfg->reserve_ratio, cfg->eos_token, cfg->vocab_size, cfg->chunk_size};
  Scheduler* s = new Scheduler(c, to_groups(groups, n_groups));
  // A portion that does not finish a history ends on a page boundary of every group; a budget below
  // that grain could never run a prompt longer than itself.
  int32_t least = cfg->chunk_size > 0 ? cfg->chunk_size : cfg->max_batch_tokens;
  if (least < s->grain()) {
    g_error = "max_batch_tokens and chunk_size must be at least " + std::to_string(s->grain()) +
              " (a portion ends on a page boundary of every cache group)";
    delete s;
    return nullptr;
  }
  return s;
}

void r2_sched_destroy(void* sched) { delete static_cast<Scheduler*>(sched); }

#define SC(p) (static_cast<Scheduler*>(p))
#define CSC(p) (static_cast<const Scheduler*>(p))

void* r2_sched_cache(void* sched) { return &SC(sched)->cache(); }

int32_t r2_sched_submit(void* sched, const int32_t* prompt, int32_t n, int32_t max_new, float temperature,
                        int32_t top_k, uint64_t seed, const int32_t* stops, int32_t n_stops) {
  return SC(sched)->submit(prompt, n, max_new, temperature, top_k, seed, stops, n_stops);
}
int32_t r2_sched_cancel(void* sched, int32_t id) { return SC(sched)->cancel(id); }

int32_t r2_sched_plan(void* sched, R2Plan* out) {
  int32_t status = SC(sched)->plan();
  if (status != r2::SCHED_OK) return status;
  const r2::Plan& p = SC(sched)->current_plan();
  out->n_entries = p.n_entries();
  out->n_tokens = p.n_tokens;
  out->req = p.req.data();
  out->start = p.start.data();
  out->rows = p.rows.data();
  out->emits = p.emits.data();
  out->kind = p.kind.data();
  out->input_ids = p.input_ids.data();
  out->temperature = p.temperature.data();
  out->top_k = p.top_k.data();
  out->sample_pos = p.sample_pos.data();
  out->key0 = p.key0.data();
  out->key1 = p.key1.data();
  return r2::SCHED_OK;
}

int32_t r2_sched_fill_step_batch(void* sched, const R2StepBatch* out) { return SC(sched)->fill_step_batch(*out); }
int32_t r2_step_batch_check(const R2StepBatch* b, int32_t t, int32_t r, int32_t vocab_size, int32_t max_seq_len,
                            const R2GroupSpec* groups, const int32_t* table_widths, int32_t n_groups, int32_t* where) {
  *where = -1;
  if (t <= 0) return 0;
  if (t > b->t_cap || r < 1 || r > b->r_cap) return 1;
  for (int32_t i = 0; i < t; ++i) {
    const int32_t e = b->row_entry[i];
    if (e < 0 || e >= r) return 1;
  }
  // an entry's rows are its newest positions (the reference asserts this on the device:
  // kelpie-models/kelpie_models/kernels/ops/paged_attention.py:143-157)
  for (int32_t i = 0; i < t; ++i) {
    const int32_t e = b->row_entry[i];
    const int32_t first = b->q_start[e], end = b->q_start[e + 1];
    if (i < first || i >= end || b->positions[i] != b->seq_lens[e] - (end - i)) {
      *where = e;
      return 2;
    }
  }
  for (int32_t i = 0; i < t; ++i) {
    if (b->input_ids[i] < 0 || b->input_ids[i] >= vocab_size) return 3;
  }
  const int32_t* tables = b->block_tables;
  for (int32_t g = 0; g < n_groups; ++g) {
    *where = g;
    const int32_t page = groups[g].page_size;
    const int64_t limit = (int64_t(groups[g].num_pages) + 1) * page;
    const int32_t* slots = b->slot_mapping + size_t(g) * b->t_cap;
    for (int32_t i = 0; i < t; ++i) {
      if (slots[i] < page || slots[i] >= limit) return 4;
    }
    const int32_t width = table_widths[g];
    for (int64_t i = 0; i < int64_t(r) * width; ++i) {
      if (tables[i] < 0 || tables[i] > groups[g].num_pages) return 5;
    }
    tables += size_t(b->r_cap) * width;
  }
  *where = -1;
  for (int32_t e = 0; e < r; ++e) {
    if (b->seq_lens[e] > max_seq_len) return 6;
  }
  return 0;
}

int32_t r2_sched_commit(void* sched, const int32_t* tokens, int32_t n) { return SC(sched)->commit(tokens, n); }
int32_t r2_sched_poll(void* sched, int32_t id, int32_t* out, int32_t cap, int32_t* finished, int32_t* state) {
  return SC(sched)->poll(id, out, cap, finished, state);
}
int32_t r2_sched_stall(const void* sched, R2Stall* out) {
  std::memcpy(out, &CSC(sched)->stall(), sizeof(R2Stall));
  return out->stalled;
}
int32_t r2_sched_event(const void* sched, R2StepEvent* out) {
  std::memcpy(out, &CSC(sched)->last_event(), sizeof(R2StepEvent));
  return 0;
}
int32_t r2_sched_counts(const void* sched, int32_t* n_running, int32_t* n_waiting) {
  *n_running = CSC(sched)->n_running();
  *n_waiting = CSC(sched)->n_waiting();
  return 0;
}
int32_t r2_sched_request_info(const void* sched, int32_t id, int32_t* state, int32_t* n_prompt, int32_t* n_tokens,
                              int32_t* n_computed, int32_t* n_preempted) {
  const r2::Request* r = CSC(sched)->request(id);
  if (r == nullptr) return r2::SCHED_BAD_ID;
  *state = r->state;
  *n_prompt = r->n_prompt;
  *n_tokens = int32_t(r->tokens.size());
  *n_computed = r->n_computed;
  *n_preempted = r->n_preempted;
  return 0;
}
int32_t r2_sched_request_event(const void* sched, int32_t id, R2RequestEvent* out) {
  static_assert(sizeof(R2RequestEvent) == sizeof(r2::RequestEvent), "layout");
  return CSC(sched)->request_event(id, reinterpret_cast<r2::RequestEvent*>(out));
}
int32_t r2_sched_drain_request_events(void* sched, R2RequestEvent* out, int32_t cap) {
  return SC(sched)->drain_request_events(reinterpret_cast<r2::RequestEvent*>(out), cap);
}
int32_t r2_sched_grain(const void* sched) { return CSC(sched)->grain(); }
int32_t r2_sched_set(void* sched, int32_t knob, double value) {
  switch (knob) {
    case 0: return SC(sched)->set_max_batch_tokens(int32_t(value));
    case 1: return SC(sched)->set_max_batch_reqs(int32_t(value));
    case 2: return SC(sched)->set_order(int32_t(value));
    case 3: return SC(sched)->set_reserve_ratio(float(value));
    case 4: return SC(sched)->set_chunk_size(int32_t(value));
    default: return r2::SCHED_BAD_ARGS;
  }
}

}  // extern "C"
