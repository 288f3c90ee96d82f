/* The C ABI of the host library: cache manager and scheduler.
 *
 * A smaller relative of the reference's kelpie.h (kelpie-core/include/kelpie.h:13-406): the
 * host language talks to the native core through plain C functions and flat int32 arrays.
 * Every function returns 0 or a count on success and a negative status on failure; none
 * aborts the process.
 */
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define R2_ABI_VERSION 4

typedef struct {
  int32_t page_size;
  int32_t window;
  int32_t num_pages;
} R2GroupSpec;

typedef struct {
  int32_t max_requests;
  int32_t max_seq_len;
  int32_t max_batch_tokens;
  int32_t max_batch_reqs;
  int32_t order;
  float reserve_ratio;
  int32_t eos_token;
  int32_t vocab_size;
  int32_t chunk_size; /* 0: none; else the most rows of a portion that does not finish its history */
} R2SchedulerConfig;

/* Pointers into arrays that the scheduler owns; valid until the next r2_sched_plan. */
typedef struct {
  int32_t n_entries;
  int32_t n_tokens;
  const int32_t* req;
  const int32_t* start;
  const int32_t* rows;
  const int32_t* emits;
  const int32_t* kind;
  const int32_t* input_ids;
  const float* temperature;
  const int32_t* top_k;
  const int32_t* sample_pos;
  const uint32_t* key0;
  const uint32_t* key1;
} R2Plan;

/* A step batch's arrays in the caller's memory (typically one pinned buffer), with their
   capacities: t_cap rows, r_cap entries, w_cap logit rows. slot_mapping is [n_groups][t_cap],
   block_tables the concatenation over groups of [r_cap][table width]. */
typedef struct {
  int32_t t_cap, r_cap, w_cap, reserved;
  int32_t* input_ids;
  int32_t* positions;
  int32_t* row_entry;
  int32_t* q_start;
  int32_t* seq_lens;
  int32_t* state_slot;
  int32_t* fresh;
  int32_t* logit_rows;
  float* temperature;
  int32_t* top_k;
  uint32_t* key0;
  uint32_t* key1;
  int32_t* sample_pos;
  int32_t* slot_mapping;
  int32_t* block_tables;
  int32_t* entry_req;   /* host-only facts about the entries: request, first position, rows */
  int32_t* entry_start;
  int32_t* entry_rows;
} R2StepBatch;

typedef struct {
  int32_t stalled;
  int32_t req_id;
  int32_t n_work;
  int32_t need_pages; /* of the group that is shortest of pages */
  int32_t free_pages;
  int32_t group;
} R2Stall;

/* One request's life; times in nanoseconds of a monotonic clock, 0 = not yet. */
typedef struct {
  int64_t t_arrival_ns, t_first_sched_ns, t_first_token_ns, t_last_token_ns, t_finish_ns;
  int64_t first_step, last_step;
  int32_t request_id, n_prompt, n_generated, max_new;
  int32_t n_preempted, n_chunks, state, peak_pages;
} R2RequestEvent;

typedef struct {
  int64_t step;
  int32_t n_entries, n_tokens, n_prefill_rows, n_decode;
  int32_t n_admitted, n_preempted, n_finished;
  int32_t n_running, n_waiting, kv_free;
  int64_t t_plan_ns, t_commit_ns;
} R2StepEvent;

int32_t r2_abi_version(void);
int32_t r2_sizeof(int32_t which); /* 0 group spec, 1 scheduler config, 2 plan, 3 stall, 4 step event, 5 step batch, 6 request event */
const char* r2_last_error(void);

/* ---- cache manager ---- */
void* r2_cache_create(const R2GroupSpec* groups, int32_t n_groups, int32_t max_requests, int32_t max_seq_len);
void r2_cache_destroy(void* cache);
int32_t r2_cache_n_groups(const void* cache);
int32_t r2_cache_table_width(const void* cache, int32_t group);
int32_t r2_cache_n_free(const void* cache, int32_t group);
int32_t r2_cache_open(void* cache, int32_t req);
int32_t r2_cache_close(void* cache, int32_t req);
int32_t r2_cache_is_open(const void* cache, int32_t req);
int32_t r2_cache_reserve(void* cache, int32_t req, int32_t n_computed, int32_t n_total);
int32_t r2_cache_can_reserve(const void* cache, int32_t req, int32_t n_computed, int32_t n_total, int32_t spare);
int32_t r2_cache_slide(void* cache, int32_t req, int32_t n_computed);
int32_t r2_cache_pages_held(const void* cache, int32_t req, int32_t group);
int32_t r2_cache_worst_pages(const void* cache, int32_t group, int32_t n_total, int32_t max_chunk, int32_t grain);
int32_t r2_cache_table(const void* cache, int32_t req, int32_t group, int32_t* out, int32_t cap);
int32_t r2_cache_fill_batch(const void* cache, int32_t n_entries, const int32_t* req, const int32_t* start,
                            const int32_t* rows, int32_t t_stride, int32_t r_stride, int32_t* positions, int32_t* row_entry,
                            int32_t* q_start, int32_t* seq_lens, int32_t* state_slot, int32_t* fresh,
                            int32_t* slot_mapping, int32_t* block_tables);
/* Writes a description of any broken invariant into out; returns its length (0 = all hold). */
int32_t r2_cache_check(const void* cache, char* out, int32_t cap);

/* ---- scheduler ---- */
void* r2_sched_create(const R2SchedulerConfig* cfg, const R2GroupSpec* groups, int32_t n_groups);
void r2_sched_destroy(void* sched);
void* r2_sched_cache(void* sched); /* the scheduler's own cache manager; not to be destroyed */
int32_t r2_sched_submit(void* sched, const int32_t* prompt, int32_t n, int32_t max_new, float temperature,
                        int32_t top_k, uint64_t seed, const int32_t* stops, int32_t n_stops);
int32_t r2_sched_cancel(void* sched, int32_t id);
int32_t r2_sched_plan(void* sched, R2Plan* out);
/* The outstanding plan as a whole step batch: tokens, positions, slots, block tables, one logit row
   per entry (its last row) with its sampling parameters, and inert padding up to the capacities.
   Every index it writes lies inside the pool by construction. Negative on a plan that does not fit. */
int32_t r2_sched_fill_step_batch(void* sched, const R2StepBatch* out);
/* Bounds checks of a batch that the caller filled itself, in one pass over its rows: 0 if it is sound, else
   1 a row names an entry outside the batch, 2 the rows of entry *where are not its newest positions, 3 a token
   lies outside the vocabulary, 4 a slot of group *where lies outside the pool or in the null page, 5 a block
   table of group *where names a page outside the pool, 6 an entry reaches beyond max_seq_len.
   `table_widths` has the width of each group's block table. */
int32_t r2_step_batch_check(const R2StepBatch* batch, int32_t n_tokens, int32_t n_entries, int32_t vocab_size, int32_t max_seq_len,
                            const R2GroupSpec* groups, const int32_t* table_widths, int32_t n_groups, int32_t* where);
int32_t r2_sched_commit(void* sched, const int32_t* tokens, int32_t n);
int32_t r2_sched_poll(void* sched, int32_t id, int32_t* out, int32_t cap, int32_t* finished, int32_t* state);
int32_t r2_sched_stall(const void* sched, R2Stall* out);
int32_t r2_sched_event(const void* sched, R2StepEvent* out);
int32_t r2_sched_counts(const void* sched, int32_t* n_running, int32_t* n_waiting);
int32_t r2_sched_request_info(const void* sched, int32_t id, int32_t* state, int32_t* n_prompt, int32_t* n_tokens,
                              int32_t* n_computed, int32_t* n_preempted);
/* The record of a request that is queued, running, or finished and not yet polled to its end. */
int32_t r2_sched_request_event(const void* sched, int32_t id, R2RequestEvent* out);
/* Records of requests whose slots were released since the last call, oldest first; returns the count copied. */
int32_t r2_sched_drain_request_events(void* sched, R2RequestEvent* out, int32_t cap);
int32_t r2_sched_grain(const void* sched);
int32_t r2_sched_set(void* sched, int32_t knob, double value); /* 0 tokens, 1 reqs, 2 order, 3 reserve, 4 chunk size */

#ifdef __cplusplus
}
#endif
