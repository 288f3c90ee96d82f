// The cache manager: pages of keys and values, one block table per request and cache group,
// and slots for per-request state of fixed size.
//
// It owns indices only; the tensors that the indices point into belong to the model side.
// A cache group is a set of layers whose pages live and die together: "all" groups keep every
// position of a request, "window" groups keep the last `window` positions and give pages back
// as soon as the window has passed them. Every group has a pool of its own. Page id 0 of each
// pool is the null page: real memory that is never handed out; holes in a block table point
// at it. This restates the block pool of the reference's core (kelpie-core/src/kv_pool.zig:
// 17-25,183-188,254-301; block tables kelpie-core/src/request.zig:78-81,218-278) without its
// slabs, reference counts and content hashes, which serve prefix caching only.
#pragma once

#include <cstdint>
#include <deque>
#include <string>
#include <vector>

namespace r2 {

struct GroupSpec {
  int32_t page_size;  // tokens per page
  int32_t window;     // 0: keep every position; w > 0: a query at p reads keys (p - w, p]
  int32_t num_pages;  // pages that can be handed out (the null page is extra)
};

// One group's pages. Freed pages are reused in the order in which they were freed.
class PagePool {
 public:
  explicit PagePool(int32_t num_pages);
  int32_t n_free() const { return static_cast<int32_t>(free_.size()); }
  int32_t n_pages() const { return num_pages_; }
  int32_t take();            // a page id >= 1; the caller has checked n_free()
  bool give(int32_t page);   // false if the page was not held (a double free) or is the null page
  bool held(int32_t page) const { return page >= 1 && page <= num_pages_ && held_[page]; }

 private:
  int32_t num_pages_;
  std::deque<int32_t> free_;
  std::vector<uint8_t> held_;
};

enum CacheStatus : int32_t {
  CACHE_OK = 0,
  CACHE_NO_PAGES = -1,     // not enough free pages; nothing was taken
  CACHE_BAD_REQUEST = -2,  // slot out of range, not open, or already open
  CACHE_TOO_LONG = -3,     // beyond max_seq_len
  CACHE_BAD_ARG = -4,
};

class CacheManager {
 public:
  CacheManager(std::vector<GroupSpec> groups, int32_t max_requests, int32_t max_seq_len);

  int32_t n_groups() const { return static_cast<int32_t>(groups_.size()); }
  const GroupSpec& group(int32_t g) const { return groups_[g]; }
  int32_t max_requests() const { return max_requests_; }
  int32_t max_seq_len() const { return max_seq_len_; }
  int32_t table_width(int32_t g) const { return widths_[g]; }
  int32_t n_free(int32_t g) const { return pools_[g].n_free(); }
  bool is_open(int32_t req) const { return req >= 0 && req < max_requests_ && open_[req]; }

  // A request slot comes to life with empty tables and a state slot that reads as fresh.
  int32_t open(int32_t req);
  // Every page of the request goes back to its pool; the state slot is released.
  int32_t close(int32_t req);

  // First page index that group g still needs when the request's next row is at `n_computed`.
  int32_t first_needed_page(int32_t g, int32_t n_computed) const;
  // Pages that group g must take so that the request holds positions up to n_total (exclusive),
  // given that its next row is at n_computed.
  int32_t pages_to_take(int32_t req, int32_t g, int32_t n_computed, int32_t n_total) const;
  // `spare_tokens` more positions' worth of pages must stay free in every group besides.
  bool can_reserve(int32_t req, int32_t n_computed, int32_t n_total, int32_t spare_tokens) const;
  // All groups or nothing.
  int32_t reserve(int32_t req, int32_t n_computed, int32_t n_total);
  // Window groups give back the pages that no later row can read.
  int32_t slide(int32_t req, int32_t n_computed);
  // The most pages of group g that a lone request of n_total positions ever holds, when it is
  // fed in portions of at most max_chunk rows that end on multiples of `grain`.
  int32_t worst_pages(int32_t g, int32_t n_total, int32_t max_chunk, int32_t grain) const;

  const int32_t* table(int32_t req, int32_t g) const { return &tables_[g][size_t(req) * widths_[g]]; }
  int32_t pages_held(int32_t req, int32_t g) const { return held_count_[g][req]; }
  int32_t state_slot(int32_t req) const { return req; }

  // Batch arrays for entries (request, start, rows). `slot_mapping` is [n_groups][t_stride],
  // `block_tables` is the concatenation over groups of [r_stride][table_width(g)].
  int32_t fill_batch(int32_t n_entries, const int32_t* req, const int32_t* start, const int32_t* rows,
                     int32_t t_stride, int32_t r_stride, int32_t* positions, int32_t* row_entry, int32_t* q_start,
                     int32_t* seq_lens, int32_t* state_slot, int32_t* fresh, int32_t* slot_mapping,
                     int32_t* block_tables) const;

  // Debug invariant: every page is either free or held by exactly one table. Empty when it holds.
  std::string check_invariants() const;

 private:
  std::vector<GroupSpec> groups_;
  int32_t max_requests_;
  int32_t max_seq_len_;
  std::vector<int32_t> widths_;
  std::vector<PagePool> pools_;
  std::vector<std::vector<int32_t>> tables_;      // [g][req * width + i]
  std::vector<std::vector<int32_t>> held_count_;  // [g][req]
  std::vector<uint8_t> open_;
};

}  // namespace r2
