#include "cache_manager.h"

#include <algorithm>
#include <sstream>

namespace r2 {

static inline int32_t ceil_div(int32_t a, int32_t b) { return (a + b - 1) / b; }

PagePool::PagePool(int32_t num_pages) : num_pages_(num_pages), held_(size_t(num_pages) + 1, 0) {
  for (int32_t p = 1; p <= num_pages; ++p) free_.push_back(p);
}

int32_t PagePool::take() {
  int32_t page = free_.front();
  free_.pop_front();
  held_[page] = 1;
  return page;
}

bool PagePool::give(int32_t page) {
  if (page < 1 || page > num_pages_ || !held_[page]) return false;
  held_[page] = 0;
  free_.push_back(page);
  return true;
}

CacheManager::CacheManager(std::vector<GroupSpec> groups, int32_t max_requests, int32_t max_seq_len)
    : groups_(std::move(groups)), max_requests_(max_requests), max_seq_len_(max_seq_len),
      open_(size_t(max_requests), 0) {
  for (const GroupSpec& g : groups_) {
    int32_t width = ceil_div(max_seq_len_, g.page_size);
    widths_.push_back(width);
    pools_.emplace_back(g.num_pages);
    tables_.emplace_back(size_t(max_requests_) * width, 0);
    held_count_.emplace_back(size_t(max_requests_), 0);
  }
}

int32_t CacheManager::open(int32_t req) {
  if (req < 0 || req >= max_requests_ || open_[req]) return CACHE_BAD_REQUEST;
  open_[req] = 1;
  return CACHE_OK;
}

int32_t CacheManager::close(int32_t req) {
  if (!is_open(req)) return CACHE_BAD_REQUEST;
  for (int32_t g = 0; g < n_groups(); ++g) {
    int32_t* t = &tables_[g][size_t(req) * widths_[g]];
    for (int32_t i = 0; i < widths_[g]; ++i) {
      if (t[i] != 0) {
        pools_[g].give(t[i]);
        t[i] = 0;
      }
    }
    held_count_[g][req] = 0;
  }
  open_[req] = 0;
  return CACHE_OK;
}

int32_t CacheManager::first_needed_page(int32_t g, int32_t n_computed) const {
  const GroupSpec& spec = groups_[g];
  if (spec.window <= 0) return 0;
  int32_t first_key = std::max(0, n_computed - spec.window + 1);
  return first_key / spec.page_size;
}

int32_t CacheManager::pages_to_take(int32_t req, int32_t g, int32_t n_computed, int32_t n_total) const {
  const int32_t* t = table(req, g);
  int32_t end = ceil_div(n_total, groups_[g].page_size);
  int32_t need = 0;
  for (int32_t i = first_needed_page(g, n_computed); i < end; ++i) need += (t[i] == 0);
  return need;
}

bool CacheManager::can_reserve(int32_t req, int32_t n_computed, int32_t n_total, int32_t spare_tokens) const {
  if (!is_open(req) || n_total > max_seq_len_ || n_computed < 0 || n_total < n_computed) return false;
  for (int32_t g = 0; g < n_groups(); ++g) {
    int32_t spare = ceil_div(std::max(0, spare_tokens), groups_[g].page_size);
    if (pages_to_take(req, g, n_computed, n_total) + spare > pools_[g].n_free()) return false;
  }
  return true;
}

int32_t CacheManager::reserve(int32_t req, int32_t n_computed, int32_t n_total) {
  if (!is_open(req)) return CACHE_BAD_REQUEST;
  if (n_computed < 0 || n_total < n_computed) return CACHE_BAD_ARG;
  if (n_total > max_seq_len_) return CACHE_TOO_LONG;
  if (!can_reserve(req, n_computed, n_total, 0)) return CACHE_NO_PAGES;
  for (int32_t g = 0; g < n_groups(); ++g) {
    int32_t* t = &tables_[g][size_t(req) * widths_[g]];
    int32_t end = ceil_div(n_total, groups_[g].page_size);
    for (int32_t i = first_needed_page(g, n_computed); i < end; ++i) {
      if (t[i] == 0) {
        t[i] = pools_[g].take();
        held_count_[g][req] += 1;
      }
    }
  }
  return CACHE_OK;
}

int32_t CacheManager::slide(int32_t req, int32_t n_computed) {
  if (!is_open(req)) return CACHE_BAD_REQUEST;
  for (int32_t g = 0; g < n_groups(); ++g) {
    if (groups_[g].window <= 0) continue;
    int32_t* t = &tables_[g][size_t(req) * widths_[g]];
    int32_t first = std::min(first_needed_page(g, n_computed), widths_[g]);
    for (int32_t i = 0; i < first; ++i) {
      if (t[i] != 0) {
        pools_[g].give(t[i]);
        t[i] = 0;
        held_count_[g][req] -= 1;
      }
    }
  }
  return CACHE_OK;
}

int32_t CacheManager::worst_pages(int32_t g, int32_t n_total, int32_t max_chunk, int32_t grain) const {
  const GroupSpec& spec = groups_[g];
  int32_t all = ceil_div(n_total, spec.page_size);
  if (spec.window <= 0) return all;
  // A portion of rows [s, e) needs the keys from s - window + 1 up to e - 1. Portions are
  // either one decoded row at any s, or a piece of a history: it starts on a multiple of
  // `grain` and ends on one unless it reaches the history's end. The most pages over all of them:
  int32_t worst = 0;
  max_chunk = std::max(1, max_chunk);
  grain = std::max(1, grain);
  for (int32_t s = 0; s < n_total; ++s) {
    int32_t first_page = std::max(0, s - spec.window + 1) / spec.page_size;
    int32_t e = s + 1;  // the single decoded row
    if (s % grain == 0) {
      e = std::min(n_total, s + max_chunk);
      if (e < n_total) e = e / grain * grain;
      if (e <= s) e = s + 1;
    }
    worst = std::max(worst, (e - 1) / spec.page_size - first_page + 1);
  }
  return std::min(all, worst);
}

int32_t CacheManager::fill_batch(int32_t n_entries, const int32_t* req, const int32_t* start,
                                 const int32_t* rows, int32_t t_stride, int32_t r_stride, int32_t* positions,
                                 int32_t* row_entry, int32_t* q_start, int32_t* seq_lens,
                                 int32_t* state_slot_out, int32_t* fresh, int32_t* slot_mapping,
                                 int32_t* block_tables) const {
  int32_t t = 0;
  q_start[0] = 0;
  for (int32_t e = 0; e < n_entries; ++e) {
    int32_t r = req[e];
    if (!is_open(r) || rows[e] < 1 || start[e] < 0) return CACHE_BAD_REQUEST;
    if (start[e] + rows[e] > max_seq_len_) return CACHE_TOO_LONG;
    if (t + rows[e] > t_stride) return CACHE_BAD_ARG;
    for (int32_t i = 0; i < rows[e]; ++i) {
      int32_t pos = start[e] + i;
      positions[t + i] = pos;
      row_entry[t + i] = e;
      for (int32_t g = 0; g < n_groups(); ++g) {
        int32_t ps = groups_[g].page_size;
        int32_t page = table(r, g)[pos / ps];
        if (page == 0) return CACHE_NO_PAGES;  // the row's own page must have been reserved
        slot_mapping[size_t(g) * t_stride + t + i] = page * ps + pos % ps;
      }
    }
    t += rows[e];
    q_start[e + 1] = t;
    seq_lens[e] = start[e] + rows[e];
    state_slot_out[e] = state_slot(r);
    fresh[e] = start[e] == 0 ? 1 : 0;
  }
  size_t offset = 0;
  for (int32_t g = 0; g < n_groups(); ++g) {
    int32_t width = widths_[g];
    for (int32_t e = 0; e < n_entries; ++e) {
      std::copy_n(table(req[e], g), width, block_tables + offset + size_t(e) * width);
    }
    offset += size_t(r_stride) * width;
  }
  return CACHE_OK;
}

std::string CacheManager::check_invariants() const {
  std::ostringstream err;
  for (int32_t g = 0; g < n_groups(); ++g) {
    std::vector<int32_t> owner(size_t(groups_[g].num_pages) + 1, -1);
    int32_t held = 0;
    for (int32_t r = 0; r < max_requests_; ++r) {
      const int32_t* t = table(r, g);
      int32_t count = 0;
      for (int32_t i = 0; i < widths_[g]; ++i) {
        int32_t p = t[i];
        if (p == 0) continue;
        if (!open_[r]) err << "group " << g << ": closed request " << r << " holds page " << p << "; ";
        if (p < 1 || p > groups_[g].num_pages) {
          err << "group " << g << ": request " << r << " holds bad page id " << p << "; ";
          continue;
        }
        if (owner[p] >= 0) err << "group " << g << ": page " << p << " held by requests " << owner[p] << " and " << r << "; ";
        owner[p] = r;
        if (!pools_[g].held(p)) err << "group " << g << ": page " << p << " is in a table and in the free list; ";
        ++count;
      }
      if (count != held_count_[g][r]) err << "group " << g << ": request " << r << " count " << held_count_[g][r] << " != " << count << "; ";
      held += count;
    }
    if (held + pools_[g].n_free() != groups_[g].num_pages) {
      err << "group " << g << ": " << held << " held + " << pools_[g].n_free() << " free != " << groups_[g].num_pages << " pages; ";
    }
  }
  return err.str();
}

}  // namespace r2
