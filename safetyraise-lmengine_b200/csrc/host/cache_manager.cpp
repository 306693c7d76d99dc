#include "cache_manager.hpp"

#include <algorithm>

namespace srlm {

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

CacheManager::CacheManager(int max_requests, const std::vector<GroupSpec>& groups) {
  for (const GroupSpec& s : groups) {
    Group g;
    g.spec = s;
    g.free_list.reserve(s.num_pages);
    // page 0 is handed out first
    for (int p = s.num_pages - 1; p >= 0; --p) g.free_list.push_back(p);
    g.ever_used.assign(s.num_pages, 0);
    groups_.push_back(std::move(g));
  }
  slots_.resize(max_requests);
  for (int s = max_requests - 1; s >= 0; --s) free_slots_.push_back(s);
  for (Slot& s : slots_) s.tables.resize(groups_.size());
}

int CacheManager::open_request() {
  if (free_slots_.empty()) return -1;
  int slot = free_slots_.back();
  free_slots_.pop_back();
  Slot& s = slots_[slot];
  s.open = true;
  s.length = 0;
  s.reserved = 0;
  s.generation += 1;
  for (auto& t : s.tables) t.clear();
  return slot;
}

int CacheManager::close_request(int slot) {
  if (!valid(slot)) return -1;
  Slot& s = slots_[slot];
  for (size_t g = 0; g < groups_.size(); ++g) {
    for (int32_t page : s.tables[g])
      if (page >= 0) groups_[g].free_list.push_back(page);
    s.tables[g].clear();
  }
  s.open = false;
  s.length = s.reserved = 0;
  free_slots_.push_back(slot);
  return 0;
}

int CacheManager::first_needed_page(const Group& g, int length) const {
  if (g.spec.kind != GROUP_WINDOW) return 0;
  // the next query sits at position >= length and sees keys > position - window
  int first_key = std::max(0, length - g.spec.window + 1);
  return first_key / g.spec.page_size;
}

int CacheManager::reserve(int slot, int new_len) {
  if (!valid(slot) || new_len < 0) return -1;
  Slot& s = slots_[slot];
  if (new_len < s.length) return -2;
  for (size_t g = 0; g < groups_.size(); ++g) {
    int have = static_cast<int>(s.tables[g].size());
    int need = ceil_div(new_len, groups_[g].spec.page_size) - have;
    if (need > static_cast<int>(groups_[g].free_list.size())) return 0;
  }
  for (size_t g = 0; g < groups_.size(); ++g) {
    Group& grp = groups_[g];
    int want = ceil_div(new_len, grp.spec.page_size);
    while (static_cast<int>(s.tables[g].size()) < want) {
      int32_t page = grp.free_list.back();
      grp.free_list.pop_back();
      pages_taken_ += 1;
      if (grp.ever_used[page]) pages_reused_ += 1;
      grp.ever_used[page] = 1;
      s.tables[g].push_back(page);
    }
  }
  s.reserved = std::max(s.reserved, new_len);
  return 1;
}

int CacheManager::fit_tokens(int slot, int want_len) const {
  if (!valid(slot)) return -1;
  const Slot& s = slots_[slot];
  int best = want_len;
  for (size_t g = 0; g < groups_.size(); ++g) {
    const Group& grp = groups_[g];
    int have = static_cast<int>(s.tables[g].size());
    int can = (have + static_cast<int>(grp.free_list.size())) * grp.spec.page_size;
    best = std::min(best, can);
  }
  return std::max(best, s.length);
}

int CacheManager::commit(int slot, int new_len) {
  if (!valid(slot)) return -1;
  Slot& s = slots_[slot];
  if (new_len < s.length || new_len > s.reserved) return -2;
  s.length = new_len;
  for (size_t g = 0; g < groups_.size(); ++g) {
    Group& grp = groups_[g];
    int first = std::min(first_needed_page(grp, new_len), static_cast<int>(s.tables[g].size()));
    for (int p = 0; p < first; ++p) {
      if (s.tables[g][p] >= 0) {
        grp.free_list.push_back(s.tables[g][p]);
        s.tables[g][p] = -1;
      }
    }
  }
  return 0;
}

int CacheManager::truncate(int slot, int len) {
  if (!valid(slot) || len < 0) return -1;
  Slot& s = slots_[slot];
  if (len > s.reserved) return -2;
  if (len < s.length) {
    for (size_t g = 0; g < groups_.size(); ++g) {
      const Group& grp = groups_[g];
      int first = first_needed_page(grp, len);
      if (first < static_cast<int>(s.tables[g].size()) && s.tables[g][first] < 0) return -3;
    }
  }
  for (size_t g = 0; g < groups_.size(); ++g) {
    Group& grp = groups_[g];
    int keep = ceil_div(len, grp.spec.page_size);
    while (static_cast<int>(s.tables[g].size()) > keep) {
      int32_t page = s.tables[g].back();
      s.tables[g].pop_back();
      if (page >= 0) grp.free_list.push_back(page);
    }
  }
  s.length = std::min(s.length, len);
  s.reserved = len;
  return 0;
}

int CacheManager::length(int slot) const { return valid(slot) ? slots_[slot].length : -1; }
int CacheManager::reserved_tokens(int slot) const { return valid(slot) ? slots_[slot].reserved : -1; }
int CacheManager::generation(int slot) const {
  return (slot >= 0 && slot < max_requests()) ? slots_[slot].generation : -1;
}

int CacheManager::table(int group, int slot, int32_t* out, int cap) const {
  if (!valid(slot) || group < 0 || group >= num_groups()) return -1;
  const auto& t = slots_[slot].tables[group];
  int n = static_cast<int>(t.size());
  for (int i = 0; i < n && i < cap; ++i) out[i] = t[i];
  return n;
}

int CacheManager::free_pages(int group) const {
  if (group < 0 || group >= num_groups()) return -1;
  return static_cast<int>(groups_[group].free_list.size());
}

int CacheManager::peak_pages(int group, int total_len, int max_step) const {
  const GroupSpec& s = groups_[group].spec;
  int all = ceil_div(total_len, s.page_size);
  if (s.kind != GROUP_WINDOW) return all;
  // a step of max_step tokens needs its own keys and the window before its first query,
  // which may straddle one more page at each end
  return std::min(all, ceil_div(s.window + max_step, s.page_size) + 1);
}

int CacheManager::audit() const {
  for (size_t g = 0; g < groups_.size(); ++g) {
    const Group& grp = groups_[g];
    std::vector<int> seen(grp.spec.num_pages, 0);
    for (int32_t p : grp.free_list) {
      if (p < 0 || p >= grp.spec.num_pages) return 1;   // id out of range
      seen[p] += 1;
    }
    for (const Slot& s : slots_) {
      if (!s.open) {
        if (!s.tables[g].empty()) return 2;             // closed slot still holds pages
        continue;
      }
      for (int32_t p : s.tables[g]) {
        if (p < 0) continue;
        if (p >= grp.spec.num_pages) return 1;
        seen[p] += 1;
      }
    }
    for (int c : seen) {
      if (c == 0) return 3;                             // page lost
      if (c > 1) return 4;                              // page held or freed twice
    }
  }
  std::vector<int> slot_seen(slots_.size(), 0);
  for (int s : free_slots_) slot_seen[s] += 1;
  for (size_t s = 0; s < slots_.size(); ++s)
    if (slot_seen[s] + (slots_[s].open ? 1 : 0) != 1) return 5;
  return 0;
}

}  // namespace srlm
