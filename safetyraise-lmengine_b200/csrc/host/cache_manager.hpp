// Page accounting for the key/value cache and the per-request state slots.
//
// The manager owns numbers only: page ids, block tables, lengths.  The device
// memory that the ids index is allocated by the caller, one pool per group.
// A group is a set of cache entries (layers) with the same need: either every
// earlier key stays visible (kind ALL) or only a window of them (kind WINDOW),
// in which case pages that the window has passed are given back at commit.
// Each group has pages of its own.  A request holds one slot; the slot index
// also addresses the request's fixed-size state in every state group.
//
// Counterpart of PagedKvCache / SequenceState in the reference
// (src/engine/state.rs:19-224), which keeps pages per request on the heap;
// here pages come from fixed pools so that running out is an event the
// scheduler handles, not an allocation failure.
#pragma once

#include <cstdint>
#include <vector>

namespace srlm {

enum GroupKind : int { GROUP_ALL = 0, GROUP_WINDOW = 1 };

struct GroupSpec {
  int kind;
  int page_size;
  int num_pages;
  int window;  // tokens a query sees, itself included; only for GROUP_WINDOW
};

class CacheManager {
 public:
  CacheManager(int max_requests, const std::vector<GroupSpec>& groups);

  int open_request();             // slot index, or -1 when every slot is taken
  int close_request(int slot);    // gives back all pages and the slot; 0, or <0 if not open
  // Makes sure that tokens [length, new_len) have pages in every group.
  // All or nothing: 1 done, 0 not enough free pages (nothing changed), <0 bad arguments.
  int reserve(int slot, int new_len);
  // Largest L <= want_len such that reserve(slot, L) would succeed now (>= length).
  int fit_tokens(int slot, int want_len) const;
  // Tokens up to new_len are now in the cache; window groups release passed pages.
  int commit(int slot, int new_len);
  // Forgets tokens from len on and gives back pages no longer needed (ALL groups only
  // shrink; a window group cannot bring back released pages, so len must not go below
  // what its window still covers: returns <0 then).
  int truncate(int slot, int len);

  int length(int slot) const;
  int reserved_tokens(int slot) const;
  int generation(int slot) const;
  int table(int group, int slot, int32_t* out, int cap) const;  // page ids, -1 = released
  int free_pages(int group) const;
  int num_groups() const { return static_cast<int>(groups_.size()); }
  int num_pages(int group) const { return groups_[group].spec.num_pages; }
  int page_size(int group) const { return groups_[group].spec.page_size; }
  int max_requests() const { return static_cast<int>(slots_.size()); }
  // Pages a request of total_len tokens holds at most at one time in `group`.
  int peak_pages(int group, int total_len, int max_step) const;
  int64_t pages_taken_total() const { return pages_taken_; }
  int64_t pages_reused_total() const { return pages_reused_; }
  // 0 when every page of every group is either free once or held by exactly one table once.
  int audit() const;

 private:
  struct Group {
    GroupSpec spec;
    std::vector<int32_t> free_list;        // LIFO: the page freed last is used next
    std::vector<uint8_t> ever_used;
  };
  struct Slot {
    bool open = false;
    int length = 0;
    int reserved = 0;                       // tokens that have pages
    int generation = 0;
    std::vector<std::vector<int32_t>> tables;  // [group][page index] -> page id or -1
  };
  int first_needed_page(const Group& g, int length) const;
  bool valid(int slot) const { return slot >= 0 && slot < max_requests() && slots_[slot].open; }

  std::vector<Group> groups_;
  std::vector<Slot> slots_;
  std::vector<int> free_slots_;
  int64_t pages_taken_ = 0, pages_reused_ = 0;
};

}  // namespace srlm
