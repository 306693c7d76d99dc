#include "runtime_c_api.h"

#include <vector>

#include "cache_manager.hpp"
#include "scheduler.hpp"

using srlm::CacheManager;
using srlm::Scheduler;

extern "C" {

void* srlm_cache_create(int max_requests, int n_groups, const int* kinds, const int* page_sizes,
                        const int* num_pages, const int* windows) {
  if (max_requests <= 0 || n_groups < 0) return nullptr;
  std::vector<srlm::GroupSpec> groups;
  for (int g = 0; g < n_groups; ++g) {
    if (page_sizes[g] <= 0 || num_pages[g] <= 0) return nullptr;
    if (kinds[g] == srlm::GROUP_WINDOW && windows[g] <= 0) return nullptr;
    groups.push_back(srlm::GroupSpec{kinds[g], page_sizes[g], num_pages[g], windows[g]});
  }
  return new CacheManager(max_requests, groups);
}
void srlm_cache_destroy(void* c) { delete static_cast<CacheManager*>(c); }
int srlm_cache_open(void* c) { return static_cast<CacheManager*>(c)->open_request(); }
int srlm_cache_close(void* c, int slot) { return static_cast<CacheManager*>(c)->close_request(slot); }
int srlm_cache_reserve(void* c, int slot, int n) { return static_cast<CacheManager*>(c)->reserve(slot, n); }
int srlm_cache_fit_tokens(void* c, int slot, int n) { return static_cast<CacheManager*>(c)->fit_tokens(slot, n); }
int srlm_cache_commit(void* c, int slot, int n) { return static_cast<CacheManager*>(c)->commit(slot, n); }
int srlm_cache_truncate(void* c, int slot, int n) { return static_cast<CacheManager*>(c)->truncate(slot, n); }
int srlm_cache_length(void* c, int slot) { return static_cast<CacheManager*>(c)->length(slot); }
int srlm_cache_reserved(void* c, int slot) { return static_cast<CacheManager*>(c)->reserved_tokens(slot); }
int srlm_cache_generation(void* c, int slot) { return static_cast<CacheManager*>(c)->generation(slot); }
int srlm_cache_table(void* c, int group, int slot, int32_t* out, int cap) {
  return static_cast<CacheManager*>(c)->table(group, slot, out, cap);
}
int srlm_cache_free_pages(void* c, int group) { return static_cast<CacheManager*>(c)->free_pages(group); }
int srlm_cache_audit(void* c) { return static_cast<CacheManager*>(c)->audit(); }
void srlm_cache_reuse_counts(void* c, int64_t* taken, int64_t* reused) {
  *taken = static_cast<CacheManager*>(c)->pages_taken_total();
  *reused = static_cast<CacheManager*>(c)->pages_reused_total();
}

void* srlm_sched_create(void* cache, int max_active, int queue_capacity, int prefill_chunk,
                        int max_batch_tokens, int max_context) {
  if (!cache || max_active <= 0 || queue_capacity <= 0 || prefill_chunk <= 0 ||
      max_batch_tokens <= 0 || max_context <= 0)
    return nullptr;
  srlm::SchedulerConfig cfg{max_active, queue_capacity, prefill_chunk, max_batch_tokens, max_context};
  return new Scheduler(cfg, static_cast<CacheManager*>(cache));
}
void srlm_sched_destroy(void* s) { delete static_cast<Scheduler*>(s); }
int srlm_sched_submit(void* s, int64_t id, int prompt_len, int max_new) {
  return static_cast<Scheduler*>(s)->submit(id, prompt_len, max_new);
}
int srlm_sched_plan(void* s, int64_t* entries, int cap, int64_t* preempted, int* n_preempted) {
  std::vector<srlm::PlanEntry> out;
  std::vector<int64_t> pre;
  static_cast<Scheduler*>(s)->plan(&out, &pre);
  int n = 0;
  for (const srlm::PlanEntry& e : out) {
    if (n >= cap) break;
    int64_t* row = entries + 5 * n++;
    row[0] = e.id; row[1] = e.slot; row[2] = e.start; row[3] = e.count; row[4] = e.want_logits;
  }
  int np = 0;
  for (int64_t id : pre) if (np < cap) preempted[np++] = id;
  *n_preempted = np;
  return n;
}
int srlm_sched_advance(void* s, int64_t id, int count) { return static_cast<Scheduler*>(s)->advance(id, count); }
int srlm_sched_rollback(void* s, int64_t id) { return static_cast<Scheduler*>(s)->rollback(id); }
int srlm_sched_append_token(void* s, int64_t id) { return static_cast<Scheduler*>(s)->append_token(id); }
int srlm_sched_retract_token(void* s, int64_t id) { return static_cast<Scheduler*>(s)->retract_token(id); }
int srlm_sched_finish(void* s, int64_t id) { return static_cast<Scheduler*>(s)->finish(id); }
int srlm_sched_has_work(void* s) { return static_cast<Scheduler*>(s)->has_work() ? 1 : 0; }
void srlm_sched_counters(void* s, int64_t* out) {
  srlm::Counters c = static_cast<Scheduler*>(s)->counters();
  out[0] = c.submitted; out[1] = c.rejected; out[2] = c.completed; out[3] = c.preempted;
  out[4] = c.steps; out[5] = c.batched_tokens; out[6] = c.generated_tokens;
  out[7] = c.active; out[8] = c.queued;
}

}  // extern "C"
