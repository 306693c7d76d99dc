/* C interface of the host runtime (cache manager and scheduler), loaded from
 * Python with ctypes.  Handles are opaque pointers; every function returns a
 * status (>= 0 fine, < 0 an error named beside it in the C++ headers). */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

void* srlm_cache_create(int max_requests, int n_groups, const int* kinds, const int* page_sizes,
                        const int* num_pages, const int* windows);
void srlm_cache_destroy(void* cache);
int srlm_cache_open(void* cache);
int srlm_cache_close(void* cache, int slot);
int srlm_cache_reserve(void* cache, int slot, int new_len);
int srlm_cache_fit_tokens(void* cache, int slot, int want_len);
int srlm_cache_commit(void* cache, int slot, int new_len);
int srlm_cache_truncate(void* cache, int slot, int len);
int srlm_cache_length(void* cache, int slot);
int srlm_cache_reserved(void* cache, int slot);
int srlm_cache_generation(void* cache, int slot);
int srlm_cache_table(void* cache, int group, int slot, int32_t* out, int cap);
int srlm_cache_free_pages(void* cache, int group);
int srlm_cache_audit(void* cache);
void srlm_cache_reuse_counts(void* cache, int64_t* taken, int64_t* reused);

void* srlm_sched_create(void* cache, int max_active, int queue_capacity, int prefill_chunk,
                        int max_batch_tokens, int max_context);
void srlm_sched_destroy(void* sched);
int srlm_sched_submit(void* sched, int64_t id, int prompt_len, int max_new);
/* entries: 5 int64 per entry (id, slot, start, count, want_logits); returns the entry count,
 * writes the number of preempted ids to *n_preempted (ids in `preempted`, cap each). */
int srlm_sched_plan(void* sched, int64_t* entries, int cap, int64_t* preempted, int* n_preempted);
int srlm_sched_advance(void* sched, int64_t id, int count);
int srlm_sched_rollback(void* sched, int64_t id);
int srlm_sched_append_token(void* sched, int64_t id);
int srlm_sched_retract_token(void* sched, int64_t id);
int srlm_sched_finish(void* sched, int64_t id);
int srlm_sched_has_work(void* sched);
/* out[9]: submitted rejected completed preempted steps batched_tokens generated_tokens active queued */
void srlm_sched_counters(void* sched, int64_t* out);

#ifdef __cplusplus
}
#endif
