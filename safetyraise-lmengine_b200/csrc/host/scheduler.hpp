// Request scheduler: admission, portions of prompts under a token budget,
// decoding, finishing, and what happens when pages run out.
//
// The scheduler holds counts, not tokens: for every request how many tokens it
// has in all (prompt plus generated) and how many of them are in the cache.
// plan() packs one step: first one token for every request that is decoding,
// then portions of prompts, oldest request first, each at most prefill_chunk
// long, all within max_batch_tokens.  Pages for the step are reserved in
// plan(); the caller runs the step and reports back with advance().
//
// When pages run out: a prompt portion is cut to what fits, or waits.  If a
// decoding request cannot get its page, or nothing at all could be planned,
// the youngest running request is preempted: its pages and slot are given
// back, it returns to the head of the queue and will recompute its prompt and
// its generated tokens.  A request that could not fit even alone is refused at
// submit.  The oldest running request is never preempted, so it always ends.
//
// The reference bounds memory by a static budget at admission and has no such
// mechanism (src/engine/scheduler.rs:64-155, 830-940); admission, chunking
// and the finish reasons follow it (src/engine/scheduler.rs:389-487, 677-818).
#pragma once

#include <cstdint>
#include <deque>
#include <unordered_map>
#include <vector>

#include "cache_manager.hpp"

namespace srlm {

struct SchedulerConfig {
  int max_active;        // requests running at a time
  int queue_capacity;    // requests waiting at most; a submit beyond is refused
  int prefill_chunk;     // longest portion of one prompt in one step
  int max_batch_tokens;  // tokens of one step over all requests
  int max_context;       // prompt + generated tokens of one request at most
};

struct PlanEntry {
  int64_t id;
  int32_t slot;
  int32_t start;        // tokens already in the cache
  int32_t count;        // tokens to feed now: [start, start+count)
  int32_t want_logits;  // 1 when the last fed token is the request's last known token
};

enum SubmitStatus : int {
  SUBMIT_OK = 0,
  SUBMIT_QUEUE_FULL = -1,
  SUBMIT_TOO_LONG = -2,      // prompt + max_new exceeds max_context
  SUBMIT_NEVER_FITS = -3,    // would not fit the page pool even alone
  SUBMIT_INVALID = -4,       // empty prompt, max_new <= 0, duplicate id
};

struct Counters {
  int64_t submitted = 0, rejected = 0, completed = 0, preempted = 0, steps = 0,
          batched_tokens = 0, generated_tokens = 0, active = 0, queued = 0;
};

class Scheduler {
 public:
  Scheduler(const SchedulerConfig& cfg, CacheManager* cache) : cfg_(cfg), cache_(cache) {}

  int submit(int64_t id, int prompt_len, int max_new);
  // Fills `out` with the next step; ids of requests preempted while planning go to `preempted`.
  int plan(std::vector<PlanEntry>* out, std::vector<int64_t>* preempted);
  int advance(int64_t id, int count);   // the step ran: count more tokens are in the cache
  int rollback(int64_t id);             // the step failed: give back what plan() reserved
  int append_token(int64_t id);         // one sampled token joined the request
  int retract_token(int64_t id);        // the token counted last turned out not to join it (a stop token)
  int finish(int64_t id);               // any reason: frees pages and slot, forgets the request
  bool has_work() const { return !running_.empty() || !queue_.empty(); }
  Counters counters() const;

 private:
  struct Request {
    int64_t id;
    int prompt_len, max_new;
    int total_len;     // prompt + generated so far
    int fed;           // tokens in the cache
    int slot;          // -1 while queued
    int64_t order;     // admission order; larger = younger
  };
  bool preempt_youngest(std::vector<int64_t>* preempted);

  SchedulerConfig cfg_;
  CacheManager* cache_;
  std::unordered_map<int64_t, Request> requests_;
  std::deque<int64_t> queue_;
  std::vector<int64_t> running_;   // in admission order, oldest first
  int64_t next_order_ = 0;
  Counters counters_;
};

}  // namespace srlm
