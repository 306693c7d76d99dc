#include "scheduler.hpp"

#include <algorithm>

namespace srlm {

int Scheduler::submit(int64_t id, int prompt_len, int max_new) {
  counters_.submitted += 1;
  auto refuse = [&](int why) { counters_.rejected += 1; return why; };
  if (prompt_len <= 0 || max_new <= 0 || requests_.count(id)) return refuse(SUBMIT_INVALID);
  if (prompt_len + max_new > cfg_.max_context) return refuse(SUBMIT_TOO_LONG);
  for (int g = 0; g < cache_->num_groups(); ++g) {
    int step = std::min(cfg_.prefill_chunk, cfg_.max_batch_tokens);
    if (cache_->peak_pages(g, prompt_len + max_new, step) > cache_->num_pages(g))
      return refuse(SUBMIT_NEVER_FITS);
  }
  if (static_cast<int>(queue_.size()) >= cfg_.queue_capacity) return refuse(SUBMIT_QUEUE_FULL);
  Request r{id, prompt_len, max_new, prompt_len, 0, -1, -1};
  requests_.emplace(id, r);
  queue_.push_back(id);
  return SUBMIT_OK;
}

bool Scheduler::preempt_youngest(std::vector<int64_t>* preempted) {
  if (running_.size() < 2) return false;   // the oldest running request is never preempted
  int64_t victim = running_.back();
  running_.pop_back();
  Request& r = requests_[victim];
  cache_->close_request(r.slot);
  r.slot = -1;
  r.fed = 0;
  queue_.push_front(victim);
  counters_.preempted += 1;
  if (preempted) preempted->push_back(victim);
  return true;
}

int Scheduler::plan(std::vector<PlanEntry>* out, std::vector<int64_t>* preempted) {
  out->clear();
  int budget = cfg_.max_batch_tokens;
  bool any_preempted = false;

  auto is_decoding = [](const Request& r) {
    return r.total_len > r.prompt_len && r.total_len - r.fed == 1;
  };
  auto drop_planned = [&](int64_t id) {
    for (size_t i = 0; i < out->size(); ++i) {
      if ((*out)[i].id == id) {
        budget += (*out)[i].count;
        out->erase(out->begin() + i);
        return;
      }
    }
  };
  auto plan_portion = [&](Request& r) -> bool {
    int pending = r.total_len - r.fed;
    int count = std::min({cfg_.prefill_chunk, pending, budget});
    if (count <= 0) return false;
    count = std::min(count, cache_->fit_tokens(r.slot, r.fed + count) - r.fed);
    if (count <= 0) return false;
    if (cache_->reserve(r.slot, r.fed + count) != 1) return false;
    out->push_back(PlanEntry{r.id, r.slot, r.fed, count, r.fed + count == r.total_len ? 1 : 0});
    budget -= count;
    return true;
  };
  auto plan_running = [&]() {
    // one token for each request that is decoding, oldest first; a decoding request
    // that finds no page takes it from the youngest running request
    size_t i = 0;
    while (i < running_.size() && budget > 0) {
      Request& r = requests_[running_[i]];
      if (!is_decoding(r)) { ++i; continue; }
      int ok = cache_->reserve(r.slot, r.fed + 1);
      bool self_preempted = false;
      while (ok == 0 && running_.size() > 1) {
        int64_t victim = running_.back();
        preempt_youngest(preempted);
        any_preempted = true;
        drop_planned(victim);
        if (victim == r.id) { self_preempted = true; break; }
        ok = cache_->reserve(r.slot, r.fed + 1);
      }
      if (self_preempted) break;   // it was the last of the list
      if (ok == 1) {
        out->push_back(PlanEntry{r.id, r.slot, r.fed, 1, 1});
        budget -= 1;
      }
      ++i;
    }
    // portions of prompts (or of a recomputation after preemption), oldest first
    for (size_t k = 0; k < running_.size() && budget > 0; ++k) {
      Request& r = requests_[running_[k]];
      if (is_decoding(r) || r.total_len == r.fed) continue;
      plan_portion(r);
    }
  };

  plan_running();

  // admit from the queue while a first portion finds room; not in a step that preempted,
  // or the victim would come straight back and be thrown out again
  while (!any_preempted && budget > 0 && !queue_.empty() &&
         static_cast<int>(running_.size()) < cfg_.max_active) {
    Request& r = requests_[queue_.front()];
    int slot = cache_->open_request();
    if (slot < 0) break;
    // room for the whole first portion, or the request waits: a request that comes in on
    // the last free page would only be thrown out again
    const int first = std::min(cfg_.prefill_chunk, r.total_len);
    if (cache_->fit_tokens(slot, first) < first) {
      cache_->close_request(slot);
      break;
    }
    r.slot = slot;
    queue_.pop_front();
    r.order = next_order_++;
    running_.push_back(r.id);
    plan_portion(r);
  }

  // nothing to run although requests hold pages: the youngest gives way to the oldest
  while (out->empty() && running_.size() > 1) {
    preempt_youngest(preempted);
    any_preempted = true;
    plan_running();
  }

  if (!out->empty()) {
    counters_.steps += 1;
    for (const PlanEntry& e : *out) counters_.batched_tokens += e.count;
  }
  return static_cast<int>(out->size());
}

int Scheduler::advance(int64_t id, int count) {
  auto it = requests_.find(id);
  if (it == requests_.end() || it->second.slot < 0) return -1;
  Request& r = it->second;
  if (count < 0 || r.fed + count > r.total_len) return -2;
  if (cache_->commit(r.slot, r.fed + count) != 0) return -3;
  r.fed += count;
  return 0;
}

int Scheduler::rollback(int64_t id) {
  auto it = requests_.find(id);
  if (it == requests_.end() || it->second.slot < 0) return -1;
  return cache_->truncate(it->second.slot, it->second.fed);
}

int Scheduler::append_token(int64_t id) {
  auto it = requests_.find(id);
  if (it == requests_.end()) return -1;
  Request& r = it->second;
  if (r.total_len - r.prompt_len >= r.max_new) return -2;
  r.total_len += 1;
  counters_.generated_tokens += 1;
  return r.total_len - r.prompt_len;
}

int Scheduler::retract_token(int64_t id) {
  auto it = requests_.find(id);
  if (it == requests_.end()) return -1;
  Request& r = it->second;
  if (r.total_len <= r.prompt_len || r.fed >= r.total_len) return -2;   // nothing counted that was not fed yet
  r.total_len -= 1;
  counters_.generated_tokens -= 1;
  return r.total_len - r.prompt_len;
}

int Scheduler::finish(int64_t id) {
  auto it = requests_.find(id);
  if (it == requests_.end()) return -1;
  Request& r = it->second;
  if (r.slot >= 0) {
    cache_->close_request(r.slot);
    running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
  } else {
    queue_.erase(std::remove(queue_.begin(), queue_.end(), id), queue_.end());
  }
  requests_.erase(it);
  counters_.completed += 1;
  return 0;
}

Counters Scheduler::counters() const {
  Counters c = counters_;
  c.active = static_cast<int64_t>(running_.size());
  c.queued = static_cast<int64_t>(queue_.size());
  return c;
}

}  // namespace srlm
