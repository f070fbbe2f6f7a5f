// The continuous-batching scheduler of the host engine.  It keeps the reference's request states,
// finishing rules, counters and entry-point names (src/scheduler.c: submit :170-215, admission
// :337-368, preemption :429-452, the step :454-523, appending a sample :288-310, stats
// include/sgl/scheduler.h:19-31) and differs where the step function allows more:
//   * a step is mixed: one token for every running request past its prompt, then prompt portions
//     (at most `prefill_chunk` tokens each) of requests still in their prompt and of newly
//     admitted ones, until the step's token budget is full;
//   * pages are taken as a request grows, not at admission;
//   * when a step's tokens need more pages than are free, requests are preempted from the latest
//     arrival backwards until the rest fits: a preempted request gives back its pages and its
//     slot, keeps what it has generated and its random stream, and waits; readmitted, it
//     recomputes prompt plus generated tokens and continues, so its output does not change.
//     Admission never preempts: a waiting request is admitted only into free pages and a free
//     slot, which rules out two requests evicting each other in turn;
//   * a request whose prompt plus max_new can never fit the pool or the model's positions is
//     refused at submit (the reference: src/scheduler.c:818-825).
// The decisions are those of engine/scheduler.py, which tests compare it with.
#pragma once
#include <algorithm>
#include <cstdint>
#include <deque>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "pages.hpp"

namespace sglc {

struct Sampling {                 // the reference's options (include/sgl/sampling.h:12-24)
  float temperature = 0.0f;       // <= 0: greedy
  int top_k = 0;                  // <= 0: off
  float top_p = 1.0f;             // outside (0,1): off
  float min_p = 0.0f;
  float repetition_penalty = 1.0f, frequency_penalty = 0.0f, presence_penalty = 0.0f;
  int ignore_eos = 0;
  int stop_ids[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int n_stop_ids = 0;
  unsigned long long seed = 0;
  bool greedy() const { return temperature <= 0.0f; }
  bool has_penalties() const {
    return (repetition_penalty > 0.0f && repetition_penalty != 1.0f) || frequency_penalty != 0.0f ||
           presence_penalty != 0.0f;
  }
  bool is_stop(int t) const {
    for (int i = 0; i < n_stop_ids && i < 8; ++i)
      if (stop_ids[i] == t) return true;
    return false;
  }
};

// The reference's generator: xorshift64* (src/sampling.c:10-21), a request's stream seeded
// through mix64 (src/scheduler.c:95-100,195), with the caller's seed mixed in.
inline uint64_t mix64(uint64_t x) {
  x ^= x >> 33; x *= 0xFF51AFD7ED558CCDull;
  x ^= x >> 33; x *= 0xC4CEB9FE1A85EC53ull;
  x ^= x >> 33;
  return x;
}
inline uint64_t request_stream(uint64_t seed, uint64_t request_id) {
  const uint64_t s = mix64(seed ^ mix64(request_id * 0x9E3779B97F4A7C15ull + 1));
  return s ? s : 0x9E3779B97F4A7C15ull;
}
inline double next_uniform(uint64_t* state) {      // u = (next >> 11) / 2^53 in [0,1)
  uint64_t x = *state;
  x ^= x >> 12; x ^= x << 25; x ^= x >> 27;
  *state = x;
  return (double)((x * 0x2545F4914F6CDD1Dull) >> 11) / 9007199254740992.0;
}

enum ReqState { REQ_WAITING = 0, REQ_RUNNING = 1, REQ_DONE = 2 };
enum FinishReason { FIN_NONE = 0, FIN_EOS = 1, FIN_STOP = 2, FIN_LENGTH = 3, FIN_CONTEXT = 4, FIN_ABORT = 5 };

struct Request {
  long long id = 0;
  std::vector<int> prompt, gen;
  std::vector<float> logprobs;
  int max_new = 16;
  Sampling sp;
  uint64_t rng = 0;
  int state = REQ_WAITING;
  int n_computed = 0;             // tokens of prompt + gen that are in the cache
  int n_preempted = 0;
  int finish = FIN_NONE;
  int n_tokens() const { return (int)(prompt.size() + gen.size()); }
  int n_pending() const { return n_tokens() - n_computed; }
  int token(int i) const { return i < (int)prompt.size() ? prompt[i] : gen[i - (int)prompt.size()]; }
};

struct StepItem {
  Request* r;
  int n;                          // tokens of this step
  int old_len;                    // what the request held before
  bool sampled;                   // the portion reaches the request's last token: a token is sampled
};

struct SchedStats {
  long long prefill_tokens = 0, decode_tokens = 0, n_finished = 0, n_running = 0, n_waiting = 0;
  long long pool_pages = 0, pool_free = 0, n_preempt = 0, prefill_chunk = 0, n_steps = 0, recomputed_tokens = 0;
  long long steps_ahead = 0;      // steps queued before the ids of the step ahead of them were read
};

// What runs a planned step: the device engine, or a stand-in without a device.
class StepRunner {
 public:
  virtual ~StepRunner() {}
  // Queues the items' tokens as one batch over the cache (already grown for them) and the sampling
  // of one token for every item with `sampled` set, in item order, with the uniforms given in that
  // order; returns without waiting.  With `ids_on_device` every item brings one token, and these
  // are the ids the launch before this one sampled, row for row, which the host has not seen: they
  // pass from the sampler's output to the step's token array on the device.  At most two launches
  // may be uncollected.  false with `err` set: nothing was queued.
  virtual bool launch(const std::vector<StepItem>& items, const std::vector<double>& uniforms, bool want_logprobs,
                      bool ids_on_device, int* ticket, std::string* err) = 0;
  // Waits for a launch and gives its sampled ids.  false with `err` set: nothing of that step
  // (or of a step queued behind it) counts.
  virtual bool collect(int ticket, std::vector<int>* tokens, std::vector<float>* logprobs, std::string* err) = 0;
};

class Scheduler {
 public:
  Scheduler(CacheTables* cache, StepRunner* runner, int vocab, int max_positions, int eos, uint64_t seed,
            int prefill_chunk, int token_budget, bool want_logprobs, bool run_ahead)
      : cache_(cache), runner_(runner), vocab_(vocab), max_positions_(max_positions), eos_(eos), seed_(seed),
        // the reference: SGL_PREFILL_CHUNK, default 512, <= 0 means 4096 (src/scheduler.c:138-143)
        prefill_chunk_(prefill_chunk > 0 ? prefill_chunk : 4096), token_budget_(token_budget),
        want_logprobs_(want_logprobs), run_ahead_(run_ahead) {
    stats_.prefill_chunk = prefill_chunk_;
    stats_.pool_pages = cache->n_pages();
  }

  // queue a request given as token ids; its id (from 1 up), or -1 if it can never run
  long long submit_ids(const int* ids, int n, int max_new, const Sampling* sp) {
    if (max_new <= 0) max_new = 16;                                   // src/scheduler.c:193
    if (n <= 0 || n >= max_positions_) return -1;
    for (int i = 0; i < n; ++i)
      if (ids[i] < 0 || ids[i] >= vocab_) return -1;
    const long long pool_tokens = (long long)cache_->n_pages() * cache_->page_size();
    const long long need = std::min<long long>((long long)n + max_new, max_positions_);
    if (need > pool_tokens) return -1;
    std::unique_ptr<Request> r(new Request());
    r->id = next_id_++;
    r->prompt.assign(ids, ids + n);
    r->max_new = max_new;
    if (sp) r->sp = *sp;
    if (r->sp.n_stop_ids > 8) r->sp.n_stop_ids = 8;
    r->rng = request_stream(seed_ ^ r->sp.seed, (uint64_t)r->id);
    waiting_.push_back(r.get());
    const long long id = r->id;
    requests_[id] = std::move(r);
    return id;
  }
  int nactive() const { return (int)(waiting_.size() + running_.size()); }
  // one finished request not yet taken, or null; poll_take drops it
  const Request* poll_peek() const { return done_.empty() ? nullptr : done_.front(); }
  void poll_take() {
    if (done_.empty()) return;
    requests_.erase(done_.front()->id);
    done_.pop_front();
  }
  const Request* find(long long id) const {
    auto it = requests_.find(id);
    return it == requests_.end() ? nullptr : it->second.get();
  }
  int abort(long long id) {
    auto it = requests_.find(id);
    if (it == requests_.end() || it->second->state == REQ_DONE) return -1;
    Request* r = it->second.get();
    if (r->state == REQ_RUNNING) {
      cache_->free(r->id);
      running_.erase(std::find(running_.begin(), running_.end(), r));
    } else {
      waiting_.erase(std::find(waiting_.begin(), waiting_.end(), r));
    }
    finish(r, FIN_ABORT, false);
    return 0;
  }
  // what the last call of step() ran: (request, tokens, whether a token was sampled)
  struct Ran {
    long long id;
    int n;
    bool sampled;
  };
  const std::vector<Ran>& last_step() const { return last_step_; }
  SchedStats stats() {
    stats_.n_running = (long long)running_.size();
    stats_.n_waiting = (long long)waiting_.size();
    stats_.pool_free = cache_->n_free_pages();
    return stats_;
  }

  // Decide the step: (request, tokens) pairs.  Preempts as needed; admits waiting requests into
  // free pages and slots.
  std::vector<StepItem> plan_step() {
    int budget = token_budget_;
    std::vector<StepItem> chosen;
    auto decoding = [](const Request* r) { return r->n_pending() == 1 && r->n_computed > 0; };
    // 1. one token for every running request past its prompt, then portions of those in it
    for (Request* r : running_)
      if (decoding(r) && budget > 0) {
        chosen.push_back({r, 1, r->n_computed, false});
        --budget;
      }
    for (Request* r : running_)
      if (!decoding(r) && budget > 0) {
        const int n = std::min(std::min(r->n_pending(), prefill_chunk_), budget);
        chosen.push_back({r, n, r->n_computed, false});
        budget -= n;
      }
    // 2. preempt from the latest arrival backwards until the chosen tokens fit
    bool preempted = false;
    while (!chosen.empty()) {
      if (cache_->can_extend_all(wants_of(chosen))) break;
      Request* victim = *std::max_element(running_.begin(), running_.end(),
                                          [](const Request* a, const Request* b) { return a->id < b->id; });
      chosen.erase(std::remove_if(chosen.begin(), chosen.end(), [&](const StepItem& it) { return it.r == victim; }),
                   chosen.end());
      preempt(victim);
      preempted = true;
    }
    // 3. admit waiting requests, first come first served, into what is free: never in a step
    //    that had to preempt, and only if all the request holds so far fits now
    while (!waiting_.empty() && budget > 0 && cache_->n_free_slots() > 0 && !preempted) {
      Request* r = waiting_.front();
      const int n = std::min(std::min(r->n_pending(), prefill_chunk_), budget);
      if (cache_->add(r->id) < 0) break;
      auto wants = wants_of(chosen);
      wants.emplace_back(r->id, r->n_pending());
      if (!cache_->can_extend_all(wants)) {
        cache_->free(r->id);
        break;
      }
      waiting_.pop_front();
      r->state = REQ_RUNNING;
      running_.insert(std::upper_bound(running_.begin(), running_.end(), r,
                                       [](const Request* a, const Request* b) { return a->id < b->id; }),
                      r);
      chosen.push_back({r, n, r->n_computed, false});
      budget -= n;
    }
    for (StepItem& it : chosen) it.sampled = it.r->n_computed + it.n == it.r->n_tokens();
    return chosen;
  }

  // Run one step; how many requests finished in this call, or -1 with `err` set (the cache is as
  // before the failed step).
  //
  // With run_ahead, a step's sampled ids are read one call later: while every running request
  // just decodes (none waits, none can end by its length, none has penalties, pages suffice), a
  // call first queues the next step of single tokens behind the step in flight (its ids pass from
  // the sampler to the token array on the device), then waits for the ids of the step in flight
  // and appends them.  So the device always has the next step queued while the host does its
  // bookkeeping.  Whatever changes the set of running requests sends the next call down the plain
  // path: wait, plan, launch.  A request that ends while a step with it is queued has that step's
  // id dropped.
  int step(std::string* err) {
    int finished = 0;
    if (flight_.active) {
      Flight next;
      if (run_ahead_ && can_run_ahead() && launch(decode_items(), true, &next, err)) {
        const int f = collect(&flight_, &next, err);
        if (f < 0) return -1;
        flight_ = next;
        stats_.steps_ahead++;
        return f;
      }
      err->clear();
      finished = collect(&flight_, nullptr, err);
      if (finished < 0) return -1;
    }
    std::vector<StepItem> chosen = plan_step();
    if (chosen.empty()) {
      last_step_.clear();
      return finished;
    }
    Flight now;
    if (!launch(chosen, false, &now, err)) return -1;
    if (!run_ahead_) {
      const int f = collect(&now, nullptr, err);
      return f < 0 ? -1 : finished + f;
    }
    flight_ = now;
    return finished;
  }
  // a step may still be in flight when the caller asks whether anything is active
  bool in_flight() const { return flight_.active; }
  // wait for the step in flight, if any, and append its ids; requests ended by it, or -1
  int drain(std::string* err) {
    if (!flight_.active) return 0;
    return collect(&flight_, nullptr, err);
  }
  // Forget what a running request has generated beyond its first `keep` ids (and what the cache
  // holds of it); it goes on from there.  For measurements that time the same steps again and
  // again.  false: no such running request, a step in flight, or nothing to keep it running.
  bool rewind(long long id, int keep) {
    auto it = requests_.find(id);
    if (it == requests_.end() || flight_.active) return false;
    Request* r = it->second.get();
    if (r->state != REQ_RUNNING || keep < 1 || keep > (int)r->gen.size()) return false;
    const int n = (int)r->prompt.size() + keep - 1;           // the last kept id is not computed yet
    if (n > r->n_computed || !cache_->truncate(r->id, n)) return false;
    r->gen.resize((size_t)keep);
    if (r->logprobs.size() > (size_t)keep) r->logprobs.resize((size_t)keep);
    r->n_computed = n;
    return true;
  }

 private:
  struct FlightItem {
    long long id;
    int n, old_len;
    bool sampled;
    uint64_t stream;          // the request's random stream before this step drew from it
  };
  struct Flight {
    bool active = false, all_decode = false;
    int ticket = 0;
    std::vector<FlightItem> items;
  };

  // every running request was sampled in the step in flight, in this order, as a single token;
  // none waits; none can end by its length or the model's positions with the id in flight; none
  // needs its history on the host; and one more position for each fits the free pages
  bool can_run_ahead() const {
    if (!flight_.all_decode || !waiting_.empty() || running_.empty() || flight_.items.size() != running_.size()) return false;
    std::vector<std::pair<long long, int>> wants;
    for (size_t i = 0; i < running_.size(); ++i) {
      const Request* r = running_[i];
      if (r->id != flight_.items[i].id || r->sp.has_penalties()) return false;
      if ((int)r->gen.size() + 2 > r->max_new || r->n_computed + 2 > max_positions_) return false;
      wants.emplace_back(r->id, r->n_computed + 1);
    }
    return (int)running_.size() <= token_budget_ && cache_->can_extend_all(wants);
  }
  std::vector<StepItem> decode_items() const {
    std::vector<StepItem> items;
    for (Request* r : running_) items.push_back({r, 1, r->n_computed, true});
    return items;
  }

  // grow the cache, draw the uniforms and queue the step; on failure everything is as before
  bool launch(const std::vector<StepItem>& chosen, bool ids_on_device, Flight* f, std::string* err) {
    last_step_.clear();
    for (const StepItem& it : chosen) last_step_.push_back({it.r->id, it.n, it.sampled});
    for (const StepItem& it : chosen)
      if (!cache_->extend(it.r->id, it.old_len + it.n)) {            // (cannot happen after can_extend_all)
        roll_back(chosen);
        return *err = "the cache refused pages that it had promised", false;
      }
    std::vector<double> us;
    f->items.clear();
    f->all_decode = true;
    for (const StepItem& it : chosen) {
      f->items.push_back({it.r->id, it.n, it.old_len, it.sampled, it.r->rng});
      f->all_decode = f->all_decode && it.n == 1 && it.sampled;
      if (it.sampled) us.push_back(it.r->sp.greedy() ? 0.0 : next_uniform(&it.r->rng));
    }
    if (!runner_->launch(chosen, us, want_logprobs_, ids_on_device, &f->ticket, err)) {
      for (size_t i = 0; i < chosen.size(); ++i) chosen[i].r->rng = f->items[i].stream;
      roll_back(chosen);
      return false;
    }
    for (const StepItem& it : chosen) {
      if (it.old_len + it.n <= (int)it.r->prompt.size()) stats_.prefill_tokens += it.n;
      it.r->n_computed += it.n;
    }
    stats_.n_steps++;
    f->active = true;
    return true;
  }

  // Wait for a step's ids and append them; how many requests ended, or -1: the step (and `behind`,
  // a step queued after it) is undone.
  int collect(Flight* f, Flight* behind, std::string* err) {
    std::vector<int> toks;
    std::vector<float> lps;
    size_t n_sampled = 0;
    for (const FlightItem& it : f->items) n_sampled += it.sampled;
    f->active = false;
    if (!runner_->collect(f->ticket, &toks, &lps, err) || toks.size() != n_sampled) {
      if (err->empty()) *err = "the step gave fewer sampled tokens than it was asked for";
      if (behind && behind->active) {
        std::string ignored;
        std::vector<int> t2;
        std::vector<float> l2;
        runner_->collect(behind->ticket, &t2, &l2, &ignored);        // drain it; its ids rest on bad ones
        undo(*behind);
        behind->active = false;
      }
      undo(*f);
      return -1;
    }
    int finished = 0;
    size_t k = 0;
    for (const FlightItem& it : f->items) {
      if (!it.sampled) continue;
      const size_t row = k++;
      auto found = requests_.find(it.id);
      // ended or aborted after this step was queued: its id is dropped
      if (found == requests_.end() || found->second->state != REQ_RUNNING) continue;
      Request* r = found->second.get();
      finished += append(r, toks[row], want_logprobs_ && row < lps.size() ? &lps[row] : nullptr, it.old_len + it.n) ? 1 : 0;
    }
    return finished;
  }
  // a failed step: lengths, counters and random streams as before it
  void undo(const Flight& f) {
    for (const FlightItem& it : f.items) {
      auto found = requests_.find(it.id);
      if (found == requests_.end() || found->second->state != REQ_RUNNING) continue;
      Request* r = found->second.get();
      if (cache_->has(r->id) && cache_->length(r->id) > it.old_len) cache_->truncate(r->id, it.old_len);
      if (r->n_computed > it.old_len) r->n_computed = it.old_len;
      r->rng = it.stream;
    }
  }

  static std::vector<std::pair<long long, int>> wants_of(const std::vector<StepItem>& chosen) {
    std::vector<std::pair<long long, int>> w;
    for (const StepItem& it : chosen) w.emplace_back(it.r->id, it.old_len + it.n);
    return w;
  }
  void roll_back(const std::vector<StepItem>& chosen) {
    // the requests were grown for tokens whose keys and values were never written
    for (const StepItem& it : chosen)
      if (cache_->has(it.r->id) && cache_->length(it.r->id) > it.old_len) cache_->truncate(it.r->id, it.old_len);
  }
  void finish(Request* r, int reason, bool free_pages) {
    if (free_pages && cache_->has(r->id)) cache_->free(r->id);
    r->state = REQ_DONE;
    r->finish = reason;
    done_.push_back(r);
    stats_.n_finished++;
  }
  void preempt(Request* r) {
    cache_->free(r->id);
    running_.erase(std::find(running_.begin(), running_.end(), r));
    stats_.recomputed_tokens += r->n_computed;
    r->n_computed = 0;
    r->n_preempted++;
    r->state = REQ_WAITING;
    stats_.n_preempt++;
    // back into the queue by arrival order, so it is readmitted before later arrivals
    auto at = waiting_.begin();
    while (at != waiting_.end() && (*at)->id < r->id) ++at;
    waiting_.insert(at, r);
  }
  // The reference's req_sample_append (src/scheduler.c:288-310): eos or a stop id ends the
  // request without being appended; then max_new and the model's positions.
  // n_computed: the request's tokens in the cache after the step that gave `tok` (a later step
  // may be queued already).
  bool append(Request* r, int tok, const float* logprob, int n_computed) {
    auto end = [&](int reason) {
      running_.erase(std::find(running_.begin(), running_.end(), r));
      finish(r, reason, true);
      return true;
    };
    if (eos_ >= 0 && tok == eos_ && !r->sp.ignore_eos) return end(FIN_EOS);
    if (r->sp.is_stop(tok)) return end(FIN_STOP);
    r->gen.push_back(tok);
    if (logprob) r->logprobs.push_back(*logprob);
    stats_.decode_tokens++;
    if ((int)r->gen.size() >= r->max_new) return end(FIN_LENGTH);
    if (n_computed + 1 >= max_positions_) return end(FIN_CONTEXT);
    return false;
  }

  CacheTables* cache_;
  StepRunner* runner_;
  int vocab_, max_positions_, eos_;
  uint64_t seed_;
  int prefill_chunk_, token_budget_;
  bool want_logprobs_;
  bool run_ahead_;
  Flight flight_;
  long long next_id_ = 1;
  std::unordered_map<long long, std::unique_ptr<Request>> requests_;
  std::deque<Request*> waiting_;            // first come first served; preempted requests re-enter by arrival
  std::vector<Request*> running_;           // in order of arrival
  std::deque<Request*> done_;               // finished and not yet taken by poll
  SchedStats stats_;
  std::vector<Ran> last_step_;
};

}  // namespace sglc
