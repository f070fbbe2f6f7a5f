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
};

// What runs a planned step: the device engine, or a stand-in without a device.
class StepRunner {
 public:
  virtual ~StepRunner() {}
  // Runs the items' tokens as one batch over the cache (already grown for them) and samples one
  // token for every item with `sampled` set, in item order, with the uniforms given in that
  // order.  false with `err` set: nothing of the step counts.
  virtual bool run(const std::vector<StepItem>& items, const std::vector<double>& uniforms, bool want_logprobs,
                   std::vector<int>* tokens, std::vector<float>* logprobs, std::string* err) = 0;
};

class Scheduler {
 public:
  Scheduler(CacheTables* cache, StepRunner* runner, int vocab, int max_positions, int eos, uint64_t seed,
            int prefill_chunk, int token_budget, bool want_logprobs)
      : cache_(cache), runner_(runner), vocab_(vocab), max_positions_(max_positions), eos_(eos), seed_(seed),
        // the reference: SGL_PREFILL_CHUNK, default 512, <= 0 means 4096 (src/scheduler.c:138-143)
        prefill_chunk_(prefill_chunk > 0 ? prefill_chunk : 4096), token_budget_(token_budget),
        want_logprobs_(want_logprobs) {
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

  // Run one step; how many requests finished in it, or -1 with `err` set (nothing changed but
  // preemptions and admissions already made).
  int step(std::string* err) {
    std::vector<StepItem> chosen = plan_step();
    last_step_.clear();
    for (const StepItem& it : chosen) last_step_.push_back({it.r->id, it.n, it.sampled});
    if (chosen.empty()) return 0;
    for (const StepItem& it : chosen)
      if (!cache_->extend(it.r->id, it.old_len + it.n)) {            // (cannot happen after can_extend_all)
        roll_back(chosen);
        return *err = "the cache refused pages that it had promised", -1;
      }
    std::vector<double> us;
    std::vector<uint64_t> streams;            // as they were, should the step fail
    for (const StepItem& it : chosen)
      if (it.sampled) {
        streams.push_back(it.r->rng);
        us.push_back(it.r->sp.greedy() ? 0.0 : next_uniform(&it.r->rng));
      }
    std::vector<int> toks;
    std::vector<float> lps;
    if (!runner_->run(chosen, us, want_logprobs_, &toks, &lps, err) || toks.size() != us.size()) {
      if (err->empty()) *err = "the step gave fewer sampled tokens than it was asked for";
      size_t k = 0;
      for (const StepItem& it : chosen)
        if (it.sampled) it.r->rng = streams[k++];
      roll_back(chosen);
      return -1;
    }
    for (const StepItem& it : chosen) {
      if (it.old_len + it.n <= (int)it.r->prompt.size()) stats_.prefill_tokens += it.n;
      it.r->n_computed += it.n;
    }
    stats_.n_steps++;
    int finished = 0;
    size_t k = 0;
    for (const StepItem& it : chosen)
      if (it.sampled) {
        finished += append(it.r, toks[k], want_logprobs_ && k < lps.size() ? &lps[k] : nullptr) ? 1 : 0;
        ++k;
      }
    return finished;
  }

 private:
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
  bool append(Request* r, int tok, const float* logprob) {
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
    if (r->n_computed + 1 >= max_positions_) return end(FIN_CONTEXT);
    return false;
  }

  CacheTables* cache_;
  StepRunner* runner_;
  int vocab_, max_positions_, eos_;
  uint64_t seed_;
  int prefill_chunk_, token_budget_;
  bool want_logprobs_;
  long long next_id_ = 1;
  std::unordered_map<long long, std::unique_ptr<Request>> requests_;
  std::deque<Request*> waiting_;            // first come first served; preempted requests re-enter by arrival
  std::vector<Request*> running_;           // in order of arrival
  std::deque<Request*> done_;               // finished and not yet taken by poll
  SchedStats stats_;
  std::vector<Ran> last_step_;
};

}  // namespace sglc
