// The host side of the paged cache: a LIFO pool of page ids per group of calls with equal needs
// (all keys, or a window of them), a block table per live request and group, and request slots.
// Pages are taken as a request grows and go back when it ends, is preempted or truncated, or when
// a group's window has passed them.  (The reference takes all pages of a request at admission and
// returns them at its end, one position a page: src/scheduler.c:340-360, 222-225;
// src/gpt2.c:135-138, 158-182.)
#pragma once
#include <cstdint>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace sglc {

class PagePool {
 public:
  explicit PagePool(int n_pages = 0) { reset(n_pages); }
  void reset(int n_pages) {
    n_ = n_pages;
    free_.clear();
    held_.assign((size_t)n_pages, 0);
    for (int p = n_pages - 1; p >= 0; --p) free_.push_back(p);     // page 0 pops first
  }
  int n_pages() const { return n_; }
  int n_free() const { return (int)free_.size(); }
  // n pages appended to `out`, or false (nothing taken) if fewer are free
  bool alloc(int n, std::vector<int>* out) {
    if (n < 0 || n > (int)free_.size()) return false;
    for (int k = 0; k < n; ++k) {
      const int p = free_.back();
      free_.pop_back();
      held_[p] = 1;
      out->push_back(p);
    }
    return true;
  }
  // false: the page is outside the pool or not held (a double free)
  bool release(int page) {
    if (page < 0 || page >= n_ || !held_[page]) return false;
    held_[page] = 0;
    free_.push_back(page);                                          // the next one handed out
    return true;
  }
  bool held(int page) const { return page >= 0 && page < n_ && held_[page]; }
  // every page free exactly once or held
  bool check(std::string* why) const {
    std::vector<char> seen((size_t)n_, 0);
    for (int p : free_) {
      if (p < 0 || p >= n_ || seen[p]) return *why = "page " + std::to_string(p) + " is on the free stack twice", false;
      if (held_[p]) return *why = "page " + std::to_string(p) + " is free and held", false;
      seen[p] = 1;
    }
    int held = 0;
    for (char h : held_) held += h;
    if (held + (int)free_.size() != n_) return *why = "a page is neither free nor held", false;
    return true;
  }

 private:
  int n_ = 0;
  std::vector<int> free_;
  std::vector<char> held_;
};

struct CacheGroup {
  int window = 0;                         // 0: all keys
  PagePool pool;
};

struct RequestPages {
  int slot = -1;
  int length = 0;
  std::vector<std::vector<int>> tables;   // per group: page per block (-1 = given back behind the window)
};

class CacheTables {
 public:
  CacheTables(int page_size, int n_pages, int max_requests, const std::vector<int>& windows)
      : page_size_(page_size), n_pages_(n_pages), max_requests_(max_requests) {
    for (int w : windows) {
      groups_.emplace_back();
      groups_.back().window = w;
      groups_.back().pool.reset(n_pages);
    }
    for (int s = max_requests - 1; s >= 0; --s) free_slots_.push_back(s);
  }
  int page_size() const { return page_size_; }
  int n_pages() const { return n_pages_; }
  int n_groups() const { return (int)groups_.size(); }
  int n_free_slots() const { return (int)free_slots_.size(); }
  int n_free_pages() const {
    int m = n_pages_;
    for (const auto& g : groups_) m = g.pool.n_free() < m ? g.pool.n_free() : m;
    return m;
  }
  bool has(long long req) const { return reqs_.count(req) != 0; }
  int length(long long req) const { return reqs_.at(req).length; }
  int slot(long long req) const { return reqs_.at(req).slot; }
  const std::vector<int>& table(int group, long long req) const { return reqs_.at(req).tables[group]; }
  size_t n_live() const { return reqs_.size(); }

  // a slot and empty block tables; -1 when all slots are taken or the request is live already
  int add(long long req) {
    if (free_slots_.empty() || reqs_.count(req)) return -1;
    RequestPages r;
    r.slot = free_slots_.back();
    free_slots_.pop_back();
    r.tables.resize(groups_.size());
    const int slot = r.slot;
    reqs_.emplace(req, std::move(r));
    return slot;
  }
  bool free(long long req) {
    auto it = reqs_.find(req);
    if (it == reqs_.end()) return false;
    for (size_t g = 0; g < groups_.size(); ++g)
      for (int p : it->second.tables[g])
        if (p >= 0) groups_[g].pool.release(p);
    free_slots_.push_back(it->second.slot);
    reqs_.erase(it);
    return true;
  }
  // whether every (request, new length) of `wants` can grow in one step, counting the pages
  // that the windows have passed as free
  bool can_extend_all(const std::vector<std::pair<long long, int>>& wants) const {
    for (size_t g = 0; g < groups_.size(); ++g) {
      long long budget = groups_[g].pool.n_free();
      for (const auto& w : wants) {
        const RequestPages& r = reqs_.at(w.first);
        const std::vector<int>& t = r.tables[g];
        const int first = first_needed_block(groups_[g], r.length);
        for (int b = 0; b < first && b < (int)t.size(); ++b) budget += t[b] >= 0;
        const int need = blocks_for(w.second) - (int)t.size();
        if (need > 0) budget -= need;
      }
      if (budget < 0) return false;
    }
    return true;
  }
  // room for positions up to new_len (exclusive) in every group, all or nothing (but the pages
  // behind a window go back first either way)
  bool extend(long long req, int new_len) {
    RequestPages& r = reqs_.at(req);
    if (new_len < r.length) return false;
    for (size_t g = 0; g < groups_.size(); ++g) {
      std::vector<int>& t = r.tables[g];
      const int first = first_needed_block(groups_[g], r.length);
      for (int b = 0; b < first && b < (int)t.size(); ++b)
        if (t[b] >= 0) {
          groups_[g].pool.release(t[b]);
          t[b] = -1;
        }
    }
    for (size_t g = 0; g < groups_.size(); ++g)
      if (blocks_for(new_len) - (int)r.tables[g].size() > groups_[g].pool.n_free()) return false;
    for (size_t g = 0; g < groups_.size(); ++g) {
      const int need = blocks_for(new_len) - (int)r.tables[g].size();
      if (need > 0) groups_[g].pool.alloc(need, &r.tables[g]);
    }
    r.length = new_len;
    return true;
  }
  // forget what lies beyond new_len; pages filled by that alone go back.  false: not live, longer
  // than it is, or a page that new_len positions still need was given back behind a window
  bool truncate(long long req, int new_len) {
    auto it = reqs_.find(req);
    if (it == reqs_.end() || new_len < 0 || new_len > it->second.length) return false;
    RequestPages& r = it->second;
    const int keep = blocks_for(new_len);
    for (size_t g = 0; g < groups_.size(); ++g) {
      const std::vector<int>& t = r.tables[g];
      for (int b = first_needed_block(groups_[g], new_len); b < keep && b < (int)t.size(); ++b)
        if (t[b] < 0) return false;
    }
    for (size_t g = 0; g < groups_.size(); ++g) {
      std::vector<int>& t = r.tables[g];
      while ((int)t.size() > keep) {
        if (t.back() >= 0) groups_[g].pool.release(t.back());
        t.pop_back();
      }
    }
    r.length = new_len;
    return true;
  }
  // where position `pos` of the request lies in group g (page * page_size + offset), -1 if given back
  long long slot_of_position(int g, long long req, int pos) const {
    const std::vector<int>& t = reqs_.at(req).tables[g];
    const int b = pos / page_size_;
    if (b >= (int)t.size() || t[b] < 0) return -1;
    return (long long)t[b] * page_size_ + pos % page_size_;
  }
  // no page lost, held twice or freed twice; slots likewise
  bool check(std::string* why) const {
    for (size_t g = 0; g < groups_.size(); ++g) {
      if (!groups_[g].pool.check(why)) return false;
      std::vector<char> seen((size_t)n_pages_, 0);
      int held = 0;
      for (const auto& kv : reqs_)
        for (int p : kv.second.tables[g]) {
          if (p < 0) continue;
          if (p >= n_pages_ || seen[p]) return *why = "page " + std::to_string(p) + " is in two block tables", false;
          if (!groups_[g].pool.held(p)) return *why = "page " + std::to_string(p) + " is in a table and free", false;
          seen[p] = 1;
          ++held;
        }
      if (held + groups_[g].pool.n_free() != n_pages_) return *why = "a page is lost: neither free nor in a block table", false;
    }
    std::vector<char> s((size_t)max_requests_, 0);
    for (const auto& kv : reqs_) {
      if (kv.second.slot < 0 || kv.second.slot >= max_requests_ || s[kv.second.slot]) return *why = "a slot is held twice", false;
      s[kv.second.slot] = 1;
    }
    for (int f : free_slots_) {
      if (f < 0 || f >= max_requests_ || s[f]) return *why = "a slot is free and held", false;
      s[f] = 1;
    }
    if (reqs_.size() + free_slots_.size() != (size_t)max_requests_) return *why = "a slot is lost", false;
    return true;
  }

 private:
  int blocks_for(int n) const { return (n + page_size_ - 1) / page_size_; }
  int first_needed_block(const CacheGroup& g, int length) const {
    if (g.window <= 0) return 0;
    const int first_pos = length - g.window + 1;
    return first_pos > 0 ? first_pos / page_size_ : 0;
  }
  int page_size_, n_pages_, max_requests_;
  std::vector<CacheGroup> groups_;
  std::unordered_map<long long, RequestPages> reqs_;
  std::vector<int> free_slots_;
};

}  // namespace sglc
