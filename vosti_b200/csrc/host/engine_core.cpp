// Host-side core of the engine in C++: page pools, the cache manager's accounting and the
// continuous-batching scheduler. The Python classes in vosti_b200/cache and
// vosti_b200/engine are thin faces over this library (C ABI, loaded with ctypes); device
// storage stays with the Python side.
//
// Behaviour follows the reference's Rust cache scheduler (src/exec/cache_scheduler/*):
// vacant page ids start in order and a released page is the next one handed out
// (availability_queue.rs:746-780, 377, 246); published prefix pages that nobody holds wait
// in an eviction queue, leaves first, and are evicted only under pressure
// (reclamation.rs:13-334, eviction_policy.rs:34-65); a prefix match compares depth, parent
// and every token, the hash is only an index (prefix_cache.rs:3155-3469); planning takes
// decode rows first as a prefix of the running queue, then the head of the waiting queue
// only, and cuts prompts into whole pages under the token budget (planning.rs:11-49,
// 247-338, 1002-1091). Decided here and not in the reference: pages are reserved per
// portion and kept between portions, and when no row at all fits the youngest running
// request is preempted and recomputed later.
#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <list>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#define VH_API extern "C" __attribute__((visibility("default")))

namespace {

enum Code : int {
  VH_OK = 0,
  VH_OUT_OF_PAGES = -1,
  VH_ACCOUNTING = -2,
  VH_BAD_ARGUMENT = -3,
  VH_OUT_OF_SLOTS = -4,
  VH_UNKNOWN_REQUEST = -5,
};

thread_local char g_error[512] = "";
int fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return code;
}

constexpr int RELEASED = -1;

uint64_t chain_hash(uint64_t previous, const int32_t* tokens, int count) {
  uint64_t h = previous ^ 0xCBF29CE484222325ull;
  for (int i = 0; i < count; ++i) {
    h ^= (uint64_t)(int64_t)tokens[i];
    h *= 0x100000001B3ull;
  }
  return h ? h : 1;
}

struct Published {
  std::vector<int32_t> tokens;
  uint64_t hash = 0;
  int depth = 0, parent = -1;
};

class PagePool {
 public:
  explicit PagePool(int pages) : num_pages(pages), refcount(pages, 0), in_evictable(pages) {
    for (int i = 0; i < pages; ++i) free_list.push_back(i);
  }
  int available() const { return (int)free_list.size() + (int)evictable.size(); }

  int allocate(int count, std::vector<int>* out) {
    if (count < 0) return fail(VH_BAD_ARGUMENT, "cannot allocate a negative number of pages");
    if (count > available()) return fail(VH_OUT_OF_PAGES, "%d pages wanted, %d available", count, available());
    while ((int)free_list.size() < count) evict_one();
    for (int i = 0; i < count; ++i) {
      const int page = free_list.front();
      free_list.pop_front();
      if (refcount[page] != 0) return fail(VH_ACCOUNTING, "vacant page %d has holders", page);
      refcount[page] = 1;
      out->push_back(page);
    }
    return VH_OK;
  }
  int acquire(int page) {
    if (page < 0 || page >= num_pages) return fail(VH_ACCOUNTING, "page %d does not exist", page);
    if (refcount[page] == 0) {
      if (!in_evictable[page].second) return fail(VH_ACCOUNTING, "page %d is vacant and cannot be acquired", page);
      evictable.erase(in_evictable[page].first);
      in_evictable[page].second = false;
    }
    ++refcount[page];
    return VH_OK;
  }
  int release(int page) {
    if (page < 0 || page >= num_pages || refcount[page] <= 0)
      return fail(VH_ACCOUNTING, "page %d released but not held", page);
    if (--refcount[page] == 0) {
      if (published.count(page)) {
        evictable.push_back(page);
        in_evictable[page] = {std::prev(evictable.end()), true};
      } else {
        free_list.push_front(page);
      }
    }
    return VH_OK;
  }
  // Returns the hash of the page; *parent_out is the page a following page names as parent.
  uint64_t publish(int page, const int32_t* tokens, int count, uint64_t previous, int depth, int parent, int* parent_out) {
    const uint64_t h = chain_hash(previous, tokens, count);
    *parent_out = page;
    if (published.count(page)) return h;
    auto owner = hash_to_page.find(h);
    if (owner != hash_to_page.end()) {
      const Published& twin = published[owner->second];
      if (twin.depth == depth && twin.parent == parent && (int)twin.tokens.size() == count &&
          std::equal(twin.tokens.begin(), twin.tokens.end(), tokens))
        *parent_out = owner->second;               // equal content: chain through the first writer
      return h;                                    // (else a true collision: this page stays private)
    }
    Published p;
    p.tokens.assign(tokens, tokens + count);
    p.hash = h;
    p.depth = depth;
    p.parent = parent;
    published[page] = std::move(p);
    hash_to_page[h] = page;
    return h;
  }
  void match(const int32_t* tokens, int count, int page_size, std::vector<int>* out) const {
    uint64_t previous = 0;
    int parent = -1;
    const int limit = count > 0 ? (count - 1) / page_size : 0;
    for (int j = 0; j < limit; ++j) {
      const int32_t* chunk = tokens + (int64_t)j * page_size;
      const uint64_t h = chain_hash(previous, chunk, page_size);
      auto it = hash_to_page.find(h);
      if (it == hash_to_page.end()) break;
      const Published& info = published.at(it->second);
      if (info.depth != j + 1 || info.parent != parent || (int)info.tokens.size() != page_size ||
          !std::equal(info.tokens.begin(), info.tokens.end(), chunk))
        break;
      out->push_back(it->second);
      previous = h;
      parent = it->second;
    }
  }
  int check(const std::map<int, int>& holders) const {
    std::vector<char> seen(num_pages, 0);
    for (int page : free_list) {
      if (seen[page] || refcount[page] != 0 || published.count(page))
        return fail(VH_ACCOUNTING, "page %d is in the free list wrongly", page);
      seen[page] = 1;
    }
    for (int page : evictable) {
      if (seen[page] || refcount[page] != 0 || !published.count(page))
        return fail(VH_ACCOUNTING, "page %d is in the evictable queue wrongly", page);
      seen[page] = 1;
    }
    int count_seen = 0;
    for (int page = 0; page < num_pages; ++page) {
      auto it = holders.find(page);
      const int count = it == holders.end() ? 0 : it->second;
      if (refcount[page] != count)
        return fail(VH_ACCOUNTING, "page %d: reference count %d, %d holders", page, refcount[page], count);
      if (count > 0) {
        if (seen[page]) return fail(VH_ACCOUNTING, "page %d is held and also vacant", page);
        seen[page] = 1;
      }
      count_seen += seen[page];
    }
    if (count_seen != num_pages) return fail(VH_ACCOUNTING, "pages lost: %d of %d accounted for", count_seen, num_pages);
    for (auto& kv : hash_to_page) {
      auto it = published.find(kv.second);
      if (it == published.end() || it->second.hash != kv.first)
        return fail(VH_ACCOUNTING, "hash index names page %d wrongly", kv.second);
    }
    return VH_OK;
  }

  int num_pages;
  std::deque<int> free_list;
  std::vector<int> refcount;
  std::map<int, Published> published;
  std::unordered_map<uint64_t, int> hash_to_page;
  std::list<int> evictable;                               // oldest first
  std::vector<std::pair<std::list<int>::iterator, bool>> in_evictable;
  int64_t evictions = 0;

 private:
  void evict_one() {
    const int page = evictable.front();
    evictable.pop_front();
    in_evictable[page].second = false;
    auto it = published.find(page);
    auto owner = hash_to_page.find(it->second.hash);
    if (owner != hash_to_page.end() && owner->second == page) hash_to_page.erase(owner);
    published.erase(it);
    free_list.push_front(page);
    ++evictions;
  }
};

struct Residency {
  int64_t id = 0;
  int slot = 0, length = 0, cached_prefix_pages = 0, published_pages = 0, last_parent = -1;
  uint64_t last_hash = 0;
  std::vector<std::vector<int>> pages;
};

class CacheCore {
 public:
  CacheCore(int groups, const int* group_windows, int pages, int page, int requests, bool reuse, bool has_state)
      : page_size(page), num_pages(pages), max_requests(requests), has_state(has_state) {
    for (int g = 0; g < groups; ++g) {
      windows.push_back(group_windows[g]);
      pools.emplace_back(new PagePool(pages));
    }
    prefix_reuse = reuse && groups == 1 && windows[0] == 0 && !has_state;
    for (int s = requests - 1; s >= 0; --s) free_slots.push_back(s);
  }
  int pages_for(int tokens) const { return (tokens + page_size - 1) / page_size; }
  int available_pages() const {
    int best = num_pages;
    for (auto& p : pools) best = std::min(best, p->available());
    return best;
  }
  Residency* find(int64_t id) {
    auto it = live.find(id);
    return it == live.end() ? nullptr : &it->second;
  }
  int begin(int64_t id, const int32_t* prompt, int count) {
    if (live.count(id)) return fail(VH_BAD_ARGUMENT, "request is already live");
    if (free_slots.empty()) return fail(VH_OUT_OF_SLOTS, "all %d request slots are taken", max_requests);
    Residency res;
    res.id = id;
    res.slot = free_slots.back();
    free_slots.pop_back();
    res.pages.resize(pools.size());
    if (prefix_reuse && prompt != nullptr && count > 0) {
      std::vector<int> matched;
      pools[0]->match(prompt, count, page_size, &matched);
      for (int page : matched) {
        const int rc = pools[0]->acquire(page);
        if (rc != VH_OK) return rc;
      }
      if (!matched.empty()) {
        res.pages[0] = matched;
        res.length = (int)matched.size() * page_size;
        res.cached_prefix_pages = res.published_pages = (int)matched.size();
        res.last_hash = pools[0]->published.at(matched.back()).hash;
        res.last_parent = matched.back();
        reused_prefix_pages += (int64_t)matched.size();
        ++requests_with_reuse;
      }
    }
    const int slot = res.slot;
    live[id] = std::move(res);
    // A slot of per-request state still holds what its last tenant left: whoever owns the
    // device storage takes this list before the next step and clears those slots.
    if (has_state) fresh_slots.push_back(slot);
    return slot;
  }
  int pages_needed(const Residency& res, int new_tokens) const {
    const int need = pages_for(res.length + new_tokens);
    int most = 0;
    for (size_t g = 0; g < pools.size(); ++g) most = std::max(most, need - (int)res.pages[g].size());
    return most;
  }
  bool can_extend(const Residency& res, int new_tokens) const {
    const int need = pages_for(res.length + new_tokens);
    for (size_t g = 0; g < pools.size(); ++g)
      if (need - (int)res.pages[g].size() > pools[g]->available()) return false;
    return true;
  }
  // slots_out: [groups][new_tokens]
  int extend(Residency& res, int new_tokens, int32_t* slots_out) {
    if (new_tokens <= 0) return fail(VH_BAD_ARGUMENT, "extend needs at least one token");
    if (!can_extend(res, new_tokens)) return fail(VH_OUT_OF_PAGES, "not enough pages for %d more tokens", new_tokens);
    const int need = pages_for(res.length + new_tokens);
    for (size_t g = 0; g < pools.size(); ++g) {
      const int extra = need - (int)res.pages[g].size();
      if (extra > 0) {
        const int rc = pools[g]->allocate(extra, &res.pages[g]);
        if (rc != VH_OK) return rc;
      }
      if (slots_out) {
        for (int i = 0; i < new_tokens; ++i) {
          const int pos = res.length + i;
          slots_out[g * (int64_t)new_tokens + i] = res.pages[g][pos / page_size] * page_size + pos % page_size;
        }
      }
    }
    res.length += new_tokens;
    return VH_OK;
  }
  int trim(Residency& res) {
    int freed = 0;
    for (size_t g = 0; g < pools.size(); ++g) {
      if (windows[g] <= 0) continue;
      const int first_needed = res.length - windows[g] + 1;
      if (first_needed <= 0) continue;
      const int upto = std::min(first_needed / page_size, (int)res.pages[g].size());
      for (int index = 0; index < upto; ++index) {
        if (res.pages[g][index] != RELEASED) {
          const int rc = pools[g]->release(res.pages[g][index]);
          if (rc != VH_OK) return rc;
          res.pages[g][index] = RELEASED;
          ++freed;
        }
      }
    }
    return freed;
  }
  int publish(Residency& res, const int32_t* tokens, int count) {
    if (!prefix_reuse) return 0;
    const int full = res.length / page_size;
    if (count < full * page_size) return fail(VH_BAD_ARGUMENT, "publish needs the tokens of every full page");
    int done = 0;
    while (res.published_pages < full) {
      const int i = res.published_pages;
      int parent_out = -1;
      res.last_hash = pools[0]->publish(res.pages[0][i], tokens + (int64_t)i * page_size, page_size, res.last_hash,
                                        i + 1, res.last_parent, &parent_out);
      res.last_parent = parent_out;
      ++res.published_pages;
      ++done;
    }
    return done;
  }
  int finish(int64_t id) {
    auto it = live.find(id);
    if (it == live.end()) return fail(VH_UNKNOWN_REQUEST, "request is not live");
    Residency& res = it->second;
    for (size_t g = 0; g < pools.size(); ++g)
      for (auto page = res.pages[g].rbegin(); page != res.pages[g].rend(); ++page)   // leaves before their parents
        if (*page != RELEASED) {
          const int rc = pools[g]->release(*page);
          if (rc != VH_OK) return rc;
        }
    free_slots.push_back(res.slot);
    live.erase(it);
    return VH_OK;
  }
  int check() const {
    std::set<int> slots;
    for (auto& kv : live)
      if (!slots.insert(kv.second.slot).second) return fail(VH_ACCOUNTING, "a state slot is held twice");
    for (int s : free_slots)
      if (slots.count(s)) return fail(VH_ACCOUNTING, "a state slot is held and also free");
    if ((int)(slots.size() + free_slots.size()) != max_requests) return fail(VH_ACCOUNTING, "a state slot was lost");
    for (size_t g = 0; g < pools.size(); ++g) {
      std::map<int, int> holders;
      for (auto& kv : live) {
        std::set<int> own;
        for (int page : kv.second.pages[g]) {
          if (page == RELEASED) continue;
          if (!own.insert(page).second) return fail(VH_ACCOUNTING, "a request lists page %d twice", page);
          ++holders[page];
        }
      }
      if (!prefix_reuse)
        for (auto& kv : holders)
          if (kv.second > 1) return fail(VH_ACCOUNTING, "page %d is held by two requests without prefix reuse", kv.first);
      const int rc = pools[g]->check(holders);
      if (rc != VH_OK) return rc;
    }
    return VH_OK;
  }

  int page_size, num_pages, max_requests;
  bool has_state = false;
  std::vector<int> fresh_slots;                           // handed out by begin() since they were last taken
  bool prefix_reuse = false;
  std::vector<int> windows;
  std::vector<std::unique_ptr<PagePool>> pools;
  std::map<int64_t, Residency> live;
  std::vector<int> free_slots;
  int64_t reused_prefix_pages = 0, requests_with_reuse = 0;
};

// ------------------------------------------------------------------ scheduler
enum Admission : int {
  ACCEPTED = 0, DUPLICATE_ID = 1, EMPTY_PROMPT = 2, BAD_EOS = 3, ZERO_BUDGET = 4, TOO_LONG = 5, BAD_TOKEN = 6,
  BAD_SAMPLING = 7,
};
enum FinishReason : int { NOT_FINISHED = 0, LENGTH = 1, EOS = 2, CAPACITY = 3, ABORTED = 4 };

struct Request {
  int64_t id = 0;
  std::vector<int32_t> tokens;          // prompt followed by what was generated
  int prompt_len = 0, max_tokens = 0, computed = 0, preemptions = 0, finish_reason = NOT_FINISHED;
  int32_t eos[3] = {0, 0, 0};
  int n_eos = 0;
  bool ignore_eos = false;
  int generated() const { return (int)tokens.size() - prompt_len; }
  int remaining() const { return (int)tokens.size() - computed; }
  bool decoding() const { return generated() > 0 && remaining() == 1; }
};

struct PlanRow {
  int64_t id;
  int32_t start, count, sample;
};

class SchedulerCore {
 public:
  SchedulerCore(CacheCore* cache, int max_seqs, int budget, int chunk, int vocab, int context)
      : cache(cache), max_num_seqs(max_seqs), max_batched_tokens(budget), chunk_size(chunk), vocab_size(vocab),
        max_context(context) {}

  int add(int64_t id, const int32_t* prompt, int count, int max_tokens, const int32_t* eos, int n_eos, bool ignore_eos,
          float temperature) {
    if (accepted.count(id)) return DUPLICATE_ID;
    if (count <= 0) return EMPTY_PROMPT;
    if (!ignore_eos && (n_eos < 1 || n_eos > 3)) return BAD_EOS;
    if (n_eos > 3) return BAD_EOS;
    if (max_tokens <= 0) return ZERO_BUDGET;
    if (!(temperature >= 0.0f && temperature < 3.0e38f)) return BAD_SAMPLING;
    if (max_context && count + max_tokens > max_context) return TOO_LONG;
    if (vocab_size)
      for (int i = 0; i < count; ++i)
        if (prompt[i] < 0 || prompt[i] >= vocab_size) return BAD_TOKEN;
    accepted.insert(id);
    auto request = std::make_shared<Request>();
    request->id = id;
    request->tokens.assign(prompt, prompt + count);
    request->prompt_len = count;
    request->max_tokens = max_tokens;
    request->n_eos = n_eos;
    for (int i = 0; i < n_eos; ++i) request->eos[i] = eos[i];
    request->ignore_eos = ignore_eos;
    requests[id] = request;
    waiting.push_back(request);
    return ACCEPTED;
  }
  bool abort(int64_t id) {
    for (auto* queue : {&waiting, &running}) {
      for (auto it = queue->begin(); it != queue->end(); ++it) {
        if ((*it)->id == id) {
          auto request = *it;
          queue->erase(it);
          if (cache->find(id)) cache->finish(id);
          request->finish_reason = ABORTED;
          return true;
        }
      }
    }
    return false;
  }
  bool unfinished() const { return !waiting.empty() || !running.empty(); }

  int chunk(int remaining, int budget) const {
    int cap = budget;
    if (chunk_size) cap = std::min(cap, chunk_size);
    if (remaining <= cap) return remaining;
    return cap / cache->page_size * cache->page_size;
  }
  void plan_once(std::vector<PlanRow>* rows) {
    int budget = max_batched_tokens, reserved = 0;
    for (auto& request : running) {                       // 1. decode rows: a prefix of the running queue
      if (!request->decoding()) continue;
      if ((int)rows->size() >= max_num_seqs) break;
      const int need = cache->pages_needed(*cache->find(request->id), 1);
      if (reserved + need > cache->available_pages()) break;
      rows->push_back({request->id, request->computed, 1, 1});
      reserved += need;
      budget -= 1;
    }
    for (auto& request : running) {                       // 2. running requests in the middle of their prompt
      if (request->decoding() || (int)rows->size() >= max_num_seqs) continue;
      const int count = chunk(request->remaining(), std::max(budget, 0));
      if (count <= 0) continue;
      const int need = cache->pages_needed(*cache->find(request->id), count);
      if (reserved + need > cache->available_pages()) continue;
      rows->push_back({request->id, request->computed, count, count == request->remaining()});
      reserved += need;
      budget -= count;
    }
    while (!waiting.empty() && (int)rows->size() < max_num_seqs && budget > 0) {   // 3. the head of the waiting queue
      if ((int)running.size() >= cache->max_requests || cache->free_slots.empty()) break;
      auto request = waiting.front();
      if (cache->begin(request->id, request->tokens.data(), (int)request->tokens.size()) < 0) break;
      Residency* res = cache->find(request->id);
      request->computed = res->length;
      const int count = chunk(request->remaining(), budget);
      const int need = count > 0 ? cache->pages_needed(*res, count) : 0;
      if (count <= 0 || reserved + need > cache->available_pages()) {
        if (res->cached_prefix_pages > 0) {               // roll back: nothing of it is held or counted
          cache->reused_prefix_pages -= res->cached_prefix_pages;
          --cache->requests_with_reuse;
        }
        cache->finish(request->id);
        request->computed = 0;
        break;
      }
      waiting.pop_front();
      running.push_back(request);
      ++admitted;
      rows->push_back({request->id, request->computed, count, count == request->remaining()});
      reserved += need;
      budget -= count;
    }
  }
  void plan(std::vector<PlanRow>* rows, std::vector<int64_t>* preempted, std::vector<int64_t>* dropped) {
    while (true) {
      rows->clear();
      plan_once(rows);
      if (!rows->empty() || !unfinished()) break;
      if (!running.empty()) {
        auto victim = running.back();                     // the youngest
        running.pop_back();
        cache->finish(victim->id);
        victim->computed = 0;
        ++victim->preemptions;
        ++preemptions;
        waiting.push_front(victim);
        preempted->push_back(victim->id);
        continue;
      }
      auto victim = waiting.front();                      // no cache of this size can hold it
      waiting.pop_front();
      victim->finish_reason = CAPACITY;
      dropped->push_back(victim->id);
    }
    last_plan = *rows;
  }
  // sampled[i]: token of row i, ignored for rows that do not sample. emitted_out: 1 if the row emitted.
  int commit(const int32_t* sampled, int count, int32_t* finished_out) {
    if (count != (int)last_plan.size()) return fail(VH_BAD_ARGUMENT, "commit of %d rows, the plan has %zu", count, last_plan.size());
    for (int i = 0; i < count; ++i) {
      const PlanRow& row = last_plan[i];
      auto request = requests.at(row.id);
      request->computed += row.count;
      Residency* res = cache->find(row.id);
      if (res == nullptr) return fail(VH_UNKNOWN_REQUEST, "a planned request is not live");
      const int rc = cache->publish(*res, request->tokens.data(), request->computed);
      if (rc < 0) return rc;
      finished_out[i] = NOT_FINISHED;
      if (!row.sample) continue;
      const int32_t token = sampled[i];
      request->tokens.push_back(token);
      bool done = false;
      if (request->generated() >= request->max_tokens) {
        request->finish_reason = LENGTH;
        done = true;
      } else if (!request->ignore_eos) {
        for (int e = 0; e < request->n_eos; ++e)
          if (request->eos[e] == token) {
            request->finish_reason = EOS;
            done = true;
          }
      }
      if (done) {
        finished_out[i] = request->finish_reason;
        running.erase(std::find(running.begin(), running.end(), request));
        const int rc2 = cache->finish(row.id);
        if (rc2 != VH_OK) return rc2;
      }
    }
    last_plan.clear();
    return VH_OK;
  }

  // ---- the same commit in two halves, for an engine that launches step n + 1 before it has read
  // step n's tokens. commit_ahead applies everything that does not need the token values: the
  // computed counts, page publication (it only needs tokens that were inputs of the step), and
  // the end by length, which is known from the count; a sampling row gets the token PENDING.
  // resolve, called once the tokens are on the host and before the next commit_ahead, writes
  // them in and applies the end by EOS. A request whose newest token is pending is planned like
  // any other (the engine feeds that token from the device); if resolve ends it, a row it
  // already has in the launched step is ignored by the commit_ahead and resolve of that step.
  static constexpr int32_t PENDING = -1;
  static constexpr int32_t IGNORED = -1;                 // in finished_out: the row's request had ended before
  int commit_ahead(int32_t* finished_out) {
    const int count = (int)last_plan.size();
    for (int i = 0; i < count; ++i) {
      const PlanRow& row = last_plan[i];
      finished_out[i] = IGNORED;
      auto found = requests.find(row.id);
      if (found == requests.end() || found->second->finish_reason != NOT_FINISHED) continue;
      auto request = found->second;
      Residency* res = cache->find(row.id);
      if (res == nullptr) continue;
      request->computed += row.count;
      const int rc = cache->publish(*res, request->tokens.data(), request->computed);
      if (rc < 0) return rc;
      finished_out[i] = NOT_FINISHED;
      if (!row.sample) continue;
      request->tokens.push_back(PENDING);
      if (request->generated() >= request->max_tokens) {
        request->finish_reason = LENGTH;
        finished_out[i] = LENGTH;
        running.erase(std::find(running.begin(), running.end(), request));
        const int rc2 = cache->finish(row.id);
        if (rc2 != VH_OK) return rc2;
      }
    }
    ahead_plan = last_plan;
    ahead_state.assign(finished_out, finished_out + count);
    last_plan.clear();
    return count;
  }
  // sampled[i]: the token of row i of the plan commit_ahead took. finished_out[i]: IGNORED for a
  // row that emits nothing, else the request's finish reason after this token.
  int resolve(const int32_t* sampled, int count, int32_t* finished_out) {
    if (count != (int)ahead_plan.size()) return fail(VH_BAD_ARGUMENT, "resolve of %d rows, the step had %zu", count, ahead_plan.size());
    for (int i = 0; i < count; ++i) {
      const PlanRow& row = ahead_plan[i];
      finished_out[i] = IGNORED;
      if (!row.sample || ahead_state[i] == IGNORED) continue;
      auto found = requests.find(row.id);
      if (found == requests.end()) continue;
      auto request = found->second;
      const int index = row.start + row.count;            // where the sampled token went
      if (index >= (int)request->tokens.size() || request->tokens[index] != PENDING) continue;
      if (request->finish_reason == ABORTED) continue;
      const int32_t token = sampled[i];
      request->tokens[index] = token;
      finished_out[i] = request->finish_reason;           // LENGTH if commit_ahead ended it
      if (request->finish_reason != NOT_FINISHED || request->ignore_eos) continue;
      for (int e = 0; e < request->n_eos; ++e)
        if (request->eos[e] == token) {
          abort(row.id);                                  // leaves its queue, gives back what it holds
          request->finish_reason = EOS;
          finished_out[i] = EOS;
          break;
        }
    }
    ahead_plan.clear();
    ahead_state.clear();
    return VH_OK;
  }
  std::vector<PlanRow> ahead_plan;
  std::vector<int32_t> ahead_state;

  CacheCore* cache;
  int max_num_seqs, max_batched_tokens, chunk_size, vocab_size, max_context;
  std::deque<std::shared_ptr<Request>> waiting, running;
  std::map<int64_t, std::shared_ptr<Request>> requests;
  std::set<int64_t> accepted;
  std::vector<PlanRow> last_plan;
  int64_t admitted = 0, preemptions = 0;
};

struct Host {
  std::unique_ptr<CacheCore> cache;
  std::unique_ptr<SchedulerCore> scheduler;
};

}  // namespace

// ------------------------------------------------------------------ C ABI
VH_API const char* vh_last_error() { return g_error; }
VH_API uint64_t vh_chain_hash(uint64_t previous, const int32_t* tokens, int count) { return chain_hash(previous, tokens, count); }

// ---- a pool on its own
VH_API void* vh_pool_create(int pages) { return pages > 0 ? new PagePool(pages) : nullptr; }
VH_API void vh_pool_destroy(void* pool) { delete (PagePool*)pool; }
VH_API int vh_pool_available(void* pool) { return ((PagePool*)pool)->available(); }
VH_API int vh_pool_num_pages(void* pool) { return ((PagePool*)pool)->num_pages; }
VH_API int64_t vh_pool_evictions(void* pool) { return ((PagePool*)pool)->evictions; }
VH_API int vh_pool_refcount(void* pool, int page) { return ((PagePool*)pool)->refcount[page]; }
VH_API int vh_pool_allocate(void* pool, int count, int32_t* out) {
  std::vector<int> pages;
  const int rc = ((PagePool*)pool)->allocate(count, &pages);
  if (rc != VH_OK) return rc;
  std::copy(pages.begin(), pages.end(), out);
  return VH_OK;
}
VH_API int vh_pool_acquire(void* pool, int page) { return ((PagePool*)pool)->acquire(page); }
VH_API int vh_pool_release(void* pool, int page) { return ((PagePool*)pool)->release(page); }
VH_API uint64_t vh_pool_publish(void* pool, int page, const int32_t* tokens, int count, uint64_t previous, int depth,
                                int parent, int32_t* parent_out) {
  int next_parent = -1;
  const uint64_t h = ((PagePool*)pool)->publish(page, tokens, count, previous, depth, parent, &next_parent);
  *parent_out = next_parent;
  return h;
}
VH_API int vh_pool_match(void* pool, const int32_t* tokens, int count, int page_size, int32_t* out, int capacity) {
  std::vector<int> pages;
  ((PagePool*)pool)->match(tokens, count, page_size, &pages);
  const int n = std::min((int)pages.size(), capacity);
  std::copy(pages.begin(), pages.begin() + n, out);
  return (int)pages.size();
}
VH_API int vh_pool_list(void* pool, int which, int32_t* out, int capacity) {   // 0: free, 1: evictable, 2: published
  PagePool* p = (PagePool*)pool;
  std::vector<int> pages;
  if (which == 0) pages.assign(p->free_list.begin(), p->free_list.end());
  else if (which == 1) pages.assign(p->evictable.begin(), p->evictable.end());
  else for (auto& kv : p->published) pages.push_back(kv.first);
  const int n = std::min((int)pages.size(), capacity);
  std::copy(pages.begin(), pages.begin() + n, out);
  return (int)pages.size();
}
// Test hook: overwrite the tokens a published page is remembered with (as a hash collision would look).
VH_API int vh_pool_set_published_tokens(void* pool, int page, const int32_t* tokens, int count) {
  PagePool* p = (PagePool*)pool;
  auto it = p->published.find(page);
  if (it == p->published.end()) return fail(VH_BAD_ARGUMENT, "page %d is not published", page);
  it->second.tokens.assign(tokens, tokens + count);
  return VH_OK;
}
VH_API int vh_pool_check(void* pool, const int32_t* pages, const int32_t* counts, int n) {
  std::map<int, int> holders;
  for (int i = 0; i < n; ++i) holders[pages[i]] = counts[i];
  return ((PagePool*)pool)->check(holders);
}

// ---- cache manager and scheduler
VH_API void* vh_create(int groups, const int32_t* windows, int num_pages, int page_size, int max_requests,
                       int prefix_reuse, int has_state, int max_num_seqs, int max_batched_tokens, int chunk_size,
                       int vocab_size, int max_context) {
  if (groups < 0 || num_pages <= 0 || page_size <= 0 || max_requests <= 0) return nullptr;
  Host* h = new Host;
  h->cache.reset(new CacheCore(groups, windows, num_pages, page_size, max_requests, prefix_reuse != 0, has_state != 0));
  h->scheduler.reset(new SchedulerCore(h->cache.get(), max_num_seqs, max_batched_tokens, chunk_size, vocab_size, max_context));
  return h;
}
VH_API void vh_destroy(void* host) { delete (Host*)host; }
VH_API void vh_configure_scheduler(void* host, int max_num_seqs, int max_batched_tokens, int chunk_size, int vocab_size,
                                   int max_context) {
  SchedulerCore* s = ((Host*)host)->scheduler.get();
  s->max_num_seqs = max_num_seqs;
  s->max_batched_tokens = max_batched_tokens;
  s->chunk_size = chunk_size;
  s->vocab_size = vocab_size;
  s->max_context = max_context;
}
VH_API void* vh_group_pool(void* host, int group) { return ((Host*)host)->cache->pools[group].get(); }
VH_API int vh_prefix_reuse(void* host) { return ((Host*)host)->cache->prefix_reuse ? 1 : 0; }
VH_API int vh_available_pages(void* host) { return ((Host*)host)->cache->available_pages(); }
VH_API int64_t vh_counter(void* host, int which) {
  Host* h = (Host*)host;
  switch (which) {
    case 0: return h->cache->reused_prefix_pages;
    case 1: return h->cache->requests_with_reuse;
    case 2: return h->scheduler->admitted;
    case 3: return h->scheduler->preemptions;
    case 4: return (int64_t)h->cache->free_slots.size();
    case 5: return (int64_t)h->cache->live.size();
    default: return -1;
  }
}
VH_API int vh_begin(void* host, int64_t id, const int32_t* prompt, int count) { return ((Host*)host)->cache->begin(id, prompt, count); }
VH_API int vh_is_live(void* host, int64_t id) { return ((Host*)host)->cache->find(id) != nullptr; }
#define VH_RES(host, id)                                                     \
  Residency* res = ((Host*)host)->cache->find(id);                           \
  if (res == nullptr) return fail(VH_UNKNOWN_REQUEST, "request is not live")
VH_API int vh_pages_needed(void* host, int64_t id, int tokens) { VH_RES(host, id); return ((Host*)host)->cache->pages_needed(*res, tokens); }
VH_API int vh_can_extend(void* host, int64_t id, int tokens) { VH_RES(host, id); return ((Host*)host)->cache->can_extend(*res, tokens) ? 1 : 0; }
VH_API int vh_extend(void* host, int64_t id, int tokens, int32_t* slots_out) { VH_RES(host, id); return ((Host*)host)->cache->extend(*res, tokens, slots_out); }
VH_API int vh_trim(void* host, int64_t id) { VH_RES(host, id); return ((Host*)host)->cache->trim(*res); }
VH_API int vh_publish(void* host, int64_t id, const int32_t* tokens, int count) { VH_RES(host, id); return ((Host*)host)->cache->publish(*res, tokens, count); }
VH_API int vh_finish(void* host, int64_t id) { return ((Host*)host)->cache->finish(id); }
VH_API int vh_length(void* host, int64_t id) { VH_RES(host, id); return res->length; }
VH_API int vh_slot(void* host, int64_t id) { VH_RES(host, id); return res->slot; }
VH_API int vh_residency_field(void* host, int64_t id, int which) {
  VH_RES(host, id);
  return which == 0 ? res->cached_prefix_pages : res->published_pages;
}
VH_API int vh_block_row(void* host, int64_t id, int group, int32_t* out, int capacity) {
  VH_RES(host, id);
  const auto& row = res->pages[group];
  const int n = std::min((int)row.size(), capacity);
  std::copy(row.begin(), row.begin() + n, out);
  return (int)row.size();
}
VH_API int vh_free_slots(void* host, int32_t* out, int capacity) {
  const auto& slots = ((Host*)host)->cache->free_slots;
  const int n = std::min((int)slots.size(), capacity);
  std::copy(slots.begin(), slots.begin() + n, out);
  return (int)slots.size();
}
VH_API int vh_live_ids(void* host, int64_t* out, int capacity) {
  int n = 0;
  for (auto& kv : ((Host*)host)->cache->live)
    if (n < capacity) out[n++] = kv.first;
  return (int)((Host*)host)->cache->live.size();
}
VH_API int vh_check(void* host) { return ((Host*)host)->cache->check(); }
// The state slots begin() handed out since the last call (a slot may appear more than once, and a
// slot whose admission was rolled back may appear although nobody holds it); the list is cleared.
VH_API int vh_take_fresh_slots(void* host, int32_t* out, int capacity) {
  auto& slots = ((Host*)host)->cache->fresh_slots;
  std::sort(slots.begin(), slots.end());
  slots.erase(std::unique(slots.begin(), slots.end()), slots.end());
  const int n = std::min((int)slots.size(), capacity);
  std::copy(slots.begin(), slots.begin() + n, out);
  slots.clear();
  return n;
}

VH_API int vh_add_request(void* host, int64_t id, const int32_t* prompt, int count, int max_tokens, const int32_t* eos,
                          int n_eos, int ignore_eos, float temperature) {
  return ((Host*)host)->scheduler->add(id, prompt, count, max_tokens, eos, n_eos, ignore_eos != 0, temperature);
}
VH_API int vh_abort(void* host, int64_t id) { return ((Host*)host)->scheduler->abort(id) ? 1 : 0; }
VH_API int vh_unfinished(void* host) { return ((Host*)host)->scheduler->unfinished() ? 1 : 0; }
VH_API int vh_queue(void* host, int which, int64_t* out, int capacity) {   // 0: waiting, 1: running
  auto& queue = which == 0 ? ((Host*)host)->scheduler->waiting : ((Host*)host)->scheduler->running;
  int n = 0;
  for (auto& r : queue)
    if (n < capacity) out[n++] = r->id;
  return (int)queue.size();
}
// rows_out: [capacity][4] = (start, count, sample, state slot of the request), ids in ids_out.
VH_API int vh_plan(void* host, int64_t* ids_out, int32_t* rows_out, int capacity, int64_t* preempted_out,
                   int32_t* n_preempted, int64_t* dropped_out, int32_t* n_dropped, int side_capacity) {
  std::vector<PlanRow> rows;
  std::vector<int64_t> preempted, dropped;
  ((Host*)host)->scheduler->plan(&rows, &preempted, &dropped);
  if ((int)rows.size() > capacity || (int)preempted.size() > side_capacity || (int)dropped.size() > side_capacity)
    return fail(VH_BAD_ARGUMENT, "plan does not fit the buffers given");
  for (size_t i = 0; i < rows.size(); ++i) {
    ids_out[i] = rows[i].id;
    rows_out[4 * i] = rows[i].start;
    rows_out[4 * i + 1] = rows[i].count;
    rows_out[4 * i + 2] = rows[i].sample;
    const Residency* res = ((Host*)host)->cache->find(rows[i].id);
    rows_out[4 * i + 3] = res != nullptr ? res->slot : -1;
  }
  std::copy(preempted.begin(), preempted.end(), preempted_out);
  std::copy(dropped.begin(), dropped.end(), dropped_out);
  *n_preempted = (int32_t)preempted.size();
  *n_dropped = (int32_t)dropped.size();
  return (int)rows.size();
}
VH_API int vh_commit(void* host, const int32_t* sampled, int count, int32_t* finished_out) {
  return ((Host*)host)->scheduler->commit(sampled, count, finished_out);
}
VH_API int vh_commit_ahead(void* host, int32_t* finished_out) { return ((Host*)host)->scheduler->commit_ahead(finished_out); }
VH_API int vh_resolve(void* host, const int32_t* sampled, int count, int32_t* finished_out) {
  return ((Host*)host)->scheduler->resolve(sampled, count, finished_out);
}
// which: 0 computed, 1 generated count, 2 preemptions, 3 finish reason, 4 total tokens
VH_API int vh_request_field(void* host, int64_t id, int which) {
  auto& requests = ((Host*)host)->scheduler->requests;
  auto it = requests.find(id);
  if (it == requests.end()) return fail(VH_UNKNOWN_REQUEST, "unknown request");
  const Request& r = *it->second;
  switch (which) {
    case 0: return r.computed;
    case 1: return r.generated();
    case 2: return r.preemptions;
    case 3: return r.finish_reason;
    default: return (int)r.tokens.size();
  }
}
VH_API int vh_request_tokens(void* host, int64_t id, int from, int count, int32_t* out) {
  auto& requests = ((Host*)host)->scheduler->requests;
  auto it = requests.find(id);
  if (it == requests.end()) return fail(VH_UNKNOWN_REQUEST, "unknown request");
  const auto& tokens = it->second->tokens;
  if (from < 0 || count < 0 || from + count > (int)tokens.size()) return fail(VH_BAD_ARGUMENT, "token range outside the request");
  std::copy(tokens.begin() + from, tokens.begin() + from + count, out);
  return count;
}
// Forget a finished request's record (ids stay taken).
VH_API void vh_forget(void* host, int64_t id) { ((Host*)host)->scheduler->requests.erase(id); }

// ---- a whole step at once (the engine's hot path)
// Reserve cache entries for every entry of a step, all or nothing. starts_out[i]: position of
// entry i's first token; widest_out[g]: the longest block-table row of group g after the step.
// No request may reach beyond `position_limit` tokens (0: no limit).
VH_API int vh_step_extend(void* host, const int64_t* ids, const int32_t* counts, int n, int position_limit,
                          int32_t* starts_out, int32_t* widest_out) {
  CacheCore* cache = ((Host*)host)->cache.get();
  std::vector<Residency*> rows(n);
  for (int i = 0; i < n; ++i) {
    rows[i] = cache->find(ids[i]);
    if (rows[i] == nullptr) return fail(VH_UNKNOWN_REQUEST, "entry %d names a request that is not live", i);
    if (counts[i] <= 0) return fail(VH_BAD_ARGUMENT, "entry %d brings no tokens", i);
    if (position_limit > 0 && rows[i]->length + counts[i] > position_limit)
      return fail(VH_BAD_ARGUMENT, "entry %d would reach position %d, the model's limit is %d", i,
                  rows[i]->length + counts[i], position_limit);
    for (int j = 0; j < i; ++j)
      if (ids[j] == ids[i]) return fail(VH_BAD_ARGUMENT, "a request appears twice in one step");
  }
  for (size_t g = 0; g < cache->pools.size(); ++g) {
    int64_t need = 0;
    for (int i = 0; i < n; ++i)
      need += std::max(0, cache->pages_for(rows[i]->length + counts[i]) - (int)rows[i]->pages[g].size());
    if (need > cache->pools[g]->available())
      return fail(VH_OUT_OF_PAGES, "step needs %lld pages in group %zu, %d available", (long long)need, g,
                  cache->pools[g]->available());
  }
  for (size_t g = 0; g < cache->pools.size(); ++g) widest_out[g] = 1;
  for (int i = 0; i < n; ++i) {
    starts_out[i] = rows[i]->length;
    const int rc = cache->extend(*rows[i], counts[i], nullptr);
    if (rc != VH_OK) return rc;
    for (size_t g = 0; g < cache->pools.size(); ++g)
      widest_out[g] = std::max(widest_out[g], (int32_t)rows[i]->pages[g].size());
  }
  return VH_OK;
}
// Fill the step's index arrays (already extended): positions, request_of [T]; cu_q [n+1]; kv_len,
// state_slot [n]; for each group g: slot_mapping[g] [T] and block_table[g] [n, widths[g]].
VH_API int vh_step_fill(void* host, const int64_t* ids, const int32_t* counts, const int32_t* starts, int n,
                        int32_t* positions, int32_t* request_of, int32_t* cu_q, int32_t* kv_len, int32_t* state_slot,
                        int32_t** slot_mapping, int32_t** block_table, const int32_t* widths) {
  CacheCore* cache = ((Host*)host)->cache.get();
  const int P = cache->page_size;
  int cursor = 0;
  cu_q[0] = 0;
  for (int i = 0; i < n; ++i) {
    Residency* res = cache->find(ids[i]);
    if (res == nullptr) return fail(VH_UNKNOWN_REQUEST, "entry %d names a request that is not live", i);
    for (int j = 0; j < counts[i]; ++j) {
      positions[cursor + j] = starts[i] + j;
      request_of[cursor + j] = i;
    }
    kv_len[i] = starts[i] + counts[i];
    state_slot[i] = res->slot;
    for (size_t g = 0; g < cache->pools.size(); ++g) {
      const auto& row = res->pages[g];
      if ((int)row.size() > widths[g]) return fail(VH_BAD_ARGUMENT, "block-table width %d too small", widths[g]);
      for (int j = 0; j < counts[i]; ++j) {
        const int pos = starts[i] + j;
        slot_mapping[g][cursor + j] = row[pos / P] * P + pos % P;
      }
      int32_t* dst = block_table[g] + (int64_t)i * widths[g];
      std::copy(row.begin(), row.end(), dst);
      std::fill(dst + row.size(), dst + widths[g], 0);
    }
    cursor += counts[i];
    cu_q[i + 1] = cursor;
  }
  return VH_OK;
}
