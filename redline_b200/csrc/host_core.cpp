// The host side of the cache, of the scheduler and of a step's metadata, in C++: page pools with
// LIFO reuse, per-request block tables for every cache group, window release, state slots, the
// scheduler's plan of a step (at the end of the file), and the routine that fills a step's pinned
// metadata buffer.  No CUDA in this file: it is
// compiled as a host-only shared object and bound with ctypes (redline_b200/cache/manager.py,
// redline_b200/engine/scheduler.py, redline_b200/engine/batch.py).
//
// Policy of the reference's block allocator (src/core/block_allocator.cpp:7-35): pages are
// handed out lowest id first and reused last-freed first; page 0 of every pool is never handed
// out (padded rows of a fixed-shape batch write there).  A reservation is all or nothing.  In
// a window group a page goes back as soon as every key on it is older than the window of all
// tokens still to come.
//
// Error codes (returned negative by the functions below; the Python side raises):
//   -1 not a page of this pool   -2 page freed twice   -3 no such request   -4 no free state slot
//   -5 bad argument
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

namespace {

struct Pool {
  int num_pages = 0, reserved = 1;
  std::vector<int32_t> free_list;     // back() is the next page to hand out
  std::vector<uint8_t> held;

  void init(int n, int r) {
    num_pages = n;
    reserved = r;
    free_list.clear();
    for (int p = n - 1; p >= r; --p) free_list.push_back(p);   // the lowest id is handed out first
    held.assign(n, 0);
  }
  int usable() const { return num_pages - reserved; }
  int allocate() {
    if (free_list.empty()) return -1;
    const int p = free_list.back();
    free_list.pop_back();
    held[p] = 1;
    return p;
  }
  // Gives pages back; the first of `pages` is the next to be handed out again.  Stops at the first
  // bad id (what came after it in the list has been given back by then).
  int give_back(const int32_t* pages, int n, int* bad) {
    for (int i = n - 1; i >= 0; --i) {
      const int p = pages[i];
      if (p < reserved || p >= num_pages) {
        *bad = p;
        return -1;
      }
      if (!held[p]) {
        *bad = p;
        return -2;
      }
      held[p] = 0;
      free_list.push_back(p);
    }
    return 0;
  }
};

struct Request {
  bool open = false;
  int state_slot = -1;
  int num_tokens = 0;
  std::vector<std::vector<int32_t>> tables;   // per group: page id per block; 0 once released by a window
  std::vector<int> released_upto;             // per group: blocks below this index were released
};

struct Core {
  int page_size = 16;
  std::vector<Pool> pools;
  std::vector<int> windows;                    // per group; 0: every key is kept
  std::vector<int> free_slots;
  int num_state_slots = 0;
  std::vector<Request> reqs;
  std::vector<int> free_rids;
  int num_open = 0;

  Request* get(int rid) {
    if (rid < 0 || rid >= static_cast<int>(reqs.size()) || !reqs[rid].open) return nullptr;
    return &reqs[rid];
  }
  int blocks_for(int tokens) const { return (tokens + page_size - 1) / page_size; }
};

}  // namespace

extern "C" {

// ------------------------------------------------------------------ a pool alone
void* rl_pool_create(int num_pages, int reserved) {
  if (num_pages <= reserved || reserved < 0) return nullptr;
  Pool* p = new Pool;
  p->init(num_pages, reserved);
  return p;
}
void rl_pool_destroy(void* h) { delete static_cast<Pool*>(h); }
int rl_pool_allocate(void* h) { return static_cast<Pool*>(h)->allocate(); }
int rl_pool_free(void* h, const int32_t* pages, int n, int* bad) { return static_cast<Pool*>(h)->give_back(pages, n, bad); }
int rl_pool_num_free(void* h) { return static_cast<int>(static_cast<Pool*>(h)->free_list.size()); }
int rl_pool_num_usable(void* h) { return static_cast<Pool*>(h)->usable(); }
int rl_pool_is_held(void* h, int page) {
  Pool* p = static_cast<Pool*>(h);
  return page >= 0 && page < p->num_pages ? p->held[page] : 0;
}

// ------------------------------------------------------------------ the cache manager
void* rl_hc_create(int num_groups, const int32_t* pages_per_group, const int32_t* windows, int page_size,
                   int num_state_slots) {
  if (num_groups < 0 || page_size <= 0 || num_state_slots < 0) return nullptr;
  for (int g = 0; g < num_groups; ++g)
    if (pages_per_group[g] <= 1) return nullptr;
  Core* c = new Core;
  c->page_size = page_size;
  c->pools.resize(num_groups);
  c->windows.assign(windows, windows + num_groups);
  for (int g = 0; g < num_groups; ++g) c->pools[g].init(pages_per_group[g], 1);
  c->num_state_slots = num_state_slots;
  for (int s = num_state_slots - 1; s >= 0; --s) c->free_slots.push_back(s);   // slot 0 first
  return c;
}
void rl_hc_destroy(void* h) { delete static_cast<Core*>(h); }

// A new request: its id (>= 0), or -4 when no state slot is free.
int rl_hc_open(void* h) {
  Core* c = static_cast<Core*>(h);
  if (c->free_slots.empty()) return -4;
  int rid;
  if (!c->free_rids.empty()) {
    rid = c->free_rids.back();
    c->free_rids.pop_back();
  } else {
    rid = static_cast<int>(c->reqs.size());
    c->reqs.emplace_back();
  }
  Request& r = c->reqs[rid];
  r.open = true;
  r.state_slot = c->free_slots.back();
  c->free_slots.pop_back();
  r.num_tokens = 0;
  r.tables.assign(c->pools.size(), std::vector<int32_t>());
  r.released_upto.assign(c->pools.size(), 0);
  ++c->num_open;
  return rid;
}

// Gives back every page and the state slot of the request.
int rl_hc_close(void* h, int rid, int* bad) {
  Core* c = static_cast<Core*>(h);
  Request* r = c->get(rid);
  if (!r) return -3;
  int rc = 0;
  for (size_t g = 0; g < c->pools.size() && rc == 0; ++g) {
    const std::vector<int32_t>& t = r->tables[g];
    const int from = std::min<int>(r->released_upto[g], static_cast<int>(t.size()));
    rc = c->pools[g].give_back(t.data() + from, static_cast<int>(t.size()) - from, bad);
  }
  c->free_slots.push_back(r->state_slot);
  r->open = false;
  r->tables.clear();
  c->free_rids.push_back(rid);
  --c->num_open;
  return rc;
}

// Makes sure pages exist for positions < new_len in every group.  1: done; 0: not enough pages (what
// this call took has been given back).
int rl_hc_reserve(void* h, int rid, int new_len) {
  Core* c = static_cast<Core*>(h);
  Request* r = c->get(rid);
  if (!r) return -3;
  const int need = c->blocks_for(new_len);
  const size_t G = c->pools.size();
  std::vector<int> taken(G, 0);
  for (size_t g = 0; g < G; ++g) {
    std::vector<int32_t>& t = r->tables[g];
    while (static_cast<int>(t.size()) < need) {
      const int p = c->pools[g].allocate();
      if (p < 0) {
        // roll back in reverse order of taking: the pools hand the same pages out again, in the same order
        for (int gg = static_cast<int>(g); gg >= 0; --gg) {
          std::vector<int32_t>& tt = r->tables[gg];
          for (int k = 0; k < taken[gg]; ++k) {
            const int32_t pp = tt.back();
            tt.pop_back();
            int bad = 0;
            c->pools[gg].give_back(&pp, 1, &bad);
          }
        }
        return 0;
      }
      t.push_back(p);
      ++taken[g];
    }
  }
  r->num_tokens = std::max(r->num_tokens, new_len);
  return 1;
}

// After num_computed positions are in the cache: in window groups, frees the pages whose keys no
// later token can see (key j is dead when j <= n - window for the next position n).  Pages freed.
int rl_hc_release_passed(void* h, int rid, int num_computed) {
  Core* c = static_cast<Core*>(h);
  Request* r = c->get(rid);
  if (!r) return -3;
  int freed = 0;
  for (size_t g = 0; g < c->pools.size(); ++g) {
    const int w = c->windows[g];
    if (w <= 0) continue;
    const int dead_keys = num_computed - w + 1;               // keys 0 .. dead_keys-1 are dead
    int dead_blocks = std::max(0, dead_keys) / c->page_size;
    dead_blocks = std::min<int>(dead_blocks, static_cast<int>(r->tables[g].size()));
    if (dead_blocks > r->released_upto[g]) {
      std::vector<int32_t>& t = r->tables[g];
      const int from = r->released_upto[g];
      int bad = 0;
      const int rc = c->pools[g].give_back(t.data() + from, dead_blocks - from, &bad);
      if (rc < 0) return rc;
      for (int i = from; i < dead_blocks; ++i) t[i] = 0;
      freed += dead_blocks - from;
      r->released_upto[g] = dead_blocks;
    }
  }
  return freed;
}

int rl_hc_state_slot(void* h, int rid) {
  Request* r = static_cast<Core*>(h)->get(rid);
  return r ? r->state_slot : -3;
}
int rl_hc_num_tokens(void* h, int rid) {
  Request* r = static_cast<Core*>(h)->get(rid);
  return r ? r->num_tokens : -3;
}
int rl_hc_released_upto(void* h, int rid, int group) {
  Core* c = static_cast<Core*>(h);
  Request* r = c->get(rid);
  if (!r || group < 0 || group >= static_cast<int>(c->pools.size())) return -3;
  return r->released_upto[group];
}
// The block table of a request in one group: its length; *ptr points at the entries (valid until the
// request's next reserve or close).
int rl_hc_table(void* h, int rid, int group, const int32_t** ptr) {
  Core* c = static_cast<Core*>(h);
  Request* r = c->get(rid);
  if (!r || group < 0 || group >= static_cast<int>(c->pools.size())) return -3;
  *ptr = r->tables[group].data();
  return static_cast<int>(r->tables[group].size());
}
int rl_hc_num_free(void* h, int group) { return static_cast<int>(static_cast<Core*>(h)->pools[group].free_list.size()); }
int rl_hc_num_usable(void* h, int group) { return static_cast<Core*>(h)->pools[group].usable(); }
int rl_hc_num_open(void* h) { return static_cast<Core*>(h)->num_open; }

// No page lost, none held twice: every usable page is either free or in exactly one live table entry;
// the same for state slots.  0, or 1 with a message.
int rl_hc_check(void* h, char* msg, int cap) {
  Core* c = static_cast<Core*>(h);
  for (size_t g = 0; g < c->pools.size(); ++g) {
    Pool& a = c->pools[g];
    std::vector<int> owner(a.num_pages, -1);
    int seen = 0;
    for (size_t rid = 0; rid < c->reqs.size(); ++rid) {
      const Request& r = c->reqs[rid];
      if (!r.open) continue;
      const std::vector<int32_t>& t = r.tables[g];
      for (int i = r.released_upto[g]; i < static_cast<int>(t.size()); ++i) {
        const int p = t[i];
        if (p < 0 || p >= a.num_pages) {
          std::snprintf(msg, cap, "group %zu: request %zu holds page id %d outside the pool", g, rid, p);
          return 1;
        }
        if (owner[p] >= 0) {
          std::snprintf(msg, cap, "group %zu: page %d held by requests %d and %zu", g, p, owner[p], rid);
          return 1;
        }
        if (!a.held[p]) {
          std::snprintf(msg, cap, "group %zu: page %d of request %zu is on the free list", g, p, rid);
          return 1;
        }
        owner[p] = static_cast<int>(rid);
        ++seen;
      }
    }
    if (seen + static_cast<int>(a.free_list.size()) != a.usable()) {
      std::snprintf(msg, cap, "group %zu: %d pages lost", g, a.usable() - static_cast<int>(a.free_list.size()) - seen);
      return 1;
    }
  }
  std::vector<uint8_t> slot_used(std::max(c->num_state_slots, 1), 0);
  int slots = 0;
  for (const Request& r : c->reqs) {
    if (!r.open) continue;
    if (r.state_slot < 0 || r.state_slot >= c->num_state_slots || slot_used[r.state_slot]) {
      std::snprintf(msg, cap, "state slots lost or held twice");
      return 1;
    }
    slot_used[r.state_slot] = 1;
    ++slots;
  }
  if (slots + static_cast<int>(c->free_slots.size()) != c->num_state_slots) {
    std::snprintf(msg, cap, "state slots lost or held twice");
    return 1;
  }
  return 0;
}

// ------------------------------------------------------------------ a step's metadata
// Offsets (in 32-bit words) of the fields of the metadata buffer, as the Python side lays them out.
struct RlLayout {
  int32_t token_ids, token_src, positions, seq_of_token;
  int32_t state_slot, decode_info, tile_seq, tile_tok, tile_rows;
  int32_t logit_rows, temperature, top_k, top_p, seed_lo, seed_hi, sample_pos;
  int32_t words;
};

// One segment of a step: a request's next tokens.
struct RlSegment {
  int32_t rid, start_pos, num_tokens, src_row;     // src_row >= 0: the single token is fed on the device
  int32_t token_off, want_off, num_want;           // into the flat token and want arrays
  int32_t has_sampling;
  float temperature, top_p;
  int32_t top_k;
  uint32_t seed_lo, seed_hi;
};

// Results: [0] decode items, [1] tiles, [2] longest context among decode items, [3] any token fed on the
// device, [4] any sampling parameters, [5] the segment an error refers to, [6] a number for the message.
// Errors: -10 empty segment, -11 beyond max_seq_len, -12 a device-fed segment has more than one token,
// -13 pages reserved for fewer positions ([6] = positions covered), -14 wanted index outside, -3 no such
// request.
int rl_hc_build(void* h, int32_t* out, const RlLayout* lay, const int32_t* slots_off, const int32_t* table_off,
                int G, int B, int S, const RlSegment* segs, const int32_t* tokens, const int32_t* want,
                int max_seq_len, int tile_rows, int32_t* result) {
  Core* c = static_cast<Core*>(h);
  const int ps = c->page_size;
  if (G != static_cast<int>(c->pools.size())) return -5;
  std::memset(out, 0, sizeof(int32_t) * static_cast<size_t>(lay->words));
  int t = 0, r = 0, nd = 0, li = 0, max_ctx = 1, has_src = 0, any_sampling = 0;
  for (int si = 0; si < S; ++si) {
    const RlSegment& s = segs[si];
    result[5] = si;
    const int n = s.num_tokens, end = s.start_pos + n;
    if (n <= 0) return -10;
    if (end > max_seq_len) {
      result[6] = end;
      return -11;
    }
    Request* rq = c->get(s.rid);
    if (!rq) return -3;
    if (s.src_row >= 0) {
      if (n != 1) return -12;
      out[lay->token_src + t] = s.src_row;
      has_src = 1;
    } else {
      std::memcpy(out + lay->token_ids + t, tokens + s.token_off, sizeof(int32_t) * n);
      for (int i = 0; i < n; ++i) out[lay->token_src + t + i] = -1;
    }
    for (int i = 0; i < n; ++i) {
      out[lay->positions + t + i] = s.start_pos + i;
      out[lay->seq_of_token + t + i] = si;
    }
    for (int g = 0; g < G; ++g) {
      const std::vector<int32_t>& tb = rq->tables[g];
      if (static_cast<int>(tb.size()) * ps < end) {
        result[6] = static_cast<int>(tb.size()) * ps;
        return -13;
      }
      int32_t* sl = out + slots_off[g] + t;
      for (int i = 0; i < n; ++i) {
        const int pos = s.start_pos + i;
        sl[i] = tb[pos / ps] * ps + pos % ps;
      }
      const int nb = std::min<int>(static_cast<int>(tb.size()), B);
      std::memcpy(out + table_off[g] + static_cast<size_t>(si) * B, tb.data(), sizeof(int32_t) * nb);
    }
    out[lay->state_slot + si] = rq->state_slot;
    if (n == 1) {
      int32_t* d = out + lay->decode_info + 4 * nd;
      d[0] = t;
      d[1] = si;
      d[2] = end;
      ++nd;
      max_ctx = std::max(max_ctx, end);
    } else {
      for (int r0 = 0; r0 < n; r0 += tile_rows) {
        out[lay->tile_seq + li] = si;
        out[lay->tile_tok + li] = t + r0;
        out[lay->tile_rows + li] = std::min(tile_rows, n - r0);
        ++li;
      }
    }
    for (int k = 0; k < s.num_want; ++k) {
      const int wi = want[s.want_off + k];
      if (wi < 0 || wi >= n) {
        result[6] = wi;
        return -14;
      }
      out[lay->logit_rows + r] = t + wi;
      float one = 1.0f;
      if (s.has_sampling) {
        any_sampling = 1;
        std::memcpy(out + lay->temperature + r, &s.temperature, 4);
        out[lay->top_k + r] = s.top_k;
        std::memcpy(out + lay->top_p + r, &s.top_p, 4);
        std::memcpy(out + lay->seed_lo + r, &s.seed_lo, 4);
        std::memcpy(out + lay->seed_hi + r, &s.seed_hi, 4);
      } else {
        std::memcpy(out + lay->top_p + r, &one, 4);
      }
      out[lay->sample_pos + r] = s.start_pos + wi + 1;   // position of the token being drawn
      ++r;
    }
    t += n;
  }
  result[0] = nd;
  result[1] = li;
  result[2] = max_ctx;
  result[3] = has_src;
  result[4] = any_sampling;
  return 0;
}

// The dummy rows that pad a step of single tokens up to a fixed shape: token 0 at position 0 of a
// sequence whose table is all page 0.
void rl_hc_pad(int32_t* out, const RlLayout* lay, int from, int to) {
  const float one = 1.0f;
  for (int i = from; i < to; ++i) {
    out[lay->token_src + i] = -1;
    out[lay->seq_of_token + i] = i;
    int32_t* d = out + lay->decode_info + 4 * i;
    d[0] = i;
    d[1] = i;
    d[2] = 1;
    out[lay->logit_rows + i] = i;
    std::memcpy(out + lay->top_p + i, &one, 4);
    out[lay->sample_pos + i] = 1;
  }
}

}  // extern "C"

// ------------------------------------------------------------------ the scheduler's plan of one step
// Policy of the reference's scheduler (src/core/scheduler.cpp:104-218): under a token budget, first one
// token for every running sequence that is decoding, then portions of prompts (running sequences that
// are mid-prompt first, then admissions from the front of the waiting queue while a watermark of pages
// stays free, unless nothing is running).  A decoding sequence that cannot get its next page preempts
// the newest running sequence that is not in the plan yet (all its pages go back, it is queued again at
// the front), or itself if there is none.  If nothing could be planned while sequences are stuck
// mid-prompt, the newest are freed until the oldest goes on.
//
// The caller passes the running sequences in admission order followed by the front of the waiting
// queue; the planner works on the cache manager's state directly (opens, reserves, closes) and gives
// back, per sequence, its new request id, computed count and queue, the queues' new orders and the
// entries of the plan.
struct RlSchedSeq {
  int32_t rid;            // in/out: the sequence's request in the cache manager, -1: none
  int32_t known;          // tokens the host knows (prompt + received samples)
  int32_t pending;        // tokens sampled on the GPU that the host has not read yet
  int32_t computed;       // in/out: positions whose cache writes have been enqueued
  int32_t prompt_len;
  int32_t max_new;
  int32_t pending_ok;     // the pending token is the previous step's: it can be read on the device
  int32_t pending_row;
  int32_t where;          // in/out: 0 running, 1 waiting; out also 2: parked (preempted with a token in flight)
  int32_t preempted;      // out: times preempted in this call
  int32_t cache_changed;  // out: its request was opened or closed in this call
};

struct RlSchedCfg {
  int32_t max_num_seqs, budget, max_seq_len, mix;
  double watermark;       // fraction of a group's pages that an admission must leave free
};

struct RlSchedEntry {
  int32_t seq, start_pos, num_tokens, sample, from_device, src_row;
};

namespace {

struct Planner {
  Core* c;
  RlSchedCfg cfg;
  RlSchedSeq* s;
  std::vector<int> running, waiting, parked;
  std::vector<RlSchedEntry> plan;
  int budget = 0, num_preempted = 0, error_seq = -1;

  int total(int i) const { return s[i].known + s[i].pending; }
  int uncomputed(int i) const { return total(i) - s[i].computed; }
  bool needs_compute(int i) const {
    const int u = uncomputed(i);
    if (u > 1) return true;
    if (u == 0) return false;
    if (total(i) - s[i].prompt_len >= s[i].max_new) return false;
    return total(i) < cfg.max_seq_len;
  }
  bool ensure(int i, int positions) {
    if (s[i].rid < 0) {
      const int rid = rl_hc_open(c);
      if (rid < 0) return false;
      s[i].rid = rid;
      s[i].cache_changed = 1;
    }
    return rl_hc_reserve(c, s[i].rid, positions) == 1;
  }
  void drop_cache(int i) {
    if (s[i].rid >= 0) {
      int bad = 0;
      rl_hc_close(c, s[i].rid, &bad);
      s[i].rid = -1;
      s[i].cache_changed = 1;
    }
  }
  void preempt(int i) {
    drop_cache(i);
    s[i].computed = 0;
    ++s[i].preempted;
    running.erase(std::remove(running.begin(), running.end(), i), running.end());
    if (s[i].pending > 0) {
      s[i].where = 2;
      parked.push_back(i);
    } else {
      s[i].where = 1;
      waiting.insert(waiting.begin(), i);
    }
  }
  bool add_entry(int i, int n) {
    RlSchedEntry e;
    e.seq = i;
    e.start_pos = s[i].computed;
    e.num_tokens = n;
    e.sample = (s[i].computed + n == total(i)) ? 1 : 0;
    e.from_device = 0;
    e.src_row = -1;
    if (e.start_pos >= s[i].known) {
      if (!(n == 1 && s[i].pending > 0 && s[i].pending_ok)) {
        error_seq = i;
        return false;
      }
      e.from_device = 1;
      e.src_row = s[i].pending_row;
    }
    s[i].computed += n;
    budget -= n;
    plan.push_back(e);
    return true;
  }
  bool schedule_prefill() {
    const std::vector<int> snapshot = running;
    for (int i : snapshot) {
      if (budget <= 0) return true;
      if (uncomputed(i) <= 1) continue;
      // a pending token cannot be part of a multi-token portion
      const int chunk = std::min(s[i].pending > 0 ? s[i].known - s[i].computed : uncomputed(i), budget);
      if (chunk <= 0) continue;
      if (!ensure(i, s[i].computed + chunk)) return true;
      if (!add_entry(i, chunk)) return false;
    }
    while (!waiting.empty() && budget > 0 && static_cast<int>(running.size()) < cfg.max_num_seqs) {
      const int i = waiting.front();
      const int chunk = std::min(uncomputed(i), budget);
      if (!running.empty()) {
        const int need = c->blocks_for(s[i].computed + chunk);
        for (size_t g = 0; g < c->pools.size(); ++g) {
          const int mark = static_cast<int>(cfg.watermark * c->pools[g].usable());
          if (static_cast<int>(c->pools[g].free_list.size()) - need < mark) return true;
        }
      }
      if (c->num_open >= c->num_state_slots && s[i].rid < 0) return true;
      if (!ensure(i, s[i].computed + chunk)) {
        drop_cache(i);
        return true;
      }
      waiting.erase(waiting.begin());
      s[i].where = 0;
      running.push_back(i);
      if (!add_entry(i, chunk)) return false;
    }
    return true;
  }
  bool schedule_decode() {
    size_t k = 0;
    while (k < running.size()) {
      const int i = running[k];
      if (budget <= 0) break;
      if (uncomputed(i) != 1 || !needs_compute(i)) {
        ++k;
        continue;
      }
      bool self_preempted = false;
      while (!ensure(i, s[i].computed + 1)) {
        const int victim = running.back();
        bool in_plan = false;
        for (const RlSchedEntry& e : plan) in_plan = in_plan || e.seq == victim;
        if (victim == i || in_plan) {
          preempt(i);
          self_preempted = true;
          break;
        }
        preempt(victim);
        ++num_preempted;
      }
      if (self_preempted) {
        ++num_preempted;
        continue;                        // running shrank at position k
      }
      if (!add_entry(i, 1)) return false;
      ++k;
    }
    return true;
  }
  bool run() {
    budget = cfg.budget;
    if (cfg.mix) {
      if (!schedule_decode() || !schedule_prefill()) return false;
    } else {
      if (!schedule_prefill()) return false;
      if (plan.empty() && !schedule_decode()) return false;
    }
    // sequences stuck mid-prompt can hold every page with none able to go on
    while (plan.empty() && running.size() > 1) {
      bool any = false;
      for (int i : running) any = any || needs_compute(i);
      if (!any) break;
      preempt(running.back());
      ++num_preempted;
      if (!schedule_prefill()) return false;
      if (plan.empty() && !schedule_decode()) return false;
    }
    return true;
  }
};

}  // namespace

extern "C" {

// seqs: num_running running sequences (oldest first), then num_waiting from the front of the waiting
// queue.  Out: entries (capacity: one per sequence), the new running order, the new order of the passed
// part of the waiting queue (preempted sequences in front), the parked ones; counts in n_out[0..3] =
// entries, running, waiting, parked, n_out[4] = preemptions.  Returns 0, or -10 when a sequence would
// need a device token that is not available (n_out[5] = its index), -5 for bad arguments.
int rl_sched_plan(void* h, const RlSchedCfg* cfg, RlSchedSeq* seqs, int num_running, int num_waiting,
                  RlSchedEntry* entries, int32_t* running_out, int32_t* waiting_out, int32_t* parked_out,
                  int32_t* n_out) {
  if (!h || !cfg || num_running < 0 || num_waiting < 0) return -5;
  Planner p;
  p.c = static_cast<Core*>(h);
  p.cfg = *cfg;
  p.s = seqs;
  const int n = num_running + num_waiting;
  for (int i = 0; i < n; ++i) {
    seqs[i].preempted = 0;
    seqs[i].cache_changed = 0;
    seqs[i].where = i < num_running ? 0 : 1;
    (i < num_running ? p.running : p.waiting).push_back(i);
  }
  const bool ok = p.run();
  // a sequence is planned at most once in a step (one token, or one portion)
  n_out[0] = static_cast<int32_t>(p.plan.size());
  n_out[1] = static_cast<int32_t>(p.running.size());
  n_out[2] = static_cast<int32_t>(p.waiting.size());
  n_out[3] = static_cast<int32_t>(p.parked.size());
  n_out[4] = p.num_preempted;
  n_out[5] = p.error_seq;
  std::copy(p.plan.begin(), p.plan.end(), entries);
  std::copy(p.running.begin(), p.running.end(), running_out);
  std::copy(p.waiting.begin(), p.waiting.end(), waiting_out);
  std::copy(p.parked.begin(), p.parked.end(), parked_out);
  return ok ? 0 : -10;
}

}  // extern "C"
