// Continuous-batching scheduler core: slot table, admission policy and step planning.
//
// Behavioural counterpart of the reference's GrimoireScheduler::run (grimoire.cpp:24370-24993):
//  * admission hold: a fresh arrival waits a few milliseconds (longer for long prompts) for a burst
//    of arrivals so several prompts are admitted together (:24420-24463);
//  * batched admission of short prompts under a token budget (<= 32768 tokens, admit_batch :12071);
//  * interleaved admission: while conversations are decoding, a long prompt is read in chunks of
//    `interleave_chunk` tokens between decode steps (admit_begin/chunk/end :12183-12223);
//  * a step covers every live conversation; speculative depth comes from a table indexed by the
//    number of live conversations (:11401-11431);
//  * cancellation takes effect at the next plan; finished jobs free their slot at once.
// The engine calls themselves (prefill / decode rows) are made by the Python scheduler thread that
// owns the engine; this core only decides what to run next, so it is testable without a device.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <map>
#include <vector>

namespace {

enum JobState : int { PENDING = 0, ADMITTING = 1, LIVE = 2, DONE = 3 };

struct Job {
  int64_t id;
  int prompt_len, prefilled, max_new, emitted;
  int state, slot;
  double arrival_ms;
  bool cancelled;
  int reused;   // tokens served by the prefix cache
};

struct Config {
  int width;              // conversation slots stepped together (GRIMOIRE_MAX_BATCH)
  int max_ctx;
  int interleave_chunk;   // GRIMOIRE_INTERLEAVE_CHUNK (1024)
  int prefill_chunk;      // GRIMOIRE_PREFILL_CHUNK (4096)
  int admit_budget;       // tokens of one batched admission (32768)
  int long_prompt;        // prompts at least this long use the long hold
  double hold_ms, hold_long_ms;
  int depths[16];
  int n_depths;
  int spec_rows;          // row budget of one verify step
};

struct Sched {
  Config cfg;
  std::map<int64_t, Job> jobs;
  std::deque<int64_t> pending;
  std::vector<int64_t> slots;   // slot -> job id or -1
  int64_t steps = 0, admitted = 0, cancelled = 0;
};

}  // namespace

extern "C" {

// plan kinds (bit mask)
enum { GRM_PLAN_IDLE = 0, GRM_PLAN_ADMIT = 1, GRM_PLAN_STEP = 2, GRM_PLAN_WAIT = 4 };

struct GrmPlan {
  int kind;
  double wait_ms;
  int n_admit;
  int64_t admit_job[64];
  int admit_slot[64];
  int admit_from[64];
  int admit_to[64];
  int n_live;
  int64_t live_job[64];
  int live_slot[64];
  int draft_depth;      // per conversation, from the depth table
  int n_retired;
  int64_t retired_job[64];
  int retired_slot[64];
};

void* grm_sched_new(int width, int max_ctx, int interleave_chunk, int prefill_chunk, int admit_budget, int long_prompt,
                    double hold_ms, double hold_long_ms, const int* depths, int n_depths, int spec_rows) {
  if (width < 1 || width > 64) return nullptr;
  Sched* s = new Sched();
  s->cfg = Config{width, max_ctx, interleave_chunk, prefill_chunk, admit_budget, long_prompt, hold_ms, hold_long_ms, {0}, 0, spec_rows};
  s->cfg.n_depths = std::min(n_depths, 16);
  for (int i = 0; i < s->cfg.n_depths; ++i) s->cfg.depths[i] = depths[i];
  s->slots.assign(width, -1);
  return s;
}

void grm_sched_delete(void* h) { delete static_cast<Sched*>(h); }

int grm_sched_width(void* h) { return static_cast<Sched*>(h)->cfg.width; }

// returns 0, or -1 when the prompt cannot fit the context (the caller answers HTTP 400)
int grm_sched_submit(void* h, int64_t id, int prompt_len, int max_new, int reused, double now_ms) {
  Sched* s = static_cast<Sched*>(h);
  if (prompt_len <= 0 || prompt_len >= s->cfg.max_ctx) return -1;
  if (s->jobs.count(id)) return -2;
  Job j{id, prompt_len, std::min(reused, prompt_len - 1), std::min(max_new, s->cfg.max_ctx - prompt_len), 0, PENDING, -1, now_ms, false, reused};
  s->jobs[id] = j;
  s->pending.push_back(id);
  return 0;
}

int grm_sched_cancel(void* h, int64_t id) {
  Sched* s = static_cast<Sched*>(h);
  auto it = s->jobs.find(id);
  if (it == s->jobs.end()) return -1;
  it->second.cancelled = true;
  return 0;
}

static int depth_for(const Config& c, int live) {
  if (c.n_depths == 0) return 0;
  return c.depths[std::min(std::max(live, 1), c.n_depths) - 1];
}

// Decide what the engine thread does next.  Retired jobs (finished or cancelled) are reported once
// so the caller can cache / release their KV.
void grm_sched_plan(void* h, double now_ms, GrmPlan* out) {
  Sched* s = static_cast<Sched*>(h);
  const Config& c = s->cfg;
  std::memset(out, 0, sizeof(*out));
  // ---- retire ----
  for (int sl = 0; sl < c.width; ++sl) {
    const int64_t id = s->slots[sl];
    if (id < 0) continue;
    Job& j = s->jobs[id];
    if (j.state == DONE || j.cancelled) {
      if (out->n_retired < 64) {
        out->retired_job[out->n_retired] = id;
        out->retired_slot[out->n_retired] = sl;
        ++out->n_retired;
      }
      if (j.cancelled && j.state != DONE) ++s->cancelled;
      s->slots[sl] = -1;
      s->jobs.erase(id);
    }
  }
  // cancelled before admission
  for (auto it = s->pending.begin(); it != s->pending.end();) {
    Job& j = s->jobs[*it];
    if (j.cancelled) {
      if (out->n_retired < 64) { out->retired_job[out->n_retired] = j.id; out->retired_slot[out->n_retired] = -1; ++out->n_retired; }
      ++s->cancelled;
      s->jobs.erase(*it);
      it = s->pending.erase(it);
    } else {
      ++it;
    }
  }
  int live = 0, admitting = 0, free_slots = 0;
  for (int sl = 0; sl < c.width; ++sl) {
    const int64_t id = s->slots[sl];
    if (id < 0) { ++free_slots; continue; }
    const Job& j = s->jobs[id];
    if (j.state == LIVE) ++live;
    if (j.state == ADMITTING) ++admitting;
  }
  // ---- admission hold: wait for a burst only when nothing is decoding ----
  if (!s->pending.empty() && free_slots > 0 && live == 0 && admitting == 0) {
    double newest = 0, hold = c.hold_ms;
    for (int64_t id : s->pending) {
      const Job& j = s->jobs[id];
      newest = std::max(newest, j.arrival_ms);
      if (j.prompt_len >= c.long_prompt) hold = std::max(hold, c.hold_long_ms);
    }
    const bool burst_full = (int)s->pending.size() >= free_slots;
    if (!burst_full && now_ms - newest < hold) {
      out->kind = GRM_PLAN_WAIT;
      out->wait_ms = hold - (now_ms - newest);
      return;
    }
  }
  // ---- move pending jobs into free slots ----
  while (!s->pending.empty() && free_slots > 0) {
    const int64_t id = s->pending.front();
    s->pending.pop_front();
    Job& j = s->jobs[id];
    for (int sl = 0; sl < c.width; ++sl)
      if (s->slots[sl] < 0) { s->slots[sl] = id; j.slot = sl; break; }
    j.state = ADMITTING;
    --free_slots;
    ++admitting;
    ++s->admitted;
  }
  // ---- admission work of this round ----
  int budget = c.admit_budget;
  for (int sl = 0; sl < c.width && out->n_admit < 64; ++sl) {
    const int64_t id = s->slots[sl];
    if (id < 0) continue;
    Job& j = s->jobs[id];
    if (j.state != ADMITTING) continue;
    const int left = j.prompt_len - j.prefilled;
    // while others decode, read long prompts in interleave chunks; otherwise whole prefill chunks
    int take = (live > 0) ? std::min(left, c.interleave_chunk) : std::min(left, std::max(c.prefill_chunk, 1));
    take = std::min(take, budget);
    if (take <= 0) continue;
    out->admit_job[out->n_admit] = id;
    out->admit_slot[out->n_admit] = sl;
    out->admit_from[out->n_admit] = j.prefilled;
    out->admit_to[out->n_admit] = j.prefilled + take;
    ++out->n_admit;
    budget -= take;
    if (live > 0) break;   // one interleave chunk per decode step
  }
  if (out->n_admit) out->kind |= GRM_PLAN_ADMIT;
  // ---- decode step over the live conversations ----
  for (int sl = 0; sl < c.width; ++sl) {
    const int64_t id = s->slots[sl];
    if (id < 0) continue;
    const Job& j = s->jobs[id];
    if (j.state == LIVE && out->n_live < 64) {
      out->live_job[out->n_live] = id;
      out->live_slot[out->n_live] = sl;
      ++out->n_live;
    }
  }
  if (out->n_live) {
    out->kind |= GRM_PLAN_STEP;
    int d = depth_for(c, out->n_live);
    if (c.spec_rows > 0) d = std::min(d, std::max(0, c.spec_rows / out->n_live - 1));
    out->draft_depth = d;
    ++s->steps;
  }
}

// n tokens of the prompt are now in the cache; the job turns LIVE when the prompt is complete
int grm_sched_on_prefilled(void* h, int64_t id, int upto) {
  Sched* s = static_cast<Sched*>(h);
  auto it = s->jobs.find(id);
  if (it == s->jobs.end()) return -1;
  Job& j = it->second;
  j.prefilled = std::max(j.prefilled, std::min(upto, j.prompt_len));
  if (j.prefilled >= j.prompt_len && j.state == ADMITTING) j.state = LIVE;
  return j.state;
}

// n tokens were emitted for the job; finished != 0 (eos / failure) or an exhausted budget ends it
int grm_sched_on_tokens(void* h, int64_t id, int n, int finished) {
  Sched* s = static_cast<Sched*>(h);
  auto it = s->jobs.find(id);
  if (it == s->jobs.end()) return -1;
  Job& j = it->second;
  j.emitted += n;
  if (finished || j.emitted >= j.max_new) j.state = DONE;
  return j.state;
}

int grm_sched_remaining(void* h, int64_t id) {
  Sched* s = static_cast<Sched*>(h);
  auto it = s->jobs.find(id);
  if (it == s->jobs.end()) return 0;
  return std::max(0, it->second.max_new - it->second.emitted);
}

void grm_sched_counts(void* h, int64_t* out4) {
  Sched* s = static_cast<Sched*>(h);
  int busy = 0;
  for (int64_t v : s->slots) busy += v >= 0;
  out4[0] = s->steps; out4[1] = s->admitted; out4[2] = (int64_t)s->pending.size(); out4[3] = busy;
}

}  // extern "C"
