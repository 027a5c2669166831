// Host runtime of the serving engine: paged KV-cache block allocator and the
// continuous-batching scheduler.  Plain C++ behind a C ABI (loaded with ctypes).
//
// The reference server collects a static batch under a deadline, pads it and runs
// every request to the longest max_new_tokens with a dense, never-freed cache
// (rumus-serve/src/scheduler.rs:29-95, gpu_worker.rs:77-150).  Here requests join
// and leave between decode steps, prompt prefill is chunked under a per-step
// token budget, and the KV cache is a pool of fixed-size blocks handed out per
// sequence and returned the moment a sequence finishes.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace {

struct Seq {
  int64_t id;
  int prompt_len;
  int max_new;
  int computed;    // prompt tokens whose KV is already in the cache
  int generated;   // tokens generated so far
  bool running;    // admitted (has blocks)
  std::vector<int> blocks;
};

struct Engine {
  int num_blocks, block_size;
  int max_batch;        // max sequences decoded per step
  int token_budget;     // max tokens (prefill chunk + decode) per step
  std::vector<int> free_list;
  std::unordered_map<int64_t, Seq> seqs;
  std::deque<int64_t> waiting;
  std::vector<int64_t> running;
  std::mutex mu;
  int64_t preemptions = 0;
};

int blocks_needed(int tokens, int bs) { return (tokens + bs - 1) / bs; }

bool grow(Engine& e, Seq& s, int total_tokens) {
  const int need = blocks_needed(total_tokens, e.block_size);
  const int extra = need - (int)s.blocks.size();
  if (extra <= 0) return true;
  if ((int)e.free_list.size() < extra) return false;
  for (int i = 0; i < extra; ++i) {
    s.blocks.push_back(e.free_list.back());
    e.free_list.pop_back();
  }
  return true;
}

void release(Engine& e, Seq& s) {
  for (int b : s.blocks) e.free_list.push_back(b);
  s.blocks.clear();
}

}  // namespace

extern "C" {

void* rbs_create(int num_blocks, int block_size, int max_batch, int token_budget) {
  Engine* e = new Engine();
  e->num_blocks = num_blocks;
  e->block_size = block_size;
  e->max_batch = max_batch;
  e->token_budget = token_budget;
  e->free_list.reserve(num_blocks);
  for (int i = num_blocks - 1; i >= 0; --i) e->free_list.push_back(i);
  return e;
}

void rbs_destroy(void* h) { delete static_cast<Engine*>(h); }

int rbs_num_free_blocks(void* h) {
  Engine* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> lk(e->mu);
  return (int)e->free_list.size();
}

int rbs_num_waiting(void* h) {
  Engine* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> lk(e->mu);
  return (int)e->waiting.size();
}

int rbs_num_running(void* h) {
  Engine* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> lk(e->mu);
  return (int)e->running.size();
}

long long rbs_num_preemptions(void* h) { return static_cast<Engine*>(h)->preemptions; }

// Returns 0, or -1 when the request can never fit (prompt + max_new exceeds the whole pool).
int rbs_add_request(void* h, long long id, int prompt_len, int max_new) {
  Engine* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> lk(e->mu);
  if (blocks_needed(prompt_len + max_new, e->block_size) > e->num_blocks) return -1;
  if (e->seqs.count(id)) return -2;
  Seq s{id, prompt_len, max_new, 0, 0, false, {}};
  e->seqs.emplace(id, std::move(s));
  e->waiting.push_back(id);
  return 0;
}

// Plans one engine step.
//   decode_ids[n_decode]                      sequences that produce one token this step
//   prefill_ids / prefill_start / prefill_len  prompt chunks processed this step
// A sequence whose last prompt chunk is processed this step also yields its first token.
// Returns the total number of tokens scheduled.
int rbs_schedule(void* h, long long* decode_ids, int* n_decode, long long* prefill_ids,
                 int* prefill_start, int* prefill_len, int* n_prefill, int max_out) {
  Engine* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> lk(e->mu);
  int nd = 0, np = 0, tokens = 0;
  // 1. running sequences that finished their prompt decode one token each (they need room for it)
  for (size_t i = 0; i < e->running.size();) {
    Seq& s = e->seqs[e->running[i]];
    if (s.computed < s.prompt_len) { ++i; continue; }
    const int total = s.prompt_len + s.generated + 1;
    if (!grow(*e, s, total)) {
      // out of blocks: preempt the youngest running sequence (recompute later), retry this one
      int64_t victim = e->running.back();
      Seq& v = e->seqs[victim];
      release(*e, v);
      v.running = false;
      v.computed = 0;
      v.prompt_len += v.generated;  // generated tokens become part of the prompt to recompute
      v.max_new -= v.generated;
      v.generated = 0;
      e->running.pop_back();
      e->waiting.push_front(victim);
      ++e->preemptions;
      if (victim == s.id) break;
      continue;
    }
    if (nd < max_out && nd < e->max_batch && tokens < e->token_budget) {
      decode_ids[nd++] = s.id;
      ++tokens;
    }
    ++i;
  }
  // 2. continue partially prefilled running sequences, then admit waiting ones
  auto plan_prefill = [&](Seq& s) -> bool {
    const int remaining = s.prompt_len - s.computed;
    int chunk = std::min(remaining, e->token_budget - tokens);
    if (chunk <= 0 || np >= max_out) return false;
    if (!grow(*e, s, s.computed + chunk)) {
      // take what fits
      const int fit = ((int)s.blocks.size() + (int)e->free_list.size()) * e->block_size - s.computed;
      chunk = std::min(chunk, fit);
      if (chunk <= 0 || !grow(*e, s, s.computed + chunk)) return false;
    }
    prefill_ids[np] = s.id;
    prefill_start[np] = s.computed;
    prefill_len[np] = chunk;
    ++np;
    tokens += chunk;
    return true;
  };
  for (int64_t id : e->running) {
    Seq& s = e->seqs[id];
    if (s.computed < s.prompt_len && tokens < e->token_budget) plan_prefill(s);
  }
  while (!e->waiting.empty() && tokens < e->token_budget && (int)e->running.size() < e->max_batch) {
    Seq& s = e->seqs[e->waiting.front()];
    if (!plan_prefill(s)) break;
    s.running = true;
    e->running.push_back(s.id);
    e->waiting.pop_front();
  }
  *n_decode = nd;
  *n_prefill = np;
  return tokens;
}

// Commit the step planned by rbs_schedule: advances counters; sequences that reached
// max_new (or were reported finished via `eos_ids`) are retired and their blocks freed.
// finished_ids receives the retired ids; returns their count.
int rbs_commit(void* h, const long long* decode_ids, int n_decode, const long long* prefill_ids,
               const int* prefill_len, int n_prefill, const long long* eos_ids, int n_eos,
               long long* finished_ids, int max_out) {
  Engine* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> lk(e->mu);
  int nf = 0;
  auto retire = [&](Seq& s) {
    release(*e, s);
    if (nf < max_out) finished_ids[nf++] = s.id;
    e->running.erase(std::remove(e->running.begin(), e->running.end(), s.id), e->running.end());
    e->seqs.erase(s.id);
  };
  for (int i = 0; i < n_prefill; ++i) {
    auto it = e->seqs.find(prefill_ids[i]);
    if (it == e->seqs.end()) continue;
    Seq& s = it->second;
    s.computed += prefill_len[i];
    if (s.computed >= s.prompt_len) {
      s.generated += 1;  // the last prompt chunk yields the first token
      if (s.generated >= s.max_new) retire(s);
    }
  }
  for (int i = 0; i < n_decode; ++i) {
    auto it = e->seqs.find(decode_ids[i]);
    if (it == e->seqs.end()) continue;
    Seq& s = it->second;
    s.generated += 1;
    if (s.generated >= s.max_new) retire(s);
  }
  for (int i = 0; i < n_eos; ++i) {
    auto it = e->seqs.find(eos_ids[i]);
    if (it != e->seqs.end()) retire(it->second);
  }
  return nf;
}

// Copies the block table of a sequence; returns the number of blocks (or -1 if unknown).
int rbs_block_table(void* h, long long id, int* out, int max_blocks) {
  Engine* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> lk(e->mu);
  auto it = e->seqs.find(id);
  if (it == e->seqs.end()) return -1;
  const int n = std::min((int)it->second.blocks.size(), max_blocks);
  std::memcpy(out, it->second.blocks.data(), sizeof(int) * n);
  return (int)it->second.blocks.size();
}

// Block tables of `n` sequences at once, into a row-major int32 [n, max_blocks] array (unused
// entries zero); `counts[i]` receives the number of blocks of sequence i (-1 if unknown).  One call
// per decode step instead of one per sequence.
int rbs_block_tables(void* h, const long long* ids, int n, int* out, int max_blocks, int* counts) {
  Engine* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> lk(e->mu);
  std::memset(out, 0, sizeof(int) * (size_t)n * (size_t)max_blocks);
  int missing = 0;
  for (int i = 0; i < n; ++i) {
    auto it = e->seqs.find(ids[i]);
    if (it == e->seqs.end()) {
      counts[i] = -1;
      ++missing;
      continue;
    }
    const int nb = std::min((int)it->second.blocks.size(), max_blocks);
    std::memcpy(out + (size_t)i * max_blocks, it->second.blocks.data(), sizeof(int) * nb);
    counts[i] = (int)it->second.blocks.size();
  }
  return missing;
}

// Context length (tokens whose KV is cached, counting generated ones) of a sequence.
int rbs_context_len(void* h, long long id) {
  Engine* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> lk(e->mu);
  auto it = e->seqs.find(id);
  if (it == e->seqs.end()) return -1;
  const Seq& s = it->second;
  return s.computed + std::max(0, s.generated - (s.computed >= s.prompt_len ? 1 : 0));
}

void rbs_abort(void* h, long long id) {
  Engine* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> lk(e->mu);
  auto it = e->seqs.find(id);
  if (it == e->seqs.end()) return;
  release(*e, it->second);
  e->running.erase(std::remove(e->running.begin(), e->running.end(), id), e->running.end());
  e->waiting.erase(std::remove(e->waiting.begin(), e->waiting.end(), id), e->waiting.end());
  e->seqs.erase(it);
}
}
