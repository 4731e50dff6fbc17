// Paged-KV block manager and continuous-batching scheduler of the rollout
// engine (C ABI, loaded with ctypes).
//
// The scheduler owns, per request, the token list (prompt + generated), the
// generated tokens' logprobs and the list of KV pages. Each engine iteration
// asks for a plan:
//   * PREFILL – waiting requests are admitted while sequence slots, pages and
//     the token budget last; the plan lists their packed tokens, positions,
//     cu_seqlens and the flat KV slot of every token;
//   * DECODE  – every running request contributes its last token, position,
//     slot, sequence length and page table row.
// After the model step the engine commits one sampled token (+ logprob) per
// planned sequence; the scheduler applies stop-token and length limits, frees
// the pages of finished requests and reports them. When pages run out the
// youngest running request is preempted: its pages are released and it goes
// back to the head of the waiting queue to be re-prefilled with everything it
// has produced so far. abort_all() (used when generation is paused for a weight
// update) finishes every live request with reason ABORT and returns partial
// outputs, which is what makes generation interruptible.
//
// The reference delegates all of this to an external SGLang / vLLM server
// (areal/engine/sglang_remote.py, areal/api/cli_args.py:1624-1890).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

enum FinishReason : int { kRunning = 0, kStop = 1, kLength = 2, kAbort = 3 };
enum PlanKind : int { kIdle = 0, kPrefill = 1, kDecode = 2 };

struct Request {
  int64_t id;
  std::vector<int32_t> tokens;   // prompt + generated
  std::vector<float> logprobs;   // generated only
  int32_t prompt_len = 0;
  int32_t max_new_tokens = 0;
  int32_t min_new_tokens = 0;
  bool ignore_eos = false;
  std::vector<int32_t> stop_ids;
  std::vector<int32_t> blocks;
  int32_t cached_len = 0;  // tokens whose K/V are in the cache
  int finish = kRunning;
  int64_t arrival = 0;
  uint64_t prompt_hash = 0;
  bool kv_ready = false;   // the prompt's K/V have been written (its prefill step was committed)
  // The first share_len tokens are common to a group of requests (the samples of one prompt). For a fresh
  // request that is the whole prompt; a request re-submitted after an interruption carries prompt + partial
  // output as its prompt and names the original prompt's length here.
  int32_t share_len = 0;
  uint64_t share_hash = 0;
};

struct Scheduler {
  int num_blocks, block_size, max_num_seqs, max_batched_tokens, max_blocks_per_seq;
  std::vector<int32_t> free_blocks;
  std::vector<int32_t> refcnt;  // pages may be shared by requests with the same prompt (read-only full pages)
  std::unordered_map<uint64_t, int64_t> prompt_leader;  // prompt hash -> request whose prompt pages can be shared
  bool share_prompts = true;
  int64_t n_forked = 0, n_shared_pages = 0, n_dedup_pages = 0;
  // common-prefix hash -> request whose prefilled prefix pages later arrivals of the group adopt
  std::unordered_map<uint64_t, int64_t> prefix_leader;
  std::unordered_map<int64_t, Request> reqs;
  std::deque<int64_t> waiting;
  std::vector<int64_t> running;
  std::vector<int64_t> planned;  // sequences of the outstanding plan, in plan order
  int planned_kind = kIdle;
  std::deque<int64_t> finished;
  int64_t next_id = 1;
  int64_t clock = 0;
  int64_t n_preempt = 0;
  std::mutex mu;

  bool ensure_blocks(Request& r, int32_t need_tokens) {
    const int32_t need = (need_tokens + block_size - 1) / block_size;
    if (need > max_blocks_per_seq) return false;
    while (static_cast<int32_t>(r.blocks.size()) < need) {
      if (free_blocks.empty()) return false;
      const int32_t b = free_blocks.back();
      free_blocks.pop_back();
      refcnt[b] = 1;
      r.blocks.push_back(b);
    }
    return true;
  }
  void release(Request& r) {
    for (int32_t b : r.blocks)
      if (--refcnt[b] == 0) free_blocks.push_back(b);
    r.blocks.clear();
    r.cached_len = 0;
    r.kv_ready = false;
  }
  // A running request with the same prompt whose prompt pages are in the cache, or nullptr.
  Request* leader_for(const Request& r) {
    auto it = prompt_leader.find(r.prompt_hash);
    if (it == prompt_leader.end() || it->second == r.id) return nullptr;
    auto rq = reqs.find(it->second);
    if (rq == reqs.end()) return nullptr;
    Request& l = rq->second;
    if (l.finish != kRunning || l.prompt_len != r.prompt_len || l.blocks.empty()) return nullptr;
    if (!std::equal(r.tokens.begin(), r.tokens.begin() + r.prompt_len, l.tokens.begin())) return nullptr;
    return &l;
  }
  void finish(Request& r, int reason) {
    r.finish = reason;
    release(r);
    finished.push_back(r.id);
  }
  int64_t slot_of(const Request& r, int32_t pos) const {
    return static_cast<int64_t>(r.blocks[pos / block_size]) * block_size + pos % block_size;
  }
};

}  // namespace

extern "C" {

void* b200_sched_create(int num_blocks, int block_size, int max_num_seqs, int max_batched_tokens,
                        int max_blocks_per_seq) {
  auto* s = new Scheduler();
  s->num_blocks = num_blocks;
  s->block_size = block_size;
  s->max_num_seqs = max_num_seqs;
  s->max_batched_tokens = max_batched_tokens;
  s->max_blocks_per_seq = max_blocks_per_seq;
  s->free_blocks.reserve(num_blocks);
  s->refcnt.assign(num_blocks, 0);
  for (int b = num_blocks - 1; b >= 0; --b) s->free_blocks.push_back(b);
  return s;
}

void b200_sched_destroy(void* h) { delete static_cast<Scheduler*>(h); }

// Returns the request id (> 0) or -1 when the prompt can never fit. share_len: number of leading tokens that
// the other samples of the same group also start with (<= 0: the whole prompt).
int64_t b200_sched_add_shared(void* h, const int32_t* prompt, int n_prompt, int max_new_tokens,
                              int min_new_tokens, const int32_t* stop_ids, int n_stop, int ignore_eos,
                              int share_len) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  const int64_t total = static_cast<int64_t>(n_prompt) + max_new_tokens;
  if (n_prompt <= 0 || n_prompt > s->max_batched_tokens ||
      (n_prompt + s->block_size - 1) / s->block_size > s->max_blocks_per_seq)
    return -1;
  (void)total;
  Request r;
  r.id = s->next_id++;
  r.tokens.assign(prompt, prompt + n_prompt);
  r.prompt_len = n_prompt;
  r.max_new_tokens = max_new_tokens;
  r.min_new_tokens = min_new_tokens;
  r.ignore_eos = ignore_eos != 0;
  r.stop_ids.assign(stop_ids, stop_ids + n_stop);
  r.arrival = s->clock++;
  uint64_t hsh = 1469598103934665603ull;  // FNV-1a over the prompt tokens
  for (int i = 0; i < n_prompt; ++i) {
    hsh ^= static_cast<uint32_t>(prompt[i]);
    hsh *= 1099511628211ull;
  }
  r.prompt_hash = hsh;
  r.share_len = (share_len <= 0 || share_len > n_prompt) ? n_prompt : share_len;
  uint64_t ph = 1469598103934665603ull;
  for (int i = 0; i < r.share_len; ++i) {
    ph ^= static_cast<uint32_t>(prompt[i]);
    ph *= 1099511628211ull;
  }
  r.share_hash = ph ^ (static_cast<uint64_t>(r.share_len) << 40);
  const int64_t id = r.id;
  s->reqs.emplace(id, std::move(r));
  s->waiting.push_back(id);
  return id;
}

int64_t b200_sched_add(void* h, const int32_t* prompt, int n_prompt, int max_new_tokens,
                       int min_new_tokens, const int32_t* stop_ids, int n_stop, int ignore_eos) {
  return b200_sched_add_shared(h, prompt, n_prompt, max_new_tokens, min_new_tokens, stop_ids, n_stop,
                               ignore_eos, 0);
}

struct PlanHeader {
  int32_t kind;
  int32_t n_seqs;
  int32_t n_tokens;
  int32_t max_seq_len;
  int32_t n_copies;  // page copies (src, dst pairs in copy_pairs) to perform before the step runs
  int32_t pad;
};

// Buffers must hold: seq_ids[max_num_seqs], cu_seqlens[max_num_seqs+1],
// tokens/positions/slots[max(max_batched_tokens, max_num_seqs)],
// seq_lens[max_num_seqs], block_table[max_num_seqs * max_blocks_per_seq].
// copy_pairs: int32 [2 * max_num_seqs].
//
// Prompt sharing: a fresh request whose prompt equals that of a running request with its prompt
// already in the cache does not prefill. It references the leader's full prompt pages (read-only,
// reference-counted), gets a private copy of the page that holds the last prompt positions, and
// enters decoding with the LAST PROMPT TOKEN as its input: the ordinary decode step recomputes that
// one position and samples the first new token. The n samples of a GRPO group thus prefill once, and
// their decode attention reads the same prompt pages (adjacent sequences, so the reads hit in L2).
int b200_sched_plan(void* h, PlanHeader* hdr, int64_t* seq_ids, int32_t* cu_seqlens,
                    int32_t* tokens, int32_t* positions, int64_t* slots, int32_t* seq_lens,
                    int32_t* block_table, int32_t* copy_pairs) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  hdr->kind = kIdle;
  hdr->n_seqs = hdr->n_tokens = hdr->max_seq_len = 0;
  hdr->n_copies = 0;
  s->planned.clear();
  s->planned_kind = kIdle;

  // ---- prefill admission
  if (!s->waiting.empty() && static_cast<int>(s->running.size()) < s->max_num_seqs) {
    int budget = s->max_batched_tokens;
    int n_tok = 0;
    cu_seqlens[0] = 0;
    std::vector<int64_t> deferred;  // followers whose leader is being prefilled by this very plan
    while (!s->waiting.empty() && static_cast<int>(s->running.size()) < s->max_num_seqs) {
      const int64_t id = s->waiting.front();
      Request& r = s->reqs[id];
      const int32_t L = static_cast<int32_t>(r.tokens.size());
      if (s->share_prompts && copy_pairs != nullptr && L == r.prompt_len && L >= 2) {
        if (Request* ld = s->leader_for(r)) {
          if (!ld->kv_ready) {  // wait one step for the leader's prefill
            s->waiting.pop_front();
            deferred.push_back(id);
            continue;
          }
          const int32_t bs = s->block_size;
          const int32_t nshare = (L - 1) / bs, rem = (L - 1) % bs;
          if (static_cast<int32_t>(ld->blocks.size()) > nshare) {
            for (int32_t b = 0; b < nshare; ++b) {
              r.blocks.push_back(ld->blocks[b]);
              s->refcnt[ld->blocks[b]]++;
            }
            if (s->ensure_blocks(r, L + 1)) {
              if (rem > 0) {
                copy_pairs[2 * hdr->n_copies] = ld->blocks[nshare];
                copy_pairs[2 * hdr->n_copies + 1] = r.blocks[nshare];
                hdr->n_copies++;
              }
              s->waiting.pop_front();
              r.cached_len = L - 1;
              r.kv_ready = true;
              s->running.push_back(id);
              s->n_forked++;
              s->n_shared_pages += nshare;
              continue;
            }
            s->release(r);  // no page for the private tail: fall back to waiting
            break;
          }
        }
      }
      if (L > budget) break;
      // keep one page of head-room per running sequence so decode can proceed
      if (!s->ensure_blocks(r, L + 1)) {
        s->release(r);
        break;
      }
      s->waiting.pop_front();
      for (int32_t p = 0; p < L; ++p) {
        tokens[n_tok] = r.tokens[p];
        positions[n_tok] = p;
        slots[n_tok] = s->slot_of(r, p);
        ++n_tok;
      }
      r.cached_len = L;
      budget -= L;
      seq_ids[hdr->n_seqs] = id;
      seq_lens[hdr->n_seqs] = L;
      cu_seqlens[hdr->n_seqs + 1] = n_tok;
      hdr->max_seq_len = std::max(hdr->max_seq_len, L);
      hdr->n_seqs++;
      s->running.push_back(id);
      s->planned.push_back(id);
      if (L == r.prompt_len) s->prompt_leader[r.prompt_hash] = id;
    }
    for (auto it = deferred.rbegin(); it != deferred.rend(); ++it) s->waiting.push_front(*it);
    if (hdr->n_seqs > 0) {
      hdr->kind = kPrefill;
      hdr->n_tokens = n_tok;
      s->planned_kind = kPrefill;
      return kPrefill;
    }
  }

  // ---- decode
  if (s->running.empty()) return kIdle;
  // make sure every running sequence has a page for its next token; preempt the youngest otherwise
  for (size_t i = 0; i < s->running.size();) {
    Request& r = s->reqs[s->running[i]];
    const int32_t L = static_cast<int32_t>(r.tokens.size());
    if (s->ensure_blocks(r, L)) {
      ++i;
      continue;
    }
    if (static_cast<int32_t>((L + s->block_size - 1) / s->block_size) > s->max_blocks_per_seq) {
      // context limit reached
      const int64_t id = r.id;
      s->finish(r, kLength);
      s->running.erase(s->running.begin() + i);
      (void)id;
      continue;
    }
    // out of pages: preempt the most recently arrived running request (not necessarily r)
    size_t victim = 0;
    for (size_t j = 1; j < s->running.size(); ++j)
      if (s->reqs[s->running[j]].arrival > s->reqs[s->running[victim]].arrival) victim = j;
    Request& v = s->reqs[s->running[victim]];
    s->release(v);
    s->waiting.push_front(v.id);
    s->running.erase(s->running.begin() + victim);
    s->n_preempt++;
    if (s->running.empty()) return kIdle;
    i = 0;  // re-check from the start with the freed pages
  }
  // Sequences that share prefix pages sit next to each other in the batch (equal first page): the attention
  // kernel's blocks of one group then run at about the same time and read the shared pages from L2.
  std::vector<int64_t> order(s->running.begin(), s->running.end());
  std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) {
    return s->reqs[a].blocks[0] < s->reqs[b].blocks[0];
  });
  int n = 0;
  for (int64_t id : order) {
    Request& r = s->reqs[id];
    const int32_t L = static_cast<int32_t>(r.tokens.size());
    seq_ids[n] = id;
    tokens[n] = r.tokens[L - 1];
    positions[n] = L - 1;
    slots[n] = s->slot_of(r, L - 1);
    seq_lens[n] = L;
    int32_t* row = block_table + static_cast<int64_t>(n) * s->max_blocks_per_seq;
    std::memcpy(row, r.blocks.data(), r.blocks.size() * sizeof(int32_t));
    hdr->max_seq_len = std::max(hdr->max_seq_len, L);
    r.cached_len = L;
    s->planned.push_back(id);
    ++n;
  }
  hdr->kind = kDecode;
  hdr->n_seqs = n;
  hdr->n_tokens = n;
  s->planned_kind = kDecode;
  return kDecode;
}

// One sampled token and logprob per planned sequence, in plan order.
// Returns the number of requests that finished with this commit.
int b200_sched_commit(void* h, const int32_t* sampled, const float* logprobs, int n) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  if (n != static_cast<int>(s->planned.size())) return -1;
  const bool was_prefill = s->planned_kind == kPrefill;
  int done = 0;
  for (int i = 0; i < n; ++i) {
    auto it = s->reqs.find(s->planned[i]);
    if (it == s->reqs.end()) continue;
    Request& r = it->second;
    if (r.finish != kRunning) continue;  // aborted between plan and commit
    if (was_prefill) {
      r.kv_ready = true;
      // Prefix pages of a group are kept once: the first request of the group to finish its prefill becomes
      // the holder, later ones (same leading tokens, computed under the same weights) adopt its full prefix
      // pages and return their own copies. After a weight update every request is re-submitted with
      // prompt + partial output, so this is what keeps a group's prompt shared for its whole life.
      const int32_t bs = s->block_size;
      const int32_t nshare = r.share_len / bs;
      if (s->share_prompts && nshare > 0 && static_cast<int32_t>(r.blocks.size()) > nshare) {
        Request* ld = nullptr;
        auto pl = s->prefix_leader.find(r.share_hash);
        if (pl != s->prefix_leader.end() && pl->second != r.id) {
          auto rq = s->reqs.find(pl->second);
          if (rq != s->reqs.end()) {
            Request& c = rq->second;
            if (c.finish == kRunning && c.kv_ready && c.share_len == r.share_len &&
                static_cast<int32_t>(c.blocks.size()) > nshare &&
                std::equal(r.tokens.begin(), r.tokens.begin() + r.share_len, c.tokens.begin()))
              ld = &c;
          }
        }
        if (ld != nullptr) {
          for (int32_t b = 0; b < nshare; ++b) {
            const int32_t mine = r.blocks[b], theirs = ld->blocks[b];
            if (mine == theirs) continue;
            r.blocks[b] = theirs;
            s->refcnt[theirs]++;
            if (--s->refcnt[mine] == 0) s->free_blocks.push_back(mine);
            s->n_dedup_pages++;
          }
        } else {
          s->prefix_leader[r.share_hash] = r.id;
        }
      }
    }
    r.tokens.push_back(sampled[i]);
    r.logprobs.push_back(logprobs[i]);
    const int32_t n_new = static_cast<int32_t>(r.tokens.size()) - r.prompt_len;
    int reason = kRunning;
    if (!r.ignore_eos && n_new >= r.min_new_tokens &&
        std::find(r.stop_ids.begin(), r.stop_ids.end(), sampled[i]) != r.stop_ids.end())
      reason = kStop;
    else if (n_new >= r.max_new_tokens)
      reason = kLength;
    if (reason != kRunning) {
      s->finish(r, reason);
      s->running.erase(std::remove(s->running.begin(), s->running.end(), r.id), s->running.end());
      ++done;
    }
  }
  s->planned.clear();
  s->planned_kind = kIdle;
  return done;
}

// Finishes every live request (running and waiting) with reason ABORT.
int b200_sched_abort_all(void* h) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  int n = 0;
  for (int64_t id : s->running) {
    s->finish(s->reqs[id], kAbort);
    ++n;
  }
  s->running.clear();
  for (int64_t id : s->waiting) {
    s->finish(s->reqs[id], kAbort);
    ++n;
  }
  s->waiting.clear();
  s->planned.clear();
  s->planned_kind = kIdle;
  return n;
}

int b200_sched_abort(void* h, int64_t id) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end() || it->second.finish != kRunning) return 0;
  s->finish(it->second, kAbort);
  s->running.erase(std::remove(s->running.begin(), s->running.end(), id), s->running.end());
  s->waiting.erase(std::remove(s->waiting.begin(), s->waiting.end(), id), s->waiting.end());
  return 1;
}

// Pops one finished request: returns its id (0 if none) and writes reason and
// the number of generated tokens.
int64_t b200_sched_pop_finished(void* h, int32_t* reason, int32_t* n_generated) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  if (s->finished.empty()) return 0;
  const int64_t id = s->finished.front();
  s->finished.pop_front();
  const Request& r = s->reqs[id];
  *reason = r.finish;
  *n_generated = static_cast<int32_t>(r.tokens.size()) - r.prompt_len;
  return id;
}

// Copies the generated tokens / logprobs of a finished request and forgets it.
int b200_sched_take_output(void* h, int64_t id, int32_t* out_tokens, float* out_logprobs, int cap) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end()) return -1;
  const Request& r = it->second;
  const int n = static_cast<int>(r.tokens.size()) - r.prompt_len;
  if (n > cap) return -2;
  if (n > 0) {  // an aborted request may have produced nothing: its vectors hold no storage to copy from
    std::memcpy(out_tokens, r.tokens.data() + r.prompt_len, n * sizeof(int32_t));
    std::memcpy(out_logprobs, r.logprobs.data(), n * sizeof(float));
  }
  s->reqs.erase(it);
  return n;
}

// stats[0]=waiting, [1]=running, [2]=free blocks, [3]=preemptions, [4]=live requests,
// [5]=requests that skipped their prefill by sharing a prompt, [6]=pages shared that way (cumulative),
// [7]=prefix pages given back after a prefill because another request of the group already held them
void b200_sched_stats(void* h, int64_t* stats) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  stats[0] = static_cast<int64_t>(s->waiting.size());
  stats[1] = static_cast<int64_t>(s->running.size());
  stats[2] = static_cast<int64_t>(s->free_blocks.size());
  stats[3] = s->n_preempt;
  stats[4] = static_cast<int64_t>(s->reqs.size());
  stats[5] = s->n_forked;
  stats[6] = s->n_shared_pages;
  stats[7] = s->n_dedup_pages;
}

void b200_sched_set_prompt_sharing(void* h, int on) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  s->share_prompts = on != 0;
}

}  // extern "C"
