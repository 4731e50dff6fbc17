// Standalone stress driver for the host runtime, meant to be built with sanitizers
// (-fsanitize=address,undefined or -fsanitize=thread) and run without Python or a GPU:
//   g++ -std=c++17 -O1 -g -fsanitize=thread -pthread selftest.cpp seqpack.cpp rollout_scheduler.cpp -o selftest
// Part 1 drives the packers on random sizes and checks their invariants. Part 2 drives the paged-KV
// scheduler from two threads the way the rollout engine does: a client thread submits (and sometimes
// aborts) requests, among them groups with identical prompts (prompt sharing), while the engine thread
// plans, commits random tokens and collects finished requests. Every plan is checked: token and
// sequence counts within the budgets, slots and block-table entries inside the cache, no page written
// by two sequences in one step. At the end every page must be free again. Exit code 0 = all checks held.

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <set>
#include <thread>
#include <vector>

extern "C" {
struct PlanHeader {
  int32_t kind, n_seqs, n_tokens, max_seq_len, n_copies, pad;
};
void* b200_sched_create(int, int, int, int, int);
void b200_sched_destroy(void*);
int64_t b200_sched_add(void*, const int32_t*, int, int, int, const int32_t*, int, int);
int b200_sched_plan(void*, PlanHeader*, int64_t*, int32_t*, int32_t*, int32_t*, int64_t*, int32_t*, int32_t*, int32_t*);
int b200_sched_commit(void*, const int32_t*, const float*, int);
int b200_sched_abort(void*, int64_t);
int64_t b200_sched_pop_finished(void*, int32_t*, int32_t*);
int b200_sched_take_output(void*, int64_t, int32_t*, float*, int);
void b200_sched_stats(void*, int64_t*);
void b200_sched_set_prompt_sharing(void*, int);
int b200_ffd_allocate(const int64_t*, int, int64_t, int, int32_t*);
int b200_kk_partition(const int64_t*, int, int, int, int32_t*);
int b200_partition_balanced(const int64_t*, int, int, int, int32_t*);
int b200_greedy_partition(const int64_t*, int, int, int, int32_t*);
}

static int g_fail = 0;
#define CHECK(cond)                                                        \
  do {                                                                     \
    if (!(cond)) {                                                         \
      std::fprintf(stderr, "CHECK failed %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      ++g_fail;                                                            \
    }                                                                      \
  } while (0)

static void test_packers(unsigned seed) {
  std::mt19937 rng(seed);
  for (int round = 0; round < 200; ++round) {
    const int n = 1 + rng() % 200;
    std::vector<int64_t> sizes(n);
    for (auto& s : sizes) s = 1 + rng() % 4096;
    const int64_t cap = 4096 + rng() % 8192;
    std::vector<int32_t> bin(n);
    const int nb = b200_ffd_allocate(sizes.data(), n, cap, 1 + rng() % 4, bin.data());
    CHECK(nb >= 1);
    std::vector<int64_t> load(nb > 0 ? nb : 1, 0);
    for (int i = 0; i < n; ++i) {
      CHECK(bin[i] >= 0 && bin[i] < nb);
      if (bin[i] >= 0 && bin[i] < nb) load[bin[i]] += sizes[i];
    }
    for (int b = 0; b < nb; ++b) CHECK(load[b] <= cap);
    const int k = 1 + rng() % (n < 8 ? n : 8);
    std::vector<int32_t> grp(n);
    CHECK(b200_kk_partition(sizes.data(), n, k, 0, grp.data()) == k);
    for (int i = 0; i < n; ++i) CHECK(grp[i] >= 0 && grp[i] < k);
    CHECK(b200_greedy_partition(sizes.data(), n, k, 0, grp.data()) == k);
    for (int i = 0; i < n; ++i) CHECK(grp[i] >= 0 && grp[i] < k);
    std::vector<int32_t> bounds(k + 1);
    CHECK(b200_partition_balanced(sizes.data(), n, k, 1, bounds.data()) == 0);
    CHECK(bounds[0] == 0 && bounds[k] == n);
    for (int j = 0; j < k; ++j) CHECK(bounds[j] < bounds[j + 1]);
  }
}

static void test_scheduler(unsigned seed, bool share) {
  const int num_blocks = 96, block = 16, max_seqs = 24, max_tok = 512, max_bps = 24;
  void* h = b200_sched_create(num_blocks, block, max_seqs, max_tok, max_bps);
  b200_sched_set_prompt_sharing(h, share ? 1 : 0);
  const int total = 300;
  std::atomic<int> submitted{0}, collected{0};
  std::atomic<bool> client_done{false};

  std::thread client([&] {
    std::mt19937 rng(seed);
    std::vector<int64_t> mine;
    int made = 0;
    while (made < total) {
      const int n_prompt = 1 + rng() % 120;
      std::vector<int32_t> prompt(n_prompt);
      for (auto& t : prompt) t = rng() % 1000;
      const int group = 1 + rng() % 4;  // identical prompts: candidates for sharing
      for (int g = 0; g < group && made < total; ++g) {
        const int32_t stop = 7;
        const int64_t id = b200_sched_add(h, prompt.data(), n_prompt, 1 + rng() % 60, 0, &stop, 1, rng() % 2);
        CHECK(id > 0);
        mine.push_back(id);
        ++made;
        submitted.fetch_add(1);
      }
      if (rng() % 5 == 0 && !mine.empty()) b200_sched_abort(h, mine[rng() % mine.size()]);
      if (rng() % 3 == 0) std::this_thread::yield();
    }
    client_done.store(true);
  });

  std::thread engine([&] {
    std::mt19937 rng(seed + 1);
    std::vector<int64_t> seq_ids(max_seqs), slots(max_tok);
    std::vector<int32_t> cu(max_seqs + 1), tokens(max_tok), positions(max_tok), seq_lens(max_seqs),
        table(max_seqs * max_bps), copies(2 * max_seqs), sampled(max_seqs), out_tok(4096);
    std::vector<float> logp(max_seqs, -1.f), out_lp(4096);
    long idle = 0;
    while (!(client_done.load() && collected.load() >= submitted.load())) {
      PlanHeader hdr;
      const int kind = b200_sched_plan(h, &hdr, seq_ids.data(), cu.data(), tokens.data(), positions.data(), slots.data(),
                                       seq_lens.data(), table.data(), copies.data());
      if (hdr.n_seqs > 0) {
        idle = 0;
        CHECK(hdr.n_seqs <= max_seqs && hdr.n_tokens <= max_tok && hdr.n_copies <= max_seqs);
        std::set<int64_t> written;
        for (int t = 0; t < hdr.n_tokens; ++t) {
          CHECK(slots[t] >= 0 && slots[t] < static_cast<int64_t>(num_blocks) * block);
          CHECK(written.insert(slots[t]).second);  // two tokens never write the same cache slot
          CHECK(positions[t] >= 0 && tokens[t] >= 0);
        }
        for (int c = 0; c < hdr.n_copies; ++c) {
          CHECK(copies[2 * c] >= 0 && copies[2 * c] < num_blocks);
          CHECK(copies[2 * c + 1] >= 0 && copies[2 * c + 1] < num_blocks && copies[2 * c] != copies[2 * c + 1]);
        }
        for (int i = 0; i < hdr.n_seqs; ++i) sampled[i] = rng() % 40;  // 7 ends a request now and then
        CHECK(b200_sched_commit(h, sampled.data(), logp.data(), hdr.n_seqs) >= 0);
      } else if (++idle > 2000000) {
        CHECK(!"scheduler made no progress");
        break;
      }
      (void)kind;
      int32_t reason, n_gen;
      while (int64_t id = b200_sched_pop_finished(h, &reason, &n_gen)) {
        CHECK(n_gen >= 0 && n_gen <= 4096);
        CHECK(b200_sched_take_output(h, id, out_tok.data(), out_lp.data(), 4096) == n_gen);
        collected.fetch_add(1);
      }
    }
  });
  client.join();
  engine.join();
  int64_t st[8] = {0};
  b200_sched_stats(h, st);
  CHECK(st[0] == 0 && st[1] == 0 && st[4] == 0);
  CHECK(st[2] == num_blocks);  // every page returned, shared ones included
  if (share) CHECK(st[5] >= 0);
  std::printf("scheduler(share=%d): %d requests, %lld preemptions, %lld forks, %lld shared pages\n", share ? 1 : 0,
              collected.load(), static_cast<long long>(st[3]), static_cast<long long>(st[5]),
              static_cast<long long>(st[6]));
  b200_sched_destroy(h);
}

int main(int argc, char** argv) {
  const unsigned seed = argc > 1 ? static_cast<unsigned>(std::atoi(argv[1])) : 1u;
  test_packers(seed);
  test_scheduler(seed, true);
  test_scheduler(seed + 7, false);
  if (g_fail) {
    std::fprintf(stderr, "%d checks failed\n", g_fail);
    return 1;
  }
  std::puts("host selftest ok");
  return 0;
}
