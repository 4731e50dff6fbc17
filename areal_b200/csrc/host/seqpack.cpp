// Host-side sequence packing / partitioning (C ABI, loaded with ctypes).
//
//  * ffd_allocate        first-fit-decreasing bin packing under a token capacity
//  * kk_partition        Karmarkar–Karp (largest differencing) k-way partition
//  * partition_balanced  contiguous k-way partition minimising the largest part
//                        (dynamic programme over prefix sums)
//  * greedy_partition    longest-processing-time greedy into k groups, with an
//                        optional equal-cardinality constraint
//
// These are the native counterparts of the reference's numba / Python
// partitioners (areal/utils/seqpack.py:22,234,337,446,540).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <functional>
#include <limits>
#include <numeric>
#include <queue>
#include <vector>

extern "C" {

// Packs items (sizes[n]) into bins of `capacity`, each bin holding at least
// `min_groups` bins overall. Writes bin index per item into out_bin[n] and
// returns the number of bins (or -1 if an item exceeds the capacity).
int b200_ffd_allocate(const int64_t* sizes, int n, int64_t capacity, int min_groups,
                      int32_t* out_bin) {
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return sizes[a] > sizes[b]; });
  std::vector<int64_t> load;
  std::vector<int> count;
  if (min_groups > 0) {
    load.assign(min_groups, 0);
    count.assign(min_groups, 0);
  }
  for (int idx : order) {
    const int64_t s = sizes[idx];
    if (s > capacity) return -1;
    int chosen = -1;
    if (min_groups > 0) {
      // while some of the mandatory bins are still empty, fill those first
      for (int b = 0; b < min_groups; ++b)
        if (count[b] == 0) {
          chosen = b;
          break;
        }
    }
    if (chosen < 0) {
      for (size_t b = 0; b < load.size(); ++b)
        if (load[b] + s <= capacity) {
          chosen = static_cast<int>(b);
          break;
        }
    }
    if (chosen < 0) {
      load.push_back(0);
      count.push_back(0);
      chosen = static_cast<int>(load.size()) - 1;
    }
    load[chosen] += s;
    count[chosen] += 1;
    out_bin[idx] = chosen;
  }
  return static_cast<int>(load.size());
}

namespace {
struct KKState {
  // k partial sets sorted by descending sum
  std::vector<int64_t> sums;
  std::vector<std::vector<int>> sets;
  int64_t spread() const { return sums.front() - sums.back(); }
};
struct KKCmp {
  bool operator()(const KKState* a, const KKState* b) const {
    if (a->spread() != b->spread()) return a->spread() < b->spread();
    return a->sums.front() < b->sums.front();
  }
};
}  // namespace

// Karmarkar–Karp k-way partition. equal_size != 0 forces group cardinalities to
// differ by at most one (items are merged in blocks of k). Writes group per item.
int b200_kk_partition(const int64_t* sizes, int n, int k, int equal_size, int32_t* out_group) {
  if (k <= 0) return -1;
  std::vector<KKState*> owned;
  std::priority_queue<KKState*, std::vector<KKState*>, KKCmp> heap;
  auto make = [&]() {
    auto* s = new KKState();
    s->sums.assign(k, 0);
    s->sets.assign(k, {});
    owned.push_back(s);
    return s;
  };
  if (equal_size) {
    std::vector<int> order(n);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return sizes[a] > sizes[b]; });
    for (int i = 0; i < n; i += k) {
      auto* s = make();
      for (int j = 0; j < k && i + j < n; ++j) {
        s->sums[j] = sizes[order[i + j]];
        s->sets[j].push_back(order[i + j]);
      }
      heap.push(s);
    }
  } else {
    for (int i = 0; i < n; ++i) {
      auto* s = make();
      s->sums[0] = sizes[i];
      s->sets[0].push_back(i);
      heap.push(s);
    }
  }
  if (heap.empty()) return 0;
  while (heap.size() > 1) {
    KKState* a = heap.top();
    heap.pop();
    KKState* b = heap.top();
    heap.pop();
    // merge: largest of a with smallest of b, and so on
    auto* m = make();
    std::vector<std::pair<int64_t, std::vector<int>>> parts(k);
    for (int j = 0; j < k; ++j) {
      parts[j].first = a->sums[j] + b->sums[k - 1 - j];
      parts[j].second = a->sets[j];
      parts[j].second.insert(parts[j].second.end(), b->sets[k - 1 - j].begin(),
                             b->sets[k - 1 - j].end());
    }
    std::stable_sort(parts.begin(), parts.end(),
                     [](const auto& x, const auto& y) { return x.first > y.first; });
    for (int j = 0; j < k; ++j) {
      m->sums[j] = parts[j].first;
      m->sets[j] = std::move(parts[j].second);
    }
    heap.push(m);
  }
  KKState* fin = heap.top();
  for (int j = 0; j < k; ++j)
    for (int idx : fin->sets[j]) out_group[idx] = j;
  for (auto* s : owned) delete s;
  return k;
}

// Contiguous partition of sizes[n] into k parts minimising the maximum part sum,
// each part holding at least min_size items. Writes k+1 boundaries; returns 0,
// or -1 when n < k * min_size.
int b200_partition_balanced(const int64_t* sizes, int n, int k, int min_size, int32_t* out_bounds) {
  if (k <= 0 || n < static_cast<int64_t>(k) * min_size) return -1;
  std::vector<int64_t> pre(n + 1, 0);
  for (int i = 0; i < n; ++i) pre[i + 1] = pre[i] + sizes[i];
  const int64_t INF = std::numeric_limits<int64_t>::max() / 4;
  std::vector<std::vector<int64_t>> dp(k + 1, std::vector<int64_t>(n + 1, INF));
  std::vector<std::vector<int32_t>> arg(k + 1, std::vector<int32_t>(n + 1, -1));
  dp[0][0] = 0;
  for (int j = 1; j <= k; ++j) {
    for (int i = j * min_size; i <= n - (k - j) * min_size; ++i) {
      for (int p = (j - 1) * min_size; p <= i - min_size; ++p) {
        if (dp[j - 1][p] >= INF) continue;
        const int64_t cost = std::max(dp[j - 1][p], pre[i] - pre[p]);
        if (cost < dp[j][i]) {
          dp[j][i] = cost;
          arg[j][i] = p;
        }
      }
    }
  }
  if (dp[k][n] >= INF) return -1;
  int i = n;
  out_bounds[k] = n;
  for (int j = k; j >= 1; --j) {
    i = arg[j][i];
    out_bounds[j - 1] = i;
  }
  return 0;
}

// Longest-processing-time greedy: items in descending size go to the lightest
// group; with equal_size each group takes at most ceil(n/k) items.
int b200_greedy_partition(const int64_t* sizes, int n, int k, int equal_size, int32_t* out_group) {
  if (k <= 0) return -1;
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return sizes[a] > sizes[b]; });
  std::vector<int64_t> load(k, 0);
  std::vector<int> count(k, 0);
  const int cap = (n + k - 1) / k;
  for (int idx : order) {
    int best = -1;
    for (int g = 0; g < k; ++g) {
      if (equal_size && count[g] >= cap) continue;
      if (best < 0 || load[g] < load[best]) best = g;
    }
    if (best < 0) best = 0;
    load[best] += sizes[idx];
    count[best] += 1;
    out_group[idx] = best;
  }
  return k;
}

}  // extern "C"
