// Static memory planner for graph executors: given every tensor's size and the first / last node index at which it
// is alive, assign byte offsets inside ONE shared buffer so that tensors whose lifetimes overlap never overlap in
// memory.  Algorithm: "greedy by size" offset assignment (Pisarchyk & Lee, arXiv 2001.03288): visit tensors from the
// largest to the smallest and place each at the lowest offset that does not collide with an already placed tensor
// whose lifetime intersects.  A self-check verifies the plan.
//
// Counterpart of lightseq2's lsflow MemoryManager (oslo/lightseq2/csrc/lsflow/manager.cpp:29-232).
#include <algorithm>
#include <cstdint>
#include <vector>

namespace {
struct Item {
  int id;
  long long size, first, last, offset;
};
inline bool lifetimes_overlap(const Item& a, const Item& b) { return a.first <= b.last && b.first <= a.last; }
}  // namespace

// sizes / first_use / last_use: [n]; offsets_out: [n].  alignment: every offset is a multiple of it.
// Returns the total buffer size, or -1 on invalid input.
extern "C" long long oslo_plan_memory(const long long* sizes, const long long* first_use, const long long* last_use, int n,
                                      long long alignment, long long* offsets_out) {
  if (n < 0 || alignment <= 0) return -1;
  std::vector<Item> items(n);
  for (int i = 0; i < n; ++i) {
    if (sizes[i] < 0 || first_use[i] > last_use[i]) return -1;
    const long long sz = (sizes[i] + alignment - 1) / alignment * alignment;
    items[i] = Item{i, sz, first_use[i], last_use[i], -1};
  }
  std::vector<int> order(n);
  for (int i = 0; i < n; ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return items[a].size > items[b].size; });
  std::vector<int> placed;
  long long total = 0;
  for (int idx : order) {
    Item& t = items[idx];
    std::vector<std::pair<long long, long long>> busy;  // [offset, end) of conflicting tensors
    for (int p : placed)
      if (lifetimes_overlap(t, items[p]) && items[p].size > 0) busy.emplace_back(items[p].offset, items[p].offset + items[p].size);
    std::sort(busy.begin(), busy.end());
    long long best = 0;
    for (auto& iv : busy) {
      if (best + t.size <= iv.first) break;  // fits in the gap before this interval
      best = std::max(best, iv.second);
    }
    t.offset = best;
    total = std::max(total, best + t.size);
    placed.push_back(idx);
  }
  for (int i = 0; i < n; ++i) offsets_out[i] = items[i].offset;
  return total;
}

// 0 when no two tensors with intersecting lifetimes intersect in memory, else 1 + index of the first offender.
extern "C" int oslo_check_memory_plan(const long long* sizes, const long long* first_use, const long long* last_use,
                                      const long long* offsets, int n) {
  for (int i = 0; i < n; ++i)
    for (int j = i + 1; j < n; ++j) {
      const bool live = first_use[i] <= last_use[j] && first_use[j] <= last_use[i];
      const bool mem = offsets[i] < offsets[j] + sizes[j] && offsets[j] < offsets[i] + sizes[i];
      if (live && mem && sizes[i] > 0 && sizes[j] > 0) return 1 + i;
    }
  return 0;
}
