#include "device_arena.h"

#include <algorithm>
#include <numeric>

namespace b200 {

namespace {
inline size_t AlignUp(size_t v) { return (v + kArenaAlignment - 1) / kArenaAlignment * kArenaAlignment; }
}  // namespace

size_t PlanArena(const std::vector<ArenaRequest>& requests, int num_ops, std::vector<size_t>* offsets) {
  const size_t n = requests.size();
  offsets->assign(n, 0);
  std::vector<size_t> order(n);
  std::iota(order.begin(), order.end(), 0);
  auto whole = [&](size_t i) { return requests[i].first_use <= 0 && requests[i].last_use >= num_ops - 1; };
  std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) {
    const bool wa = whole(a), wb = whole(b);
    if (wa != wb) return wa;
    if (requests[a].bytes != requests[b].bytes) return requests[a].bytes > requests[b].bytes;
    return requests[a].first_use < requests[b].first_use;
  });

  struct Placed {
    size_t offset, size;
    int first, last;
  };
  std::vector<Placed> placed;  // kept sorted by offset
  size_t high_water = 0;
  for (size_t idx : order) {
    const ArenaRequest& r = requests[idx];
    if (r.bytes == 0) continue;
    const size_t size = AlignUp(r.bytes);
    // best fit: the smallest gap, among the allocations alive at the same time, that still
    // holds the tensor; the open end of the slab only when no gap does
    size_t cursor = 0, candidate = 0, best_gap = static_cast<size_t>(-1);
    bool found = false;
    for (const Placed& p : placed) {
      if (p.last < r.first_use || p.first > r.last_use) continue;  // never alive together
      if (cursor + size <= p.offset && p.offset - cursor < best_gap) {
        best_gap = p.offset - cursor;
        candidate = cursor;
        found = true;
      }
      cursor = std::max(cursor, p.offset + p.size);
      if (best_gap == 0) break;
    }
    if (!found) candidate = cursor;
    (*offsets)[idx] = candidate;
    Placed np{candidate, size, r.first_use, r.last_use};
    placed.insert(std::upper_bound(placed.begin(), placed.end(), np,
                                   [](const Placed& a, const Placed& b) { return a.offset < b.offset; }),
                  np);
    high_water = std::max(high_water, candidate + size);
  }
  return high_water;
}

bool DeviceArena::Commit(const std::vector<ArenaRequest>& requests, int num_ops) {
  std::vector<size_t> offsets;
  const size_t need = PlanArena(requests, num_ops, &offsets);
  if (need > capacity_) {
    void* fresh = alloc_(user_, need);
    if (!fresh) return false;
    if (base_) free_(user_, base_);
    base_ = fresh;
    capacity_ = need;
  }
  planned_ = need;
  offsets_.swap(offsets);
  return true;
}

void DeviceArena::Release() {
  if (base_) free_(user_, base_);
  base_ = nullptr;
  capacity_ = planned_ = 0;
  offsets_.clear();
}

}  // namespace b200
