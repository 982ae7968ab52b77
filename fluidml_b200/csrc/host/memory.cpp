#include "memory.h"
#include <algorithm>
#include <map>

namespace fluidml {
namespace memory {

namespace {
size_t AlignUp(size_t v, size_t a) { return a <= 1 ? v : (v + a - 1) / a * a; }

// Disjoint busy byte ranges [start, end), kept sorted; ranges that overlap or touch merge,
// as the reference's slice list does (greedy.cpp:97-174).
class BusySet {
public:
  void Busy(size_t start, size_t end) {
    if (start >= end) return;
    auto it = ranges_.lower_bound(start);
    if (it != ranges_.begin()) {
      auto prev = std::prev(it);
      if (prev->second >= start) it = prev;
    }
    while (it != ranges_.end() && it->first <= end) {
      start = std::min(start, it->first);
      end = std::max(end, it->second);
      it = ranges_.erase(it);
    }
    ranges_[start] = end;
  }
  // Smallest gap between two consecutive busy ranges that holds `size` (after aligning its
  // start), else the end of the last range; 0 when nothing is busy.
  size_t Alloc(size_t size, size_t alignment) const {
    if (ranges_.empty()) return 0;
    size_t best = (size_t)-1, best_gap = (size_t)-1;
    for (auto it = ranges_.begin(); std::next(it) != ranges_.end(); ++it) {
      const size_t gap_start = AlignUp(it->second, alignment), gap_end = std::next(it)->first;
      if (gap_end < gap_start) continue;
      const size_t free_size = gap_end - gap_start;
      // the reference compares the raw gap; with alignment 1 the two are the same
      if (free_size >= size && (gap_end - it->second) < best_gap) {
        best = gap_start;
        best_gap = gap_end - it->second;
      }
    }
    if (best != (size_t)-1) return best;
    return AlignUp(ranges_.rbegin()->second, alignment);
  }

private:
  std::map<size_t, size_t> ranges_;
};
}  // namespace

size_t Index::GetMaximum() const {
  size_t m = 0;
  for (const auto &kv : map_) m = std::max(m, kv.second.first + kv.second.second);
  return m;
}

Index LinearPlan::Run(Infos &infos) const {
  Index index;
  size_t top = 0;
  while (!infos.IsEmpty()) {
    Info info = infos.Pop();
    const size_t offset = AlignUp(top, alignment_);
    index.Set(info.name, offset, info.size);
    top = std::max(top, offset + info.size);
  }
  return index;
}

Index GreedyPlan::Run(Infos &infos) const {
  struct Placed { size_t start, end, life_start, life_end; };
  std::vector<Placed> placed;
  Index index;
  while (!infos.IsEmpty()) {
    Info cur = infos.Pop();
    const size_t life_start = cur.start, life_end = cur.end + 1;
    BusySet busy;
    for (const Placed &p : placed)
      if (p.life_start <= life_end && p.life_end >= life_start) busy.Busy(p.start, p.end);
    const size_t offset = busy.Alloc(cur.size, alignment_);
    placed.push_back({offset, offset + cur.size, life_start, life_end});
    index.Set(cur.name, offset, cur.size);
  }
  return index;
}

}  // namespace memory
}  // namespace fluidml
