// Offsets of the activation tensors of one forward inside a shared arena.
//
// nncv plans buffer reuse with "greedy by size for offset calculation" (Pisarchyk & Lee, "Efficient
// Memory Management for Deep Neural Net Inference", 2020; nncv: include/nncv/compiler/Optimizer/
// MemSolver.hpp:55-70, src/nncv/compiler/Optimizer/MemSolver.cpp:15-50, known answer 124 in
// tests/MemSolver/test.cpp:17-37).  Each tensor has a size and a usage interval [first op, last op]
// (both ends included); tensors whose intervals intersect must not overlap in memory.  Tensors are
// taken in non-increasing order of size; each goes into the smallest gap, between tensors already
// placed whose intervals intersect its own, that is large enough, else behind the last of them.
// Host code only.
#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <numeric>
#include <vector>

#include "kernels.h"

namespace nncv_b200 {

size_t arena_plan(std::vector<ArenaTensor>& tensors, size_t align) {
  if (align == 0) align = 1;
  auto up = [&](size_t v) { return (v + align - 1) / align * align; };
  std::vector<size_t> order(tensors.size());
  std::iota(order.begin(), order.end(), (size_t)0);
  // larger first; equal sizes keep their registration order (stable), which makes the plan reproducible
  std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return tensors[a].size > tensors[b].size; });
  std::vector<size_t> placed;   // indices of placed tensors, ordered by offset
  size_t total = 0;
  for (size_t idx : order) {
    ArenaTensor& t = tensors[idx];
    const size_t need = up(t.size);
    size_t prev_end = 0, best = SIZE_MAX, best_gap = SIZE_MAX;
    for (size_t j : placed) {
      const ArenaTensor& x = tensors[j];
      if (std::max(t.first, x.first) > std::min(t.last, x.last)) continue;   // never alive together
      if (x.offset > prev_end) {
        const size_t gap = x.offset - prev_end;
        if (gap >= need && gap < best_gap) { best_gap = gap; best = prev_end; }
      }
      prev_end = std::max(prev_end, x.offset + up(x.size));
    }
    t.offset = best != SIZE_MAX ? best : prev_end;
    total = std::max(total, t.offset + need);
    placed.insert(std::upper_bound(placed.begin(), placed.end(), idx,
                                   [&](size_t a, size_t b) { return tensors[a].offset < tensors[b].offset; }),
                  idx);
  }
  return total;
}

}  // namespace nncv_b200
