// First-fit-decreasing bin packing of sequence lengths into fixed-capacity bins, in groups.
// Plain C++ replacement for the numba-jitted packer of the reference
// (src/xorl/data/prepare/packing.py:30-190).
#include <algorithm>
#include <cstdint>
#include <numeric>
#include <vector>

extern "C" {

// lengths[n] -> bin_of[n] (bin ids are global, increasing with the group index).
// Sequences longer than `capacity` get a bin of their own.  Returns the number of bins.
// group_size <= 0 packs everything as one group.
int64_t xb_ffd_pack(const int64_t* lengths, int64_t n, int64_t capacity, int64_t group_size,
                    int64_t* bin_of) {
  if (n <= 0) return 0;
  if (group_size <= 0) group_size = n;
  int64_t next_bin = 0;
  std::vector<int64_t> order;
  std::vector<int64_t> space;  // remaining space per open bin of the current group
  for (int64_t g0 = 0; g0 < n; g0 += group_size) {
    const int64_t g1 = std::min(n, g0 + group_size);
    order.resize(g1 - g0);
    std::iota(order.begin(), order.end(), g0);
    std::stable_sort(order.begin(), order.end(),
                     [&](int64_t a, int64_t b) { return lengths[a] > lengths[b]; });
    space.clear();
    const int64_t base = next_bin;
    for (int64_t idx : order) {
      const int64_t len = lengths[idx];
      int64_t chosen = -1;
      for (size_t b = 0; b < space.size(); ++b) {
        if (space[b] >= len) { chosen = (int64_t)b; break; }
      }
      if (chosen < 0) {
        space.push_back(std::max<int64_t>(capacity - len, 0));
        chosen = (int64_t)space.size() - 1;
      } else {
        space[chosen] -= len;
      }
      bin_of[idx] = base + chosen;
    }
    next_bin = base + (int64_t)space.size();
  }
  return next_bin;
}

// Sequential packing: walk the samples in order, open a new bin when the next one does not fit.
int64_t xb_sequential_pack(const int64_t* lengths, int64_t n, int64_t capacity, int64_t* bin_of) {
  int64_t bin = 0, used = 0;
  for (int64_t i = 0; i < n; ++i) {
    if (used > 0 && used + lengths[i] > capacity) { ++bin; used = 0; }
    bin_of[i] = bin;
    used += lengths[i];
  }
  return n > 0 ? bin + 1 : 0;
}

}  // extern "C"
