// Exercises the C++ host runtime (packer, delta codec) under AddressSanitizer and
// UndefinedBehaviorSanitizer: exact-size heap buffers, so any read or write past an end aborts.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

extern "C" {
int64_t xb_ffd_pack(const int64_t* lengths, int64_t n, int64_t capacity, int64_t group_size, int64_t* bin_of);
int64_t xb_sequential_pack(const int64_t* lengths, int64_t n, int64_t capacity, int64_t* bin_of);
long long xb_delta_bound(long long n);
long long xb_delta_encode(const uint16_t* prev, const uint16_t* cur, long long n, uint8_t* out, long long cap);
long long xb_delta_apply(uint16_t* weights, long long n, const uint8_t* buf, long long len);
}

static uint32_t rng_state = 12345u;
static uint32_t rnd() { rng_state = rng_state * 1664525u + 1013904223u; return rng_state >> 8; }

#define CHECK(c) do { if (!(c)) { std::fprintf(stderr, "check failed: %s (line %d)\n", #c, __LINE__); return 1; } } while (0)

int main() {
  // packer: every sequence in exactly one bin, no bin over capacity unless it holds one long sequence
  for (int trial = 0; trial < 20; ++trial) {
    const int64_t n = 1 + rnd() % 500, cap = 64 + rnd() % 512, group = (trial % 3 == 0) ? 0 : 1 + rnd() % 64;
    std::vector<int64_t> len(n), bin(n, -1);
    for (auto& l : len) l = 1 + rnd() % (cap + cap / 4);
    const int64_t bins = (trial % 2) ? xb_ffd_pack(len.data(), n, cap, group, bin.data())
                                     : xb_sequential_pack(len.data(), n, cap, bin.data());
    CHECK(bins > 0 && bins <= n);
    std::vector<int64_t> fill(bins, 0), count(bins, 0);
    for (int64_t i = 0; i < n; ++i) {
      CHECK(bin[i] >= 0 && bin[i] < bins);
      fill[bin[i]] += len[i];
      count[bin[i]] += 1;
    }
    for (int64_t b = 0; b < bins; ++b) CHECK(count[b] >= 1 && (fill[b] <= cap || count[b] == 1));
  }
  CHECK(xb_ffd_pack(nullptr, 0, 128, 0, nullptr) == 0);
  // delta codec: encode / apply round trip at several densities, and a too-small buffer is refused
  for (int trial = 0; trial < 12; ++trial) {
    const long long n = (trial == 0) ? 1 : 1 + rnd() % 200000;
    std::vector<uint16_t> prev(n), cur(n);
    const uint32_t every = 1 + rnd() % (trial % 2 ? 3 : 5000);
    for (long long i = 0; i < n; ++i) {
      prev[i] = (uint16_t)rnd();
      cur[i] = (rnd() % every == 0) ? (uint16_t)rnd() : prev[i];
    }
    std::vector<uint8_t> buf(xb_delta_bound(n));
    const long long used = xb_delta_encode(prev.data(), cur.data(), n, buf.data(), (long long)buf.size());
    CHECK(used >= 16 && used <= (long long)buf.size());
    std::vector<uint8_t> exact(buf.begin(), buf.begin() + used);        // exact-size copy for the reader
    std::vector<uint16_t> w(prev);
    CHECK(xb_delta_apply(w.data(), n, exact.data(), used) >= 0);
    CHECK(w == cur);
    std::vector<uint8_t> tiny(8);
    CHECK(xb_delta_encode(prev.data(), cur.data(), n, tiny.data(), 8) == -1);
    if (used > 20) {                                                      // truncated stream: refused, no overrun
      std::vector<uint8_t> cut(exact.begin(), exact.begin() + used - 3);
      std::vector<uint16_t> w2(prev);
      (void)xb_delta_apply(w2.data(), n, cut.data(), (long long)cut.size());
    }
  }
  std::puts("host runtime clean under asan+ubsan");
  return 0;
}
