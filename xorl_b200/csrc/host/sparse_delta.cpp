// Sparse weight-delta codec for incremental weight sync to inference engines.
//
// Between two syncs most bf16 weights of an RL-trained model do not change at all (the update is
// below half a bf16 ulp).  The codec compares the new 16-bit words against the previously synced
// ones and emits only the changed positions:
//
//   header   : u64 n_elems, u64 n_changed
//   gaps     : LEB128 varints, gap from the previous changed index (first gap is the index itself)
//   values   : n_changed little-endian u16 words (the NEW words, not arithmetic differences, so
//              applying a delta is exact and idempotent)
//
// Plays the role of the optional native escape extension of the reference's delta-encoding
// package (src/xorl/server/weight_sync/sparse_delta_files.py:60-92).
#include <cstdint>
#include <cstring>

extern "C" {

// Upper bound of the encoded size for n elements (all changed, 5-byte gaps never occur for all of
// them, but the bound is simple and safe).
long long xb_delta_bound(long long n) { return 16 + n * 2 + n * 2 + 16; }

// Returns the number of bytes written, or -1 when `cap` is too small.
long long xb_delta_encode(const uint16_t* prev, const uint16_t* cur, long long n, uint8_t* out,
                          long long cap) {
  if (cap < 16) return -1;
  // pass 1: count, so the value block can be placed right after the gap block
  long long changed = 0;
  for (long long i = 0; i < n; ++i) changed += prev[i] != cur[i];
  uint8_t* p = out + 16;
  uint8_t* const end = out + cap;
  long long last = 0;
  bool first = true;
  for (long long i = 0; i < n; ++i) {
    if (prev[i] == cur[i]) continue;
    uint64_t gap = first ? (uint64_t)i : (uint64_t)(i - last);
    first = false;
    last = i;
    do {
      if (p >= end) return -1;
      uint8_t b = gap & 0x7f;
      gap >>= 7;
      *p++ = b | (gap ? 0x80 : 0);
    } while (gap);
  }
  if (p + changed * 2 > end) return -1;
  for (long long i = 0; i < n; ++i) {
    if (prev[i] == cur[i]) continue;
    std::memcpy(p, &cur[i], 2);
    p += 2;
  }
  uint64_t hn = (uint64_t)n, hc = (uint64_t)changed;
  std::memcpy(out, &hn, 8);
  std::memcpy(out + 8, &hc, 8);
  return p - out;
}

// Applies an encoded delta to `weights` (n elements) in place.  Returns the number of changed
// elements, -1 on a malformed or mismatching buffer.
long long xb_delta_apply(uint16_t* weights, long long n, const uint8_t* buf, long long len) {
  if (len < 16) return -1;
  uint64_t hn, hc;
  std::memcpy(&hn, buf, 8);
  std::memcpy(&hc, buf + 8, 8);
  if ((long long)hn != n) return -1;
  const uint8_t* p = buf + 16;
  const uint8_t* const end = buf + len;
  // first walk the gap block to find where the values start
  const uint8_t* q = p;
  for (uint64_t c = 0; c < hc; ++c) {
    while (true) {
      if (q >= end) return -1;
      if (!(*q++ & 0x80)) break;
    }
  }
  const uint8_t* vals = q;
  if (vals + hc * 2 > end) return -1;
  long long idx = 0;
  for (uint64_t c = 0; c < hc; ++c) {
    uint64_t gap = 0;
    int shift = 0;
    while (true) {
      uint8_t b = *p++;
      gap |= (uint64_t)(b & 0x7f) << shift;
      shift += 7;
      if (!(b & 0x80)) break;
      if (shift > 63) return -1;
    }
    idx = c == 0 ? (long long)gap : idx + (long long)gap;
    if (idx < 0 || idx >= n) return -1;
    std::memcpy(&weights[idx], vals + c * 2, 2);
  }
  return (long long)hc;
}

}  // extern "C"
