// Lean warp-level exact top-k for candidate lists of a few thousand (score, index) entries.
//
// Same ordering rule as gw_select.cuh (score descending, index ascending), specialised for the common case so
// that it costs about two dozen instructions per candidate: 32-bit score keys, one histogram pass over 1024
// linear bins of the key range [lo, hi] (keys outside are clamped into the end bins, which keeps the binning
// monotone), a conflict-free scan, one output pass that emits every bin above the boundary bin through
// ballot compaction, and a direct ranking of the boundary bin's entries (at most TS_SIDE of them; otherwise
// the caller falls back to the general routine).
#pragma once

#include "gw_common.cuh"

namespace gw {

constexpr int TS_BINS = 1024;
constexpr int TS_SIDE = 128;
constexpr int TS_U = 8;  // entries fetched per lane before any is processed

struct TightSmem {
  uint32_t hist[TS_BINS + TS_BINS / 32];  // one pad word per 32 bins: lane t scans bins 32t..32t+31 without conflicts
  unsigned long long side[TS_SIDE];
};

__device__ __forceinline__ uint32_t ts_bin(uint32_t key, uint32_t lo, int shift) {
  const uint32_t d = key > lo ? (key - lo) >> shift : 0u;
  return d < TS_BINS - 1 ? d : TS_BINS - 1;
}

// Sources come in segments.  A source provides segments(), count(seg), bits(seg, i) and entry(seg, i).
// nseg arrays of (score bits, index), `cap` entries apart, with their lengths in cnt[0..nseg):
struct TightLists {
  const uint2* __restrict__ base;
  const int* __restrict__ cnt;
  int cap;
  int nseg;
  __device__ __forceinline__ int segments() const { return nseg; }
  __device__ __forceinline__ int count(int seg) const { return cnt[seg]; }
  __device__ __forceinline__ uint32_t bits(int seg, int i) const { return base[static_cast<size_t>(seg) * cap + i].x; }
  __device__ __forceinline__ uint2 entry(int seg, int i) const { return base[static_cast<size_t>(seg) * cap + i]; }
};
// One dense row of fp32 scores, index = column:
struct TightDenseRow {
  const float* __restrict__ row;
  int n;
  __device__ __forceinline__ int segments() const { return 1; }
  __device__ __forceinline__ int count(int) const { return n; }
  __device__ __forceinline__ uint32_t bits(int, int i) const { return __float_as_uint(row[i]); }
  __device__ __forceinline__ uint2 entry(int, int i) const { return make_uint2(__float_as_uint(row[i]), static_cast<uint32_t>(i)); }
};

// Select the k largest of the n = na + nb entries (n > k).  sink(pos, bits, idx) is called once per selected
// entry with a unique pos in [0, k).  Returns k on success and -1 when the boundary bin holds more than
// TS_SIDE entries (nothing useful has been emitted then; use the general routine).
// When kth_bits is non-null nothing is emitted and *kth_bits receives the score bits of the k-th largest entry.
template <class Lists, class Sink>
__device__ int warp_select_tight(const Lists& L, int k, uint32_t lo, uint32_t hi, TightSmem& sm, int lane,
                                 const Sink& sink, uint32_t* kth_bits) {
  // Up to three histogram levels: [lo, hi] is only a hint (keys outside are clamped into the end bins of the
  // first level), and score keys are logarithmic in the score, so the first boundary bin can be crowded.
  uint32_t cur_lo = lo, cur_hi = hi > lo ? hi : lo;
  int kk = k;
  uint32_t cntb = 0;
  for (int level = 0; level < 3; ++level) {
    const uint32_t span = cur_hi - cur_lo;
    const int bits = 32 - __clz(span);
    const int shift = bits > 10 ? bits - 10 : 0;
#pragma unroll
    for (int j = 0; j < (TS_BINS + TS_BINS / 32) / 32; ++j) sm.hist[lane + 32 * j] = 0;
    __syncwarp();
    // ---- histogram of the undecided keys ----
#pragma unroll 1
    for (int seg = 0; seg < L.segments(); ++seg) {
      const int n = L.count(seg);
      for (int base = lane; base < n; base += 32 * TS_U) {
        uint32_t sb[TS_U];
#pragma unroll
        for (int u = 0; u < TS_U; ++u) {
          const int i = base + 32 * u;
          sb[u] = i < n ? L.bits(seg, i) : 0u;
        }
#pragma unroll
        for (int u = 0; u < TS_U; ++u) {
          if (base + 32 * u < n) {
            const uint32_t key = score_key(__uint_as_float(sb[u]));
            if (level == 0 || (key >= cur_lo && key <= cur_hi)) {
              const uint32_t bn = ts_bin(key, cur_lo, shift);
              atomicAdd(&sm.hist[bn + (bn >> 5)], 1u);
            }
          }
        }
      }
    }
    __syncwarp();
    // ---- scan from the top bin down: lane t owns bins 32t..32t+31 ----
    uint32_t mysum = 0;
#pragma unroll
    for (int j = 0; j < 32; ++j) mysum += sm.hist[33 * lane + j];
    uint32_t above = mysum;  // becomes the count in all lanes above this one
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint32_t v = __shfl_down_sync(0xffffffffu, above, d);
      if (lane + d < 32) above += v;
    }
    above -= mysum;
    const bool mine = above < static_cast<uint32_t>(kk) && static_cast<uint32_t>(kk) <= above + mysum;
    const uint32_t owner_mask = __ballot_sync(0xffffffffu, mine);
    if (owner_mask == 0) return -1;  // fewer than k entries: the caller guarantees this cannot happen
    const int owner = __ffs(owner_mask) - 1;
    uint32_t b_star = 0, cnt_above = 0;
    cntb = 0;
    if (lane == owner) {
      uint32_t run = above;
      for (int j = 31; j >= 0; --j) {
        const uint32_t c = sm.hist[33 * lane + j];
        if (run + c >= static_cast<uint32_t>(kk)) {
          b_star = 32 * lane + j;
          cnt_above = run;
          cntb = c;
          break;
        }
        run += c;
      }
    }
    b_star = __shfl_sync(0xffffffffu, b_star, owner);
    cnt_above = __shfl_sync(0xffffffffu, cnt_above, owner);
    cntb = __shfl_sync(0xffffffffu, cntb, owner);
    __syncwarp();
    kk -= static_cast<int>(cnt_above);
    // the boundary bin becomes the new range (the end bins of the first level are open-ended)
    const uint32_t new_lo = (level == 0 && b_star == 0) ? 0u : cur_lo + (b_star << shift);
    uint32_t new_hi = cur_lo + (b_star << shift) + ((1u << shift) - 1u);
    if (new_hi < cur_lo) new_hi = 0xffffffffu;  // the bin's upper edge lies beyond the key space
    // Below the first level the range is closed (keys outside it were not counted), so its last bin may be cut
    // short.  On the first level hi is a hint: keys above it were still counted in the bin their value falls in,
    // and cutting that bin at hi would make the output pass take them on top of the k it was promised.
    if (level > 0 && new_hi > cur_hi) new_hi = cur_hi;
    if (level == 0 && b_star == TS_BINS - 1) new_hi = 0xffffffffu;
    cur_lo = new_lo;
    cur_hi = new_hi;
    if (cntb <= TS_SIDE || shift == 0) break;
  }
  if (cntb > TS_SIDE) return -1;
  const int need = kk;  // entries to take from the boundary range [cur_lo, cur_hi]

  // ---- output pass: emit everything above the boundary range, stash the boundary range ----
  int out_n = 0, side_n = 0;
#pragma unroll 1
  for (int seg = 0; seg < L.segments(); ++seg) {
    const int n = L.count(seg);
    for (int base0 = 0; base0 < n; base0 += 32 * TS_U) {
      uint2 e[TS_U];
#pragma unroll
      for (int u = 0; u < TS_U; ++u) {
        const int i = base0 + 32 * u + lane;
        e[u] = i < n ? L.entry(seg, i) : make_uint2(0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < TS_U; ++u) {
        if (base0 + 32 * u >= n) break;
        const bool valid = base0 + 32 * u + lane < n;
        const uint32_t key = score_key(__uint_as_float(e[u].x));
        const bool take = valid && key > cur_hi;
        const bool inb = valid && key >= cur_lo && key <= cur_hi;
        const uint32_t bt = __ballot_sync(0xffffffffu, take);
        const uint32_t bi = __ballot_sync(0xffffffffu, inb);
        const uint32_t lt = (1u << lane) - 1u;
        if (take && kth_bits == nullptr) sink(out_n + __popc(bt & lt), e[u].x, e[u].y);
        if (inb) {
          const int sp = side_n + __popc(bi & lt);
          if (sp < TS_SIDE) sm.side[sp] = composite(key, e[u].y);
        }
        out_n += __popc(bt);
        side_n += __popc(bi);
      }
    }
  }
  __syncwarp();

  // ---- rank the boundary bin directly: composites are distinct, so ranks are a permutation ----
  const int m = side_n < TS_SIDE ? side_n : TS_SIDE;
  uint32_t found_bits = 0;
  bool found = false;
  for (int j = lane; j < m; j += 32) {
    const unsigned long long cj = sm.side[j];
    int rank = 0;
    for (int i = 0; i < m; ++i) {
      const unsigned long long ci = sm.side[i];
      rank += (ci > cj) || (ci == cj && i < j);
    }
    if (kth_bits != nullptr) {
      if (rank == need - 1) {
        found_bits = __float_as_uint(key_score(composite_key(cj)));
        found = true;
      }
    } else if (rank < need) {
      sink(out_n + rank, __float_as_uint(key_score(composite_key(cj))), composite_idx(cj));
    }
  }
  __syncwarp();
  if (kth_bits != nullptr) {
    const uint32_t who = __ballot_sync(0xffffffffu, found);
    if (who == 0) return -1;
    *kth_bits = __shfl_sync(0xffffffffu, found_bits, __ffs(who) - 1);
  }
  return k;
}

}  // namespace gw
