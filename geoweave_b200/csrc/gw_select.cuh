// Exact top-k selection by adaptive-range radix select, shared by every kernel of the library.
//
// A thread group (one warp, or NT threads of a CTA) selects the k largest of n candidates, each given as a
// 64-bit composite (score key << 32 | ~index), so "largest" means (score descending, index ascending) and
// all candidates with distinct indices are distinct.  Each level histograms the still-undecided candidates
// into NB equal-width bins of the current [lo, hi] composite range, finds the bin that holds the k-th
// candidate, and either finishes (the bin is taken whole, or it is small enough to be ranked directly, or
// it is a single value) or recurses into that bin.  The width adapts to the actual range, so candidate
// lists whose scores differ only in low mantissa bits still spread over all bins in the first level.
#pragma once

#include "gw_common.cuh"

namespace gw {

constexpr int kSideCap = 64;  // boundary bins up to this size are ranked directly

template <int NB>
struct SelectSmem {
  uint32_t hist[NB];
  unsigned long long side[kSideCap];
  unsigned long long kth;
  uint32_t warp_sums[32];
  uint32_t side_n, out_n, tie_n, b_star, above, cntb, found;
};

template <int NT>
__device__ __forceinline__ void group_sync(int bar_id) {
  if (NT == 32)
    __syncwarp();
  else
    named_bar_sync(bar_id, NT);
}

// Select the k largest of src(0..n-1) inside the composite range [lo, hi] (candidates outside the range
// are ignored; the range must hold at least k of them, otherwise all of them are taken).
//   src(i)        -> composite of candidate i (0 marks an empty slot; it loses to everything)
//   sink(pos, c)  -> called once per selected candidate with a unique pos in [0, #selected)
// Returns the number selected; *kth_out (optional) receives the smallest selected composite.
// `tid` is the caller's rank in the group (0..NT-1); all NT threads must call this together.
// With NT == 32 sink may write into the storage src reads (in-place compaction): a write to pos never
// targets a candidate that has not been read yet.
//   soft_hi       -> `hi` is only an estimate: candidates above it are counted in the top bin of the first level
//   U             -> candidates fetched per thread before any is processed (hides the latency of src)
template <int NT, int NB, class Src, class Sink, int U = 8>
__device__ int group_select_topk(const Src& src, int n, int k, unsigned long long lo, unsigned long long hi,
                                 SelectSmem<NB>& sm, int tid, int bar_id, const Sink& sink,
                                 unsigned long long* kth_out, bool soft_hi = false) {
  static_assert(NB % NT == 0, "bins must divide evenly over the group");
  constexpr int BPT = NB / NT;  // bins per thread
  constexpr int LOG_NB = (NB == 512) ? 9 : (NB == 1024) ? 10 : (NB == 2048) ? 11 : (NB == 4096) ? 12 : -1;
  static_assert(LOG_NB > 0, "NB must be 512..4096");
  const int lane = tid & 31;
  const int wid = tid >> 5;

  if (tid == 0) {
    sm.kth = ~0ull;
    sm.out_n = 0;
    sm.side_n = 0;
    sm.tie_n = 0;
  }
  unsigned long long cur_lo = lo, cur_hi = hi;
  int kk = k;
  int mode = 0;  // 0: take everything >= cur_lo; 1: rank the boundary bin; 2: boundary bin is one value
  if (n <= k) {
    cur_lo = 0;
    cur_hi = ~0ull;
    mode = 0;
    group_sync<NT>(bar_id);
  } else {
    for (;;) {
      const unsigned long long span = cur_hi - cur_lo;
      const int bits = (span == 0) ? 0 : 64 - __clzll(static_cast<long long>(span));
      const int shift = bits > LOG_NB ? bits - LOG_NB : 0;
#pragma unroll
      for (int j = 0; j < BPT; ++j) sm.hist[tid + j * NT] = 0;
      if (tid == 0) sm.found = 0;
      group_sync<NT>(bar_id);
      for (int base = tid; base < n; base += NT * U) {
        unsigned long long c[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int i = base + u * NT;
          c[u] = (i < n) ? src(i) : 0ull;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (base + u * NT < n && c[u] >= cur_lo && (c[u] <= cur_hi || soft_hi)) {
            uint32_t bin = static_cast<uint32_t>((c[u] - cur_lo) >> shift);
            if (soft_hi && (c[u] > cur_hi || bin > NB - 1)) bin = NB - 1;
            atomicAdd(&sm.hist[bin], 1u);
          }
        }
      }
      group_sync<NT>(bar_id);
      // thread t owns bins NB-1-t*BPT ... NB-t*BPT-BPT (descending), so a scan over t walks bins downward
      uint32_t mysum = 0;
#pragma unroll
      for (int j = 0; j < BPT; ++j) mysum += sm.hist[NB - 1 - tid * BPT - j];
      uint32_t incl = mysum;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
      }
      if (NT > 32) {
        if (lane == 31) sm.warp_sums[wid] = incl;
        group_sync<NT>(bar_id);
        uint32_t before = 0;
        for (int w2 = 0; w2 < wid; ++w2) before += sm.warp_sums[w2];
        incl += before;
      }
      const uint32_t excl = incl - mysum;
      if (excl < static_cast<uint32_t>(kk) && static_cast<uint32_t>(kk) <= incl) {
        uint32_t run = excl;
        for (int j = 0; j < BPT; ++j) {
          const int bin = NB - 1 - tid * BPT - j;
          const uint32_t c = sm.hist[bin];
          if (run + c >= static_cast<uint32_t>(kk)) {
            sm.b_star = bin;
            sm.above = run;
            sm.cntb = c;
            sm.found = 1;
            break;
          }
          run += c;
        }
      }
      if (tid == NT - 1 && incl < static_cast<uint32_t>(kk)) {
        // fewer than kk candidates in range: take them all
        sm.b_star = 0;
        sm.above = incl - sm.hist[0];
        sm.cntb = sm.hist[0];
        sm.found = 2;
      }
      group_sync<NT>(bar_id);
      const uint32_t b_star = sm.b_star, above = sm.above, cntb = sm.cntb, found = sm.found;
      group_sync<NT>(bar_id);  // everyone has read the result before the next level rewrites it
      const unsigned long long new_lo = cur_lo + (static_cast<unsigned long long>(b_star) << shift);
      unsigned long long new_hi = new_lo + ((1ull << shift) - 1ull);
      if (new_hi > cur_hi || new_hi < new_lo) new_hi = cur_hi;
      if (soft_hi && b_star == NB - 1) new_hi = ~0ull;  // the top bin also holds everything above the estimate
      soft_hi = false;
      kk -= static_cast<int>(above);
      cur_lo = new_lo;
      cur_hi = new_hi;
      if (found == 2) kk = static_cast<int>(cntb);
      if (static_cast<int>(cntb) == kk) { mode = 0; break; }
      if (cntb <= static_cast<uint32_t>(kSideCap)) { mode = 1; break; }
      if (shift == 0) { mode = 2; break; }
    }
  }

  // output pass
  unsigned long long my_min = ~0ull;
  for (int base0 = 0; base0 < n; base0 += NT * U) {
   unsigned long long cu[U];
#pragma unroll
   for (int u = 0; u < U; ++u) {
     const int i = base0 + u * NT + tid;
     cu[u] = (i < n) ? src(i) : 0ull;
   }
#pragma unroll
   for (int u = 0; u < U; ++u) {
    const int base = base0 + u * NT;
    if (base >= n) break;
    const int i = base + tid;
    const unsigned long long c = cu[u];
    bool take = false;
    if (i < n) {
      if (mode == 0) {
        take = (c >= cur_lo);
      } else if (c > cur_hi) {
        take = true;
      } else if (c >= cur_lo) {
        if (mode == 1) {
          const uint32_t s = atomicAdd(&sm.side_n, 1u);
          if (s < static_cast<uint32_t>(kSideCap)) sm.side[s] = c;
        } else {
          take = atomicAdd(&sm.tie_n, 1u) < static_cast<uint32_t>(kk);
        }
      }
    }
    const uint32_t ballot = __ballot_sync(0xffffffffu, take);
    if (ballot) {
      uint32_t basepos = 0;
      if (lane == 0) basepos = atomicAdd(&sm.out_n, __popc(ballot));
      basepos = __shfl_sync(0xffffffffu, basepos, 0);
      if (take) {
        sink(static_cast<int>(basepos + __popc(ballot & ((1u << lane) - 1u))), c);
        my_min = c < my_min ? c : my_min;
      }
    }
   }
  }
  if (mode == 1) {
    group_sync<NT>(bar_id);
    const int m = static_cast<int>(sm.side_n < static_cast<uint32_t>(kSideCap) ? sm.side_n : kSideCap);
    for (int j = tid; j < m; j += NT) {
      const unsigned long long cj = sm.side[j];
      int rank = 0;
      for (int i = 0; i < m; ++i) {
        const unsigned long long ci = sm.side[i];
        rank += (ci > cj) || (ci == cj && i < j);
      }
      if (rank < kk) {
        const uint32_t pos = atomicAdd(&sm.out_n, 1u);
        sink(static_cast<int>(pos), cj);
        my_min = cj < my_min ? cj : my_min;
      }
    }
  }
  if (my_min != ~0ull) atomicMin(&sm.kth, my_min);
  group_sync<NT>(bar_id);
  const int total = static_cast<int>(sm.out_n);
  if (kth_out != nullptr) *kth_out = sm.kth;
  group_sync<NT>(bar_id);  // results read before a following call resets the scratch
  return total;
}

}  // namespace gw
