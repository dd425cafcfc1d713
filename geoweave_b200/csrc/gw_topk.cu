// Stage 2 alone: exact top-k of materialised score rows, and the merge of two top-k lists.
// Both are thin drivers around group_select_topk (gw_select.cuh).
#include <cmath>

#include "gw_common.cuh"
#include "gw_select.cuh"
#include "gw_select_tight.cuh"

namespace gw {

thread_local int g_last_cuda_error = 0;
std::atomic<unsigned> g_cache_epoch{0};
DeviceFactsSlot g_device_facts[kMaxDevices];

namespace {

constexpr int kTopkThreads = 256;
constexpr int kTopkBins = 2048;

template <typename T>
struct DenseRowSrc {
  const T* row;
  __device__ __forceinline__ unsigned long long operator()(int i) const {
    return composite(score_key(to_float(row[i])), static_cast<uint32_t>(i));
  }
};

template <typename T>
struct DenseRowSink {
  const T* row;
  int32_t* o32;
  int64_t* o64;
  T* os;
  __device__ __forceinline__ void operator()(int pos, unsigned long long c) const {
    const uint32_t idx = composite_idx(c);
    if (o32) o32[pos] = static_cast<int32_t>(idx);
    if (o64) o64[pos] = static_cast<int64_t>(idx);
    if (os) {
      // the key gives the score back exactly, except that it cannot tell -0.0 from +0.0: those are read from the row
      const uint32_t key = composite_key(c);
      os[pos] = key == 0x80000000u ? row[idx] : from_float<T>(key_score(key));
    }
  }
};

// one CTA per row: min/max pass, then adaptive radix select (rows of a few hundred KB stay in L2 between passes)
template <typename T>
__global__ void __launch_bounds__(kTopkThreads) topk_exact_kernel(const T* __restrict__ scores, int64_t cols,
                                                                   int64_t row_stride, int k, int32_t* o32,
                                                                   int64_t* o64, T* os) {
  __shared__ SelectSmem<kTopkBins> sm;
  __shared__ uint32_t s_min, s_max;
  const int tid = threadIdx.x;
  const int64_t r = blockIdx.x;
  const T* row = scores + r * row_stride;
  const int n = static_cast<int>(cols);
  if (tid == 0) {
    s_min = 0xffffffffu;
    s_max = 0u;
  }
  __syncthreads();
  uint32_t kmin = 0xffffffffu, kmax = 0u;
  for (int i = tid; i < n; i += kTopkThreads) {
    const uint32_t key = score_key(to_float(row[i]));
    kmin = min(kmin, key);
    kmax = max(kmax, key);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    kmin = min(kmin, __shfl_xor_sync(0xffffffffu, kmin, d));
    kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, d));
  }
  if ((tid & 31) == 0) {
    atomicMin(&s_min, kmin);
    atomicMax(&s_max, kmax);
  }
  __syncthreads();
  const unsigned long long lo = static_cast<unsigned long long>(s_min) << 32;
  const unsigned long long hi = (static_cast<unsigned long long>(s_max) << 32) | 0xffffffffull;
  DenseRowSrc<T> src{row};
  DenseRowSink<T> sink{row, o32 ? o32 + r * k : nullptr, o64 ? o64 + r * k : nullptr, os ? os + r * k : nullptr};
  group_select_topk<kTopkThreads, kTopkBins>(src, n, k, lo, hi, sm, tid, 1, sink, nullptr);
}

// ---------------------------------------------------------------------------------------------
// Rows that fit in shared memory.  The row is brought in once (bulk copies when it is fp32 and 16-byte aligned)
// and every later pass runs on shared memory.  Shared-memory atomics are the scarce resource (about two per
// clock per SM), so a full-row histogram is avoided when k is small against the row: a strided sample of the
// row gives a threshold that keeps a few thousand candidates, one compare-only pass compacts those, and the
// histogram levels run on the candidates.  Whenever the candidates come short of k, overflow their buffer or the
// sample is unusable, the row is selected in full instead, so the result is exact for any input.  Within either
// path up to three levels of 2048 bins narrow the boundary range until it holds at most kCtaSide entries,
// which are ranked directly; a boundary crowded with equal scores goes to the general routine.
// ---------------------------------------------------------------------------------------------
constexpr int kRowThreads = 512;
constexpr int kCtaSide = 256;
constexpr uint32_t kCopyChunk = 8192;
constexpr int kPrivSlots = 32;        // 16-bit candidate slots per thread on the sampled path
constexpr int kSegCap = 384;          // candidate columns per warp once packed
constexpr size_t kPrivBytes = sizeof(uint16_t) * kPrivSlots * kRowThreads;
constexpr size_t kSegBytes = sizeof(uint32_t) * kSegCap * (kRowThreads / 32);
constexpr uint32_t kSampleStop = 96;  // the sample's boundary range is narrowed until it holds at most this many samples
struct RowSelSmem {
  SelectSmem<kTopkBins> gen;  // scratch of the general routine; its histogram also serves the lean levels
  unsigned long long side[kCtaSide];
  uint32_t wsum[kRowThreads / 32], wmin[kRowThreads / 32], wmax[kRowThreads / 32];
  uint64_t bar;
  uint32_t b_star, cnt_above, cntb, found, copy_ok;
};
// the row in shared memory: raw fp32 bits (as copied) or score keys; every stride-th column
struct RowKeys {
  const uint32_t* w;
  bool raw;
  int stride;
  __device__ __forceinline__ uint32_t key(int i) const {
    const uint32_t v = w[i * stride];
    return raw ? score_key(__uint_as_float(v)) : v;
  }
  __device__ __forceinline__ uint32_t idx(int i) const { return static_cast<uint32_t>(i * stride); }
};
// The candidate columns of one warp, compacted into the warp's segment (entry i = element (i / 512) * 32 + lane
// of the segment of the calling thread's warp); entries past the warp's count read as key 0, below every range
// that is searched.
struct WarpSegKeys {
  const uint32_t* w;
  const uint32_t* seg;
  bool raw;
  int wcnt, lane;
  __device__ __forceinline__ int local(int i) const { return (i / kRowThreads) * 32 + lane; }
  __device__ __forceinline__ uint32_t key(int i) const {
    const int li = local(i);
    if (li >= wcnt) return 0u;
    const uint32_t v = w[seg[li]];
    return raw ? score_key(__uint_as_float(v)) : v;
  }
  __device__ __forceinline__ uint32_t idx(int i) const { return seg[local(i)]; }
};
struct WarpSegComposites {
  WarpSegKeys p;
  __device__ __forceinline__ unsigned long long operator()(int i) const {
    const uint32_t key = p.key(i);
    return key ? composite(key, p.idx(i)) : 0ull;
  }
};
struct SmemKeySrc {
  const uint32_t* keys;
  __device__ __forceinline__ unsigned long long operator()(int i) const { return composite(keys[i], static_cast<uint32_t>(i)); }
};

// smallest and largest key of src(0..n-1), returned to every thread
template <class Src>
__device__ __forceinline__ void cta_key_range(const Src& src, int n, RowSelSmem& sm, int tid, uint32_t& kmin_out, uint32_t& kmax_out) {
  constexpr int NW = kRowThreads / 32;
  const int lane = tid & 31, wid = tid >> 5;
  uint32_t kmin = 0xffffffffu, kmax = 0u;
  for (int i = tid; i < n; i += kRowThreads) {
    const uint32_t key = src.key(i);
    kmin = min(kmin, key);
    kmax = max(kmax, key);
  }
  kmin = __reduce_min_sync(0xffffffffu, kmin);
  kmax = __reduce_max_sync(0xffffffffu, kmax);
  if (lane == 0) {
    sm.wmin[wid] = kmin;
    sm.wmax[wid] = kmax;
  }
  __syncthreads();
  kmin = __reduce_min_sync(0xffffffffu, lane < NW ? sm.wmin[lane] : 0xffffffffu);
  kmax = __reduce_max_sync(0xffffffffu, lane < NW ? sm.wmax[lane] : 0u);
  __syncthreads();  // wmin / wmax are read before a following call rewrites them
  kmin_out = kmin;
  kmax_out = kmax;
}

// Histogram levels: narrows [lo, hi] to the range that holds the kk-th largest key of src (keys outside
// [lo, hi] are ignored; at least kk keys must lie inside), until that range holds at most `stop` keys or is a
// single key value.  On return kk counts from the top of the new range and cntb is its population.
// False when fewer than kk keys were in range.
template <class Src>
__device__ bool cta_find_range(const Src& src, int n, int& kk, uint32_t& lo, uint32_t& hi, uint32_t& cntb, uint32_t stop,
                               RowSelSmem& sm, int tid) {
  constexpr int NT = kRowThreads, NB = kTopkBins, BPT = NB / NT;
  const int lane = tid & 31, wid = tid >> 5;
  uint32_t* const hist = sm.gen.hist;
  for (int level = 0; level < 3; ++level) {
    const uint32_t span = hi - lo;
    const int bits = 32 - __clz(span);
    const int shift = bits > 11 ? bits - 11 : 0;
#pragma unroll
    for (int j = 0; j < BPT; ++j) hist[tid + j * NT] = 0;
    if (tid == 0) sm.found = 0;
    __syncthreads();
    for (int i = tid; i < n; i += NT) {
      const uint32_t key = src.key(i);
      if (key >= lo && key <= hi) atomicAdd(&hist[(key - lo) >> shift], 1u);
    }
    __syncthreads();
    // thread t owns bins NB-1-t*BPT-j: a scan over t walks the bins from the top down
    uint32_t mysum = 0;
#pragma unroll
    for (int j = 0; j < BPT; ++j) mysum += hist[NB - 1 - tid * BPT - j];
    uint32_t incl = mysum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += up;
    }
    if (lane == 31) sm.wsum[wid] = incl;
    __syncthreads();
    incl += __reduce_add_sync(0xffffffffu, lane < wid ? sm.wsum[lane] : 0u);  // warps before this one (wid < 32 warps)
    const uint32_t excl = incl - mysum;
    if (excl < static_cast<uint32_t>(kk) && static_cast<uint32_t>(kk) <= incl) {
      uint32_t run = excl;
      for (int j = 0; j < BPT; ++j) {
        const int bin = NB - 1 - tid * BPT - j;
        const uint32_t c = hist[bin];
        if (run + c >= static_cast<uint32_t>(kk)) {
          sm.b_star = bin;
          sm.cnt_above = run;
          sm.cntb = c;
          sm.found = 1;
          break;
        }
        run += c;
      }
    }
    __syncthreads();
    const uint32_t found = sm.found, b_star = sm.b_star, above = sm.cnt_above;
    cntb = sm.cntb;
    __syncthreads();  // everyone has read the result before the next level (or the caller) rewrites it
    if (!found) return false;
    kk -= static_cast<int>(above);
    const uint32_t new_lo = lo + (b_star << shift);
    uint32_t new_hi = new_lo + ((1u << shift) - 1u);
    if (new_hi > hi || new_hi < new_lo) new_hi = hi;
    lo = new_lo;
    hi = new_hi;
    if (cntb <= stop || shift == 0) break;
  }
  return true;
}

// Emits every entry of src above [lo, hi] (there are base_pos of them) and the `need` best of the entries
// inside [lo, hi] (at most kCtaSide, ranked directly by score, then index).  Two sweeps and no shared counter:
// the first counts per warp, a prefix over the warps gives each its output offset, the second writes.
template <class Src, class Sink>
__device__ void cta_emit(const Src& src, int n, uint32_t lo, uint32_t hi, int need, int base_pos, RowSelSmem& sm, int tid,
                         const Sink& sink) {
  constexpr int NT = kRowThreads, NW = NT / 32, OU = 4;
  const int lane = tid & 31, wid = tid >> 5;
  const uint32_t below = (1u << lane) - 1u;
  uint32_t ct = 0, ci = 0;
  for (int base = 0; base < n; base += NT * OU) {
#pragma unroll
    for (int u = 0; u < OU; ++u) {
      const int i = base + u * NT + tid;
      const uint32_t key = i < n ? src.key(i) : 0u;
      ct += __popc(__ballot_sync(0xffffffffu, i < n && key > hi));
      ci += __popc(__ballot_sync(0xffffffffu, i < n && key >= lo && key <= hi));
    }
  }
  if (lane == 0) {
    sm.wsum[wid] = ct;
    sm.wmin[wid] = ci;
  }
  __syncthreads();
  uint32_t pt = __reduce_add_sync(0xffffffffu, lane < wid ? sm.wsum[lane] : 0u);
  uint32_t pi = __reduce_add_sync(0xffffffffu, lane < wid ? sm.wmin[lane] : 0u);
  const uint32_t side_total = __reduce_add_sync(0xffffffffu, lane < NW ? sm.wmin[lane] : 0u);
  for (int base = 0; base < n; base += NT * OU) {
    uint32_t key[OU];
#pragma unroll
    for (int u = 0; u < OU; ++u) {
      const int i = base + u * NT + tid;
      key[u] = i < n ? src.key(i) : 0u;
    }
#pragma unroll
    for (int u = 0; u < OU; ++u) {
      const int i = base + u * NT + tid;
      const bool take = i < n && key[u] > hi;
      const bool inb = i < n && key[u] >= lo && key[u] <= hi;
      const uint32_t bt = __ballot_sync(0xffffffffu, take);
      const uint32_t bi = __ballot_sync(0xffffffffu, inb);
      if (take) sink(static_cast<int>(pt + __popc(bt & below)), composite(key[u], src.idx(i)));
      if (inb) {
        const uint32_t sp = pi + __popc(bi & below);
        if (sp < kCtaSide) sm.side[sp] = composite(key[u], src.idx(i));
      }
      pt += __popc(bt);
      pi += __popc(bi);
    }
  }
  __syncthreads();
  const int m = static_cast<int>(side_total < kCtaSide ? side_total : kCtaSide);
  for (int j = tid; j < m; j += NT) {
    const unsigned long long cj = sm.side[j];
    int rank = 0;
    for (int i = 0; i < m; ++i) {
      const unsigned long long ci2 = sm.side[i];
      rank += (ci2 > cj) || (ci2 == cj && i < j);
    }
    if (rank < need) sink(base_pos + rank, cj);
  }
  __syncthreads();
}

// Compare-only pass of the sampled path.  Thread t looks at columns t, t + 512, ... and notes the sweeps (column /
// 512) in which it met a value at or above the threshold, in 16-bit slots of its own (slot s of thread t is
// halfword s * 512 + t: no bank conflicts, no counter shared with anyone).  Per column: one load, one compare, a
// predicated store and a predicated bump of the slot address.  MODE 0: the buffer holds raw fp32 bits and the
// threshold is positive, so signed integer order of the bits is score order; MODE 1: raw bits, any threshold
// (the key is computed); MODE 2: the buffer holds keys.  thr is the threshold in the compared domain.
// Returns the number of slots filled, or -1 when the slots ran out before the row did.
template <int MODE>
__device__ __forceinline__ int filter_row(const uint32_t* keys, int n, int thr, uint16_t* priv, int tid) {
  constexpr int NT = kRowThreads, U = 8;
  const uint32_t off0 = smem_u32(priv + tid);
  const uint32_t off_stop = off0 + (kPrivSlots - U) * NT * 2;  // beyond this a sweep of U columns could overrun
  uint32_t off = off0;
  auto cmp_value = [](uint32_t v) -> int {
    if (MODE == 0) return static_cast<int>(v);
    if (MODE == 1) return static_cast<int>(score_key(__uint_as_float(v)) ^ 0x80000000u);
    return static_cast<int>(v ^ 0x80000000u);
  };
  auto note = [&](int x, uint32_t sweep) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ge.s32 p, %1, %2;\n\t"
        "@p st.shared.u16 [%0], %3;\n\t"
        "@p add.u32 %0, %0, 1024;\n\t}"
        : "+r"(off)
        : "r"(x), "r"(thr), "h"(static_cast<uint16_t>(sweep))
        : "memory");
  };
  const int full = n / (NT * U);  // groups of U sweeps that lie wholly inside the row
  int g = 0;
  for (; g < full; ++g) {
    uint32_t v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = keys[(g * U + u) * NT + tid];
#pragma unroll
    for (int u = 0; u < U; ++u) note(cmp_value(v[u]), static_cast<uint32_t>(g * U + u));
    if (off > off_stop) return -1;
  }
  {
    uint32_t v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = (g * U + u) * NT + tid;
      v[u] = i < n ? keys[i] : 0u;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = (g * U + u) * NT + tid;
      note(i < n ? cmp_value(v[u]) : static_cast<int>(0x80000000u), static_cast<uint32_t>(g * U + u));
    }
  }
  return static_cast<int>((off - off0) / (NT * 2));
}

// sample_step > 0: the sampled path is tried first, with (about) the sample's sample_rank-th largest key as threshold;
// the threads' candidate slots lie behind the row.
template <typename T>
__global__ void __launch_bounds__(kRowThreads, 1)
topk_row_in_smem_kernel(const T* __restrict__ scores, int64_t rows, int n, int64_t row_stride, int k, int32_t* o32, int64_t* o64,
                        T* os, int sample_step, int sample_rank) {
  constexpr int NT = kRowThreads;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  uint32_t* keys = reinterpret_cast<uint32_t*>(smem_raw);
  const size_t row_bytes = static_cast<size_t>((n + 3) / 4 * 4) * 4;
  uint16_t* priv = reinterpret_cast<uint16_t*>(smem_raw + row_bytes);
  uint32_t* segs = reinterpret_cast<uint32_t*>(smem_raw + row_bytes + kPrivBytes);
  RowSelSmem& sm = *reinterpret_cast<RowSelSmem*>(smem_raw + row_bytes + (sample_step > 0 ? kPrivBytes + kSegBytes : 0));
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  if (tid == 0) {
    mbar_init(&sm.bar, 1);
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  uint32_t phase = 0;
  bool bulk_usable = sizeof(T) == 4 && (n % 4) == 0;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* row = scores + r * row_stride;
    bool bulk = bulk_usable && (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
    // ---- the row comes into shared memory ----
    if (bulk) {
      if (tid == 0) mbar_arrive_expect_tx(&sm.bar, static_cast<uint32_t>(n) * 4u);
      __syncthreads();
      if (wid == 0) {
        // up to 32 copies of kCopyChunk bytes in flight, one per lane, all counted on one barrier; the row this
        // CTA takes next is asked into L2 meanwhile.  Every thread's accesses to the buffer for the previous row
        // lie before the barrier above; the fence orders them before the copies.
        fence_proxy_async_smem();
        const uint32_t bytes = static_cast<uint32_t>(n) * 4u;
        const int64_t rn = r + gridDim.x;
        const char* next = reinterpret_cast<const char*>(scores + rn * row_stride);
        const bool pf = rn < rows && (reinterpret_cast<uintptr_t>(next) & 15u) == 0;
        for (uint32_t off = lane * kCopyChunk; off < bytes; off += 32 * kCopyChunk) {
          const uint32_t len = bytes - off < kCopyChunk ? bytes - off : kCopyChunk;
          bulk_g2s(reinterpret_cast<char*>(keys) + off, reinterpret_cast<const char*>(row) + off, len, &sm.bar);
          if (pf) bulk_prefetch_l2(next + off, len);
        }
      }
      // one thread waits (bounded) and tells the rest; a copy that never lands switches the kernel to plain loads
      if (tid == 0) sm.copy_ok = mbar_wait_bounded(&sm.bar, phase & 1u) ? 1u : 0u;
      __syncthreads();
      ++phase;
      if (!sm.copy_ok) {
        bulk = false;
        bulk_usable = false;
      }
    }
    if (!bulk) {
      for (int base = tid; base < n; base += NT * 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = (base + u * NT < n) ? to_float(row[base + u * NT]) : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (base + u * NT < n) keys[base + u * NT] = score_key(v[u]);
      }
      __syncthreads();
    }
    bool raw = bulk;  // the buffer holds fp32 bits until the full path turns them into keys
    DenseRowSink<T> sink{row, o32 ? o32 + r * k : nullptr, o64 ? o64 + r * k : nullptr, os ? os + r * k : nullptr};
    bool done = false;

    // ---- sampled path ----
    if (sample_step > 0) {
      const RowKeys samp{keys, raw, sample_step};
      const int ns = (n + sample_step - 1) / sample_step;
      // the first level spans the whole key space (quarter-octave bins): no pass for the sample's own range
      uint32_t lo = 0u, hi = 0xffffffffu, cntb = 0;
      int kk = sample_rank;
      if (cta_find_range(samp, ns, kk, lo, hi, cntb, kSampleStop, sm, tid) && lo != 0u) {
        const uint32_t tau = lo;  // at least sample_rank sample keys are >= tau
        int cnt;
        if (raw && tau > 0x80000000u)
          cnt = filter_row<0>(keys, n, static_cast<int>(__float_as_uint(key_score(tau))), priv, tid);
        else if (raw)
          cnt = filter_row<1>(keys, n, static_cast<int>(tau ^ 0x80000000u), priv, tid);
        else
          cnt = filter_row<2>(keys, n, static_cast<int>(tau ^ 0x80000000u), priv, tid);
        // Each warp packs its threads' notes into its own segment as column numbers, and the CTA learns the number
        // of candidates, the longest segment and the largest candidate key.
        const bool over = cnt < 0;
        const int mycnt = over ? 0 : cnt;
        int incl = mycnt;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int up = __shfl_up_sync(0xffffffffu, incl, d);
          if (lane >= d) incl += up;
        }
        const int wcnt = __shfl_sync(0xffffffffu, incl, 31);
        const bool wover = __any_sync(0xffffffffu, over) || wcnt > kSegCap;
        uint32_t* const seg = segs + wid * kSegCap;
        uint32_t kmax = 0u;
        if (!wover) {
          for (int sl = 0; sl < mycnt; ++sl) {
            const uint32_t col = static_cast<uint32_t>(priv[sl * NT + tid]) * NT + tid;
            seg[incl - mycnt + sl] = col;
            const uint32_t v = keys[col];
            kmax = max(kmax, raw ? score_key(__uint_as_float(v)) : v);
          }
        }
        kmax = __reduce_max_sync(0xffffffffu, kmax);
        if (lane == 0) {
          sm.wmax[wid] = kmax;
          sm.wsum[wid] = wover ? 0x40000000u : static_cast<uint32_t>(wcnt);
        }
        __syncthreads();
        constexpr int NW = NT / 32;
        const uint32_t cmax = __reduce_max_sync(0xffffffffu, lane < NW ? sm.wmax[lane] : 0u);
        const uint32_t nc = __reduce_add_sync(0xffffffffu, lane < NW ? sm.wsum[lane] : 0u);
        const uint32_t longest = __reduce_max_sync(0xffffffffu, lane < NW ? sm.wsum[lane] : 0u);
        __syncthreads();
        if (nc >= static_cast<uint32_t>(k) && longest <= static_cast<uint32_t>(kSegCap)) {
          const WarpSegKeys ws{keys, seg, raw, wcnt, lane};
          const int slots = static_cast<int>((longest + 31) / 32) * NT;
          uint32_t clo = tau, chi = cmax;
          kk = k;
          const bool lean = cta_find_range(ws, slots, kk, clo, chi, cntb, kCtaSide, sm, tid) && cntb <= kCtaSide;
          if (lean) {
            cta_emit(ws, slots, clo, chi, kk, k - kk, sm, tid, sink);
          } else {
            const WarpSegComposites src{ws};
            group_select_topk<NT, kTopkBins>(src, slots, k, static_cast<unsigned long long>(tau) << 32,
                                             (static_cast<unsigned long long>(cmax) << 32) | 0xffffffffull, sm.gen, tid, 1, sink, nullptr);
            __syncthreads();
          }
          done = true;
        }
      }
    }

    // ---- full path ----
    if (!done) {
      if (raw) {
        for (int i = tid; i < n; i += NT) keys[i] = score_key(__uint_as_float(keys[i]));
        raw = false;
        __syncthreads();
      }
      const RowKeys full{keys, false, 1};
      uint32_t rmin, rmax;
      cta_key_range(full, n, sm, tid, rmin, rmax);
      uint32_t lo = rmin, hi = rmax, cntb = 0;
      int kk = k;
      if (cta_find_range(full, n, kk, lo, hi, cntb, kCtaSide, sm, tid) && cntb <= kCtaSide) {
        cta_emit(full, n, lo, hi, kk, k - kk, sm, tid, sink);
      } else {
        const SmemKeySrc src{keys};
        group_select_topk<NT, kTopkBins>(src, n, k, static_cast<unsigned long long>(rmin) << 32,
                                         (static_cast<unsigned long long>(rmax) << 32) | 0xffffffffull, sm.gen, tid, 1, sink, nullptr);
        __syncthreads();
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// merge of two lists: one warp per row
// ---------------------------------------------------------------------------------------------
constexpr int kMergeWarps = 4;
constexpr int kMergeBins = 1024;

template <typename T>
struct TwoListSrc {
  const T* a_s;
  const int32_t* a_i;
  const T* b_s;
  const int64_t* b_p;
  int ka;
  int64_t b_start;
  __device__ __forceinline__ unsigned long long operator()(int i) const {
    float s;
    int64_t idx;
    if (i < ka) {
      s = to_float(a_s[i]);
      idx = a_i[i];
    } else {
      s = to_float(b_s[i - ka]);
      idx = b_p[i - ka];
      idx = idx < 0 ? idx : idx + b_start;
    }
    return idx < 0 ? 0ull : composite(score_key(s), static_cast<uint32_t>(idx));
  }
};

template <typename T>
struct ListSink {
  T* os;
  int32_t* oi;
  __device__ __forceinline__ void operator()(int pos, unsigned long long c) const {
    if (c == 0ull) {  // an empty slot had to be taken: fewer than k real candidates
      oi[pos] = -1;
      os[pos] = from_float<T>(-INFINITY);
    } else {
      oi[pos] = static_cast<int32_t>(composite_idx(c));
      os[pos] = from_float<T>(key_score(composite_key(c)));
    }
  }
};

// the two lists as segments of (score bits, index) for the lean warp routine; an empty slot (negative index)
// becomes (-inf, 0xffffffff), which loses every comparison and is written back as index -1
template <typename T>
struct TwoListSegs {
  const T* a_s;
  const int32_t* a_i;
  const T* b_s;
  const int64_t* b_p;
  int ka, kb;
  int64_t b_start;
  __device__ __forceinline__ int segments() const { return 2; }
  __device__ __forceinline__ int count(int seg) const { return seg == 0 ? ka : kb; }
  __device__ __forceinline__ uint2 entry(int seg, int i) const {
    float s;
    int64_t idx;
    if (seg == 0) {
      s = to_float(a_s[i]);
      idx = a_i[i];
    } else {
      s = to_float(b_s[i]);
      idx = b_p[i];
      idx = idx < 0 ? idx : idx + b_start;
    }
    return idx < 0 ? make_uint2(0xff800000u, 0xffffffffu) : make_uint2(__float_as_uint(s), static_cast<uint32_t>(idx));
  }
  __device__ __forceinline__ uint32_t bits(int seg, int i) const { return entry(seg, i).x; }
};
template <typename T>
struct ListBitsSink {
  T* os;
  int32_t* oi;
  __device__ __forceinline__ void operator()(int pos, uint32_t bits, uint32_t idx) const {
    oi[pos] = static_cast<int32_t>(idx);
    os[pos] = from_float<T>(__uint_as_float(bits));
  }
};

struct MergeSmem {
  union {
    SelectSmem<kMergeBins> gen;
    TightSmem tight;
  };
};

// The lean warp routine first (32-bit keys, about two dozen instructions per entry); a boundary crowded with
// equal scores, or fewer than k entries in all, goes to the general routine.  Both may write over list a: an
// output position is never ahead of the entries already read into registers.
template <typename T>
__global__ void __launch_bounds__(kMergeWarps * 32) merge_two_topk_kernel(const T* a_s, const int32_t* a_i, int ka,
                                                                          const T* b_s, const int64_t* b_p, int kb,
                                                                          int64_t b_start, int64_t rows, int k, T* os,
                                                                          int32_t* oi) {
  __shared__ MergeSmem sm[kMergeWarps];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r = static_cast<int64_t>(blockIdx.x) * kMergeWarps + w;
  if (r >= rows) return;
  const int n = ka + kb;
  if (n > k) {
    const TwoListSegs<T> segs{a_s + r * ka, a_i + r * ka, b_s + r * kb, b_p + r * kb, ka, kb, b_start};
    uint32_t kmin = 0xffffffffu, kmax = 0u;
    for (int seg = 0; seg < 2; ++seg)
      for (int i = lane; i < segs.count(seg); i += 32) {
        const uint32_t key = score_key(__uint_as_float(segs.bits(seg, i)));
        kmin = min(kmin, key);
        kmax = max(kmax, key);
      }
    kmin = __reduce_min_sync(0xffffffffu, kmin);
    kmax = __reduce_max_sync(0xffffffffu, kmax);
    const ListBitsSink<T> bsink{os + r * k, oi + r * k};
    if (warp_select_tight(segs, k, kmin, kmax, sm[w].tight, lane, bsink, nullptr) == k) return;
    __syncwarp();
  }
  TwoListSrc<T> src{a_s + r * ka, a_i + r * ka, b_s + r * kb, b_p + r * kb, ka, b_start};
  unsigned long long cmin = ~0ull, cmax = 0ull;
  for (int i = lane; i < n; i += 32) {
    const unsigned long long c = src(i);
    cmin = c < cmin ? c : cmin;
    cmax = c > cmax ? c : cmax;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const unsigned long long a = __shfl_xor_sync(0xffffffffu, cmin, d);
    const unsigned long long b = __shfl_xor_sync(0xffffffffu, cmax, d);
    cmin = a < cmin ? a : cmin;
    cmax = b > cmax ? b : cmax;
  }
  ListSink<T> sink{os + r * k, oi + r * k};
  const int got = group_select_topk<32, kMergeBins>(src, n, k, cmin, cmax, sm[w].gen, lane, 0, sink, nullptr);
  for (int p = got + lane; p < k; p += 32) sink(p, 0ull);  // k > ka + kb: pad with empty slots
}

}  // namespace
}  // namespace gw

using namespace gw;

// Rows that fit in shared memory (about 55K columns) go to the kernel that keeps the row there (as many CTAs per SM as
// its footprint allows, each walking rows grid-stride); longer rows to the kernel that re-reads them from L2.
template <typename T>
static int launch_topk_exact(const void* scores, int64_t rows, int64_t cols, int64_t row_stride, int k, int32_t* o32, int64_t* o64,
                             void* out_scores, cudaStream_t st) {
  const T* sc = static_cast<const T*>(scores);
  T* os = static_cast<T*>(out_scores);
  constexpr size_t kSmemBudget = 226 * 1024;
  const size_t row_bytes = static_cast<size_t>((cols + 3) / 4 * 4) * 4;
  if (row_bytes + sizeof(RowSelSmem) <= kSmemBudget) {
    // Sampled path when k is small against the row: about 2048 samples; the threshold is at or below the sample's
    // key of rank ratio + 6.75 sqrt(ratio) + 2 (ratio = k * samples / cols), which keeps at least k candidates
    // except in one row of many millions (such a row is then selected in full).
    int step = 0, rank = 0;
    size_t cap = 0;
    if (cols >= 8192 && static_cast<int64_t>(k) * 8 <= cols) {
      step = static_cast<int>(cols / 2048) | 1;
      if (step < 3) step = 3;
      const double ns = static_cast<double>((cols + step - 1) / step);
      const double ratio = static_cast<double>(k) * ns / static_cast<double>(cols);
      rank = static_cast<int>(std::ceil(ratio + 6.75 * std::sqrt(ratio) + 2.0));
      const double per = static_cast<double>(cols) / ns;
      // each thread keeps its candidates in slots of its own, of which kPrivSlots - 8 are sure to be usable: the
      // expected load (the threshold sits up to kSampleStop samples low, half of that on average) must leave
      // four standard deviations of room, or too many rows would overflow and be selected in full
      const double load = (rank + kSampleStop / 2) * per / kRowThreads;
      cap = kPrivBytes + kSegBytes;
      if (rank >= ns || load + 4.0 * std::sqrt(load) + 1.0 > kPrivSlots - 8 || 32 * load + 4.0 * std::sqrt(32 * load) > kSegCap ||
          cols / kRowThreads >= 65535 || row_bytes + cap + sizeof(RowSelSmem) > kSmemBudget) {
        step = 0;
        rank = 0;
        cap = 0;
      }
    }
    const size_t smem = row_bytes + cap + sizeof(RowSelSmem);
    int dev = 0, per_sm = 0;
    DeviceFacts facts;
    const int frc = device_facts(&dev, &facts);
    if (frc != GW_OK) return frc;
    const int sms = facts.sms;
    // the shared-memory size depends on the row length, so the attribute is raised to the budget once per device
    static OncePerDevice smem_once;
    const int src = ensure_dynamic_smem(topk_row_in_smem_kernel<T>, kSmemBudget, smem_once, dev);
    if (src != GW_OK) return src;
    GW_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, topk_row_in_smem_kernel<T>, kRowThreads, smem));
    if (per_sm >= 1) {
      const int64_t slots = static_cast<int64_t>(sms) * per_sm;
      const unsigned grid = static_cast<unsigned>(rows < slots ? rows : slots);
      topk_row_in_smem_kernel<T><<<grid, kRowThreads, smem, st>>>(sc, rows, static_cast<int>(cols), row_stride, k, o32, o64, os, step,
                                                                  rank);
      GW_LAUNCH_CHECK();
      return GW_OK;
    }
  }
  topk_exact_kernel<T><<<static_cast<unsigned>(rows), kTopkThreads, 0, st>>>(sc, cols, row_stride, k, o32, o64, os);
  GW_LAUNCH_CHECK();
  return GW_OK;
}

extern "C" int gw_topk_exact(const void* scores, int dtype, int64_t rows, int64_t cols, int64_t row_stride, int k,
                             int32_t* out_idx32, int64_t* out_idx64, void* out_scores, gw_stream_t stream) {
  if (!scores || rows < 0 || cols <= 0 || k <= 0 || row_stride < cols) return GW_ERR_INVALID_ARG;
  if (!out_idx32 && !out_idx64) return GW_ERR_INVALID_ARG;
  if (k > cols || cols > 0x7fffffff || rows > 0x7fffffff) return GW_ERR_INVALID_ARG;
  if (rows == 0) return GW_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case GW_F32:
      return launch_topk_exact<float>(scores, rows, cols, row_stride, k, out_idx32, out_idx64, out_scores, st);
    case GW_BF16:
      return launch_topk_exact<__nv_bfloat16>(scores, rows, cols, row_stride, k, out_idx32, out_idx64, out_scores, st);
    case GW_F16:
      return launch_topk_exact<__half>(scores, rows, cols, row_stride, k, out_idx32, out_idx64, out_scores, st);
    default:
      return GW_ERR_UNSUPPORTED;
  }
}

extern "C" int gw_merge_two_topk(const void* a_scores, const int32_t* a_idx, int ka, const void* b_scores,
                                 const int64_t* b_pos, int kb, int64_t b_start, int dtype, int64_t rows, int k,
                                 void* out_scores, int32_t* out_idx, gw_stream_t stream) {
  if (!a_scores || !a_idx || !b_scores || !b_pos || !out_scores || !out_idx) return GW_ERR_INVALID_ARG;
  if (ka <= 0 || kb <= 0 || k <= 0 || rows < 0) return GW_ERR_INVALID_ARG;
  if (rows == 0) return GW_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>((rows + kMergeWarps - 1) / kMergeWarps);
  switch (dtype) {
    case GW_F32:
      merge_two_topk_kernel<float><<<grid, kMergeWarps * 32, 0, st>>>(
          static_cast<const float*>(a_scores), a_idx, ka, static_cast<const float*>(b_scores), b_pos, kb, b_start, rows,
          k, static_cast<float*>(out_scores), out_idx);
      break;
    case GW_BF16:
      merge_two_topk_kernel<__nv_bfloat16><<<grid, kMergeWarps * 32, 0, st>>>(
          static_cast<const __nv_bfloat16*>(a_scores), a_idx, ka, static_cast<const __nv_bfloat16*>(b_scores), b_pos,
          kb, b_start, rows, k, static_cast<__nv_bfloat16*>(out_scores), out_idx);
      break;
    case GW_F16:
      merge_two_topk_kernel<__half><<<grid, kMergeWarps * 32, 0, st>>>(
          static_cast<const __half*>(a_scores), a_idx, ka, static_cast<const __half*>(b_scores), b_pos, kb, b_start,
          rows, k, static_cast<__half*>(out_scores), out_idx);
      break;
    default:
      return GW_ERR_UNSUPPORTED;
  }
  GW_LAUNCH_CHECK();
  return GW_OK;
}

extern "C" const char* gw_strerror(int code) {
  switch (code) {
    case GW_OK: return "ok";
    case GW_ERR_INVALID_ARG: return "invalid argument (null pointer, bad size, misaligned pointer or stride)";
    case GW_ERR_UNSUPPORTED: return "unsupported shape or dtype (this library has no fallback path)";
    case GW_ERR_WORKSPACE: return "workspace too small";
    case GW_ERR_CUDA: return "CUDA call failed (see gw_last_cuda_error)";
    case GW_ERR_TIMEOUT: return "a bounded wait inside a kernel ran out";
    case GW_ERR_NO_SM100: return "device is not compute capability 10.x";
    case GW_ERR_TOO_LARGE: return "problem exceeds the fixed capacity of a no-allocation entry point";
    case GW_ERR_INTERNAL: return "a kernel found its own bookkeeping inconsistent and skipped the work";
    default: return "unknown geoweave_b200 status";
  }
}
extern "C" int gw_last_cuda_error(void) { return gw::g_last_cuda_error; }
extern "C" int gw_abi_version(void) { return 2; }
extern "C" int gw_device_cache_reset(void) {
  gw::g_cache_epoch.fetch_add(1u, std::memory_order_acq_rel);
  return GW_OK;
}
