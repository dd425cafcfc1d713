// Coarse-to-fine selection around the indexer: the keys the coarse stage ranks ("sources": every special token, every
// patch token outside the pooled region, every 2x2 cell of patches as the mean of its tokens) and the expansion of each
// query's kept sources back to token indices.  The reference does both with torch ops in its caller
// (easyvolcap/official_vggt/layers/dsa_attention.py:3386-3543 avg_pool2d / index_select / cat, :4079-4128 index_select /
// cumsum / argsort / gather); here each is one kernel driven by the same source -> tokens table.
#include "gw_common.cuh"

namespace gw {
namespace {

constexpr int C2F_MAX_WIDTH = 4;      // tokens per source at most (2x2 cells)
constexpr int C2F_MAX_LIST = 4096;    // sources per query at most
constexpr int C2F_MAX_OUT = 4096;     // token indices per query at most
constexpr int C2F_THREADS = 128;

// one warp per source row: mean over the row's tokens of the token's Hi*Di key values and of its Hi weights
template <typename T>
__global__ void __launch_bounds__(256) pool_sources_kernel(const T* __restrict__ k, const T* __restrict__ w,
                                                           const int32_t* __restrict__ table, int width, int N, int L, int Hi,
                                                           int row_elems, T* __restrict__ src_k, T* __restrict__ src_w) {
  constexpr int VEC = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const long long r = blockIdx.x * static_cast<long long>(blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long b = blockIdx.y;
  if (r >= L) return;
  int tok[C2F_MAX_WIDTH];
  int cnt = 0;
  for (int s = 0; s < width; ++s) {
    const int t = table[r * width + s];
    if (t >= 0 && t < N) tok[cnt++] = t;  // slots are filled from the front, in the order the mean is taken
  }
  const float inv = cnt > 0 ? 1.0f / static_cast<float>(cnt) : 0.f;
  const T* kb = k + b * N * row_elems;
  T* ko = src_k + (b * L + r) * row_elems;
  for (int e = lane * VEC; e < row_elems; e += 32 * VEC) {
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
    for (int c = 0; c < cnt; ++c) {
      const uint4 raw = *reinterpret_cast<const uint4*>(kb + static_cast<long long>(tok[c]) * row_elems + e);
      const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] += to_float(v[i]);
    }
    uint4 out;
    T* o = reinterpret_cast<T*>(&out);
#pragma unroll
    for (int i = 0; i < VEC; ++i) o[i] = from_float<T>(acc[i] * inv);
    *reinterpret_cast<uint4*>(ko + e) = out;
  }
  if (w != nullptr && lane < Hi) {
    float acc = 0.f;
    for (int c = 0; c < cnt; ++c) acc += to_float(w[(b * N + tok[c]) * Hi + lane]);
    src_w[(b * L + r) * Hi + lane] = from_float<T>(acc * inv);
  }
}

struct ExpandParams {
  const int32_t* lists;   // [B*T, m]
  const void* scores;     // [B*T, m] of score_dtype, or null: keep the given order
  const int32_t* table;   // [L, width]
  int32_t* out;           // [B*T, out_k]
  int score_dtype, width, L, m, out_k, pad_window, n_tokens;
};

__device__ __forceinline__ float load_score(const void* p, int dtype, long long i) {
  if (dtype == GW_F32) return static_cast<const float*>(p)[i];
  if (dtype == GW_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}

// one CTA per query: order the kept sources by descending score (equal scores: lower source first), then slot 0 of every
// source in that order, slot 1 of every source that has one, ... ; cut to out_k; pad a short list by cycling over its tail
__global__ void __launch_bounds__(C2F_THREADS) expand_sources_kernel(const ExpandParams p) {
  extern __shared__ __align__(16) unsigned char c2f_smem[];
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(c2f_smem);   // [P] composite (score, ~source)
  int P = 1;
  while (P < p.m) P <<= 1;
  int32_t* compact = reinterpret_cast<int32_t*>(keys + P);                     // [out_k] token indices in output order
  __shared__ int warp_count[C2F_THREADS / 32];
  __shared__ int running;
  const long long row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int32_t* list = p.lists + row * p.m;
  for (int i = tid; i < P; i += C2F_THREADS) {
    unsigned long long c = 0ull;  // sentinel: sorts behind every real entry
    if (i < p.m) {
      const int src = list[i];
      // without scores the list keeps its order: the position stands in for the score
      const uint32_t key = p.scores ? score_key(load_score(p.scores, p.score_dtype, row * p.m + i)) : 0xffffffffu - static_cast<uint32_t>(i);
      c = (static_cast<unsigned long long>(key) << 32) | static_cast<uint32_t>(~static_cast<uint32_t>(src));
      if (c == 0ull) c = 1ull;
    }
    keys[i] = c;
  }
  __syncthreads();
  // bitonic sort, descending
  for (int size = 2; size <= P; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < P / 2; i += C2F_THREADS) {
        const int lo = 2 * i - (i & (stride - 1));
        const int hi = lo + stride;
        const bool desc = (lo & size) == 0;
        const unsigned long long a = keys[lo], b = keys[hi];
        if ((a < b) == desc) {
          keys[lo] = b;
          keys[hi] = a;
        }
      }
      __syncthreads();
    }
  }
  if (tid == 0) running = 0;
  __syncthreads();
  // slot-major walk with a running count of the tokens emitted so far
  const int total = p.width * p.m;
  for (int base = 0; base < total; base += C2F_THREADS) {
    const int pos = base + tid;
    int tok = -1;
    if (pos < total) {
      const int s = pos / p.m, i = pos - s * p.m;
      const unsigned long long c = keys[i];
      const int src = static_cast<int>(~static_cast<uint32_t>(c));
      if (c != 0ull && src >= 0 && src < p.L) tok = p.table[static_cast<long long>(src) * p.width + s];
      if (tok >= p.n_tokens) tok = -1;
    }
    const uint32_t ballot = __ballot_sync(0xffffffffu, tok >= 0);
    if (lane == 0) warp_count[warp] = __popc(ballot);
    __syncthreads();
    int before = running;
    for (int wv = 0; wv < warp; ++wv) before += warp_count[wv];
    const int rank = before + __popc(ballot & ((1u << lane) - 1u));
    if (tok >= 0 && rank < p.out_k) compact[rank] = tok;
    __syncthreads();
    if (tid == 0) {
      int add = 0;
      for (int wv = 0; wv < C2F_THREADS / 32; ++wv) add += warp_count[wv];
      running += add;
    }
    __syncthreads();
    if (running >= p.out_k) break;  // uniform: read after the barrier
  }
  const int count = running < p.out_k ? running : p.out_k;
  const int n = count > 0 ? count : 1;
  int win = p.pad_window < p.out_k ? p.pad_window : p.out_k;
  if (win < 1) win = 1;
  if (win > n) win = n;
  const int start = n - win;
  int32_t* out = p.out + row * p.out_k;
  for (int j = tid; j < p.out_k; j += C2F_THREADS) {
    int v;
    if (j < count) v = compact[j];
    else v = count > 0 ? compact[start + (j - n) % win] : -1;
    out[j] = v;
  }
}

}  // namespace
}  // namespace gw

using namespace gw;

extern "C" int gw_pool_sources(const void* k, const void* w, const int32_t* source_to_fine, int dtype, int B, int N, int L, int Hi,
                               int Di, int width, void* src_k, void* src_w, gw_stream_t stream) {
  if (!k || !source_to_fine || !src_k || (w != nullptr) != (src_w != nullptr)) return GW_ERR_INVALID_ARG;  // w is optional
  if (B <= 0 || N <= 0 || L <= 0 || Hi <= 0 || Di <= 0 || B > 65535) return GW_ERR_INVALID_ARG;
  if (width < 1 || width > C2F_MAX_WIDTH || Hi > 32) return GW_ERR_UNSUPPORTED;
  const size_t es = dtype_size(dtype);
  if ((static_cast<size_t>(Hi) * Di * es) % 16 != 0 || !aligned16(k) || !aligned16(src_k)) return GW_ERR_UNSUPPORTED;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const dim3 grid(static_cast<unsigned>((L + 7) / 8), B);
  switch (dtype) {
    case GW_F32:
      pool_sources_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(k), static_cast<const float*>(w), source_to_fine, width,
                                                       N, L, Hi, Hi * Di, static_cast<float*>(src_k), static_cast<float*>(src_w));
      break;
    case GW_BF16:
      pool_sources_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(w),
                                                               source_to_fine, width, N, L, Hi, Hi * Di,
                                                               static_cast<__nv_bfloat16*>(src_k), static_cast<__nv_bfloat16*>(src_w));
      break;
    case GW_F16:
      pool_sources_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(k), static_cast<const __half*>(w), source_to_fine, width,
                                                        N, L, Hi, Hi * Di, static_cast<__half*>(src_k), static_cast<__half*>(src_w));
      break;
    default: return GW_ERR_UNSUPPORTED;
  }
  GW_LAUNCH_CHECK();
  return GW_OK;
}

extern "C" int gw_expand_sources(const int32_t* lists, const void* scores, int score_dtype, const int32_t* source_to_fine, int width,
                                 int L, int n_tokens, long long rows, int m, int out_k, int pad_window, int32_t* out,
                                 gw_stream_t stream) {
  if (!lists || !source_to_fine || !out) return GW_ERR_INVALID_ARG;
  if (rows < 0 || m <= 0 || out_k <= 0 || L <= 0 || n_tokens <= 0 || pad_window <= 0) return GW_ERR_INVALID_ARG;
  if (width < 1 || width > C2F_MAX_WIDTH || m > C2F_MAX_LIST || out_k > C2F_MAX_OUT || rows > 0x7fffffffLL) return GW_ERR_UNSUPPORTED;
  if (scores && score_dtype != GW_F32 && score_dtype != GW_BF16 && score_dtype != GW_F16) return GW_ERR_UNSUPPORTED;
  if (rows == 0) return GW_OK;
  int P = 1;
  while (P < m) P <<= 1;
  const size_t smem = static_cast<size_t>(P) * 8 + static_cast<size_t>(out_k) * 4;
  int dev = 0;
  DeviceFacts facts;
  int rc = device_facts(&dev, &facts);
  if (rc != GW_OK) return rc;
  static OncePerDevice once;
  rc = ensure_dynamic_smem(expand_sources_kernel, static_cast<size_t>(C2F_MAX_LIST) * 8 + static_cast<size_t>(C2F_MAX_OUT) * 4, once, dev);
  if (rc != GW_OK) return rc;
  ExpandParams p;
  p.lists = lists; p.scores = scores; p.table = source_to_fine; p.out = out; p.score_dtype = score_dtype; p.width = width; p.L = L;
  p.m = m; p.out_k = out_k; p.pad_window = pad_window; p.n_tokens = n_tokens;
  expand_sources_kernel<<<static_cast<unsigned>(rows), C2F_THREADS, smem, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  GW_LAUNCH_CHECK();
  return GW_OK;
}
