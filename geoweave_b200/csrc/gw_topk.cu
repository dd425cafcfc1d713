// Stage 2 alone: exact top-k of materialised score rows, and the merge of two top-k lists.
// Both are thin drivers around group_select_topk (gw_select.cuh).
#include "gw_common.cuh"
#include "gw_select.cuh"

namespace gw {

thread_local int g_last_cuda_error = 0;

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
    if (os) os[pos] = row[idx];
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

template <typename T>
__global__ void __launch_bounds__(kMergeWarps * 32) merge_two_topk_kernel(const T* a_s, const int32_t* a_i, int ka,
                                                                          const T* b_s, const int64_t* b_p, int kb,
                                                                          int64_t b_start, int64_t rows, int k, T* os,
                                                                          int32_t* oi) {
  __shared__ SelectSmem<kMergeBins> sm[kMergeWarps];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r = static_cast<int64_t>(blockIdx.x) * kMergeWarps + w;
  if (r >= rows) return;
  TwoListSrc<T> src{a_s + r * ka, a_i + r * ka, b_s + r * kb, b_p + r * kb, ka, b_start};
  const int n = ka + kb;
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
  const int got = group_select_topk<32, kMergeBins>(src, n, k, cmin, cmax, sm[w], lane, 0, sink, nullptr);
  for (int p = got + lane; p < k; p += 32) sink(p, 0ull);  // k > ka + kb: pad with empty slots
}

}  // namespace
}  // namespace gw

using namespace gw;

extern "C" int gw_topk_exact(const void* scores, int dtype, int64_t rows, int64_t cols, int64_t row_stride, int k,
                             int32_t* out_idx32, int64_t* out_idx64, void* out_scores, gw_stream_t stream) {
  if (!scores || rows < 0 || cols <= 0 || k <= 0 || row_stride < cols) return GW_ERR_INVALID_ARG;
  if (!out_idx32 && !out_idx64) return GW_ERR_INVALID_ARG;
  if (k > cols || cols > 0x7fffffff || rows > 0x7fffffff) return GW_ERR_INVALID_ARG;
  if (rows == 0) return GW_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(rows);
  switch (dtype) {
    case GW_F32:
      topk_exact_kernel<float><<<grid, kTopkThreads, 0, st>>>(static_cast<const float*>(scores), cols, row_stride, k,
                                                               out_idx32, out_idx64, static_cast<float*>(out_scores));
      break;
    case GW_BF16:
      topk_exact_kernel<__nv_bfloat16><<<grid, kTopkThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(scores), cols,
                                                                       row_stride, k, out_idx32, out_idx64,
                                                                       static_cast<__nv_bfloat16*>(out_scores));
      break;
    case GW_F16:
      topk_exact_kernel<__half><<<grid, kTopkThreads, 0, st>>>(static_cast<const __half*>(scores), cols, row_stride, k,
                                                                out_idx32, out_idx64, static_cast<__half*>(out_scores));
      break;
    default:
      return GW_ERR_UNSUPPORTED;
  }
  GW_LAUNCH_CHECK();
  return GW_OK;
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
    default: return "unknown geoweave_b200 status";
  }
}
extern "C" int gw_last_cuda_error(void) { return gw::g_last_cuda_error; }
extern "C" int gw_abi_version(void) { return 1; }
