// Diagnostics that are not part of the data path.
//
// gw_debug_bounded_wait_selftest shows the way every kernel of this library leaves a wait that can never be
// satisfied: one warp of a tiny kernel waits on an mbarrier nobody arrives at, with the limit given by the
// caller (milliseconds instead of the ~2 s of the real pipelines); when the limit passes, the warp records
// GW_ERR_TIMEOUT in the caller's status word and the kernel returns normally.  No trap, no fault, no endless
// loop: the context stays usable and the next call works.
#include "gw_common.cuh"

namespace gw {
namespace {

__global__ void bounded_wait_selftest_kernel(unsigned long long limit_ns, int* status, unsigned long long* waited_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const unsigned long long t0 = global_timer_ns();
    const bool ok = mbar_wait_limit(&bar, 0u, limit_ns);  // phase 0 never completes: no thread arrives
    if (threadIdx.x == 0) {
      if (waited_ns != nullptr) *waited_ns = global_timer_ns() - t0;
      if (!ok) report_status(status, GW_ERR_TIMEOUT);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// The gather of the sparse attention without its arithmetic: the same bulk copies (one per selected K row and
// one per V row, straight into shared memory, about 190 KB in flight per SM), nothing else.  Its rate on a given
// index list is the ceiling the attention kernel can reach on that list with this copy method -- the L2-to-SM
// path when K and V fit the L2, HBM when they do not.
// ---------------------------------------------------------------------------------------------
constexpr int GR_WARPS = 4;      // issuing warps per CTA
constexpr int GR_DEPTH = 3;      // slots per warp
constexpr int GR_KEYS = 4;       // keys per slot (a K row and a V row each)
constexpr int GR_MAX_ROW = 2048; // bytes per row

__global__ void __launch_bounds__(GR_WARPS * 32, 1)
gather_rate_kernel(const unsigned char* __restrict__ kbase, const unsigned char* __restrict__ vbase, const int32_t* __restrict__ pos,
                   int64_t T, int S, int K, int row_bytes, int64_t k_stride, int64_t v_stride, int* status) {
  extern __shared__ __align__(128) unsigned char gr_smem[];
  __shared__ uint64_t bars[GR_WARPS * GR_DEPTH];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0)
    for (int d = 0; d < GR_DEPTH; ++d) mbar_init(&bars[warp * GR_DEPTH + d], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  unsigned char* ring = gr_smem + static_cast<size_t>(warp) * GR_DEPTH * GR_KEYS * 2 * GR_MAX_ROW;
  const int per_warp = (K + GR_WARPS - 1) / GR_WARPS;
  const int j_begin = warp * per_warp, j_end = min(K, j_begin + per_warp);
  const int rounds_per_query = (per_warp + GR_KEYS - 1) / GR_KEYS;
  const int64_t my_queries = T > blockIdx.x ? (T - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int64_t rounds = my_queries * rounds_per_query;
  bool ok = true;
  for (int64_t r = 0; r < rounds + GR_DEPTH && ok; ++r) {
    const int d = static_cast<int>(r % GR_DEPTH);
    uint64_t* bar = &bars[warp * GR_DEPTH + d];
    if (r >= GR_DEPTH) ok = mbar_wait_bounded(bar, static_cast<uint32_t>((r / GR_DEPTH) - 1) & 1u);
    ok = __all_sync(0xffffffffu, ok);
    if (ok && r < rounds) {
      const int64_t t = blockIdx.x + (r / rounds_per_query) * gridDim.x;
      const int j = j_begin + static_cast<int>(r % rounds_per_query) * GR_KEYS + (lane >> 1);
      int p = -1;
      if (lane < 2 * GR_KEYS && j < j_end) p = pos[t * K + j];
      const bool valid = p >= 0 && p < S;
      const int n = __popc(__ballot_sync(0xffffffffu, valid));
      if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(n) * row_bytes);
      __syncwarp();
      if (valid) {
        const unsigned char* src = (lane & 1) ? vbase + static_cast<int64_t>(p) * v_stride : kbase + static_cast<int64_t>(p) * k_stride;
        bulk_g2s(ring + (d * GR_KEYS * 2 + lane) * GR_MAX_ROW, src, row_bytes, bar);
      }
    }
  }
  if (!ok && lane == 0) report_status(status, GW_ERR_TIMEOUT);
}

// The same gather with plain 16-byte loads instead of bulk copies (rows of 2 KB, two keys per warp step, sixteen loads in
// flight per lane): the rate of the L2 -> SM path itself, to tell a limit of the copy unit from a limit of the L2.
__global__ void __launch_bounds__(1024, 1) gather_rate_ldg_kernel(const uint4* __restrict__ k, const uint4* __restrict__ v,
                                                                  const int32_t* __restrict__ pos, long long T, int S, int K,
                                                                  unsigned* sink) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  unsigned acc = 0;
  for (long long q = blockIdx.x; q < T; q += gridDim.x) {
    const int32_t* p = pos + q * K;
    for (int j = warp * 2; j + 1 < K; j += nw * 2) {
      const uint32_t a = static_cast<uint32_t>(p[j]) < static_cast<uint32_t>(S) ? p[j] : 0;
      const uint32_t b = static_cast<uint32_t>(p[j + 1]) < static_cast<uint32_t>(S) ? p[j + 1] : 0;
      const uint4* ka = k + static_cast<long long>(a) * 128;
      const uint4* va = v + static_cast<long long>(a) * 128;
      const uint4* kb = k + static_cast<long long>(b) * 128;
      const uint4* vb = v + static_cast<long long>(b) * 128;
      uint4 r[16];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        r[i] = ka[i * 32 + lane];
        r[4 + i] = va[i * 32 + lane];
        r[8 + i] = kb[i * 32 + lane];
        r[12 + i] = vb[i * 32 + lane];
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) acc ^= r[i].x ^ r[i].y ^ r[i].z ^ r[i].w;
    }
  }
  if (acc == 0x9e3779b9u && sink != nullptr) *sink = acc;  // keeps the loads alive; practically never true
}

}  // namespace
}  // namespace gw

extern "C" int gw_debug_gather_rate_ldg(const void* k, const void* v, const int32_t* kv_pos, int64_t T, int S, int K, int max_ctas,
                                        gw_stream_t stream) {
  using namespace gw;
  if (!k || !v || !kv_pos || T < 0 || S <= 0 || K <= 0 || !aligned16(k) || !aligned16(v)) return GW_ERR_INVALID_ARG;
  if (T == 0) return GW_OK;
  int dev = 0;
  DeviceFacts facts;
  int rc = device_facts(&dev, &facts);
  if (rc != GW_OK) return rc;
  int grid = static_cast<int>(T < facts.sms ? T : facts.sms);
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  gather_rate_ldg_kernel<<<grid, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(k), static_cast<const uint4*>(v),
                                                                                   kv_pos, T, S, K, nullptr);
  GW_LAUNCH_CHECK();
  return GW_OK;
}

extern "C" int gw_debug_gather_rate_ctas(const void* k, const void* v, const int32_t* kv_pos, int64_t T, int S, int K, int row_bytes,
                                         int64_t k_row_stride_bytes, int64_t v_row_stride_bytes, int max_ctas, int* status_dev,
                                         gw_stream_t stream);

extern "C" int gw_debug_gather_rate(const void* k, const void* v, const int32_t* kv_pos, int64_t T, int S, int K, int row_bytes,
                                    int64_t k_row_stride_bytes, int64_t v_row_stride_bytes, int* status_dev, gw_stream_t stream) {
  return gw_debug_gather_rate_ctas(k, v, kv_pos, T, S, K, row_bytes, k_row_stride_bytes, v_row_stride_bytes, 0, status_dev, stream);
}

extern "C" int gw_debug_gather_rate_ctas(const void* k, const void* v, const int32_t* kv_pos, int64_t T, int S, int K, int row_bytes,
                                         int64_t k_row_stride_bytes, int64_t v_row_stride_bytes, int max_ctas, int* status_dev,
                                         gw_stream_t stream) {
  using namespace gw;
  if (!k || !v || !kv_pos || T < 0 || S <= 0 || K <= 0) return GW_ERR_INVALID_ARG;
  if (row_bytes <= 0 || row_bytes > GR_MAX_ROW || row_bytes % 16 != 0) return GW_ERR_INVALID_ARG;
  if (!aligned16(k) || !aligned16(v) || k_row_stride_bytes % 16 != 0 || v_row_stride_bytes % 16 != 0) return GW_ERR_INVALID_ARG;
  if (T == 0) return GW_OK;
  int dev = 0;
  DeviceFacts facts;
  int rc = device_facts(&dev, &facts);
  if (rc != GW_OK) return rc;
  constexpr size_t smem = static_cast<size_t>(GR_WARPS) * GR_DEPTH * GR_KEYS * 2 * GR_MAX_ROW;  // 192 KB
  static OncePerDevice once;
  rc = ensure_dynamic_smem(gather_rate_kernel, smem, once, dev);
  if (rc != GW_OK) return rc;
  int grid = static_cast<int>(T < facts.sms ? T : facts.sms);
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;  // fewer CTAs than SMs: how the rate depends on the SMs that gather
  gather_rate_kernel<<<grid, GR_WARPS * 32, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned char*>(k), static_cast<const unsigned char*>(v), kv_pos, T, S, K, row_bytes, k_row_stride_bytes,
      v_row_stride_bytes, status_dev);
  GW_LAUNCH_CHECK();
  return GW_OK;
}

extern "C" int gw_debug_bounded_wait_selftest(unsigned int limit_us, int* status_dev, unsigned long long* waited_ns_dev,
                                              gw_stream_t stream) {
  if (status_dev == nullptr || limit_us == 0 || limit_us > 100000u) return GW_ERR_INVALID_ARG;  // at most 0.1 s
  gw::bounded_wait_selftest_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<unsigned long long>(limit_us) * 1000ull, status_dev, waited_ns_dev);
  GW_LAUNCH_CHECK();
  return GW_OK;
}
