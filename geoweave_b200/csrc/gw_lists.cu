// The (query, slot) pairs of the index lists grouped by key, in a fixed order: what the backward kernels walk.
//   order[b, e] = flat position t*K + j of the e-th pair when the pairs are stably sorted by key (padding entries --
//                 positions outside [0, S) -- sort behind the last key);  start[b, s] = first e of key s, start[b, S] = where
//                 the padding begins.
// A radix sort over only the bits a key can have (the library's device-wide sort, stable by construction), the pair
// number as payload, then one binary search per key for the offsets.  The reference sorts the same pairs with torch.sort in
// its grouped backward (easyvolcap/utils/custom_flash_attn/sparse_index_flash_attn.py:2600-2700, csrc/sparse_bwd_grouped_kernel.cu:78-180).
#include <cub/device/device_radix_sort.cuh>

#include "gw_common.cuh"

namespace gw {
namespace {

__global__ void lists_prepare_kernel(const int32_t* __restrict__ pos, long long n, int S, int32_t* __restrict__ keys, int32_t* __restrict__ vals) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  const int32_t v = pos[i];
  keys[i] = static_cast<uint32_t>(v) < static_cast<uint32_t>(S) ? v : S;
  vals[i] = static_cast<int32_t>(i);
}

// start[s] = number of sorted keys < s, for s = 0..S
__global__ void lists_offsets_kernel(const int32_t* __restrict__ sorted, long long n, int S, int32_t* __restrict__ start) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s > S) return;
  long long lo = 0, hi = n;
  while (lo < hi) {
    const long long mid = (lo + hi) >> 1;
    if (sorted[mid] < s) lo = mid + 1;
    else hi = mid;
  }
  start[s] = static_cast<int32_t>(lo);
}

int key_bits(int S) {
  int bits = 1;
  while ((1ll << bits) <= S) ++bits;  // the largest key is S itself (padding)
  return bits;
}

size_t sort_temp_bytes(long long n, int bits) {
  size_t bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, bytes, static_cast<const int32_t*>(nullptr), static_cast<int32_t*>(nullptr),
                                  static_cast<const int32_t*>(nullptr), static_cast<int32_t*>(nullptr), n, 0, bits);
  return bytes;
}

}  // namespace
}  // namespace gw

using namespace gw;

extern "C" size_t gw_group_by_key_workspace_bytes(int T, int K, int S) {
  if (T <= 0 || K <= 0 || S <= 0) return 0;
  const long long n = static_cast<long long>(T) * K;
  return 3 * round_up(static_cast<size_t>(n) * 4, 256) + round_up(sort_temp_bytes(n, key_bits(S)), 256);
}

extern "C" int gw_group_by_key(const int32_t* kv_pos, int B, int T, int K, int S, int32_t* key_order, int32_t* key_start, void* workspace,
                               size_t workspace_bytes, gw_stream_t stream) {
  if (!kv_pos || !key_order || !key_start || B <= 0 || T < 0 || K <= 0 || S <= 0) return GW_ERR_INVALID_ARG;
  const long long n = static_cast<long long>(T) * K;
  if (n > 0x7fffffffLL) return GW_ERR_UNSUPPORTED;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (n == 0) {
    GW_CUDA_TRY(cudaMemsetAsync(key_start, 0, static_cast<size_t>(B) * (S + 1) * 4, st));
    return GW_OK;
  }
  const int bits = key_bits(S);
  const size_t arr = round_up(static_cast<size_t>(n) * 4, 256);
  size_t temp = sort_temp_bytes(n, bits);
  if (!workspace || workspace_bytes < 3 * arr + round_up(temp, 256) || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return GW_ERR_WORKSPACE;
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  int32_t* keys = reinterpret_cast<int32_t*>(ws);
  int32_t* keys_sorted = reinterpret_cast<int32_t*>(ws + arr);
  int32_t* vals = reinterpret_cast<int32_t*>(ws + 2 * arr);
  void* temp_ptr = ws + 3 * arr;
  for (int b = 0; b < B; ++b) {
    lists_prepare_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(kv_pos + b * n, n, S, keys, vals);
    GW_LAUNCH_CHECK();
    GW_CUDA_TRY(cub::DeviceRadixSort::SortPairs(temp_ptr, temp, keys, keys_sorted, vals, key_order + b * n, n, 0, bits, st));
    lists_offsets_kernel<<<(S + 1 + 255) / 256, 256, 0, st>>>(keys_sorted, n, S, key_start + static_cast<long long>(b) * (S + 1));
    GW_LAUNCH_CHECK();
  }
  return GW_OK;
}
