// Indexer scores for fp32 inputs (the reference's `--backend torch` arithmetic: fp32 q_idx, k_idx, w).
//
//   out[t, s] = sum_h w[s,h] * relu(scale * <q[t,h,:], k[s,h,:]>)          everything fp32
//
// fp32 operands cannot go through the 16-bit tensor-core path without changing the scores, so this is a plain
// FFMA kernel: a CTA owns a 64 x 64 block of (query, key) pairs, walks the heads, stages the head's 64 x Di
// query and key slices in shared memory (transposed, so a thread's four rows are one 16-byte read) and keeps a
// 4 x 4 register tile per thread.  The caller materialises a block of query rows at a time and selects with
// gw_topk_exact, which is exact on these scores.  It is the small-problem path (4 views of the reference's
// CPU-runnable configuration take a fraction of a millisecond); the 16-bit fused kernel is the fast one.
#include "gw_common.cuh"

namespace gw {
namespace {

constexpr int FT = 64;        // queries and keys per CTA tile
constexpr int FD = 64;        // indexer head dimension
constexpr int FTHREADS = 256; // 16 x 16 threads, 4 x 4 outputs each

__global__ void __launch_bounds__(FTHREADS) indexer_scores_f32_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                                      const float* __restrict__ w, int T, int S, int Hi, float scale,
                                                                      int64_t row0, int rows, float* __restrict__ out,
                                                                      int64_t out_stride) {
  __shared__ __align__(16) float qs[FD][FT + 4];  // [d][query]
  __shared__ __align__(16) float ks[FD][FT + 4];  // [d][key]
  const int b = blockIdx.z;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t t0 = row0 + static_cast<int64_t>(blockIdx.y) * FT;  // first query row of the tile (within the batch)
  const int s0 = blockIdx.x * FT;
  const float* qb = q + static_cast<int64_t>(b) * T * Hi * FD;
  const float* kb = k + static_cast<int64_t>(b) * S * Hi * FD;
  const float* wb = w + static_cast<int64_t>(b) * S * Hi;
  float score[4][4] = {};
  for (int h = 0; h < Hi; ++h) {
    __syncthreads();
    // 64 rows x 64 dims each: thread loads float4 pieces, 16 threads per row, 16 rows per pass
    for (int r = threadIdx.x >> 4; r < FT; r += FTHREADS / 16) {
      const int d4 = (threadIdx.x & 15) * 4;
      const int64_t tq = t0 + r;
      float4 vq = make_float4(0.f, 0.f, 0.f, 0.f), vk = vq;
      if (tq < row0 + rows && tq < T) vq = *reinterpret_cast<const float4*>(qb + (tq * Hi + h) * FD + d4);
      if (s0 + r < S) vk = *reinterpret_cast<const float4*>(kb + (static_cast<int64_t>(s0 + r) * Hi + h) * FD + d4);
      qs[d4 + 0][r] = vq.x; qs[d4 + 1][r] = vq.y; qs[d4 + 2][r] = vq.z; qs[d4 + 3][r] = vq.w;
      ks[d4 + 0][r] = vk.x; ks[d4 + 1][r] = vk.y; ks[d4 + 2][r] = vk.z; ks[d4 + 3][r] = vk.w;
    }
    __syncthreads();
    float acc[4][4] = {};
#pragma unroll 8
    for (int d = 0; d < FD; ++d) {
      const float4 a = *reinterpret_cast<const float4*>(&qs[d][ty * 4]);
      const float4 c = *reinterpret_cast<const float4*>(&ks[d][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, cv[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], cv[j], acc[i][j]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int s = s0 + tx * 4 + j;
      const float wv = s < S ? wb[static_cast<int64_t>(s) * Hi + h] : 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) score[i][j] = fmaf(fmaxf(acc[i][j] * scale, 0.f), wv, score[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t t = t0 + ty * 4 + i;
    if (t >= row0 + rows || t >= T) continue;
    float* orow = out + (static_cast<int64_t>(b) * rows + (t - row0)) * out_stride;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int s = s0 + tx * 4 + j;
      if (s < S) orow[s] = score[i][j];
    }
  }
}

}  // namespace
}  // namespace gw

extern "C" int gw_indexer_scores_f32(const float* q_idx, const float* k_idx, const float* w, int B, int T, int S, int Hi, int Di,
                                     float scale, int64_t row_begin, int rows, float* out, int64_t out_row_stride,
                                     gw_stream_t stream) {
  if (!q_idx || !k_idx || !w || !out || B <= 0 || T <= 0 || S <= 0 || Hi <= 0 || rows < 0 || row_begin < 0) return GW_ERR_INVALID_ARG;
  if (Di != gw::FD) return GW_ERR_UNSUPPORTED;
  if (row_begin + rows > T || out_row_stride < S) return GW_ERR_INVALID_ARG;
  if (!gw::aligned16(q_idx) || !gw::aligned16(k_idx)) return GW_ERR_INVALID_ARG;
  if (B > 65535) return GW_ERR_UNSUPPORTED;
  if (rows == 0) return GW_OK;
  const dim3 grid((S + gw::FT - 1) / gw::FT, (rows + gw::FT - 1) / gw::FT, B);
  if (grid.y > 65535u) return GW_ERR_UNSUPPORTED;
  gw::indexer_scores_f32_kernel<<<grid, gw::FTHREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      q_idx, k_idx, w, T, S, Hi, scale, row_begin, rows, out, out_row_stride);
  GW_LAUNCH_CHECK();
  return GW_OK;
}
