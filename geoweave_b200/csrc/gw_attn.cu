// Stage 3: sparse attention over the selected keys.  HBM/L2-gather bound: per query, K selected keys are
// fetched as whole token rows (all heads of a token are adjacent, and all heads of a query share one index
// list, so one row serves G heads), staged in shared memory by bulk (TMA) copies, and consumed by one warp
// per query with an online softmax in fp32.
//
// Work split: one warp = one query (x one group of G heads); lane l owns head l / (32/G) of the group and a
// contiguous D*G/32-element slice of it, both for the q.K dot product (finished by an xor-shuffle over the
// lanes of the head) and for the p.V accumulation.  Each warp runs its own NST-deep ring of one-key stages
// (K row slice + V row slice) with one mbarrier per stage, so there is no CTA-wide synchronisation at all.
#include <math.h>
#include <stdlib.h>

#include "gw_common.cuh"

namespace gw {
namespace {

template <int WORDS> struct WordVec;
template <> struct WordVec<4> { using type = uint4; };
template <> struct WordVec<2> { using type = uint2; };
template <> struct WordVec<1> { using type = uint32_t; };

template <int WORDS>
__device__ __forceinline__ void load_words(const void* p, uint32_t (&w)[WORDS]) {
  using V = typename WordVec<WORDS>::type;
  const V v = *reinterpret_cast<const V*>(p);
  if constexpr (WORDS == 4) { w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; }
  else if constexpr (WORDS == 2) { w[0] = v.x; w[1] = v.y; }
  else { w[0] = v; }
}
template <int WORDS>
__device__ __forceinline__ void store_words(void* p, const uint32_t (&w)[WORDS]) {
  using V = typename WordVec<WORDS>::type;
  V v;
  if constexpr (WORDS == 4) { v.x = w[0]; v.y = w[1]; v.z = w[2]; v.w = w[3]; }
  else if constexpr (WORDS == 2) { v.x = w[0]; v.y = w[1]; }
  else { v = w[0]; }
  *reinterpret_cast<V*>(p) = v;
}

// words of one chunk -> floats
template <typename T, int WORDS, int EPC>
__device__ __forceinline__ void chunk_to_float(const uint32_t (&w)[WORDS], float (&f)[EPC]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < WORDS; ++i) f[i] = __uint_as_float(w[i]);
  } else {
#pragma unroll
    for (int i = 0; i < WORDS; ++i) unpack2<T>(w[i], f[2 * i], f[2 * i + 1]);
  }
}
template <typename T, int WORDS, int EPC>
__device__ __forceinline__ void float_to_chunk(const float (&f)[EPC], uint32_t (&w)[WORDS]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < WORDS; ++i) w[i] = __float_as_uint(f[i]);
  } else {
#pragma unroll
    for (int i = 0; i < WORDS; ++i) {
      const T lo = from_float<T>(f[2 * i]);
      const T hi = from_float<T>(f[2 * i + 1]);
      w[i] = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&lo)) |
             (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&hi)) << 16);
    }
  }
}

struct AttnParams {
  const void* q;
  const void* k;
  const void* v;
  const int32_t* pos;
  void* out;
  float* lse;       // [B,H,T]
  float* attn_sum;  // [B,T,K]
  int* status;
  int64_t qs_b, qs_t, qs_h, ks_b, ks_t, ks_h, vs_b, vs_t, vs_h, os_b, os_t, os_h;
  int B, T, S, H, K;
  float scale_log2;  // softmax scale * log2(e)
  int kv_heads_contiguous;  // head stride == D for both k and v: one bulk copy per row slice
};

constexpr float kRescaleSlack = 8.0f;  // log2 units: the running reference max is raised only past this

// MODE 0: forward (out, lse).  MODE 1: attn_sum pass (reads lse, gathers K only).
template <typename T, int D, int G, int WARPS, int NST, int MODE>
__global__ void __launch_bounds__(WARPS * 32) sparse_attn_kernel(const AttnParams p) {
  constexpr int LPH = 32 / G;                      // lanes per head
  constexpr int EPL = D / LPH;                     // elements per lane
  constexpr int BPL = EPL * sizeof(T);             // bytes per lane
  constexpr int CHB = BPL >= 16 ? 16 : BPL;        // bytes per chunk
  constexpr int WORDS = CHB / 4;
  constexpr int CPL = BPL / CHB;                   // chunks per lane
  constexpr int EPC = CHB / sizeof(T);             // elements per chunk
  constexpr int SEG = G * D * sizeof(T);           // bytes of one tensor's row slice
  constexpr int NT = (MODE == 0) ? 2 : 1;          // tensors staged per key
  constexpr int STAGE = NT * SEG;
  static_assert(BPL >= 4 && (BPL % CHB) == 0 && SEG % 16 == 0, "unsupported head geometry");
  static_assert((NST & (NST - 1)) == 0, "ring depth must be a power of two");

  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char* ring = smem_raw + static_cast<size_t>(w) * NST * STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + static_cast<size_t>(WARPS) * NST * STAGE) + w * NST;

  const int t = blockIdx.x * WARPS + w;
  const int hg = blockIdx.y;  // head group
  const int b = blockIdx.z;
  if (t >= p.T) return;
  const int h0 = hg * G;
  const int head_local = lane / LPH;
  const int part = lane % LPH;
  // chunk rotation: the 8 lanes of a shared-memory wavefront hit 8 different 16-byte bank groups
  constexpr int RDIV = (CPL >= 8) ? 1 : (8 / CPL);
  const int rot = (lane / RDIV) % CPL;

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NST; ++s) mbar_init(&bars[s], 1);
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  __syncwarp();

  // query slice, pre-scaled, held in the lane's rotated chunk order
  float qf[EPL];
  {
    const T* qp = static_cast<const T*>(p.q) + b * p.qs_b + static_cast<int64_t>(t) * p.qs_t +
                  static_cast<int64_t>(h0 + head_local) * p.qs_h + part * EPL;
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
      const int c = (i + rot) % CPL;
      uint32_t wds[WORDS];
      load_words<WORDS>(qp + c * EPC, wds);
      float f[EPC];
      chunk_to_float<T, WORDS, EPC>(wds, f);
#pragma unroll
      for (int e = 0; e < EPC; ++e) qf[i * EPC + e] = f[e] * p.scale_log2;
    }
  }

  const int32_t* pos = p.pos + (static_cast<int64_t>(b) * p.T + t) * p.K;
  const unsigned char* kbase = static_cast<const unsigned char*>(p.k) + (b * p.ks_b + static_cast<int64_t>(h0) * p.ks_h) * sizeof(T);
  const unsigned char* vbase = static_cast<const unsigned char*>(p.v) + (b * p.vs_b + static_cast<int64_t>(h0) * p.vs_h) * sizeof(T);
  const int K = p.K;
  const uint32_t S = static_cast<uint32_t>(p.S);

  // stage refill: an invalid (padding) key still completes its phase so parities stay in step
  auto issue = [&](int s, int id) {
    const bool valid = static_cast<uint32_t>(id) < S;
    unsigned char* dst = ring + s * STAGE;
    if (lane == 0) {
      if (valid) mbar_arrive_expect_tx(&bars[s], STAGE);
      else mbar_arrive(&bars[s]);
    }
    if (!valid) return;
    if (p.kv_heads_contiguous) {
      if (lane == 0) {
        bulk_g2s(dst, kbase + static_cast<int64_t>(id) * p.ks_t * sizeof(T), SEG, &bars[s]);
        if (MODE == 0) bulk_g2s(dst + SEG, vbase + static_cast<int64_t>(id) * p.vs_t * sizeof(T), SEG, &bars[s]);
      }
    } else {
      __syncwarp();  // the expect_tx is posted before any completion can be counted
      if (lane < G) {
        bulk_g2s(dst + lane * D * sizeof(T), kbase + (static_cast<int64_t>(id) * p.ks_t + lane * p.ks_h) * sizeof(T),
                 D * sizeof(T), &bars[s]);
        if (MODE == 0)
          bulk_g2s(dst + SEG + lane * D * sizeof(T), vbase + (static_cast<int64_t>(id) * p.vs_t + lane * p.vs_h) * sizeof(T),
                   D * sizeof(T), &bars[s]);
      }
    }
  };

  float acc[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) acc[i] = 0.f;
  float m_ref = -INFINITY, l_sum = 0.f;
  float lse2 = 0.f;  // MODE 1: log2-domain lse of this lane's head
  if (MODE == 1) {
    const float nat = p.lse[(static_cast<int64_t>(b) * p.H + h0 + head_local) * p.T + t];
    lse2 = nat * 1.4426950408889634f;
  }
  float* asum = (MODE == 1) ? p.attn_sum + (static_cast<int64_t>(b) * p.T + t) * K : nullptr;

  int cur = (lane < K) ? pos[lane] : -1;
  int nxt = -1;
  for (int s = 0; s < NST && s < K; ++s) issue(s, __shfl_sync(0xffffffffu, cur, s));

  bool timed_out = false;
  for (int base = 0; base < K && !timed_out; base += 32) {
    nxt = (base + 32 + lane < K) ? pos[base + 32 + lane] : -1;
    const int lim = (K - base) < 32 ? (K - base) : 32;
    for (int j0 = 0; j0 < lim; j0 += NST) {
#pragma unroll
      for (int s = 0; s < NST; ++s) {
        const int jj = j0 + s;
        if (jj >= lim) break;
        const int g = base + jj;
        const int id = __shfl_sync(0xffffffffu, cur, jj);
        const bool valid = static_cast<uint32_t>(id) < S;
        const uint32_t parity = static_cast<uint32_t>(g / NST) & 1u;
        if (!mbar_wait_bounded(&bars[s], parity)) { timed_out = true; break; }
        if (valid) {
          const unsigned char* kp = ring + s * STAGE + lane * BPL;
          float dot = 0.f;
#pragma unroll
          for (int i = 0; i < CPL; ++i) {
            const int c = (i + rot) % CPL;
            uint32_t wds[WORDS];
            load_words<WORDS>(kp + c * CHB, wds);
            float f[EPC];
            chunk_to_float<T, WORDS, EPC>(wds, f);
#pragma unroll
            for (int e = 0; e < EPC; ++e) dot = fmaf(qf[i * EPC + e], f[e], dot);
          }
#pragma unroll
          for (int d = LPH / 2; d > 0; d >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, d);
          if (MODE == 0) {
            if (dot > m_ref + kRescaleSlack) {
              const float alpha = exp2f(m_ref - dot);  // 0 on the first key
              l_sum *= alpha;
#pragma unroll
              for (int i = 0; i < EPL; ++i) acc[i] *= alpha;
              m_ref = dot;
            }
            const float pj = exp2f(dot - m_ref);
            l_sum += pj;
            const unsigned char* vp = kp + SEG;
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
              const int c = (i + rot) % CPL;
              uint32_t wds[WORDS];
              load_words<WORDS>(vp + c * CHB, wds);
              float f[EPC];
              chunk_to_float<T, WORDS, EPC>(wds, f);
#pragma unroll
              for (int e = 0; e < EPC; ++e) acc[i * EPC + e] = fmaf(pj, f[e], acc[i * EPC + e]);
            }
          } else {
            // probability of this key under every head of the group, summed over the group's heads
            float pj = (part == 0) ? exp2f(dot - lse2) : 0.f;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) pj += __shfl_xor_sync(0xffffffffu, pj, d);
            if (lane == 0) {
              if (gridDim.y == 1) asum[g] = pj;
              else atomicAdd(&asum[g], pj);
            }
          }
        } else if (MODE == 1 && lane == 0 && gridDim.y == 1) {
          asum[g] = 0.f;
        }
        // refill this stage with the key NST ahead
        const int g2 = g + NST;
        if (g2 < K) {
          const int j2 = jj + NST;
          const int id2 = __shfl_sync(0xffffffffu, (j2 < 32) ? cur : nxt, j2 & 31);
          __syncwarp();
          fence_proxy_async_smem();
          issue(s, id2);
        }
      }
      if (timed_out) break;
    }
    cur = nxt;
  }
  if (timed_out) {
    report_status(p.status, GW_ERR_TIMEOUT);
    // give copies still in flight a bounded chance to land before the CTA's shared memory is released
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 1000000ull) {
    }
    return;
  }

  if (MODE == 0) {
    const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.f;
    T* op = static_cast<T*>(p.out) + b * p.os_b + static_cast<int64_t>(t) * p.os_t +
            static_cast<int64_t>(h0 + head_local) * p.os_h + part * EPL;
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
      const int c = (i + rot) % CPL;
      float f[EPC];
#pragma unroll
      for (int e = 0; e < EPC; ++e) f[e] = acc[i * EPC + e] * inv;
      uint32_t wds[WORDS];
      float_to_chunk<T, WORDS, EPC>(f, wds);
      store_words<WORDS>(op + c * EPC, wds);
    }
    if (p.lse != nullptr && part == 0) {
      const float nat = l_sum > 0.f ? (m_ref + log2f(l_sum)) * 0.6931471805599453f : -INFINITY;
      p.lse[(static_cast<int64_t>(b) * p.H + h0 + head_local) * p.T + t] = nat;
    }
  }
}

}  // namespace
}  // namespace gw
#include "gw_attn_mma.cuh"
namespace gw {
namespace {

template <typename T, int D, int G, int MODE>
int launch_attn(const AttnParams& p, cudaStream_t st) {
  constexpr int SEG = G * D * sizeof(T);
  constexpr int NST = 4;
  constexpr int NTENS = (MODE == 0) ? 2 : 1;
  constexpr int BUDGET = 192 * 1024;
  constexpr int W0 = BUDGET / (NST * NTENS * SEG);
  constexpr int WARPS = W0 > 16 ? 16 : (W0 < 1 ? 1 : W0);
  constexpr size_t SMEM = static_cast<size_t>(WARPS) * NST * NTENS * SEG + static_cast<size_t>(WARPS) * NST * 8;
  auto kern = sparse_attn_kernel<T, D, G, WARPS, NST, MODE>;
  int dev = 0;
  DeviceFacts facts;
  int rc = device_facts(&dev, &facts);
  if (rc != GW_OK) return rc;
  static OncePerDevice smem_once;
  rc = ensure_dynamic_smem(kern, SMEM, smem_once, dev);
  if (rc != GW_OK) return rc;
  dim3 grid((p.T + WARPS - 1) / WARPS, p.H / G, p.B);
  kern<<<grid, WARPS * 32, SMEM, st>>>(p);
  GW_LAUNCH_CHECK();
  return GW_OK;
}

template <typename T, int D, int MODE>
int dispatch_g(const AttnParams& p, int G, cudaStream_t st) {
  switch (G) {
    case 16: return launch_attn<T, D, 16, MODE>(p, st);
    case 8: return launch_attn<T, D, 8, MODE>(p, st);
    case 4: return launch_attn<T, D, 4, MODE>(p, st);
    case 2: return launch_attn<T, D, 2, MODE>(p, st);
    default: return GW_ERR_UNSUPPORTED;
  }
}
template <typename T, int MODE>
int dispatch_d(const AttnParams& p, int D, int G, cudaStream_t st) {
  switch (D) {
    case 32: return dispatch_g<T, 32, MODE>(p, G, st);
    case 64: return dispatch_g<T, 64, MODE>(p, G, st);
    case 128: return dispatch_g<T, 128, MODE>(p, G, st);
    default: return GW_ERR_UNSUPPORTED;
  }
}
template <int MODE>
int dispatch_t(const AttnParams& p, int dtype, int D, int G, cudaStream_t st) {
  switch (dtype) {
    case GW_BF16: return dispatch_d<__nv_bfloat16, MODE>(p, D, G, st);
    case GW_F16: return dispatch_d<__half, MODE>(p, D, G, st);
    case GW_F32: return dispatch_d<float, MODE>(p, D, G, st);
    default: return GW_ERR_UNSUPPORTED;
  }
}

}  // namespace
}  // namespace gw

using namespace gw;

extern "C" int gw_sparse_attn_fwd(const void* q, const void* k, const void* v, const int32_t* kv_pos, int dtype, int B,
                                  int T, int S, int H, int D, int K, const int64_t q_strides[3],
                                  const int64_t k_strides[3], const int64_t v_strides[3], float scale, void* out,
                                  const int64_t out_strides[3], float* lse, float* attn_sum, int* status_dev,
                                  gw_stream_t stream) {
  if (!q || !k || !v || !kv_pos || !out || !q_strides || !k_strides || !v_strides || !out_strides)
    return GW_ERR_INVALID_ARG;
  if (B <= 0 || T < 0 || S <= 0 || H <= 0 || D <= 0 || K <= 0) return GW_ERR_INVALID_ARG;
  if (T == 0) return GW_OK;
  if (attn_sum != nullptr && lse == nullptr) return GW_ERR_INVALID_ARG;  // the second pass needs the lse
  const size_t es = dtype_size(dtype);
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return GW_ERR_INVALID_ARG;
  for (int i = 0; i < 3; ++i) {
    if ((q_strides[i] * es) % 16 || (k_strides[i] * es) % 16 || (v_strides[i] * es) % 16 || (out_strides[i] * es) % 16)
      return GW_ERR_INVALID_ARG;
  }
  // head group: the largest of 16/8/4/2 that divides H
  int G = 0;
  for (int g : {16, 8, 4, 2})
    if (H % g == 0) { G = g; break; }
  if (G == 0) return GW_ERR_UNSUPPORTED;
  if (static_cast<size_t>(D) * G * es / 32 < 4) return GW_ERR_UNSUPPORTED;
  if (B > 65535 || H / G > 65535) return GW_ERR_UNSUPPORTED;

  AttnParams p;
  p.q = q; p.k = k; p.v = v; p.pos = kv_pos; p.out = out; p.lse = lse; p.attn_sum = attn_sum; p.status = status_dev;
  p.qs_b = q_strides[0]; p.qs_t = q_strides[1]; p.qs_h = q_strides[2];
  p.ks_b = k_strides[0]; p.ks_t = k_strides[1]; p.ks_h = k_strides[2];
  p.vs_b = v_strides[0]; p.vs_t = v_strides[1]; p.vs_h = v_strides[2];
  p.os_b = out_strides[0]; p.os_t = out_strides[1]; p.os_h = out_strides[2];
  p.B = B; p.T = T; p.S = S; p.H = H; p.K = K;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.kv_heads_contiguous = (k_strides[2] == D && v_strides[2] == D) ? 1 : 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // 16-bit token-major rows of up to 2 KB go to the tensor-core kernel, everything else to the scalar one
  const bool use_mma = dtype != GW_F32 && D == 64 && (H == 8 || H == 16) && p.kv_heads_contiguous;
  int rc;
  bool sum_done = false;
  if (use_mma) {
    // attn_sum comes out of the same kernel when the query's logits fit its shared-memory buffer
    sum_done = attn_sum != nullptr && K <= AM_SUM_MAXK;
    if (sum_done) {
      if (dtype == GW_BF16) rc = (H == 16) ? launch_attn_mma<__nv_bfloat16, 2, true>(p, st) : launch_attn_mma<__nv_bfloat16, 1, true>(p, st);
      else rc = (H == 16) ? launch_attn_mma<__half, 2, true>(p, st) : launch_attn_mma<__half, 1, true>(p, st);
    } else {
      if (dtype == GW_BF16) rc = (H == 16) ? launch_attn_mma<__nv_bfloat16, 2, false>(p, st) : launch_attn_mma<__nv_bfloat16, 1, false>(p, st);
      else rc = (H == 16) ? launch_attn_mma<__half, 2, false>(p, st) : launch_attn_mma<__half, 1, false>(p, st);
    }
  } else {
    rc = dispatch_t<0>(p, dtype, D, G, st);
  }
  if (rc != GW_OK) return rc;
  if (attn_sum != nullptr && !sum_done) {
    if (H / G > 1) GW_CUDA_TRY(cudaMemsetAsync(attn_sum, 0, sizeof(float) * static_cast<size_t>(B) * T * K, st));
    rc = dispatch_t<1>(p, dtype, D, G, st);
  }
  return rc;
}
