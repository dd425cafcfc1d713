// Backward of the sparse attention: dQ, dK, dV (and the gradient that arrives through attn_sum), reproducible --
// no floating-point atomics anywhere.
//
//   s[t,h,j] = scale * <q[t,h], K[pos[t,j],h]>      p = exp(s - lse[t,h])      o[t,h] = sum_j p V[pos[t,j],h]
//   attn_sum[t,j] = sum_h p[t,h,j]
//
//   dp'[t,h,j] = <dO[t,h], V[pos[t,j],h]> + d_attn_sum[t,j]
//   delta'[t,h] = sum_j p dp' = <dO[t,h], o[t,h]> + sum_j p[t,h,j] d_attn_sum[t,j]
//   ds = p (dp' - delta') scale
//   dQ[t,h] = sum_j ds K[pos[t,j],h]        dK[s,h] = sum_{(t,j): pos[t,j]=s} ds q[t,h]       dV[s,h] = sum_{...} p dO[t,h]
//
// 16-bit inputs with 8 or 16 heads take the tensor-core kernels of gw_attn_bwd_mma.cuh; everything else (fp32, other head
// counts) takes the two kernels of this file.
//
// Two kernels.  The query kernel (one CTA per query, one warp per head at a time, one lane per selected key)
// gathers the key's K and V slices, forms p and dp', writes both to a scratch of the shape [B,T,H,K], and gets dQ
// in the same pass from two running sums, A = sum p dp' K and Bk = sum p K, since dQ = scale (A - delta' Bk) needs
// delta' only at the end.  The key kernel (one CTA per key, one warp per head) walks the key's (query, slot) pairs --
// given by the caller as the positions of a STABLE sort of the index lists by key, so the order of the sums is
// fixed -- re-reads p, dp' and delta', gathers q and dO of those queries and accumulates dK and dV in registers.
// The reference reaches the same sums with fp32 atomic adds
// (easyvolcap/utils/custom_flash_attn/sparse_index_flash_attn.py:535-1186, 2442-2846) or, opt-in, with a sort-based
// grouped kernel (csrc/sparse_bwd_grouped_kernel.cu:78-603).
#include "gw_common.cuh"
#include "gw_attn_bwd_mma.cuh"

namespace gw {
namespace {

constexpr int BW_D = 64;
constexpr int BQ_WARPS = 8;
constexpr int BQ_MAX_H = 32;
constexpr int BK_MAX_WARPS = 16;

struct BwdParams {
  const void *q, *k, *v, *o, *d_out;
  const int32_t* pos;        // [B,T,K]
  const float* lse;          // [B,H,T] natural log
  const float* d_attn_sum;   // [B,T,K] or null
  const int32_t* key_order;  // [B,T*K] positions t*K + j, stably sorted by key (invalid positions last)
  const int32_t* key_start;  // [B,S+1] first entry of every key in key_order
  float *P, *dP, *delta;     // scratch: [B,T,H,K], [B,T,H,K], [B,T,H]
  void *dq, *dk, *dv;
  int B, T, S, H, K;
  float scale;
};

template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& raw, float (&f)[Vec16<T>::N]) {
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec16<T>::N; ++i) f[i] = to_float(e[i]);
}

template <typename T>
__global__ void __launch_bounds__(BQ_WARPS * 32, 1) attn_bwd_query_kernel(const BwdParams p) {
  constexpr int VN = Vec16<T>::N, CH = BW_D / VN;  // elements per 16-byte piece, pieces per head slice
  extern __shared__ __align__(16) float bq_smem[];
  float* qs = bq_smem;                       // [H][64]
  float* dos = qs + p.H * BW_D;              // [H][64]
  float* red = dos + p.H * BW_D;             // [warps][32][65] transposition buffer for the lane sums
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = blockIdx.x, b = blockIdx.y;
  const int H = p.H, K = p.K;
  const int64_t row = (b * p.T + t) * H;     // first head row of this query in [B,T,H,*] tensors
  const T* q = static_cast<const T*>(p.q) + row * BW_D;
  const T* dO = static_cast<const T*>(p.d_out) + row * BW_D;
  const T* o = static_cast<const T*>(p.o) + row * BW_D;
  for (int i = threadIdx.x; i < H * BW_D; i += blockDim.x) {
    qs[i] = to_float(q[i]);
    dos[i] = to_float(dO[i]);
  }
  __syncthreads();
  float* myred = red + warp * 32 * 65;
  const float log2e = 1.4426950408889634f;
  for (int h = warp; h < H; h += BQ_WARPS) {
    // delta = <dO, o> of this head
    float dl = to_float(dO[h * BW_D + lane]) * to_float(o[h * BW_D + lane]) +
               to_float(dO[h * BW_D + 32 + lane]) * to_float(o[h * BW_D + 32 + lane]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) dl += __shfl_xor_sync(0xffffffffu, dl, d);
    const float lse2 = p.lse[(b * H + h) * static_cast<int64_t>(p.T) + t] * log2e;
    const float sc2 = p.scale * log2e;
    const float* qh = qs + h * BW_D;
    const float* doh = dos + h * BW_D;
    float A[BW_D], Bk[BW_D];
#pragma unroll
    for (int d = 0; d < BW_D; ++d) A[d] = Bk[d] = 0.f;
    float corr = 0.f;
    float* Prow = p.P + (row + h) * K;
    float* dProw = p.dP + (row + h) * K;
    for (int j0 = 0; j0 < K; j0 += 32) {
      const int j = j0 + lane;
      const int pos = j < K ? p.pos[(b * p.T + t) * K + j] : -1;
      const bool valid = pos >= 0 && pos < p.S;
      float pj = 0.f, dpj = 0.f;
      if (valid) {
        const int64_t krow = ((b * p.S + pos) * H + h) * BW_D;
        const uint4* kp = reinterpret_cast<const uint4*>(static_cast<const T*>(p.k) + krow);
        const uint4* vp = reinterpret_cast<const uint4*>(static_cast<const T*>(p.v) + krow);
        uint4 kraw[CH];
#pragma unroll
        for (int c = 0; c < CH; ++c) kraw[c] = kp[c];
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          float kf[VN];
          unpack16<T>(kraw[c], kf);
#pragma unroll
          for (int i = 0; i < VN; ++i) s = fmaf(qh[c * VN + i], kf[i], s);
        }
        pj = exp2f(fmaf(s, sc2, -lse2));
        float dp = 0.f;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          float vf[VN];
          unpack16<T>(vp[c], vf);
#pragma unroll
          for (int i = 0; i < VN; ++i) dp = fmaf(doh[c * VN + i], vf[i], dp);
        }
        float da = 0.f;
        if (p.d_attn_sum != nullptr) da = p.d_attn_sum[(b * p.T + t) * K + j];
        dpj = dp + da;
        corr = fmaf(pj, da, corr);
        const float pdp = pj * dpj;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          float kf[VN];
          unpack16<T>(kraw[c], kf);
#pragma unroll
          for (int i = 0; i < VN; ++i) {
            A[c * VN + i] = fmaf(pdp, kf[i], A[c * VN + i]);
            Bk[c * VN + i] = fmaf(pj, kf[i], Bk[c * VN + i]);
          }
        }
      }
      if (j < K) {
        Prow[j] = pj;
        dProw[j] = dpj;
      }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) corr += __shfl_xor_sync(0xffffffffu, corr, d);
    const float delta = dl + corr;
    // sum A and Bk over the 32 lanes: through shared memory, lane l ends up with dimensions l and l + 32
    float out[2];
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      __syncwarp();
#pragma unroll
      for (int d = 0; d < BW_D; ++d) myred[lane * 65 + d] = which == 0 ? A[d] : Bk[d];
      __syncwarp();
      float s0 = 0.f, s1 = 0.f;
      for (int l = 0; l < 32; ++l) {
        s0 += myred[l * 65 + lane];
        s1 += myred[l * 65 + 32 + lane];
      }
      if (which == 0) {
        out[0] = s0;
        out[1] = s1;
      } else {
        out[0] = p.scale * (out[0] - delta * s0);
        out[1] = p.scale * (out[1] - delta * s1);
      }
    }
    T* dq = static_cast<T*>(p.dq) + (row + h) * BW_D;
    dq[lane] = from_float<T>(out[0]);
    dq[32 + lane] = from_float<T>(out[1]);
    if (lane == 0) p.delta[row + h] = delta;
  }
}

template <typename T>
__global__ void __launch_bounds__(BK_MAX_WARPS * 32) attn_bwd_key_kernel(const BwdParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int64_t s = blockIdx.x, b = blockIdx.y;
  const int H = p.H, K = p.K;
  const int32_t* order = p.key_order + b * static_cast<int64_t>(p.T) * K;
  const int e0 = p.key_start[b * (p.S + 1) + s], e1 = p.key_start[b * (p.S + 1) + s + 1];
  for (int h = warp; h < H; h += nwarps) {
    float dk0 = 0.f, dk1 = 0.f, dv0 = 0.f, dv1 = 0.f;
    for (int e = e0; e < e1; ++e) {
      const int f = order[e];
      const int64_t t = f / K;
      const int j = f - static_cast<int>(t) * K;
      const int64_t row = (b * p.T + t) * H + h;
      const float pv = p.P[row * K + j];
      const float dpv = p.dP[row * K + j];
      const float ds = pv * (dpv - p.delta[row]) * p.scale;
      const T* qr = static_cast<const T*>(p.q) + row * BW_D;
      const T* dor = static_cast<const T*>(p.d_out) + row * BW_D;
      dk0 = fmaf(ds, to_float(qr[lane]), dk0);
      dk1 = fmaf(ds, to_float(qr[32 + lane]), dk1);
      dv0 = fmaf(pv, to_float(dor[lane]), dv0);
      dv1 = fmaf(pv, to_float(dor[32 + lane]), dv1);
    }
    const int64_t krow = ((b * p.S + s) * H + h) * BW_D;
    T* dk = static_cast<T*>(p.dk) + krow;
    T* dv = static_cast<T*>(p.dv) + krow;
    dk[lane] = from_float<T>(dk0);
    dk[32 + lane] = from_float<T>(dk1);
    dv[lane] = from_float<T>(dv0);
    dv[32 + lane] = from_float<T>(dv1);
  }
}

template <typename T>
int launch_bwd(const BwdParams& p, cudaStream_t st) {
  int dev = 0;
  DeviceFacts facts;
  int rc = device_facts(&dev, &facts);
  if (rc != GW_OK) return rc;
  const size_t smem = (static_cast<size_t>(2) * p.H * BW_D + static_cast<size_t>(BQ_WARPS) * 32 * 65) * sizeof(float);
  static OncePerDevice once;
  rc = ensure_dynamic_smem(attn_bwd_query_kernel<T>, (static_cast<size_t>(2) * BQ_MAX_H * BW_D + static_cast<size_t>(BQ_WARPS) * 32 * 65) * sizeof(float),
                           once, dev);
  if (rc != GW_OK) return rc;
  attn_bwd_query_kernel<T><<<dim3(p.T, p.B), BQ_WARPS * 32, smem, st>>>(p);
  GW_LAUNCH_CHECK();
  const int warps = p.H < BK_MAX_WARPS ? p.H : BK_MAX_WARPS;
  attn_bwd_key_kernel<T><<<dim3(p.S, p.B), warps * 32, 0, st>>>(p);
  GW_LAUNCH_CHECK();
  return GW_OK;
}

}  // namespace
}  // namespace gw

using namespace gw;

extern "C" size_t gw_sparse_attn_bwd_workspace_bytes(int B, int T, int H, int K) {
  if (B <= 0 || T <= 0 || H <= 0 || K <= 0) return 0;
  const size_t n = static_cast<size_t>(B) * T * H;
  return round_up(n * K * sizeof(float), 256) * 2 + round_up(n * sizeof(float), 256);
}

extern "C" int gw_sparse_attn_bwd(const void* q, const void* k, const void* v, const int32_t* kv_pos, const void* out, const float* lse,
                                  const void* d_out, const float* d_attn_sum, const int32_t* key_order, const int32_t* key_start,
                                  int dtype, int B, int T, int S, int H, int D, int K, float scale, void* dq, void* dk, void* dv,
                                  void* workspace, size_t workspace_bytes, int* status_dev, gw_stream_t stream) {
  if (!q || !k || !v || !kv_pos || !out || !lse || !d_out || !key_order || !key_start || !dq || !dk || !dv)
    return GW_ERR_INVALID_ARG;
  if (B <= 0 || T < 0 || S <= 0 || H <= 0 || K <= 0 || B > 65535) return GW_ERR_INVALID_ARG;
  if (D != BW_D || H > BQ_MAX_H) return GW_ERR_UNSUPPORTED;
  if (static_cast<int64_t>(T) * K > 0x7fffffff) return GW_ERR_UNSUPPORTED;
  for (const void* ptr : {q, k, v, out, d_out, static_cast<const void*>(dq), static_cast<const void*>(dk), static_cast<const void*>(dv)})
    if (!aligned16(ptr)) return GW_ERR_INVALID_ARG;
  if (T == 0) return GW_OK;
  const size_t need = gw_sparse_attn_bwd_workspace_bytes(B, T, H, K);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return GW_ERR_WORKSPACE;
  const size_t n = static_cast<size_t>(B) * T * H;
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  BwdParams p;
  p.q = q; p.k = k; p.v = v; p.o = out; p.d_out = d_out; p.pos = kv_pos; p.lse = lse; p.d_attn_sum = d_attn_sum;
  p.key_order = key_order; p.key_start = key_start;
  p.P = reinterpret_cast<float*>(ws);
  p.dP = reinterpret_cast<float*>(ws + round_up(n * K * sizeof(float), 256));
  p.delta = reinterpret_cast<float*>(ws + 2 * round_up(n * K * sizeof(float), 256));
  p.dq = dq; p.dk = dk; p.dv = dv; p.B = B; p.T = T; p.S = S; p.H = H; p.K = K; p.scale = scale;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype != GW_F32 && (H == 8 || H == 16) && status_dev != nullptr) {
    BwdMmaParams m;
    m.q = q; m.k = k; m.v = v; m.o = out; m.d_out = d_out; m.pos = kv_pos; m.lse = lse;
    m.d_attn_sum = d_attn_sum; m.delta_extra = p.delta;
    m.key_order = key_order; m.key_start = key_start; m.pds = reinterpret_cast<uint32_t*>(ws);
    m.dq = dq; m.dk = dk; m.dv = dv; m.status = status_dev; m.B = B; m.T = T; m.S = S; m.H = H; m.K = K; m.scale = scale;
    if (dtype == GW_BF16) return H == 16 ? launch_bwd_mma<__nv_bfloat16, 2>(m, st) : launch_bwd_mma<__nv_bfloat16, 1>(m, st);
    return H == 16 ? launch_bwd_mma<__half, 2>(m, st) : launch_bwd_mma<__half, 1>(m, st);
  }
  switch (dtype) {
    case GW_F32: return launch_bwd<float>(p, st);
    case GW_BF16: return launch_bwd<__nv_bfloat16>(p, st);
    case GW_F16: return launch_bwd<__half>(p, st);
    default: return GW_ERR_UNSUPPORTED;
  }
}
