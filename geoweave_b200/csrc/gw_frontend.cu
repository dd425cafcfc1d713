// Projection front-end: from the output of the fused linear layer to the operands of the indexer and of the
// sparse attention, in one pass over HBM.
//
// A token's row of the linear layer's output holds [q | k | v | idx_q | idx_k | idx_w] (3*H*64 + 2*Hi*64 + Hi
// values).  One warp takes one token and works on four heads at a time: eight lanes per head, eight
// consecutive elements per lane (one 16-byte load and store for 16-bit types).  LayerNorm over a head is two
// reductions over its eight lanes (three shuffle steps each), and the partner of an element in the 2-D rotary
// embedding (16 columns away inside the y half or the x half of the head) sits two lanes over.  q and k:
// LayerNorm, rotary; v: copy; idx_q: rotary; idx_k: LayerNorm, rotary; idx_w: copy.  Outputs are token-major
// and contiguous -- the layout the two operators read -- so the transposes and .contiguous() copies between
// the reference's projection and its operator calls have no counterpart here.  Arithmetic is fp32, rounded
// once on the way out.
#include "gw_common.cuh"

namespace gw {
namespace {

constexpr int FE_WARPS = 8;

// Eight consecutive elements, to and from fp32.  Outputs, tables and parameters are 16-byte aligned; a row of the
// linear layer's output need not be (3588 bf16 values are 7176 bytes), so rows are read in two 8-byte halves
// when `al16` is false.
__device__ __forceinline__ void load8(const float* p, float (&x)[8], bool al16 = true) {
  if (al16) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = *reinterpret_cast<const float2*>(p + 2 * i);
      x[2 * i] = a.x;
      x[2 * i + 1] = a.y;
    }
  }
}
__device__ __forceinline__ void store8(float* p, const float (&x)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(x[4], x[5], x[6], x[7]);
}
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&x)[8], bool al16 = true) {
  uint4 raw;
  if (al16) {
    raw = *reinterpret_cast<const uint4*>(p);
  } else {
    const uint2 lo = *reinterpret_cast<const uint2*>(p), hi = *reinterpret_cast<const uint2*>(p + 4);
    raw = make_uint4(lo.x, lo.y, hi.x, hi.y);
  }
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) x[i] = to_float(e[i]);
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&x)[8]) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) e[i] = from_float<T>(x[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

struct FeParams {
  const void* fused;
  int64_t tokens, ld;
  int H, Hi;
  const int64_t* pos;  // [tokens, 2] (y, x), or null: no rotary embedding
  const float *cos_tab, *sin_tab;
  int table_rows;
  const float *qn_w, *qn_b, *kn_w, *kn_b, *in_w, *in_b;  // LayerNorm weight / bias per kind, null = no LayerNorm
  float qn_eps, kn_eps, in_eps;
  void *q, *k, *v, *q_idx, *k_idx, *w;
  int* status;
};

// sum over the eight lanes that share a head
__device__ __forceinline__ float head_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  return x;
}

// LayerNorm of a head's 64 values (eight per lane), biased variance as torch.nn.LayerNorm
__device__ __forceinline__ void head_layer_norm(float (&x)[8], const float (&w)[8], const float (&b)[8], float eps) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += x[i];
  const float mean = head_sum(s) * (1.0f / 64.0f);
  float v = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    x[i] -= mean;
    v += x[i] * x[i];
  }
  const float rstd = 1.0f / sqrtf(head_sum(v) * (1.0f / 64.0f) + eps);
#pragma unroll
  for (int i = 0; i < 8; ++i) x[i] = x[i] * rstd * w[i] + b[i];
}

// t * cos + rotate(t) * sin with rotate(t)[j] = -t[j + 16] for the first 16 columns of a half, t[j - 16] for the others;
// the partner columns are held by the lane two over
__device__ __forceinline__ void head_rope(float (&t)[8], const float (&cs)[8], const float (&sn)[8], bool first16) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float partner = __shfl_xor_sync(0xffffffffu, t[i], 2);
    t[i] = t[i] * cs[i] + (first16 ? -partner : partner) * sn[i];
  }
}

template <typename T>
__global__ void __launch_bounds__(FE_WARPS * 32, 3) project_epilogue_kernel(const FeParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = static_cast<int64_t>(blockIdx.x) * FE_WARPS + (threadIdx.x >> 5);
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * FE_WARPS;
  const int H = p.H, Hi = p.Hi;
  const int sub = lane & 7, hq = lane >> 3;  // elements 8*sub .. 8*sub+7 of head (4*group + hq)
  const int e = 8 * sub;
  const int half = sub >> 2;                 // 0: columns 0..31 turn with y, 1: columns 32..63 with x
  const int col = 8 * (sub & 3);             // first column inside the half = column of the tables
  const bool first16 = (sub & 3) < 2;
  const bool ln_q = p.qn_w != nullptr, ln_k = p.kn_w != nullptr, ln_i = p.in_w != nullptr, rope = p.pos != nullptr;
  const T* fused = static_cast<const T*>(p.fused);

  for (int64_t tok = warp0; tok < p.tokens; tok += nwarps) {
    const T* row = fused + tok * p.ld;
    const bool al16 = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;  // every head of the row starts a multiple of 128 bytes on
    float cs[8], sn[8];
    if (rope) {
      long long pp = p.pos[tok * 2 + half];
      if (pp < 0 || pp >= p.table_rows) {  // the reference's table lookup would fail here; say so and carry on
        report_status(p.status, GW_ERR_INVALID_ARG);
        pp = 0;
      }
      load8(p.cos_tab + pp * 32 + col, cs);
      load8(p.sin_tab + pp * 32 + col, sn);
    }
    T* qo = static_cast<T*>(p.q) + tok * H * 64;
    T* ko = static_cast<T*>(p.k) + tok * H * 64;
    T* vo = static_cast<T*>(p.v) + tok * H * 64;
    for (int h0 = 0; h0 < H; h0 += 4) {  // four heads of q, of k and of v per turn
      const int h = h0 + hq;
      const bool live = h < H;
      float a[8] = {}, b[8] = {}, c[8] = {};
      if (live) {
        load8(row + h * 64 + e, a, al16);
        load8(row + (H + h) * 64 + e, b, al16);
        load8(row + (2 * H + h) * 64 + e, c, al16);
      }
      // the LayerNorm vectors are re-read every turn (they stay in L1): holding them in registers would cost a
      // third of the resident warps, and this kernel lives on loads in flight
      if (ln_q) {
        float w8[8], b8[8];
        load8(p.qn_w + e, w8);
        load8(p.qn_b + e, b8);
        head_layer_norm(a, w8, b8, p.qn_eps);
      }
      if (ln_k) {
        float w8[8], b8[8];
        load8(p.kn_w + e, w8);
        load8(p.kn_b + e, b8);
        head_layer_norm(b, w8, b8, p.kn_eps);
      }
      if (rope) {
        head_rope(a, cs, sn, first16);
        head_rope(b, cs, sn, first16);
      }
      if (live) {
        store8(qo + h * 64 + e, a);
        store8(ko + h * 64 + e, b);
        store8(vo + h * 64 + e, c);
      }
    }
    const T* irow = row + 3 * H * 64;
    T* qio = static_cast<T*>(p.q_idx) + tok * Hi * 64;
    T* kio = static_cast<T*>(p.k_idx) + tok * Hi * 64;
    for (int h0 = 0; h0 < Hi; h0 += 4) {
      const int h = h0 + hq;
      const bool live = h < Hi;
      float a[8] = {}, b[8] = {};
      if (live) {
        load8(irow + h * 64 + e, a, al16);
        load8(irow + (Hi + h) * 64 + e, b, al16);
      }
      if (ln_i) {
        float iw[8], ib[8];
        load8(p.in_w + e, iw);
        load8(p.in_b + e, ib);
        head_layer_norm(b, iw, ib, p.in_eps);
      }
      if (rope) {
        head_rope(a, cs, sn, first16);
        head_rope(b, cs, sn, first16);
      }
      if (live) {
        store8(qio + h * 64 + e, a);
        store8(kio + h * 64 + e, b);
      }
    }
    if (lane < Hi) static_cast<T*>(p.w)[tok * Hi + lane] = irow[2 * Hi * 64 + lane];
  }
}

}  // namespace
}  // namespace gw

using namespace gw;

extern "C" int gw_project_epilogue(const void* fused, int dtype, int64_t tokens, int64_t ld, int H, int D, int Hi, int Di,
                                   const int64_t* pos, const float* cos_tab, const float* sin_tab, int table_rows,
                                   const float* q_norm_w, const float* q_norm_b, float q_norm_eps, const float* k_norm_w,
                                   const float* k_norm_b, float k_norm_eps, const float* idx_k_norm_w, const float* idx_k_norm_b,
                                   float idx_k_norm_eps, void* q, void* k, void* v, void* q_idx, void* k_idx, void* w,
                                   int* status_dev, gw_stream_t stream) {
  if (!fused || !q || !k || !v || !q_idx || !k_idx || !w || tokens < 0) return GW_ERR_INVALID_ARG;
  if (H <= 0 || Hi <= 0 || Hi > 32) return GW_ERR_INVALID_ARG;
  if (D != 64 || Di != 64) return GW_ERR_UNSUPPORTED;
  const int64_t width = 3ll * H * 64 + 2ll * Hi * 64 + Hi;
  if (ld < width) return GW_ERR_INVALID_ARG;
  if (pos != nullptr && (!cos_tab || !sin_tab || table_rows <= 0)) return GW_ERR_INVALID_ARG;
  if ((q_norm_w == nullptr) != (q_norm_b == nullptr) || (k_norm_w == nullptr) != (k_norm_b == nullptr) ||
      (idx_k_norm_w == nullptr) != (idx_k_norm_b == nullptr))
    return GW_ERR_INVALID_ARG;
  const size_t es = dtype_size(dtype);
  // heads are written 16 bytes at a time and read 16 or 8 bytes at a time: rows must start on 8-byte boundaries,
  // tables, parameters and outputs on 16-byte ones
  if ((ld * es) % 8 != 0 || !aligned16(fused) || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(q_idx) ||
      !aligned16(k_idx))
    return GW_ERR_INVALID_ARG;
  if (pos != nullptr && (!aligned16(cos_tab) || !aligned16(sin_tab))) return GW_ERR_INVALID_ARG;
  for (const float* t : {q_norm_w, q_norm_b, k_norm_w, k_norm_b, idx_k_norm_w, idx_k_norm_b})
    if (t != nullptr && !aligned16(t)) return GW_ERR_INVALID_ARG;
  if (tokens == 0) return GW_OK;
  FeParams p;
  p.fused = fused; p.tokens = tokens; p.ld = ld; p.H = H; p.Hi = Hi; p.pos = pos; p.cos_tab = cos_tab; p.sin_tab = sin_tab;
  p.table_rows = table_rows; p.qn_w = q_norm_w; p.qn_b = q_norm_b; p.kn_w = k_norm_w; p.kn_b = k_norm_b; p.in_w = idx_k_norm_w;
  p.in_b = idx_k_norm_b; p.qn_eps = q_norm_eps; p.kn_eps = k_norm_eps; p.in_eps = idx_k_norm_eps;
  p.q = q; p.k = k; p.v = v; p.q_idx = q_idx; p.k_idx = k_idx; p.w = w; p.status = status_dev;
  DeviceFacts facts;
  const int frc = device_facts(nullptr, &facts);
  if (frc != GW_OK) return frc;
  const int sms = facts.sms;
  const int64_t want = (tokens + FE_WARPS - 1) / FE_WARPS;
  const int64_t cap = static_cast<int64_t>(sms) * 8 * 4;  // a few waves of resident CTAs; warps walk tokens grid-stride
  const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (dtype) {
    case GW_F32: project_epilogue_kernel<float><<<grid, FE_WARPS * 32, 0, st>>>(p); break;
    case GW_BF16: project_epilogue_kernel<__nv_bfloat16><<<grid, FE_WARPS * 32, 0, st>>>(p); break;
    case GW_F16: project_epilogue_kernel<__half><<<grid, FE_WARPS * 32, 0, st>>>(p); break;
    default: return GW_ERR_UNSUPPORTED;
  }
  GW_LAUNCH_CHECK();
  return GW_OK;
}
