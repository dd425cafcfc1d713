// The layer's projection, fused with everything that follows it up to the operator boundary.
//
//   [q | k | v | idx_q | idx_k | idx_w] = x . W^T + bias          one GEMM, M = tokens, N = 3*H*64 + 2*Hi*64 + Hi, K = dim
//   q, k: LayerNorm over the head, 2-D rotary embedding;  v: as is;  idx_q: rotary;  idx_k: LayerNorm, rotary;  idx_w: as is
//
// and the six results are written token-major ([tokens, H, 64] ...), which is the layout the indexer and the
// sparse attention read.  The product never reaches memory in its raw form: the reference writes it, reads it back
// for the LayerNorms, writes q and k, reads them for the rotary embedding, and copies q, k, v once more into the
// operator layout (easyvolcap/official_vggt/layers/dsa_attention.py:545-627, :229-232, :4935-4941, :5309-5315;
// layers/indexer.py:302-328).
//
// One persistent CTA per SM walks 128 x 256 output tiles (token-major order, so the CTAs of a wave share the x tile
// in L2 and all of W stays there).  Warp 0 = TMA producer (x tile 128 x 64 and W tile 256 x 64 per K step, 128-byte
// swizzle, four stages of 48 KB), warp 1 = one thread issuing tcgen05.mma (cta_group::1, kind::f16, M = 128,
// N = 256, K = 16: 128 cycles each, the full rate of the tensor pipe), warps 2..5 = epilogue.  Two accumulators of
// 256 TMEM columns alternate, so the epilogue of a tile runs under the main loop of the next.  An epilogue thread
// owns one token row: a head's 64 columns sit side by side in its TMEM lane, so LayerNorm and the rotary pairs
// (columns j and j + 16 of each 32-column half) are plain register arithmetic -- no shuffles, no shared memory --
// in fp32, rounded once when the head is stored (eight 16-byte stores per head).
#include <cuda.h>

#include "gw_common.cuh"
#include "gw_tc.cuh"

namespace gw {
namespace {

constexpr int PM = 128;   // token rows per tile (TMEM lanes)
constexpr int PN = 256;   // output columns per tile = four heads
constexpr int PK = 64;    // K step = one 128-byte swizzle atom of 16-bit elements
constexpr int PSTG = 4;   // operand ring depth
constexpr int P_A_BYTES = PM * PK * 2;  // 16 KB
constexpr int P_B_BYTES = PN * PK * 2;  // 32 KB
constexpr int P_EPI = 4;
constexpr int P_THREADS = 64 + P_EPI * 32;
constexpr int P_TMEM_COLS = 512;

struct ProjParams {
  const void* bias;  // [ncols] of the operand dtype, nullable
  int64_t tokens;
  int dim, ncols, H, Hi;
  const int64_t* pos;  // [tokens, 2] (y, x), or null: no rotary embedding
  const float *cos_tab, *sin_tab;
  int table_rows;
  const float *qn_w, *qn_b, *kn_w, *kn_b, *in_w, *in_b;
  float qn_eps, kn_eps, in_eps;
  void *q, *k, *v, *q_idx, *k_idx, *w;
  int* status;
};

struct alignas(16) ProjShared {
  alignas(16) float ln[3][2][64];  // [q, k, idx_k][weight, bias]; read 16 bytes at a time
  uint64_t full[PSTG], empty[PSTG];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

template <typename T>
__device__ __forceinline__ void store_head(T* dst, const float (&v)[64]) {
#pragma unroll
  for (int i = 0; i < 64; i += 8) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = from_float<T>(v[i + j]);
    *reinterpret_cast<uint4*>(dst + i) = raw;
  }
}

// LayerNorm of 64 values held by one thread (biased variance, as torch.nn.LayerNorm); wb = [weight 64][bias 64] in shared memory
__device__ __forceinline__ void layer_norm64(float (&v)[64], const float* wb, float eps) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 64; ++i) s += v[i];
  const float mean = s * (1.0f / 64.0f);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < 64; ++i) {
    v[i] -= mean;
    q = fmaf(v[i], v[i], q);
  }
  const float rstd = 1.0f / sqrtf(q * (1.0f / 64.0f) + eps);
#pragma unroll
  for (int i = 0; i < 64; i += 4) {
    const float4 w4 = *reinterpret_cast<const float4*>(wb + i);
    const float4 b4 = *reinterpret_cast<const float4*>(wb + 64 + i);
    v[i] = fmaf(v[i] * rstd, w4.x, b4.x);
    v[i + 1] = fmaf(v[i + 1] * rstd, w4.y, b4.y);
    v[i + 2] = fmaf(v[i + 2] * rstd, w4.z, b4.z);
    v[i + 3] = fmaf(v[i + 3] * rstd, w4.w, b4.w);
  }
}

// 2-D rotary embedding of one head: columns 0..31 turn with the row's y position, 32..63 with x; inside a half
// column j pairs with j + 16.  cs / sn hold the 16 angles of the y half, then the 16 of the x half (the
// reference's table repeats them for columns 16..31).
__device__ __forceinline__ void rope64(float (&v)[64], const float (&cs)[32], const float (&sn)[32]) {
#pragma unroll
  for (int half = 0; half < 2; ++half)
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float a = v[32 * half + j], b = v[32 * half + j + 16];
      const float c = cs[16 * half + j], s = sn[16 * half + j];
      v[32 * half + j] = fmaf(a, c, -b * s);
      v[32 * half + j + 16] = fmaf(b, c, a * s);
    }
}

template <typename T>
__global__ void __launch_bounds__(P_THREADS, 1)
project_fused_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const ProjParams p,
                     const int ab_format) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* a_smem = smem;                       // PSTG x 16 KB
  unsigned char* b_smem = a_smem + PSTG * P_A_BYTES;  // PSTG x 32 KB
  ProjShared* sh = reinterpret_cast<ProjShared*>(b_smem + PSTG * P_B_BYTES);

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const int ksteps = p.dim / PK;
  const int n_tiles = (p.ncols + PN - 1) / PN;
  const int64_t m_tiles = (p.tokens + PM - 1) / PM;
  const int64_t total = m_tiles * n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PSTG; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->acc_full[b], 1);
      mbar_init(&sh->acc_empty[b], P_EPI);
    }
    sh->abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  for (int i = threadIdx.x; i < 3 * 2 * 64; i += P_THREADS) {
    const int kind = i / 128, which = (i / 64) & 1, c = i & 63;
    const float* src = kind == 0 ? (which ? p.qn_b : p.qn_w) : kind == 1 ? (which ? p.kn_b : p.kn_w) : (which ? p.in_b : p.in_w);
    sh->ln[kind][which][c] = src ? src[c] : (which ? 0.f : 1.f);
  }
  if (warp == 1) tmem_alloc(&sh->tmem_base, P_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, sh->tmem_base, 0);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t use = 0;
      for (int64_t t = blockIdx.x; t < total && !sh->abort_flag; t += gridDim.x) {
        const int m0 = static_cast<int>(t / n_tiles) * PM, n0 = static_cast<int>(t % n_tiles) * PN;
        for (int ks = 0; ks < ksteps; ++ks, ++use) {
          const uint32_t s = use % PSTG;
          if (!mbar_wait_bounded(&sh->empty[s], ((use / PSTG) & 1u) ^ 1u)) { sh->abort_flag = 1; break; }
          if (sh->abort_flag) break;
          mbar_arrive_expect_tx(&sh->full[s], P_A_BYTES + P_B_BYTES);
          tma_load_2d(a_smem + s * P_A_BYTES, &tmX, ks * PK, m0, &sh->full[s]);
          tma_load_2d(b_smem + s * P_B_BYTES, &tmW, ks * PK, n0, &sh->full[s]);
        }
      }
      if (sh->abort_flag) {  // let the copies in flight land before the shared memory is given up
        for (uint32_t u = use > PSTG ? use - PSTG : 0u; u < use; ++u) mbar_wait_limit(&sh->full[u % PSTG], (u / PSTG) & 1u, kDrainLimitNs);
        report_status(p.status, GW_ERR_TIMEOUT);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      uint32_t use = 0, acc_use = 0;
      const uint64_t adesc0 = make_smem_desc(smem_u32(a_smem));
      const uint64_t bdesc0 = make_smem_desc(smem_u32(b_smem));
      for (int64_t t = blockIdx.x; t < total && !sh->abort_flag; t += gridDim.x, ++acc_use) {
        const int n0 = static_cast<int>(t % n_tiles) * PN;
        // the last column tile may hold only the few idx_w columns: issue no wider than needed (N a multiple of 16)
        const int left = p.ncols - n0;
        const int n_eff = left >= PN ? PN : ((left + 15) / 16) * 16;
        const uint32_t idesc = make_idesc_mn(ab_format, PM, n_eff);
        const uint32_t b = acc_use & 1u;
        if (!mbar_wait_bounded(&sh->acc_empty[b], ((acc_use >> 1) & 1u) ^ 1u)) { sh->abort_flag = 1; break; }
        const uint32_t d = tmem_base + b * PN;
        for (int ks = 0; ks < ksteps; ++ks, ++use) {
          const uint32_t s = use % PSTG;
          if (!mbar_wait_bounded(&sh->full[s], (use / PSTG) & 1u)) { sh->abort_flag = 1; break; }
          if (sh->abort_flag) break;
          tc_fence_after();
          const uint64_t ad = adesc0 + s * (P_A_BYTES >> 4), bd = bdesc0 + s * (P_B_BYTES >> 4);
#pragma unroll
          for (int kk = 0; kk < PK / 16; ++kk) tc_mma_f16(d, ad + 2 * kk, bd + 2 * kk, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
          tc_commit(&sh->empty[s]);
        }
        if (sh->abort_flag) break;
        tc_commit(&sh->acc_full[b]);
      }
      if (sh->abort_flag) report_status(p.status, GW_ERR_TIMEOUT);
    }
  } else {
    // ------------------------------ epilogue: bias, LayerNorm, rotary embedding, token-major stores ------------------------------
    const int lq = warp & 3;  // TMEM lane quarter this warp may read
    const int row_in_tile = lq * 32 + lane;
    const T* bias = static_cast<const T*>(p.bias);
    const int H = p.H, Hi = p.Hi;
    uint32_t acc_use = 0;
    int64_t cur_m = -1;
    float cs[32], sn[32];
    bool rope_row = false;
    for (int64_t t = blockIdx.x; t < total; t += gridDim.x, ++acc_use) {
      const int64_t mt = t / n_tiles;
      const int n0 = static_cast<int>(t % n_tiles) * PN;
      const int64_t row = mt * PM + row_in_tile;
      const bool live = row < p.tokens;
      if (mt != cur_m) {  // the row's angles serve all heads of all its tiles: y half, then x half
        cur_m = mt;
        rope_row = p.pos != nullptr && live;
        if (rope_row) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            long long pp = p.pos[row * 2 + half];
            if (pp < 0 || pp >= p.table_rows) {  // the reference's table lookup would fail here; say so and carry on
              report_status(p.status, GW_ERR_INVALID_ARG);
              pp = 0;
            }
#pragma unroll
            for (int j = 0; j < 16; j += 4) {
              const float4 c4 = *reinterpret_cast<const float4*>(p.cos_tab + pp * 32 + j);
              const float4 s4 = *reinterpret_cast<const float4*>(p.sin_tab + pp * 32 + j);
              cs[16 * half + j] = c4.x; cs[16 * half + j + 1] = c4.y; cs[16 * half + j + 2] = c4.z; cs[16 * half + j + 3] = c4.w;
              sn[16 * half + j] = s4.x; sn[16 * half + j + 1] = s4.y; sn[16 * half + j + 2] = s4.z; sn[16 * half + j + 3] = s4.w;
            }
          }
        }
      }
      const uint32_t b = acc_use & 1u;
      if (!mbar_wait_bounded(&sh->acc_full[b], (acc_use >> 1) & 1u)) { sh->abort_flag = 1; break; }
      if (sh->abort_flag) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lq * 32) << 16) + b * PN;
#pragma unroll 1
      for (int hh = 0; hh < PN / 64; ++hh) {
        const int c0 = n0 + hh * 64;  // first output column of this head slot
        if (c0 >= p.ncols) break;
        float v[64];
        {
          uint32_t r0[32], r1[32];
          tmem_ld_x32(taddr + hh * 64, r0);
          tmem_ld_x32(taddr + hh * 64 + 32, r1);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            v[i] = __uint_as_float(r0[i]);
            v[32 + i] = __uint_as_float(r1[i]);
          }
        }
        const int g = c0 / 64;  // head slot in the concatenated output: q heads, k heads, v heads, idx_q, idx_k, then idx_w
        if (g >= 3 * H + 2 * Hi) {
          // the idx_w columns: a few values per token, copied (plus bias)
          if (live)
            for (int c = 0; c < Hi && c0 + c < p.ncols; ++c) {
              float x = v[0];
#pragma unroll
              for (int i = 1; i < 32; ++i) x = (c == i) ? v[i] : x;  // Hi <= 32: select without dynamic register indexing
              if (bias != nullptr) x += to_float(bias[c0 + c]);
              static_cast<T*>(p.w)[row * Hi + c] = from_float<T>(x);
            }
          continue;
        }
        if (bias != nullptr) {
#pragma unroll
          for (int i = 0; i < 64; i += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(bias + c0 + i);
            const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i + j] += to_float(e[j]);
          }
        }
        T* dst;
        int ln_kind = -1;
        float eps = 0.f;
        bool rope = rope_row;
        if (g < H) {
          dst = static_cast<T*>(p.q) + (row * H + g) * 64;
          if (p.qn_w != nullptr) { ln_kind = 0; eps = p.qn_eps; }
        } else if (g < 2 * H) {
          dst = static_cast<T*>(p.k) + (row * H + (g - H)) * 64;
          if (p.kn_w != nullptr) { ln_kind = 1; eps = p.kn_eps; }
        } else if (g < 3 * H) {
          dst = static_cast<T*>(p.v) + (row * H + (g - 2 * H)) * 64;
          rope = false;
        } else if (g < 3 * H + Hi) {
          dst = static_cast<T*>(p.q_idx) + (row * Hi + (g - 3 * H)) * 64;
        } else {
          dst = static_cast<T*>(p.k_idx) + (row * Hi + (g - 3 * H - Hi)) * 64;
          if (p.in_w != nullptr) { ln_kind = 2; eps = p.in_eps; }
        }
        if (ln_kind >= 0) layer_norm64(v, &sh->ln[ln_kind][0][0], eps);
        if (rope) rope64(v, cs, sn);
        if (live) store_head<T>(dst, v);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->acc_empty[b]);
    }
    if (sh->abort_flag) report_status(p.status, GW_ERR_TIMEOUT);
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, P_TMEM_COLS);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [rows, cols] 16-bit row-major matrix, box = 64 columns x box_rows, 128-byte swizzle; rows and columns beyond the
// matrix read as zero
int make_matrix_map(CUtensorMap* map, const void* base, int dtype, int64_t rows, int64_t cols, int box_rows) {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess) return (EncodeTiledFn) nullptr;
    return q == cudaDriverEntryPointSuccess ? reinterpret_cast<EncodeTiledFn>(ptr) : (EncodeTiledFn) nullptr;
  }();
  if (!fn) return GW_ERR_CUDA;
  const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {PK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, dtype == GW_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                        const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return GW_ERR_CUDA;
  }
  return GW_OK;
}

}  // namespace
}  // namespace gw

using namespace gw;

extern "C" int gw_project_fused(const void* x, const void* weight, const void* bias, int dtype, int64_t tokens, int dim, int H, int D,
                                int Hi, int Di, const int64_t* pos, const float* cos_tab, const float* sin_tab, int table_rows,
                                const float* q_norm_w, const float* q_norm_b, float q_norm_eps, const float* k_norm_w,
                                const float* k_norm_b, float k_norm_eps, const float* idx_k_norm_w, const float* idx_k_norm_b,
                                float idx_k_norm_eps, void* q, void* k, void* v, void* q_idx, void* k_idx, void* w, int* status_dev,
                                gw_stream_t stream) {
  if (!x || !weight || !q || !k || !v || !q_idx || !k_idx || !w || tokens < 0) return GW_ERR_INVALID_ARG;
  if (H <= 0 || Hi <= 0 || Hi > 32 || dim <= 0) return GW_ERR_INVALID_ARG;
  if (D != 64 || Di != 64) return GW_ERR_UNSUPPORTED;
  if (dtype != GW_BF16 && dtype != GW_F16) return GW_ERR_UNSUPPORTED;  // fp32 operands: library GEMM + gw_project_epilogue
  if (dim % PK != 0) return GW_ERR_UNSUPPORTED;
  if (pos != nullptr && (!cos_tab || !sin_tab || table_rows <= 0)) return GW_ERR_INVALID_ARG;
  if ((q_norm_w == nullptr) != (q_norm_b == nullptr) || (k_norm_w == nullptr) != (k_norm_b == nullptr) ||
      (idx_k_norm_w == nullptr) != (idx_k_norm_b == nullptr))
    return GW_ERR_INVALID_ARG;
  for (const void* ptr : {x, weight, bias, static_cast<const void*>(cos_tab), static_cast<const void*>(sin_tab), static_cast<const void*>(q),
                          static_cast<const void*>(k), static_cast<const void*>(v), static_cast<const void*>(q_idx),
                          static_cast<const void*>(k_idx)})
    if (ptr != nullptr && !aligned16(ptr)) return GW_ERR_INVALID_ARG;
  if (tokens == 0) return GW_OK;
  if (tokens > 0x7fffff00) return GW_ERR_UNSUPPORTED;
  int dev = 0;
  DeviceFacts facts;
  int rc = device_facts(&dev, &facts);
  if (rc != GW_OK) return rc;
  if (facts.cc_major != 10) return GW_ERR_NO_SM100;
  const int ncols = 3 * H * 64 + 2 * Hi * 64 + Hi;
  CUtensorMap mx, mw;
  rc = make_matrix_map(&mx, x, dtype, tokens, dim, PM);
  if (rc != GW_OK) return rc;
  rc = make_matrix_map(&mw, weight, dtype, ncols, dim, PN);
  if (rc != GW_OK) return rc;
  ProjParams p;
  p.bias = bias; p.tokens = tokens; p.dim = dim; p.ncols = ncols; p.H = H; p.Hi = Hi; p.pos = pos; p.cos_tab = cos_tab; p.sin_tab = sin_tab;
  p.table_rows = table_rows; p.qn_w = q_norm_w; p.qn_b = q_norm_b; p.kn_w = k_norm_w; p.kn_b = k_norm_b; p.in_w = idx_k_norm_w;
  p.in_b = idx_k_norm_b; p.qn_eps = q_norm_eps; p.kn_eps = k_norm_eps; p.in_eps = idx_k_norm_eps;
  p.q = q; p.k = k; p.v = v; p.q_idx = q_idx; p.k_idx = k_idx; p.w = w; p.status = status_dev;
  const size_t smem = 1024 + static_cast<size_t>(PSTG) * (P_A_BYTES + P_B_BYTES) + sizeof(ProjShared);
  const int64_t total = ((tokens + PM - 1) / PM) * ((ncols + PN - 1) / PN);
  const int grid = static_cast<int>(total < facts.sms ? total : facts.sms);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == GW_BF16) {
    static OncePerDevice once;
    rc = ensure_dynamic_smem(project_fused_kernel<__nv_bfloat16>, smem, once, dev);
    if (rc != GW_OK) return rc;
    project_fused_kernel<__nv_bfloat16><<<grid, P_THREADS, smem, st>>>(mx, mw, p, 1);
  } else {
    static OncePerDevice once;
    rc = ensure_dynamic_smem(project_fused_kernel<__half>, smem, once, dev);
    if (rc != GW_OK) return rc;
    project_fused_kernel<__half><<<grid, P_THREADS, smem, st>>>(mx, mw, p, 0);
  }
  GW_LAUNCH_CHECK();
  return GW_OK;
}
