// Stage 1+2: indexer score on tcgen05 tensor cores with the exact top-k kept in the epilogue.
//
//   score[t,s] = sum_h w[s,h] * relu(scale * <q[t,h,:], k[s,h,:]>)            q,k bf16/fp16, fp32 accumulate
//
// One CTA owns a block of 128 query rows and walks all keys in tiles of 64.  Per tile and indexer head one
// 128x64x64 product is issued as four tcgen05.mma (K=16 each) from shared-memory operands that TMA loaded
// with the 128-byte swizzle; the Hi accumulators of a tile sit side by side in tensor memory, and two such
// sets (2 x 256 columns) alternate so the tensor cores work on tile j+1 while tile j is being reduced.
//
// Warp roles (320 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2..9 = epilogue.
// Epilogue thread = one query row (its TMEM lane); the eight warps form two streams of four, stream p
// reduces the tiles held in accumulator set p.  A thread reads its row of the accumulators with
// tcgen05.ld, forms the score, and appends (score, key) to its row's candidate list in global memory when
// score >= tau, tau being a per-row lower bound on the final k-th score.  Whenever a list is nearly full the
// warp compacts it to its exact top-k (gw_select.cuh) and raises tau to just above the new k-th score.  After
// the last tile the two streams' lists of a row are merged by one more exact selection, which writes the
// result.  The N x N score matrix never exists in memory.
//
// This is the robust form: it is exact from tau = -inf whatever the data and is used for small key sets, for the
// dense score mode (verification, and the sampled pass that seeds the thresholds of the fast form in
// gw_indexer_fast.cuh) and to redo the row blocks the fast form flags.
#include <cuda.h>
#include <math.h>
#include <stdlib.h>

#include "gw_common.cuh"
#include "gw_select.cuh"
#include "gw_tc.cuh"

namespace gw {
namespace {

constexpr int BM = 128;           // query rows per CTA (TMEM lanes)
constexpr int BN = 64;            // keys per tile
constexpr int DI = 64;            // indexer head dim = one 128-byte swizzle atom of bf16
constexpr int NSTG = 3;           // key-tile ring depth
constexpr int EPI_WARPS = 8;
constexpr int NTHREADS = 64 + EPI_WARPS * 32;
constexpr int ACC_COLS = 256;     // TMEM columns per accumulator set (Hi * BN <= 256)
constexpr int TMEM_COLS = 512;
constexpr int SEL_BINS = 1024;
constexpr int Q_HEAD_BYTES = BM * DI * 2;   // 16 KB
constexpr int K_HEAD_BYTES = BN * DI * 2;   // 8 KB
constexpr int MAX_SLOTS = 160;    // upper bound on resident CTAs (one per SM)

enum { MODE_TOPK = 0, MODE_SCORES = 1 };

struct IdxParams {
  const float4* wsc;       // [S_pad] w * scale, four floats per key (heads beyond Hi are 0)
  const float* wtile;      // fast path: w * scale per 64-key tile, [tile][4 heads][64]
  const float* tau_in;     // [T] initial thresholds, or null for -inf
  int32_t* out_idx;        // [T,k]
  void* out_scores;        // [T,k] of out_dtype, nullable
  int out_dtype;
  float* dense_out;        // score mode: [T, S] with row stride dense_stride
  int64_t dense_stride;
  uint2* cand;             // [slots][BM][2][caph] (score bits, key index)
  int caph;
  int T, S, k;
  int key_step;            // score mode: column j is key j * key_step
  const float* smax_in;    // [T] fast path: estimate of the row maximum (binning range of the final selection)
  int row_begin, row_end;  // fast path: rows of this launch (row_begin a multiple of the row block)
  int* list_cnt;           // fast path: [rows of the launch][nsplit][2 column halves] list lengths (caph + 1 = overflowed)
  int* item_counter;       // fast path: work items handed out beyond the first one of every CTA (zero at launch)
  int nsplit;              // fast path: key splits per row block (lists and their capacity caph are per split)
  int* block_flags;        // [row blocks] fast kernel: sets 1 for blocks with a row to redo; robust kernel, when
                           // non-null: processes only the flagged blocks
  float* tau_redo;         // [T] fast kernel output: -inf for rows to redo, +inf for finished rows
  int* status;
  int profile;             // non-zero: the fast kernel fills its cycle counters (gw_debug_indexer_profile)
};

struct TwoSegSrc {
  const uint2* a;
  const uint2* b;
  int na;
  __device__ __forceinline__ unsigned long long operator()(int i) const {
    const uint2 e = (i < na) ? a[i] : b[i - na];
    return composite(score_key(__uint_as_float(e.x)), e.y);
  }
};
struct CompactSink {  // in-place: the survivors move to the front of the same list
  uint2* dst;
  __device__ __forceinline__ void operator()(int pos, unsigned long long c) const {
    dst[pos] = make_uint2(__float_as_uint(key_score(composite_key(c))), composite_idx(c));
  }
};
struct FinalSink {
  int32_t* oi;
  void* os;
  int dtype;
  __device__ __forceinline__ void operator()(int pos, unsigned long long c) const {
    oi[pos] = static_cast<int32_t>(composite_idx(c));
    if (os != nullptr) {
      const float s = key_score(composite_key(c));
      if (dtype == GW_BF16) static_cast<__nv_bfloat16*>(os)[pos] = __float2bfloat16_rn(s);
      else if (dtype == GW_F16) static_cast<__half*>(os)[pos] = __float2half_rn(s);
      else static_cast<float*>(os)[pos] = s;
    }
  }
};

struct alignas(8) IdxShared {
  uint64_t q_full, q_empty;
  uint64_t k_full[NSTG], k_empty[NSTG];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
  int cnt[2][BM];
  float smin[2][BM];
  float smax[2][BM];
};

template <int HI, int MODE>
__global__ void __launch_bounds__(NTHREADS, 1)
indexer_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const IdxParams p,
               const uint32_t idesc) {
  extern __shared__ unsigned char smem_raw[];
  // operand tiles need 1024-byte alignment for the 128-byte swizzle
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* q_smem = smem;                                  // HI x 16 KB
  unsigned char* k_smem = q_smem + HI * Q_HEAD_BYTES;            // NSTG x HI x 8 KB
  SelectSmem<SEL_BINS>* sel = reinterpret_cast<SelectSmem<SEL_BINS>*>(k_smem + NSTG * HI * K_HEAD_BYTES);
  IdxShared* sh = reinterpret_cast<IdxShared*>(sel + EPI_WARPS);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwork = ((p.row_end > 0 ? p.row_end : p.T) + BM - 1) / BM;
  const int work0 = p.row_begin / BM;  // a launch may cover a range of rows (both multiples of the row block)
  const int ntiles = (p.S + BN - 1) / BN;

  if (threadIdx.x == 0) {
    mbar_init(&sh->q_full, 1);
    mbar_init(&sh->q_empty, 1);
    for (int s = 0; s < NSTG; ++s) {
      mbar_init(&sh->k_full[s], 1);
      mbar_init(&sh->k_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->acc_full[b], 1);
      mbar_init(&sh->acc_empty[b], 4);
    }
    sh->abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) tmem_alloc(&sh->tmem_base, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t kuse = 0, nblk = 0;
      for (int wi = work0 + blockIdx.x; wi < nwork && !sh->abort_flag; wi += gridDim.x) {
        if (p.block_flags && !p.block_flags[wi]) continue;
        const int rb = wi;
        if (!mbar_wait_bounded(&sh->q_empty, (nblk & 1u) ^ 1u)) { sh->abort_flag = 1; break; }
        ++nblk;
        mbar_arrive_expect_tx(&sh->q_full, HI * Q_HEAD_BYTES);
#pragma unroll
        for (int h = 0; h < HI; ++h) tma_load_2d(q_smem + h * Q_HEAD_BYTES, &tmQ, h * DI, rb * BM, &sh->q_full);
        for (int j = 0; j < ntiles; ++j, ++kuse) {
          const uint32_t s = kuse % NSTG, n = kuse / NSTG;
          if (!mbar_wait_bounded(&sh->k_empty[s], (n & 1u) ^ 1u)) { sh->abort_flag = 1; break; }
          if (sh->abort_flag) break;
          mbar_arrive_expect_tx(&sh->k_full[s], HI * K_HEAD_BYTES);
#pragma unroll
          for (int h = 0; h < HI; ++h)
            tma_load_2d(k_smem + (s * HI + h) * K_HEAD_BYTES, &tmK, h * DI, j * BN, &sh->k_full[s]);
        }
      }
      if (sh->abort_flag) {
        // leaving early: let the copies this thread started land before the CTA's shared memory is given up
        if (nblk > 0) mbar_wait_limit(&sh->q_full, (nblk - 1u) & 1u, kDrainLimitNs);
        for (uint32_t u = kuse > NSTG ? kuse - NSTG : 0u; u < kuse; ++u)
          mbar_wait_limit(&sh->k_full[u % NSTG], (u / NSTG) & 1u, kDrainLimitNs);
        report_status(p.status, GW_ERR_TIMEOUT);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      uint32_t kuse = 0, nblk = 0, use0 = 0, use1 = 0;
      for (int wi = work0 + blockIdx.x; wi < nwork && !sh->abort_flag; wi += gridDim.x) {
        if (p.block_flags && !p.block_flags[wi]) continue;
        if (!mbar_wait_bounded(&sh->q_full, nblk & 1u)) { sh->abort_flag = 1; break; }
        ++nblk;
        for (int j = 0; j < ntiles; ++j, ++kuse) {
          const uint32_t b = j & 1;
          const uint32_t n = b ? use1 : use0;
          if (!mbar_wait_bounded(&sh->acc_empty[b], (n & 1u) ^ 1u)) { sh->abort_flag = 1; break; }
          const uint32_t s = kuse % NSTG;
          if (!mbar_wait_bounded(&sh->k_full[s], (kuse / NSTG) & 1u)) { sh->abort_flag = 1; break; }
          if (sh->abort_flag) break;
          tc_fence_after();
#pragma unroll
          for (int h = 0; h < HI; ++h) {
            const uint64_t adesc = make_smem_desc(smem_u32(q_smem + h * Q_HEAD_BYTES));
            const uint64_t bdesc = make_smem_desc(smem_u32(k_smem + (s * HI + h) * K_HEAD_BYTES));
            const uint32_t d = tmem_base + b * ACC_COLS + h * BN;
#pragma unroll
            for (int kk = 0; kk < DI / 16; ++kk)  // +32 bytes along K per step = +2 in the address field
              tc_mma_f16(d, adesc + 2 * kk, bdesc + 2 * kk, idesc, kk > 0 ? 1u : 0u);
          }
          tc_commit(&sh->k_empty[s]);
          tc_commit(&sh->acc_full[b]);
          if (b) ++use1; else ++use0;
        }
        tc_commit(&sh->q_empty);
      }
      if (sh->abort_flag) report_status(p.status, GW_ERR_TIMEOUT);
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int e = warp - 2;
    const int strm = e >> 2;          // which accumulator set / candidate stream
    const int lq = warp & 3;          // TMEM lane quarter this warp may read
    const int row_in_tile = lq * 32 + lane;
    const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(lq * 32) << 16) + strm * ACC_COLS;
    uint32_t acc_use = 0;
    uint2* const mybuf = (MODE == MODE_TOPK)
                             ? p.cand + ((static_cast<size_t>(blockIdx.x) * BM + row_in_tile) * 2 + strm) * p.caph
                             : nullptr;
    const int compact_at = p.caph - BN;

    for (int wi = work0 + blockIdx.x; wi < nwork; wi += gridDim.x) {
      if (p.block_flags && !p.block_flags[wi]) continue;
      const int rb = wi;
      const int row = rb * BM + row_in_tile;
      float tau = INFINITY;
      if (row < p.T) tau = p.tau_in ? p.tau_in[row] : -INFINITY;
      const bool active = tau < INFINITY;
      int cnt = 0;
      float smin = INFINITY, smax = -INFINITY;

      for (int j = strm; j < ntiles; j += 2) {
        if (sh->abort_flag) break;
        if (!mbar_wait_bounded(&sh->acc_full[strm], acc_use & 1u)) { sh->abort_flag = 1; break; }
        tc_fence_after();
        const int col_base = j * BN;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          uint32_t a[HI][16];
#pragma unroll
          for (int h = 0; h < HI; ++h) tmem_ld_x16(taddr_row + h * BN + c0, a[h]);
          tmem_wait_ld();
          float sc[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const int col = col_base + c0 + c;
            const float4 w4 = __ldg(p.wsc + static_cast<size_t>(col) * p.key_step);
            float s = 0.f;
            s = fmaf(fmaxf(__uint_as_float(a[0][c]), 0.f), w4.x, s);
            if (HI > 1) s = fmaf(fmaxf(__uint_as_float(a[1 % HI][c]), 0.f), w4.y, s);
            if (HI > 2) s = fmaf(fmaxf(__uint_as_float(a[2 % HI][c]), 0.f), w4.z, s);
            if (HI > 3) s = fmaf(fmaxf(__uint_as_float(a[3 % HI][c]), 0.f), w4.w, s);
            sc[c] = s;
          }
          if (MODE == MODE_TOPK) {
#pragma unroll
            for (int c = 0; c < 16; ++c) {
              const int col = col_base + c0 + c;
              if (sc[c] >= tau && col < p.S) {
                mybuf[cnt] = make_uint2(__float_as_uint(sc[c]), static_cast<uint32_t>(col));
                ++cnt;
                smin = fminf(smin, sc[c]);
                smax = fmaxf(smax, sc[c]);
              }
            }
          } else if (row < p.T) {
            float* orow = p.dense_out + static_cast<int64_t>(row) * p.dense_stride + col_base + c0;
            if (col_base + c0 + 16 <= p.S && (p.dense_stride & 3) == 0) {
#pragma unroll
              for (int c = 0; c < 16; c += 4)
                *reinterpret_cast<float4*>(orow + c) = make_float4(sc[c], sc[c + 1], sc[c + 2], sc[c + 3]);
            } else {
#pragma unroll
              for (int c = 0; c < 16; ++c)
                if (col_base + c0 + c < p.S) orow[c] = sc[c];
            }
          }
        }
        // hand the accumulator set back to the MMA warp
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->acc_empty[strm]);
        ++acc_use;

        if (MODE == MODE_TOPK) {
          // lists that could overflow during the next tile are cut back to their exact top-k now
          uint32_t need = __ballot_sync(0xffffffffu, cnt > compact_at);
          while (need) {
            const int r = __ffs(need) - 1;
            need &= need - 1;
            uint2* buf = reinterpret_cast<uint2*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(mybuf), r));
            const int n = __shfl_sync(0xffffffffu, cnt, r);
            const float lo_s = __shfl_sync(0xffffffffu, smin, r);
            const float hi_s = __shfl_sync(0xffffffffu, smax, r);
            __syncwarp();
            TwoSegSrc src{buf, buf, n};
            CompactSink sink{buf};
            unsigned long long kth = 0;
            const int kept = group_select_topk<32, SEL_BINS>(
                src, n, p.k, composite(score_key(lo_s), 0xffffffffu), composite(score_key(hi_s), 0u), sel[e], lane, 0,
                sink, &kth);
            if (lane == r && n > p.k) {
              cnt = kept;
              const uint32_t kk = composite_key(kth);
              smin = key_score(kk);
              tau = key_score(kk + 1u);  // later keys have larger indices: only a strictly larger score can enter
            }
            __syncwarp();
          }
        }
      }

      if (MODE == MODE_TOPK) {
        sh->cnt[strm][row_in_tile] = active ? cnt : -1;
        sh->smin[strm][row_in_tile] = smin;
        sh->smax[strm][row_in_tile] = smax;
        named_bar_sync(1, EPI_WARPS * 32);
        // merge the two streams of each row: exact top-k of their union
        for (int r = e; r < BM; r += EPI_WARPS) {
          const int n0 = sh->cnt[0][r], n1 = sh->cnt[1][r];
          const int grow = rb * BM + r;
          if (n0 < 0 || grow >= p.T || sh->abort_flag) continue;
          const int n = n0 + n1;
          const uint2* b0 = p.cand + ((static_cast<size_t>(blockIdx.x) * BM + r) * 2 + 0) * p.caph;
          const uint2* b1 = b0 + p.caph;
          const float lo_s = fminf(sh->smin[0][r], sh->smin[1][r]);
          const float hi_s = fmaxf(sh->smax[0][r], sh->smax[1][r]);
          TwoSegSrc src{b0, b1, n0};
          FinalSink sink{p.out_idx + static_cast<int64_t>(grow) * p.k,
                         p.out_scores ? static_cast<unsigned char*>(p.out_scores) +
                                            static_cast<int64_t>(grow) * p.k * (p.out_dtype == GW_F32 ? 4 : 2)
                                      : nullptr,
                         p.out_dtype};
          group_select_topk<32, SEL_BINS>(src, n, p.k, composite(score_key(lo_s), 0xffffffffu),
                                          composite(score_key(hi_s), 0u), sel[e], lane, 0, sink, nullptr);
        }
        // the eight warps must take the same way out: the flag is combined through the barrier itself, so a
        // flag raised between two warps' reads cannot send one of them on to the next row block alone
        if (named_bar_or(1, EPI_WARPS * 32, sh->abort_flag != 0)) break;
      } else if (sh->abort_flag) {
        break;  // score mode: the warps share no barrier, each may leave on its own
      }
    }
    if (sh->abort_flag) report_status(p.status, GW_ERR_TIMEOUT);
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace
}  // namespace gw
#include "gw_indexer_fast.cuh"
namespace gw {
namespace {

// w * scale as fp32, four per key; rows beyond S (tile padding) are zero
template <typename T>
__global__ void prep_w_kernel(const T* w, int S, int Hi, float scale, float4* wsc, int s_pad) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= s_pad) return;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (s < S)
    for (int h = 0; h < Hi; ++h) v[h] = to_float(w[static_cast<size_t>(s) * Hi + h]) * scale;
  wsc[s] = make_float4(v[0], v[1], v[2], v[3]);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess) return (EncodeTiledFn) nullptr;
    return q == cudaDriverEntryPointSuccess ? reinterpret_cast<EncodeTiledFn>(ptr) : (EncodeTiledFn) nullptr;
  }();
  return fn;
}

// rows x (Hi*64) 16-bit matrix, row pitch `pitch_bytes`; box = 64 columns x box_rows, 128-byte swizzle.
// An encoded map is a pure function of these arguments, so the last few are kept per host thread: a model that
// calls the indexer layer after layer with the same buffers encodes each map once.
struct MapKey {
  const void* base;
  int64_t rows, pitch;
  int dtype, Hi, box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && pitch == o.pitch && dtype == o.dtype && Hi == o.Hi && box_rows == o.box_rows;
  }
};
struct MapEntry {
  MapKey key;
  CUtensorMap map;
  bool valid;
};
constexpr int kMapCacheSize = 32;
thread_local MapEntry g_map_cache[kMapCacheSize];

int make_map(CUtensorMap* map, const void* base, int dtype, int64_t rows, int Hi, int64_t pitch_bytes, int box_rows) {
  const MapKey key{base, rows, pitch_bytes, dtype, Hi, box_rows};
  uint64_t h = reinterpret_cast<uintptr_t>(base) >> 8;
  h = (h ^ (static_cast<uint64_t>(rows) * 0x9E3779B97F4A7C15ull) ^ (static_cast<uint64_t>(pitch_bytes) << 7) ^
       static_cast<uint64_t>(box_rows)) * 0xD6E8FEB86659FD93ull;
  MapEntry& slot = g_map_cache[(h >> 32) % kMapCacheSize];
  if (slot.valid && slot.key == key) {
    *map = slot.map;
    return GW_OK;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return GW_ERR_CUDA;
  const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(Hi) * DI, static_cast<cuuint64_t>(rows)};
  const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(pitch_bytes)};
  const cuuint32_t box[2] = {DI, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, dtype == GW_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                        const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return GW_ERR_CUDA;
  }
  slot.key = key;
  slot.map = *map;
  slot.valid = true;
  return GW_OK;
}

size_t smem_bytes(int Hi) {
  return 1024 + static_cast<size_t>(Hi) * Q_HEAD_BYTES + static_cast<size_t>(NSTG) * Hi * K_HEAD_BYTES +
         EPI_WARPS * sizeof(SelectSmem<SEL_BINS>) + sizeof(IdxShared);
}

int device_info(int* sms, int* dev) {
  DeviceFacts f;
  const int rc = device_facts(dev, &f);
  if (rc != GW_OK) return rc;
  *sms = f.sms;
  return f.cc_major == 10 ? GW_OK : GW_ERR_NO_SM100;
}

// cycle counters of the fast kernel: off unless switched on through gw_debug_indexer_profile_enable
std::atomic<int> g_profile_on{0};
inline int profiling_enabled() { return g_profile_on.load(std::memory_order_relaxed); }

template <int MODE>
int launch_indexer(int Hi, const CUtensorMap& mq, const CUtensorMap& mk, const IdxParams& p, uint32_t idesc, int grid, int dev,
                   cudaStream_t st) {
  const size_t smem = smem_bytes(Hi);
#define GW_IDX_CASE(H)                                                  \
  case H: {                                                             \
    auto kern = indexer_kernel<H, MODE>;                                \
    static OncePerDevice once;                                          \
    const int arc = ensure_dynamic_smem(kern, smem, once, dev);         \
    if (arc != GW_OK) return arc;                                       \
    kern<<<grid, NTHREADS, smem, st>>>(mq, mk, p, idesc);               \
    break;                                                              \
  }
  switch (Hi) {
    GW_IDX_CASE(1)
    GW_IDX_CASE(2)
    GW_IDX_CASE(3)
    GW_IDX_CASE(4)
    default: return GW_ERR_UNSUPPORTED;
  }
#undef GW_IDX_CASE
  GW_LAUNCH_CHECK();
  return GW_OK;
}

int launch_indexer_fast(int Hi, const CUtensorMap& mq, const CUtensorMap& mk, const IdxParams& p, uint32_t idesc, int grid,
                        int dev, cudaStream_t st) {
  const size_t smem = fast_smem_bytes(Hi);
#define GW_IDXF_CASE(H)                                                 \
  case H: {                                                             \
    auto kern = indexer_fast_kernel<H>;                                 \
    static OncePerDevice once;                                          \
    const int arc = ensure_dynamic_smem(kern, smem, once, dev);         \
    if (arc != GW_OK) return arc;                                       \
    kern<<<grid, F_THREADS, smem, st>>>(mq, mk, p, idesc);              \
    break;                                                              \
  }
  switch (Hi) {
    GW_IDXF_CASE(1)
    GW_IDXF_CASE(2)
    GW_IDXF_CASE(3)
    GW_IDXF_CASE(4)
    default: return GW_ERR_UNSUPPORTED;
  }
#undef GW_IDXF_CASE
  GW_LAUNCH_CHECK();
  return GW_OK;
}

int launch_prep_w(const void* w, int dtype, int S, int Hi, float scale, float4* wsc, int s_pad, cudaStream_t st) {
  const int thr = 256, grid = (s_pad + thr - 1) / thr;
  if (dtype == GW_BF16)
    prep_w_kernel<__nv_bfloat16><<<grid, thr, 0, st>>>(static_cast<const __nv_bfloat16*>(w), S, Hi, scale, wsc, s_pad);
  else
    prep_w_kernel<__half><<<grid, thr, 0, st>>>(static_cast<const __half*>(w), S, Hi, scale, wsc, s_pad);
  GW_LAUNCH_CHECK();
  return GW_OK;
}

// sampling plan for the initial threshold
struct SamplePlan {
  int step;  // 0 = no sampling
  int m;     // sampled keys
  int rank;  // tau = rank-th largest sampled score
};
SamplePlan plan_sample(int S, int k) {
  SamplePlan sp{0, 0, 0};
  if (S < 4096 || static_cast<int64_t>(S) < 8ll * k) return sp;
  // every step-th key is sampled.  The count of keys above the rank-th sampled score scatters like
  // step * sqrt(rank), so the relative precision of the estimate is set by k / step: keep it near 32, with at
  // least 1024 sampled keys and at most one key in 16 (the sampled pass is extra tensor-core work)
  int step = k / 32;
  if (step < 16) step = 16;
  // very long key sets: no more than about 4096 sampled keys (the sampled pass and the threshold kernel grow
  // with their number), as long as k / step stays at 8 or more; the lists then hold somewhat more candidates
  if (S / 4096 > step) step = S / 4096 < k / 8 ? S / 4096 : (k / 8 > step ? k / 8 : step);
  if (step > S / 1024) step = S / 1024;
  if (step < 2) return sp;
  step |= 1;  // odd: never in lock-step with an even token grid
  const int m = (S + step - 1) / step;
  const double ratio = static_cast<double>(k) / step;
  // a row that comes up short costs a slow redo of its whole row block, so aim about 4.7 standard deviations
  // above k (rank - ratio = 6.75 sqrt(ratio) is 4.7 sqrt(rank) at ratio 32)
  const int rank = static_cast<int>(ceil(ratio + 6.75 * sqrt(ratio) + 2.0));
  if (rank * 2 >= m) return sp;
  sp.step = step;
  sp.m = m;
  sp.rank = rank;
  return sp;
}

// list capacity per (row, stream).  The robust kernel keeps up to k after a compaction and refills to 2k; the fast
// kernel needs room for the candidates the sampled threshold lets through: rank * step expected, scatter
// step * sqrt(rank), split over two streams with some imbalance.
int cand_capacity(int S, int k) {
  int c = 2 * k;
  if (c < 1024) c = 1024;
  const SamplePlan sp = plan_sample(S, k);
  if (sp.step > 0) {
    const double total = static_cast<double>(sp.rank) * sp.step + 7.0 * sp.step * sqrt(static_cast<double>(sp.rank));
    const int need = static_cast<int>(total * 0.5 * 1.15) + 2 * FBN;
    if (need > c) c = need;
  }
  return static_cast<int>(round_up(static_cast<size_t>(c), 64));
}

// Key splits per row block for a fast-path launch over `blocks` row blocks on `sms` SMs: the smallest split
// count (up to 8) whose makespan, in units of one whole row block, is within 3 % of the best one.
int plan_splits(int blocks, int sms, int ntiles) {
  double best = 1e30;
  double span[9];
  for (int ns = 1; ns <= 8; ++ns) {
    const long long items = static_cast<long long>(blocks) * ns;
    span[ns] = static_cast<double>((items + sms - 1) / sms) / ns;
    if (ns * 8 > ntiles) span[ns] = 1e30;  // keep at least 8 key tiles per item
    if (span[ns] < best) best = span[ns];
  }
  for (int ns = 1; ns <= 8; ++ns)
    if (span[ns] <= best * 1.03) return ns;
  return 1;
}
constexpr int kPlanSms = 148;  // SM count assumed when sizing the workspace (any split count is valid on any device)

// capacity of one fast-path list (row, key split, column group): its share of the row's expected candidates
// (2 * caph covers the sampling scatter) with a quarter on top for the uneven spread over the lists, plus room
// for the guard (a warp's 16 columns of a tile must always fit)
int seg_capacity(int caph, int nsplit) {
  return static_cast<int>(round_up(static_cast<size_t>(2) * caph * 5 / (4 * F_NQ * nsplit) + 4 * F_QCOLS, 32));
}

// The fast kernel moves only the low 32 bits of its list addresses, so no list may cross a 4 GiB boundary: when
// such a boundary falls inside the list area, the area is shifted (by less than one list) so that the boundary
// lies between two lists.  kListShiftSlack bytes are reserved behind the area for that.
constexpr size_t kListShiftSlack = 1 << 20;
uint2* place_lists(unsigned char* area, size_t area_bytes, size_t list_bytes) {
  const uintptr_t base = reinterpret_cast<uintptr_t>(area);
  const uintptr_t boundary = (base + 0xffffffffull) & ~static_cast<uintptr_t>(0xffffffffull);
  if (boundary >= base + area_bytes + kListShiftSlack || list_bytes == 0 || list_bytes > kListShiftSlack) return reinterpret_cast<uint2*>(area);
  return reinterpret_cast<uint2*>(area + (boundary - base) % list_bytes);
}

struct WsLayout {
  size_t wsc, wtile, tau0, smax, tau_redo, flags, counter, sample, list_cnt, cand, total;
  size_t list_cnt_bytes, cand_bytes;
  int s_pad, m_pad, slots, caph, chunk_rows, nsplit, cap_split;
};
WsLayout ws_layout(int T, int S, int k) {
  WsLayout L;
  const int nblocks = (T + BM - 1) / BM;
  const SamplePlan sp = plan_sample(S, k);
  // the sampled pass reads w at key j*step for j up to the end of its last tile
  L.s_pad = static_cast<int>(round_up(static_cast<size_t>(S), BN)) + BN * (sp.step > 1 ? sp.step : 1) + BN;
  L.slots = nblocks < MAX_SLOTS ? nblocks : MAX_SLOTS;
  L.caph = cand_capacity(S, k);
  L.m_pad = static_cast<int>(round_up(static_cast<size_t>(sp.m), 4));
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off += round_up(bytes, 256);
    return at;
  };
  L.wsc = take(static_cast<size_t>(L.s_pad) * 16);
  L.wtile = take(sp.step > 0 ? (static_cast<size_t>(S) / FBN + 2) * W_TILE_BYTES : 0);
  L.tau0 = take(static_cast<size_t>(T) * 4);
  L.smax = take(static_cast<size_t>(T) * 4);
  L.tau_redo = take(static_cast<size_t>(T) * 4);
  L.flags = take(static_cast<size_t>(nblocks) * 4);
  L.counter = take(256);
  // fast path: the lists of all rows of a launch are kept until the finalize kernel has run, so long inputs are
  // processed in chunks of whole waves of row blocks (about 2 GiB of lists per chunk)
  const size_t robust_row_bytes = static_cast<size_t>(2) * L.caph * 8;
  int chunk_blocks = static_cast<int>((static_cast<size_t>(2) << 30) / (robust_row_bytes * 5 / 4) / BM);
  if (sp.m > 0) {  // the sampled scores of a chunk (fp32 [rows, m]) stay below about 1 GiB as well
    const int by_sample = static_cast<int>((static_cast<size_t>(1) << 30) / (static_cast<size_t>(L.m_pad) * 4) / BM);
    if (by_sample < chunk_blocks) chunk_blocks = by_sample;
  }
  chunk_blocks = chunk_blocks >= 2 * MAX_SLOTS ? chunk_blocks / kPlanSms * kPlanSms : (chunk_blocks > 0 ? chunk_blocks : 1);
  if (chunk_blocks > nblocks) chunk_blocks = nblocks;
  L.chunk_rows = sp.step > 0 ? chunk_blocks * BM : 0;
  // key splits even out a launch with few row blocks or a ragged last wave; every split gets its own lists,
  // each with a 25 % larger share of the capacity than an even division would give
  L.nsplit = sp.step > 0 ? plan_splits(chunk_blocks, kPlanSms, (S + FBN - 1) / FBN) : 1;
  L.cap_split = seg_capacity(L.caph, L.nsplit);
  const size_t fast_row_bytes = static_cast<size_t>(L.nsplit) * F_NQ * L.cap_split * 8;
  L.list_cnt_bytes = static_cast<size_t>(L.chunk_rows) * L.nsplit * F_NQ * 4;
  L.list_cnt = take(L.list_cnt_bytes);
  L.sample = take(static_cast<size_t>(L.chunk_rows) * L.m_pad * 4);  // sampled scores of one chunk of rows
  const size_t robust_bytes = static_cast<size_t>(L.slots) * BM * robust_row_bytes;
  const size_t fast_bytes = static_cast<size_t>(L.chunk_rows) * fast_row_bytes;
  L.cand_bytes = robust_bytes > fast_bytes ? robust_bytes : fast_bytes;
  L.cand = take(L.cand_bytes + kListShiftSlack);
  L.total = off;
  return L;
}

int check_common(const void* q, const void* k, const void* w, int dtype, int B, int T, int S, int Hi, int Di) {
  if (!q || !k || !w || B <= 0 || T < 0 || S <= 0 || Hi <= 0 || Di <= 0) return GW_ERR_INVALID_ARG;
  if (dtype != GW_BF16 && dtype != GW_F16) return GW_ERR_UNSUPPORTED;
  if (Di != DI || Hi > 4) return GW_ERR_UNSUPPORTED;
  if (!aligned16(q) || !aligned16(k)) return GW_ERR_INVALID_ARG;
  return GW_OK;
}

}  // namespace
}  // namespace gw

using namespace gw;

extern "C" size_t gw_indexer_topk_workspace_bytes(int B, int T, int S, int Hi, int Di, int k) {
  (void)B; (void)Hi; (void)Di;
  if (T <= 0 || S <= 0 || k <= 0) return 0;
  return ws_layout(T, S, k).total;
}

extern "C" int gw_debug_indexer_profile(unsigned long long* host_out, int max_entries) {
  const int total = MAX_SLOTS * (F_THREADS / 32) * PROF_SLOTS;  // [CTA][11 warps][8 slots]
  if (!host_out || max_entries < 4) return GW_ERR_INVALID_ARG;
  // first four entries: finalize statistics since the last call (overflowed / short / general / lean rows)
  GW_CUDA_TRY(cudaMemcpyFromSymbol(host_out, g_fin_stats, sizeof(unsigned long long) * 4));
  const unsigned long long zero[4] = {0, 0, 0, 0};
  GW_CUDA_TRY(cudaMemcpyToSymbol(g_fin_stats, zero, sizeof(zero)));
  const int n = max_entries - 4 < total ? max_entries - 4 : total;
  if (n > 0) GW_CUDA_TRY(cudaMemcpyFromSymbol(host_out + 4, g_idx_prof, sizeof(unsigned long long) * n));
  return n + 4;
}

extern "C" int gw_debug_indexer_profile_enable(int on) {
  g_profile_on.store(on ? 1 : 0, std::memory_order_relaxed);
  return GW_OK;
}

extern "C" int gw_indexer_topk_launch_count(int B, int T, int S, int k) {
  if (B <= 0 || T <= 0 || S <= 0 || k <= 0) return 0;
  // w scaling + fused pass, plus sampled scores + threshold pick + redo pass when sampling is on
  const WsLayout L = ws_layout(T, S, k);
  if (L.chunk_rows == 0) return B * 2;
  const int chunks = (T + L.chunk_rows - 1) / L.chunk_rows;
  return B * (3 + 4 * chunks);  // 2 x w scaling, redo pass + (sampled scores, thresholds, filter, finalize) per chunk; memsets not counted
}

extern "C" int gw_indexer_scores(const void* q_idx, const void* k_idx, const void* w, int dtype, int B, int T, int S,
                                 int Hi, int Di, float scale, int key_step, float* out, int64_t out_row_stride,
                                 int* status_dev, gw_stream_t stream) {
  int rc = check_common(q_idx, k_idx, w, dtype, B, T, S, Hi, Di);
  if (rc != GW_OK) return rc;
  if (!out || key_step <= 0) return GW_ERR_INVALID_ARG;
  const int m = (S + key_step - 1) / key_step;
  if (out_row_stride < m) return GW_ERR_INVALID_ARG;
  if (T == 0) return GW_OK;
  int sms = 0, dev = 0;
  rc = device_info(&sms, &dev);
  if (rc != GW_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // this debug/verification entry owns a small scratch for w*scale (stream-ordered allocation)
  const int s_pad = static_cast<int>(round_up(static_cast<size_t>(S), BN)) + BN * key_step + BN;
  float4* wsc = nullptr;
  GW_CUDA_TRY(cudaMallocAsync(reinterpret_cast<void**>(&wsc), static_cast<size_t>(s_pad) * 16, st));
  const size_t row_bytes = static_cast<size_t>(Hi) * DI * 2;
  const int nblocks = (T + BM - 1) / BM;
  const int grid = nblocks < sms ? nblocks : sms;
  for (int b = 0; b < B && rc == GW_OK; ++b) {
    const unsigned char* qb = static_cast<const unsigned char*>(q_idx) + static_cast<size_t>(b) * T * row_bytes;
    const unsigned char* kb = static_cast<const unsigned char*>(k_idx) + static_cast<size_t>(b) * S * row_bytes;
    const unsigned char* wb = static_cast<const unsigned char*>(w) + static_cast<size_t>(b) * S * Hi * 2;
    rc = launch_prep_w(wb, dtype, S, Hi, scale, wsc, s_pad, st);
    if (rc != GW_OK) break;
    CUtensorMap mq, mk;
    rc = make_map(&mq, qb, dtype, T, Hi, row_bytes, BM);
    if (rc != GW_OK) break;
    rc = make_map(&mk, kb, dtype, m, Hi, row_bytes * key_step, BN);
    if (rc != GW_OK) break;
    IdxParams p{};
    p.wsc = wsc;
    p.dense_out = out + static_cast<int64_t>(b) * T * out_row_stride;
    p.dense_stride = out_row_stride;
    p.T = T;
    p.S = m;
    p.k = 0;
    p.key_step = key_step;
    p.status = status_dev;
    rc = launch_indexer<MODE_SCORES>(Hi, mq, mk, p, make_idesc_mn(dtype == GW_BF16 ? 1 : 0, BM, BN), grid, dev, st);
  }
  const cudaError_t fe = cudaFreeAsync(wsc, st);
  if (rc == GW_OK && fe != cudaSuccess) return cuda_fail(fe);
  return rc;
}

extern "C" int gw_indexer_topk_fused(const void* q_idx, const void* k_idx, const void* w, int dtype, int B, int T, int S,
                                     int Hi, int Di, float scale, int k, int32_t* out_idx, void* out_scores,
                                     void* workspace, size_t workspace_bytes, int* status_dev, gw_stream_t stream) {
  int rc = check_common(q_idx, k_idx, w, dtype, B, T, S, Hi, Di);
  if (rc != GW_OK) return rc;
  if (!out_idx || k <= 0 || k > S) return GW_ERR_INVALID_ARG;
  if (T == 0) return GW_OK;
  const WsLayout L = ws_layout(T, S, k);
  if (!workspace || workspace_bytes < L.total) return GW_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return GW_ERR_INVALID_ARG;
  int sms = 0, dev = 0;
  rc = device_info(&sms, &dev);
  if (rc != GW_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  float4* wsc = reinterpret_cast<float4*>(ws + L.wsc);
  float* tau0 = reinterpret_cast<float*>(ws + L.tau0);
  float* tau_redo = reinterpret_cast<float*>(ws + L.tau_redo);
  float* smax = reinterpret_cast<float*>(ws + L.smax);
  int* flags = reinterpret_cast<int*>(ws + L.flags);
  int* list_cnt = reinterpret_cast<int*>(ws + L.list_cnt);
  float* wtile = reinterpret_cast<float*>(ws + L.wtile);
  float* sample = reinterpret_cast<float*>(ws + L.sample);
  uint2* cand = reinterpret_cast<uint2*>(ws + L.cand);

  const SamplePlan sp = plan_sample(S, k);
  const size_t row_bytes = static_cast<size_t>(Hi) * DI * 2;
  const int nblocks = (T + BM - 1) / BM;
  int grid = nblocks < sms ? nblocks : sms;
  if (grid > L.slots) grid = L.slots;
  const uint32_t idesc = make_idesc_mn(dtype == GW_BF16 ? 1 : 0, BM, BN);
  const size_t out_es = dtype_size(dtype);

  for (int b = 0; b < B; ++b) {
    const unsigned char* qb = static_cast<const unsigned char*>(q_idx) + static_cast<size_t>(b) * T * row_bytes;
    const unsigned char* kb = static_cast<const unsigned char*>(k_idx) + static_cast<size_t>(b) * S * row_bytes;
    const unsigned char* wb = static_cast<const unsigned char*>(w) + static_cast<size_t>(b) * S * Hi * 2;
    rc = launch_prep_w(wb, dtype, S, Hi, scale, wsc, L.s_pad, st);
    if (rc != GW_OK) return rc;
    CUtensorMap mq, mk;
    rc = make_map(&mq, qb, dtype, T, Hi, row_bytes, BM);
    if (rc != GW_OK) return rc;

    rc = make_map(&mk, kb, dtype, S, Hi, row_bytes, BN);
    if (rc != GW_OK) return rc;
    IdxParams p{};
    p.wsc = wsc;
    p.out_idx = out_idx + static_cast<int64_t>(b) * T * k;
    p.out_scores = out_scores ? static_cast<unsigned char*>(out_scores) + static_cast<size_t>(b) * T * k * out_es : nullptr;
    p.out_dtype = dtype;
    p.cand = cand;
    p.caph = L.caph;
    p.T = T;
    p.S = S;
    p.k = k;
    p.key_step = 1;
    p.status = status_dev;
    p.profile = profiling_enabled();
    if (sp.step == 0) {
      // small key sets: the streaming kernel from tau = -inf
      rc = launch_indexer<MODE_TOPK>(Hi, mq, mk, p, idesc, grid, dev, st);
      if (rc != GW_OK) return rc;
      continue;
    }
    GW_CUDA_TRY(cudaMemsetAsync(flags, 0, static_cast<size_t>(nblocks) * 4, st));
    p.tau_in = tau0;
    p.smax_in = smax;
    p.tau_redo = tau_redo;
    p.block_flags = flags;
    p.list_cnt = list_cnt;
    p.item_counter = reinterpret_cast<int*>(ws + L.counter);
    p.wtile = wtile;
    p.nsplit = L.nsplit;
    p.caph = L.cap_split;
    {
      const int ntiles = (S + FBN - 1) / FBN, n = ntiles * W_TILE_FLOATS;
      if (dtype == GW_BF16)
        prep_w_tiled_kernel<__nv_bfloat16><<<(n + 255) / 256, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(wb), S, Hi, scale, wtile, ntiles);
      else
        prep_w_tiled_kernel<__half><<<(n + 255) / 256, 256, 0, st>>>(reinterpret_cast<const __half*>(wb), S, Hi, scale, wtile, ntiles);
      GW_LAUNCH_CHECK();
    }
    CUtensorMap mkf;
    rc = make_map(&mkf, kb, dtype, S, Hi, row_bytes, FBN);
    if (rc != GW_OK) return rc;
    const uint32_t idesc_fast = make_idesc_mn(dtype == GW_BF16 ? 1 : 0, BM, FBN);
    CUtensorMap ms;
    rc = make_map(&ms, kb, dtype, sp.m, Hi, row_bytes * sp.step, BN);
    if (rc != GW_OK) return rc;
    for (int r0 = 0; r0 < T; r0 += L.chunk_rows) {
      p.row_begin = r0;
      p.row_end = r0 + L.chunk_rows < T ? r0 + L.chunk_rows : T;
      const int cblocks = (p.row_end - p.row_begin + BM - 1) / BM;
      const int crows = p.row_end - p.row_begin;
      {
        // threshold estimate for this chunk of rows: dense scores against every step-th key, then their
        // rank-th largest per row
        IdxParams ps{};
        ps.wsc = wsc;
        ps.dense_out = sample - static_cast<int64_t>(r0) * L.m_pad;  // the kernel indexes rows globally
        ps.dense_stride = L.m_pad;
        ps.T = T;
        ps.S = sp.m;
        ps.key_step = sp.step;
        ps.row_begin = p.row_begin;
        ps.row_end = p.row_end;
        ps.status = status_dev;
        rc = launch_indexer<MODE_SCORES>(Hi, mq, ms, ps, idesc, cblocks < grid ? cblocks : grid, dev, st);
        if (rc != GW_OK) return rc;
        sample_threshold_kernel<<<(crows + FIN_WARPS - 1) / FIN_WARPS, FIN_WARPS * 32, 0, st>>>(sample, sp.m, L.m_pad, crows, sp.rank,
                                                                                             tau0 + r0, smax + r0);
        GW_LAUNCH_CHECK();
      }
      // a shorter last chunk gets a split count of its own (few row blocks on many SMs would otherwise run one
      // full-length wave at low occupancy), provided its lists still fit the buffers sized for a full chunk
      p.nsplit = L.nsplit;
      p.caph = L.cap_split;
      if (crows < L.chunk_rows) {
        const int ns_try = plan_splits(cblocks, sms, (S + FBN - 1) / FBN);
        const int cap_try = seg_capacity(L.caph, ns_try);
        const size_t rows_pad = static_cast<size_t>(cblocks) * BM;
        if (rows_pad * ns_try * F_NQ * cap_try * 8 <= L.cand_bytes && rows_pad * ns_try * F_NQ * 4 <= L.list_cnt_bytes) {
          p.nsplit = ns_try;
          p.caph = cap_try;
        }
      }
      const int citems = cblocks * p.nsplit;
      p.cand = place_lists(ws + L.cand, L.cand_bytes, static_cast<size_t>(p.caph) * 8);
      GW_CUDA_TRY(cudaMemsetAsync(p.item_counter, 0, sizeof(int), st));
      rc = launch_indexer_fast(Hi, mq, mkf, p, idesc_fast, citems < sms ? citems : sms, dev, st);
      if (rc != GW_OK) return rc;
      finalize_lists_kernel<<<(p.row_end - p.row_begin + FIN_WARPS - 1) / FIN_WARPS, FIN_WARPS * 32, 0, st>>>(p);
      GW_LAUNCH_CHECK();
    }
    // blocks with a row whose lists overflowed or came up short (normally none): streaming kernel from -inf
    IdxParams pr = p;
    pr.tau_in = tau_redo;
    pr.smax_in = nullptr;
    pr.tau_redo = nullptr;
    pr.list_cnt = nullptr;
    pr.item_counter = nullptr;
    pr.cand = cand;
    pr.nsplit = 1;
    pr.caph = L.caph;
    pr.row_begin = 0;
    pr.row_end = 0;
    pr.profile = 0;
    rc = launch_indexer<MODE_TOPK>(Hi, mq, mk, pr, idesc, grid, dev, st);
    if (rc != GW_OK) return rc;
  }
  return GW_OK;
}

// ---------------------------------------------------------------------------------------------
// gw_indexer_scores without any allocation: the w*scale table lives in a fixed array of the library image
// ---------------------------------------------------------------------------------------------
namespace gw {
namespace {

static __device__ __align__(256) float4 g_noalloc_wsc[GW_NOALLOC_MAX_KEYS];  // 4 MiB per GPU that loads the library

float4* g_noalloc_ptr[kMaxDevices] = {};  // device address of the array above, per device (host code cannot use the symbol itself)
unsigned g_noalloc_epoch[kMaxDevices] = {};  // value of g_cache_epoch + 1 when the address was looked up (0 = never)

// Host code sees g_noalloc_wsc only as a stand-in symbol; the kernels need its device address, which differs per
// device and is looked up once, with that device current (and again after gw_device_cache_reset).
int noalloc_scratch(float4** out) {
  int dev = 0;
  GW_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return GW_ERR_UNSUPPORTED;
  const unsigned want = g_cache_epoch.load(std::memory_order_acquire) + 1u;
  float4* ptr = nullptr;
  if (__atomic_load_n(&g_noalloc_epoch[dev], __ATOMIC_ACQUIRE) == want) ptr = __atomic_load_n(&g_noalloc_ptr[dev], __ATOMIC_RELAXED);
  if (ptr == nullptr) {
    void* addr = nullptr;
    GW_CUDA_TRY(cudaGetSymbolAddress(&addr, g_noalloc_wsc));
    ptr = static_cast<float4*>(addr);
    __atomic_store_n(&g_noalloc_ptr[dev], ptr, __ATOMIC_RELAXED);  // racing first calls store the same value
    __atomic_store_n(&g_noalloc_epoch[dev], want, __ATOMIC_RELEASE);
  }
  *out = ptr;
  return GW_OK;
}

}  // namespace
}  // namespace gw

extern "C" int gw_indexer_scores_noalloc(const void* q_idx, const void* k_idx, const void* w, int dtype, int B, int T,
                                         int S, int Hi, int Di, float scale, int key_step, float* out,
                                         int64_t out_row_stride, int* status_dev, gw_stream_t stream) {
  int rc = check_common(q_idx, k_idx, w, dtype, B, T, S, Hi, Di);
  if (rc != GW_OK) return rc;
  if (!out || key_step <= 0) return GW_ERR_INVALID_ARG;
  const int m = (S + key_step - 1) / key_step;
  if (out_row_stride < m) return GW_ERR_INVALID_ARG;
  const int64_t s_pad = static_cast<int64_t>(round_up(static_cast<size_t>(S), BN)) + static_cast<int64_t>(BN) * key_step + BN;
  if (s_pad > GW_NOALLOC_MAX_KEYS) return GW_ERR_TOO_LARGE;
  if (T == 0) return GW_OK;
  int sms = 0, dev = 0;
  rc = device_info(&sms, &dev);
  if (rc != GW_OK) return rc;
  float4* wsc = nullptr;
  rc = noalloc_scratch(&wsc);
  if (rc != GW_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t row_bytes = static_cast<size_t>(Hi) * DI * 2;
  const int nblocks = (T + BM - 1) / BM;
  const int grid = nblocks < sms ? nblocks : sms;
  for (int b = 0; b < B; ++b) {
    const unsigned char* qb = static_cast<const unsigned char*>(q_idx) + static_cast<size_t>(b) * T * row_bytes;
    const unsigned char* kb = static_cast<const unsigned char*>(k_idx) + static_cast<size_t>(b) * S * row_bytes;
    const unsigned char* wb = static_cast<const unsigned char*>(w) + static_cast<size_t>(b) * S * Hi * 2;
    // every table entry the score kernel reads (keys 0 .. s_pad-1, zero beyond S) is rewritten here first
    rc = launch_prep_w(wb, dtype, S, Hi, scale, wsc, static_cast<int>(s_pad), st);
    if (rc != GW_OK) return rc;
    CUtensorMap mq, mk;
    rc = make_map(&mq, qb, dtype, T, Hi, row_bytes, BM);
    if (rc != GW_OK) return rc;
    rc = make_map(&mk, kb, dtype, m, Hi, row_bytes * key_step, BN);
    if (rc != GW_OK) return rc;
    IdxParams p{};
    p.wsc = wsc;
    p.dense_out = out + static_cast<int64_t>(b) * T * out_row_stride;
    p.dense_stride = out_row_stride;
    p.T = T;
    p.S = m;
    p.k = 0;
    p.key_step = key_step;
    p.status = status_dev;
    rc = launch_indexer<MODE_SCORES>(Hi, mq, mk, p, make_idesc_mn(dtype == GW_BF16 ? 1 : 0, BM, BN), grid, dev, st);
    if (rc != GW_OK) return rc;
  }
  return GW_OK;
}
