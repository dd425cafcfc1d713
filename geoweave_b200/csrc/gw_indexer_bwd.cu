// Backward of the indexer's selected scores: gradients of q_idx, k_idx and w given the gradient of the top-k scores.
//
//   z[t,j,h]   = scale * <q[t,h], k[idx[t,j],h]>                 score[t,j] = sum_h w[idx[t,j],h] * relu(z[t,j,h])
//   f[t,j,h]   = g[t,j] * w[idx[t,j],h] * [z > 0] * scale         (g = d loss / d score[t,j])
//   dq[t,h]    = sum_j f * k[idx[t,j],h]
//   dk[s,h]    = sum_{(t,j): idx[t,j]=s} f * q[t,h]               dw[s,h] = sum_{(t,j): idx[t,j]=s} g * relu(z)
//
// The reference does this in one Triton kernel per (query, head) with fp32 atomic adds into dk and dw
// (easyvolcap/utils/custom_indexer/sparse_topk_indexer.py:757-895, 1847-2044).  Here, as in the attention backward,
// there is no float atomic: a query kernel forms z, f and dq and leaves {f, g relu(z)} per (query, slot, head) in a
// scratch of one 32-byte line per pair; a key kernel walks each key's (query, slot) pairs in the order of a stable sort
// of the index lists by key (given by the caller) and sums dk and dw in that fixed order.
//
// Both kernels: persistent CTAs, four per SM, of one producer warp and one compute warp per indexer head.  The producer
// gathers 16 rows per batch with one bulk copy each (k rows or q rows of Hi x 64 elements) into a ring of four slots; the
// compute warps run mma.sync m16n8k16 with the vector operand in column 0 of B: z = K_h . q_h from the rows as stored,
// dq^T += K_h^T . f and dk^T += q_h^T . f from ldmatrix.trans of the same rows.  The small per-pair values (the key's w,
// the pair's scratch entry) are read by the compute warps themselves with plain loads issued one batch ahead: as bulk
// copies of 16 or 32 bytes they doubled the number of copies, and the copy rate is what bounds these kernels.
#include "gw_common.cuh"

namespace gw {
namespace {

constexpr int IB_D = 64;
constexpr int IB_BATCH = 16;
constexpr int IB_NB = 4;
constexpr int IB_CTAS_PER_SM = 4;
constexpr int IB_LINE = 32;  // scratch bytes per pair: 4 heads x {f, g relu(z)} fp32

__device__ __forceinline__ void ib_ldmatrix_x4(uint32_t saddr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr));
}
__device__ __forceinline__ void ib_ldmatrix_x4_trans(uint32_t saddr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr));
}
template <typename T>
__device__ __forceinline__ void ib_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void ib_mma<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void ib_mma<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T>
__device__ __forceinline__ uint32_t ib_pack2(float lo, float hi) {
  const T a = from_float<T>(lo), b = from_float<T>(hi);
  return static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&a)) |
         (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&b)) << 16);
}

struct IbShared {
  uint64_t full[IB_NB], empty[IB_NB];
};

struct IbParams {
  const void *q, *k, *w;       // contiguous [B,T,Hi,64], [B,S,Hi,64], [B,S,Hi]
  const int32_t* idx;          // [B,T,K]
  const float* g;              // [B,T,K]
  const int32_t* key_order;    // [B,T*K]
  const int32_t* key_start;    // [B,S+1]
  float2* fr;                  // scratch [B,T,K,4]: {f, g relu(z)}
  void *dq, *dk, *dw;
  int* status;
  int B, T, S, K;
  float scale;
};

// a producer that leaves after a timeout lets the copies it started land first (bounded), so that none arrives in
// shared memory the CTA has already given up
__device__ __forceinline__ void ib_drain(uint64_t* full, uint32_t it) {
  for (uint32_t u = it > IB_NB ? it - IB_NB : 0u; u < it; ++u) mbar_wait_limit(&full[u % IB_NB], (u / IB_NB) & 1u, kDrainLimitNs);
}

template <int HI>
__device__ __forceinline__ void ib_init_barriers(IbShared* sh) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < IB_NB; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], HI);
    }
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------------------------------------
// query kernel: dq and the {f, g relu(z)} scratch
// ------------------------------------------------------------------------------------------------------------------
template <typename T, int HI>
__global__ void __launch_bounds__((HI + 1) * 32, IB_CTAS_PER_SM) indexer_bwd_query_kernel(const IbParams p) {
  constexpr int ROW = HI * IB_D * 2;
  constexpr int RS = ROW + 16;
  constexpr int ROWS = IB_BATCH * RS;
  constexpr int SLOT = ROWS;
  extern __shared__ __align__(128) unsigned char ib_smem[];
  IbShared* sh = reinterpret_cast<IbShared*>(ib_smem + IB_NB * SLOT);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = p.K;
  const int nbatch = (K + IB_BATCH - 1) / IB_BATCH;
  const long long nq = static_cast<long long>(p.B) * p.T;
  ib_init_barriers<HI>(sh);

  if (warp == HI) {
    // producer: lanes 0..15 fetch the k rows of a batch's keys
    const uint32_t S = static_cast<uint32_t>(p.S);
    const int key = lane & 15;
    uint32_t it = 0;
    for (long long qi = blockIdx.x; qi < nq; qi += gridDim.x) {
      const long long b = qi / p.T;
      const int32_t* idx = p.idx + qi * K;
      int id_next = (key < K) ? idx[key] : -1;
      for (int bt = 0; bt < nbatch; ++bt, ++it) {
        const int id = id_next;
        const int kn = (bt + 1) * IB_BATCH + key;
        id_next = (bt + 1 < nbatch && kn < K) ? idx[kn] : -1;
        const bool valid = static_cast<uint32_t>(id) < S;
        const uint32_t slot = it % IB_NB;
        if (!mbar_wait_bounded(&sh->empty[slot], ((it / IB_NB) & 1u) ^ 1u)) {
          ib_drain(sh->full, it);
          report_status(p.status, GW_ERR_TIMEOUT);
          return;
        }
        if (lane == 0) mbar_arrive_expect_tx(&sh->full[slot], IB_BATCH * ROW);
        __syncwarp();
        const long long src = b * p.S + (valid ? id : 0);  // a padding entry gathers key 0 and weighs nothing below
        if (lane < IB_BATCH)
          bulk_g2s(ib_smem + slot * SLOT + key * RS, static_cast<const unsigned char*>(p.k) + src * ROW, ROW, &sh->full[slot]);
      }
    }
    return;
  }

  // compute warp = head
  const int h = warp;
  const int g8 = lane >> 2, t4 = lane & 3;
  const uint32_t row_lane_off = static_cast<uint32_t>(((lane & 7) + 8 * ((lane >> 3) & 1)) * RS + (lane >> 4) * 16);
  const uint32_t trans_lane_off = static_cast<uint32_t>(((lane & 7) + 8 * (lane >> 4)) * RS + ((lane >> 3) & 1) * 16);
  const uint32_t smem_base = smem_u32(ib_smem);
  uint32_t it = 0;

  for (long long qi = blockIdx.x; qi < nq; qi += gridDim.x) {
    const uint32_t* qrow = reinterpret_cast<const uint32_t*>(static_cast<const T*>(p.q) + (qi * HI + h) * IB_D);
    uint32_t qb[4][2];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      qb[ks][0] = (lane < 4) ? qrow[ks * 8 + t4] : 0u;
      qb[ks][1] = (lane < 4) ? qrow[ks * 8 + t4 + 4] : 0u;
    }
    float acc[4][4];
#pragma unroll
    for (int db = 0; db < 4; ++db)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[db][r] = 0.f;
    const float* gq = p.g + qi * K;
    const int32_t* iq = p.idx + qi * K;
    const T* wb = static_cast<const T*>(p.w) + (qi / p.T) * p.S * HI + h;
    float2* frq = p.fr + qi * K * 4;
    // this lane's two keys of a batch (g8 and g8 + 8): index two batches ahead, weight and gradient one batch ahead
    const uint32_t S = static_cast<uint32_t>(p.S);
    auto load_id = [&](int j) { return j < K ? iq[j] : -1; };
    auto load_w = [&](int id) { return static_cast<uint32_t>(id) < S ? to_float(wb[static_cast<long long>(id) * HI]) : 0.f; };
    int id0n = load_id(g8), id1n = load_id(g8 + 8);
    int id0nn = load_id(g8 + IB_BATCH), id1nn = load_id(g8 + 8 + IB_BATCH);
    float g0n = (g8 < K) ? gq[g8] : 0.f, g1n = (g8 + 8 < K) ? gq[g8 + 8] : 0.f;
    float w0n = load_w(id0n), w1n = load_w(id1n);

    for (int bt = 0; bt < nbatch; ++bt, ++it) {
      const int j0 = bt * IB_BATCH + g8, j1 = j0 + 8;
      const float g0 = g0n, g1 = g1n, w0 = w0n, w1 = w1n;
      const bool ok0 = static_cast<uint32_t>(id0n) < S, ok1 = static_cast<uint32_t>(id1n) < S;
      id0n = id0nn;
      id1n = id1nn;
      id0nn = load_id(j0 + 2 * IB_BATCH);
      id1nn = load_id(j1 + 2 * IB_BATCH);
      w0n = load_w(id0n);
      w1n = load_w(id1n);
      g0n = (j0 + IB_BATCH < K) ? gq[j0 + IB_BATCH] : 0.f;
      g1n = (j1 + IB_BATCH < K) ? gq[j1 + IB_BATCH] : 0.f;
      const uint32_t slot = it % IB_NB;
      if (!mbar_wait_bounded(&sh->full[slot], (it / IB_NB) & 1u)) {
        report_status(p.status, GW_ERR_TIMEOUT);
        return;
      }
      const uint32_t kbase = smem_base + slot * SLOT;
      float z[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t a[4];
        ib_ldmatrix_x4(kbase + row_lane_off + h * (IB_D * 2) + ks * 32, a);
        ib_mma<T>(z, a, qb[ks][0], qb[ks][1]);
      }
      // column 0 lives in the lanes with t4 == 0: element 0 = key g8, element 2 = key g8 + 8
      const float z0 = z[0] * p.scale, z1 = z[2] * p.scale;
      const bool on0 = ok0 && z0 > 0.f, on1 = ok1 && z1 > 0.f;
      const float f0 = on0 ? g0 * w0 * p.scale : 0.f, f1 = on1 ? g1 * w1 * p.scale : 0.f;
      const float r0 = on0 ? g0 * z0 : 0.f, r1 = on1 ? g1 * z1 : 0.f;
      if (t4 == 0) {
        if (j0 < K) frq[static_cast<long long>(j0) * 4 + h] = make_float2(f0, r0);
        if (j1 < K) frq[static_cast<long long>(j1) * 4 + h] = make_float2(f1, r1);
      }
      // B fragment of f: lanes 0..3 need keys 2t,2t+1 (word 0) and 2t+8,2t+9 (word 1); key kk sits in lane 4 kk
      const float fa = __shfl_sync(0xffffffffu, f0, 8 * t4);
      const float fb = __shfl_sync(0xffffffffu, f0, 8 * t4 + 4);
      const float fc = __shfl_sync(0xffffffffu, f1, 8 * t4);
      const float fd = __shfl_sync(0xffffffffu, f1, 8 * t4 + 4);
      const uint32_t fb0 = (lane < 4) ? ib_pack2<T>(fa, fb) : 0u;
      const uint32_t fb1 = (lane < 4) ? ib_pack2<T>(fc, fd) : 0u;
#pragma unroll
      for (int db = 0; db < 4; ++db) {
        uint32_t a[4];
        ib_ldmatrix_x4_trans(kbase + trans_lane_off + h * (IB_D * 2) + db * 32, a);
        ib_mma<T>(acc[db], a, fb0, fb1);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->empty[slot]);
    }

    if (t4 == 0) {  // these lanes hold dims g8 and g8+8 of every 16-dim block
      T* dq = static_cast<T*>(p.dq) + (qi * HI + h) * IB_D;
#pragma unroll
      for (int db = 0; db < 4; ++db) {
        dq[db * 16 + g8] = from_float<T>(acc[db][0]);
        dq[db * 16 + g8 + 8] = from_float<T>(acc[db][2]);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// key kernel: dk and dw
// ------------------------------------------------------------------------------------------------------------------
template <typename T, int HI>
__global__ void __launch_bounds__((HI + 1) * 32, IB_CTAS_PER_SM) indexer_bwd_key_kernel(const IbParams p) {
  constexpr int ROW = HI * IB_D * 2;
  constexpr int RS = ROW + 16;
  constexpr int ROWS = IB_BATCH * RS;
  constexpr int SLOT = ROWS;
  extern __shared__ __align__(128) unsigned char ib_smem[];
  IbShared* sh = reinterpret_cast<IbShared*>(ib_smem + IB_NB * SLOT);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = p.K;
  const long long nkeys = static_cast<long long>(p.B) * p.S;
  const long long TK = static_cast<long long>(p.T) * K;
  ib_init_barriers<HI>(sh);

  if (warp == HI) {
    // producer: lanes 0..15 fetch the q rows of a batch's pairs
    const int ent = lane & 15;
    uint32_t it = 0;
    for (long long ki = blockIdx.x; ki < nkeys; ki += gridDim.x) {
      const long long b = ki / p.S, s = ki % p.S;
      const int e0 = p.key_start[b * (p.S + 1) + s], e1 = p.key_start[b * (p.S + 1) + s + 1];
      const int n = e1 - e0;
      if (n <= 0) continue;
      const int nb = (n + IB_BATCH - 1) / IB_BATCH;
      const int32_t* order = p.key_order + b * TK + e0;
      const int f_first = order[0];
      int f_next = (ent < n) ? order[ent] : f_first;
      for (int bt = 0; bt < nb; ++bt, ++it) {
        const int f = f_next;  // rows past the end of the list repeat the first pair (finite values, weight zero below)
        const int en = (bt + 1) * IB_BATCH + ent;
        f_next = (en < n) ? order[en] : f_first;
        const long long tq = f / K;
        const uint32_t slot = it % IB_NB;
        if (!mbar_wait_bounded(&sh->empty[slot], ((it / IB_NB) & 1u) ^ 1u)) {
          ib_drain(sh->full, it);
          report_status(p.status, GW_ERR_TIMEOUT);
          return;
        }
        if (lane == 0) mbar_arrive_expect_tx(&sh->full[slot], IB_BATCH * ROW);
        __syncwarp();
        if (lane < IB_BATCH)
          bulk_g2s(ib_smem + slot * SLOT + ent * RS, static_cast<const unsigned char*>(p.q) + (b * p.T + tq) * ROW, ROW,
                   &sh->full[slot]);
      }
    }
    return;
  }

  const int h = warp;
  const int g8 = lane >> 2, t4 = lane & 3;
  const uint32_t trans_lane_off = static_cast<uint32_t>(((lane & 7) + 8 * (lane >> 4)) * RS + ((lane >> 3) & 1) * 16);
  const uint32_t smem_base = smem_u32(ib_smem);
  uint32_t it = 0;

  for (long long ki = blockIdx.x; ki < nkeys; ki += gridDim.x) {
    const long long b = ki / p.S, s = ki % p.S;
    const int e0 = p.key_start[b * (p.S + 1) + s], e1 = p.key_start[b * (p.S + 1) + s + 1];
    const int n = e1 - e0;
    const int nb = n > 0 ? (n + IB_BATCH - 1) / IB_BATCH : 0;
    float acc[4][4];
#pragma unroll
    for (int db = 0; db < 4; ++db)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[db][r] = 0.f;
    float dw_part = 0.f;
    // lane l < 16 owns pair l of a batch: its position two batches ahead, its scratch entry {f, g relu(z)} one batch ahead
    const int32_t* order = p.key_order + b * TK + e0;
    const float2* frb = p.fr + b * TK * 4 + h;
    const int pl = lane & 15;
    auto load_f = [&](int e) { return e < n ? order[e] : -1; };
    auto load_fr = [&](int f) { return f >= 0 ? frb[static_cast<long long>(f) * 4] : make_float2(0.f, 0.f); };
    int fn = load_f(pl), fnn = load_f(pl + IB_BATCH);
    float2 frn = load_fr(fn);

    for (int bt = 0; bt < nb; ++bt, ++it) {
      const float2 fr = frn;   // zero for a pair past the end of the list
      fn = fnn;
      fnn = load_f((bt + 2) * IB_BATCH + pl);
      frn = load_fr(fn);
      const uint32_t slot = it % IB_NB;
      if (!mbar_wait_bounded(&sh->full[slot], (it / IB_NB) & 1u)) {
        report_status(p.status, GW_ERR_TIMEOUT);
        return;
      }
      const uint32_t qbase = smem_base + slot * SLOT;
      if (lane < IB_BATCH) dw_part += fr.y;
      // B fragment of f: lanes 0..3 need pairs 2t,2t+1 (word 0) and 2t+8,2t+9 (word 1); pair l sits in lane l
      const float fa = __shfl_sync(0xffffffffu, fr.x, 2 * t4);
      const float fb = __shfl_sync(0xffffffffu, fr.x, 2 * t4 + 1);
      const float fc = __shfl_sync(0xffffffffu, fr.x, 2 * t4 + 8);
      const float fd = __shfl_sync(0xffffffffu, fr.x, 2 * t4 + 9);
      const uint32_t fb0 = (lane < 4) ? ib_pack2<T>(fa, fb) : 0u;
      const uint32_t fb1 = (lane < 4) ? ib_pack2<T>(fc, fd) : 0u;
#pragma unroll
      for (int db = 0; db < 4; ++db) {
        uint32_t a[4];
        ib_ldmatrix_x4_trans(qbase + trans_lane_off + h * (IB_D * 2) + db * 32, a);
        ib_mma<T>(acc[db], a, fb0, fb1);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->empty[slot]);
    }

#pragma unroll
    for (int d = 16; d > 0; d >>= 1) dw_part += __shfl_xor_sync(0xffffffffu, dw_part, d);
    if (lane == 0) static_cast<T*>(p.dw)[ki * HI + h] = from_float<T>(dw_part);
    if (t4 == 0) {
      T* dk = static_cast<T*>(p.dk) + (ki * HI + h) * IB_D;
#pragma unroll
      for (int db = 0; db < 4; ++db) {
        dk[db * 16 + g8] = from_float<T>(acc[db][0]);
        dk[db * 16 + g8 + 8] = from_float<T>(acc[db][2]);
      }
    }
  }
}

template <typename T, int HI>
int launch_indexer_bwd(const IbParams& p, cudaStream_t st) {
  constexpr size_t ROWS = static_cast<size_t>(IB_BATCH) * (HI * IB_D * 2 + 16);
  constexpr size_t SMEM_Q = IB_NB * ROWS + sizeof(IbShared);
  constexpr size_t SMEM_K = IB_NB * ROWS + sizeof(IbShared);
  int dev = 0;
  DeviceFacts facts;
  int rc = device_facts(&dev, &facts);
  if (rc != GW_OK) return rc;
  static OncePerDevice once_q, once_k;
  rc = ensure_dynamic_smem(indexer_bwd_query_kernel<T, HI>, SMEM_Q, once_q, dev);
  if (rc != GW_OK) return rc;
  rc = ensure_dynamic_smem(indexer_bwd_key_kernel<T, HI>, SMEM_K, once_k, dev);
  if (rc != GW_OK) return rc;
  const long long nk = static_cast<long long>(p.B) * p.S, nq = static_cast<long long>(p.B) * p.T;
  const long long cap = static_cast<long long>(facts.sms) * IB_CTAS_PER_SM;
  indexer_bwd_query_kernel<T, HI><<<static_cast<int>(nq < cap ? nq : cap), (HI + 1) * 32, SMEM_Q, st>>>(p);
  GW_LAUNCH_CHECK();
  indexer_bwd_key_kernel<T, HI><<<static_cast<int>(nk < cap ? nk : cap), (HI + 1) * 32, SMEM_K, st>>>(p);
  GW_LAUNCH_CHECK();
  return GW_OK;
}

template <typename T>
int dispatch_heads(const IbParams& p, int Hi, cudaStream_t st) {
  switch (Hi) {
    case 1: return launch_indexer_bwd<T, 1>(p, st);
    case 2: return launch_indexer_bwd<T, 2>(p, st);
    case 3: return launch_indexer_bwd<T, 3>(p, st);
    case 4: return launch_indexer_bwd<T, 4>(p, st);
    default: return GW_ERR_UNSUPPORTED;
  }
}

}  // namespace
}  // namespace gw

using namespace gw;

extern "C" size_t gw_indexer_topk_bwd_workspace_bytes(int B, int T, int S, int K) {
  if (B <= 0 || T <= 0 || S <= 0 || K <= 0) return 0;
  (void)S;
  return round_up(static_cast<size_t>(B) * T * K * IB_LINE, 256);
}

extern "C" int gw_indexer_topk_bwd(const void* q, const void* k, const void* w, const int32_t* topk_idx, const float* grad_scores,
                                   const int32_t* key_order, const int32_t* key_start, int dtype, int B, int T, int S, int Hi,
                                   int Di, int K, float scale, void* dq, void* dk, void* dw, void* workspace,
                                   size_t workspace_bytes, int* status_dev, gw_stream_t stream) {
  if (!q || !k || !w || !topk_idx || !grad_scores || !key_order || !key_start || !dq || !dk || !dw || !status_dev)
    return GW_ERR_INVALID_ARG;
  if (B <= 0 || T < 0 || S <= 0 || Hi <= 0 || K <= 0) return GW_ERR_INVALID_ARG;
  if (dtype != GW_BF16 && dtype != GW_F16) return GW_ERR_UNSUPPORTED;
  if (Di != IB_D || Hi > 4) return GW_ERR_UNSUPPORTED;
  if (static_cast<int64_t>(T) * K > 0x7fffffff) return GW_ERR_UNSUPPORTED;
  for (const void* ptr : {q, k, static_cast<const void*>(dq), static_cast<const void*>(dk)})
    if (!aligned16(ptr)) return GW_ERR_INVALID_ARG;
  if (T == 0) return GW_OK;
  const size_t need = gw_indexer_topk_bwd_workspace_bytes(B, T, S, K);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return GW_ERR_WORKSPACE;
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  IbParams p;
  p.q = q; p.k = k; p.w = w; p.idx = topk_idx; p.g = grad_scores; p.key_order = key_order; p.key_start = key_start;
  p.fr = reinterpret_cast<float2*>(ws);
  p.dq = dq; p.dk = dk; p.dw = dw; p.status = status_dev; p.B = B; p.T = T; p.S = S; p.K = K; p.scale = scale;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return dtype == GW_BF16 ? dispatch_heads<__nv_bfloat16>(p, Hi, st) : dispatch_heads<__half>(p, Hi, st);
}
