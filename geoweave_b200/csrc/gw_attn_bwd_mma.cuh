// Backward of the sparse attention, tensor-core form for 16-bit inputs with token-major rows of 8 or 16 heads x 64.
// (Included by gw_attn_bwd.cu.)
//
// Both kernels are the forward's machine turned to other operands: one persistent CTA per SM, four producer warps that
// gather whole token rows with one bulk copy each into a ring of three batch slots (16 rows per tensor per batch, rows
// padded by 16 bytes for conflict-free ldmatrix), eight compute warps that split the heads and run mma.sync m16n8k16
// with the vector operand in column 0 of B.
//
//   query kernel (one query at a time, batches of 16 selected keys; gathers K rows and V rows)
//     s  = K_h . q_h            p  = exp2(s * scale * log2e - lse)            (A = key rows as stored)
//     dp = V_h . dO_h           ds = p (dp - delta) scale, delta = <dO_h, o_h>   (A = value rows as stored)
//     dQ_h^T += K_h^T . ds                                                   (A = ldmatrix.trans of the key rows)
//     and one 32-bit word {p, ds} (both rounded to the input type, as the MMA operands are) per (query, slot, head)
//     into a scratch of the shape [B,T,K,H]: all heads of an entry lie in one 64-byte line.
//   key kernel (one key at a time, batches of 16 of the (query, slot) pairs that selected it; gathers q rows, dO rows
//     and the pairs' scratch lines)
//     dK_h^T += q_h^T . ds      dV_h^T += dO_h^T . p                          (A = ldmatrix.trans of the gathered rows)
//   The pairs of a key come from a stable sort of the index lists by key, so every sum runs in a fixed order.
//   With a gradient g = d_attn_sum[t,j] arriving through attn_sum (the same for all heads of a pair) dp becomes dp + g and
//   delta becomes delta + sum_j p g.  That sum needs p before ds can be formed, so a pre-pass of the query kernel (MODE 2:
//   gathers the K rows only, s and p as above) writes it per (query, head); the main pass (MODE 1) reads it back.
#pragma once

namespace gw {
namespace {

constexpr int BM_WARPS = 8;    // compute warps
constexpr int BM_PROD = 4;     // producer warps
constexpr int BM_THREADS = (BM_WARPS + BM_PROD) * 32;
constexpr int BM_BATCH = 16;   // rows per batch (M of the row-wise MMAs, K of the transposed ones)
constexpr int BM_NB = 3;       // batch slots
constexpr int BM_KPP = BM_BATCH / BM_PROD;  // rows per producer warp

__device__ __forceinline__ void bm_ldmatrix_x4(uint32_t saddr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr));
}
__device__ __forceinline__ void bm_ldmatrix_x4_trans(uint32_t saddr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr));
}
template <typename T>
__device__ __forceinline__ void bm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void bm_mma<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void bm_mma<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T>
__device__ __forceinline__ uint32_t bm_pack2(float lo, float hi) {
  const T a = from_float<T>(lo), b = from_float<T>(hi);
  return static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&a)) |
         (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&b)) << 16);
}

struct BmShared {
  uint64_t full[BM_NB], empty[BM_NB];
  uint32_t mask[BM_NB][BM_PROD];  // query kernel: validity bits of each producer's four keys
};

struct BwdMmaParams {
  const void *q, *k, *v, *o, *d_out;   // contiguous [B,T,H,64] / [B,S,H,64]
  const int32_t* pos;                  // [B,T,K]
  const float* lse;                    // [B,H,T]
  const float* d_attn_sum;             // [B,T,K] or null
  float* delta_extra;                  // [B,T,H]: sum_j p d_attn_sum (written by MODE 2, read by MODE 1)
  const int32_t* key_order;            // [B,T*K]
  const int32_t* key_start;            // [B,S+1]
  uint32_t* pds;                       // scratch [B,T,K,H]: low half p, high half ds, both of the input type
  void *dq, *dk, *dv;
  int* status;
  int B, T, S, H, K;
  float scale;
};

// a producer that leaves after a timeout lets the copies it started land first (bounded), so that none arrives in
// shared memory the CTA has already given up
__device__ __forceinline__ void bm_drain(uint64_t* full, uint32_t it) {
  for (uint32_t u = it > BM_NB ? it - BM_NB : 0u; u < it; ++u) mbar_wait_limit(&full[u % BM_NB], (u / BM_NB) & 1u, kDrainLimitNs);
}

__device__ __forceinline__ void bm_init_barriers(BmShared* sh) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < BM_NB; ++s) {
      mbar_init(&sh->full[s], BM_PROD);
      mbar_init(&sh->empty[s], BM_WARPS);
    }
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------------------------------------
// query kernel: dQ and the {p, ds} scratch
// ------------------------------------------------------------------------------------------------------------------
// MODE 0: dQ and the scratch.  MODE 1: the same with d_attn_sum.  MODE 2: only sum_j p d_attn_sum per (query, head).
template <typename T, int HPW, int MODE>
__global__ void __launch_bounds__(BM_THREADS, 1) attn_bwd_query_mma_kernel(const BwdMmaParams p) {
  constexpr int D = 64;
  constexpr int H = BM_WARPS * HPW;
  constexpr int ROW = H * D * 2;
  constexpr int RS = ROW + 16;
  constexpr int TENS = BM_BATCH * RS;
  constexpr int SLOT = 2 * TENS;
  extern __shared__ __align__(128) unsigned char bm_smem[];
  BmShared* sh = reinterpret_cast<BmShared*>(bm_smem + BM_NB * SLOT);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = p.K;
  const int nbatch = (K + BM_BATCH - 1) / BM_BATCH;
  const long long nq = static_cast<long long>(p.B) * p.T;
  bm_init_barriers(sh);

  if (warp >= BM_WARPS) {
    // producers: each warp gathers 4 of a batch's 16 keys, the K row and the V row of each
    const uint32_t S = static_cast<uint32_t>(p.S);
    const int pw = warp - BM_WARPS;
    const int key = pw * BM_KPP + (lane % BM_KPP), tens = (lane / BM_KPP) & 1;
    uint32_t it = 0;
    for (long long qi = blockIdx.x; qi < nq; qi += gridDim.x) {
      const long long b = qi / p.T;
      const int32_t* pos = p.pos + qi * K;
      const unsigned char* src0 = static_cast<const unsigned char*>(tens ? p.v : p.k) + b * p.S * ROW;
      int id_next = (key < K) ? pos[key] : -1;
      for (int bt = 0; bt < nbatch; ++bt, ++it) {
        const int id = id_next;
        const int kn = (bt + 1) * BM_BATCH + key;
        id_next = (bt + 1 < nbatch && kn < K) ? pos[kn] : -1;
        const bool valid = static_cast<uint32_t>(id) < S;
        const uint32_t mask = __ballot_sync(0xffffffffu, valid) & ((1u << BM_KPP) - 1u);
        const uint32_t slot = it % BM_NB;
        if (!mbar_wait_bounded(&sh->empty[slot], ((it / BM_NB) & 1u) ^ 1u)) {
          bm_drain(sh->full, it);
          report_status(p.status, GW_ERR_TIMEOUT);
          return;
        }
        if (lane == 0) {
          sh->mask[slot][pw] = mask;
          mbar_arrive_expect_tx(&sh->full[slot], (MODE == 2 ? 1 : 2) * BM_KPP * ROW);
        }
        __syncwarp();
        // a padding entry gathers key 0 (finite values) and weighs nothing below; the pre-pass needs the K rows only
        if (lane < (MODE == 2 ? 1 : 2) * BM_KPP)
          bulk_g2s(bm_smem + slot * SLOT + tens * TENS + key * RS, src0 + static_cast<int64_t>(valid ? id : 0) * ROW, ROW,
                   &sh->full[slot]);
      }
    }
    return;
  }

  // compute warps
  const int g = lane >> 2, t4 = lane & 3;
  const int h0 = warp * HPW;
  const uint32_t row_lane_off = static_cast<uint32_t>(((lane & 7) + 8 * ((lane >> 3) & 1)) * RS + (lane >> 4) * 16);
  const uint32_t trans_lane_off = static_cast<uint32_t>(((lane & 7) + 8 * (lane >> 4)) * RS + ((lane >> 3) & 1) * 16);
  const uint32_t smem_base = smem_u32(bm_smem);
  const float log2e = 1.4426950408889634f;
  const float scale_log2 = p.scale * log2e;
  uint32_t it = 0;

  for (long long qi = blockIdx.x; qi < nq; qi += gridDim.x) {
    const long long b = qi / p.T;
    const long long t = qi % p.T;
    const uint32_t* qrow = reinterpret_cast<const uint32_t*>(static_cast<const T*>(p.q) + qi * (H * D));
    const uint32_t* dorow = reinterpret_cast<const uint32_t*>(static_cast<const T*>(p.d_out) + qi * (H * D));
    const uint32_t* orow = reinterpret_cast<const uint32_t*>(static_cast<const T*>(p.o) + qi * (H * D));
    // B fragments of q and dO: column 0 only, i.e. lanes 0..3 hold the 32-bit words (two elements) of the rows
    uint32_t qb[HPW][4][2], dob[HPW][4][2];
    float delta[HPW], lse2[HPW];
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
      const int h = h0 + i;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        qb[i][ks][0] = (lane < 4) ? qrow[h * 32 + ks * 8 + t4] : 0u;
        qb[i][ks][1] = (lane < 4) ? qrow[h * 32 + ks * 8 + t4 + 4] : 0u;
        dob[i][ks][0] = (lane < 4) ? dorow[h * 32 + ks * 8 + t4] : 0u;
        dob[i][ks][1] = (lane < 4) ? dorow[h * 32 + ks * 8 + t4 + 4] : 0u;
      }
      float a0, a1, c0, c1;
      unpack2<T>(dorow[h * 32 + lane], a0, a1);
      unpack2<T>(orow[h * 32 + lane], c0, c1);
      float dl = fmaf(a0, c0, a1 * c1);
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) dl += __shfl_xor_sync(0xffffffffu, dl, d);
      delta[i] = MODE == 1 ? dl + p.delta_extra[qi * H + h] : dl;
      lse2[i] = p.lse[(b * H + h) * static_cast<long long>(p.T) + t] * log2e;
    }
    float corr[HPW];
#pragma unroll
    for (int i = 0; i < HPW; ++i) corr[i] = 0.f;
    const float* da = MODE != 0 ? p.d_attn_sum + qi * K : nullptr;
    float da0n = 0.f, da1n = 0.f;  // this lane's two keys of the next batch (g and g + 8)
    if (MODE != 0) {
      da0n = g < K ? da[g] : 0.f;
      da1n = g + 8 < K ? da[g + 8] : 0.f;
    }
    float acc[HPW][4][4];
#pragma unroll
    for (int i = 0; i < HPW; ++i)
#pragma unroll
      for (int db = 0; db < 4; ++db)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[i][db][r] = 0.f;
    uint32_t* pds_q = p.pds + qi * K * H;

    for (int bt = 0; bt < nbatch; ++bt, ++it) {
      const uint32_t slot = it % BM_NB;
      if (!mbar_wait_bounded(&sh->full[slot], (it / BM_NB) & 1u)) {
        report_status(p.status, GW_ERR_TIMEOUT);
        return;
      }
      uint32_t mask = 0;
#pragma unroll
      for (int pw = 0; pw < BM_PROD; ++pw) mask |= sh->mask[slot][pw] << (pw * BM_KPP);
      const uint32_t kbase = smem_base + slot * SLOT, vbase = kbase + TENS;
      const bool ok0 = (mask >> g) & 1u, ok1 = (mask >> (g + 8)) & 1u;  // keys g and g+8 of the batch
      const int j0 = bt * BM_BATCH + g, j1 = j0 + 8;
      const float da0 = da0n, da1 = da1n;
      if (MODE != 0) {
        da0n = j0 + BM_BATCH < K ? da[j0 + BM_BATCH] : 0.f;
        da1n = j1 + BM_BATCH < K ? da[j1 + BM_BATCH] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < HPW; ++i) {
        const int h = h0 + i;
        float s[4] = {0.f, 0.f, 0.f, 0.f}, dp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          uint32_t a[4];
          bm_ldmatrix_x4(kbase + row_lane_off + h * (D * 2) + ks * 32, a);
          bm_mma<T>(s, a, qb[i][ks][0], qb[i][ks][1]);
          if (MODE != 2) {
            bm_ldmatrix_x4(vbase + row_lane_off + h * (D * 2) + ks * 32, a);
            bm_mma<T>(dp, a, dob[i][ks][0], dob[i][ks][1]);
          }
        }
        // column 0 lives in the lanes with t4 == 0: element 0 = key g, element 2 = key g + 8
        const float p0 = ok0 ? exp2f(fmaf(s[0], scale_log2, -lse2[i])) : 0.f;
        const float p1 = ok1 ? exp2f(fmaf(s[2], scale_log2, -lse2[i])) : 0.f;
        if (MODE == 2) {
          corr[i] = fmaf(p0, da0, fmaf(p1, da1, corr[i]));
          continue;
        }
        const float ds0 = p0 * (dp[0] + da0 - delta[i]) * p.scale;
        const float ds1 = p1 * (dp[2] + da1 - delta[i]) * p.scale;
        const uint32_t w0 = bm_pack2<T>(p0, ds0), w1 = bm_pack2<T>(p1, ds1);
        if (t4 == 0) {
          if (j0 < K) pds_q[static_cast<long long>(j0) * H + h] = w0;
          if (j1 < K) pds_q[static_cast<long long>(j1) * H + h] = w1;
        }
        // B fragment of ds: lanes 0..3 need keys 2t,2t+1 (word 0) and 2t+8,2t+9 (word 1); key kk sits in lane 4 kk
        const uint32_t wa = __shfl_sync(0xffffffffu, w0, 8 * t4);
        const uint32_t wb = __shfl_sync(0xffffffffu, w0, 8 * t4 + 4);
        const uint32_t wc = __shfl_sync(0xffffffffu, w1, 8 * t4);
        const uint32_t wd = __shfl_sync(0xffffffffu, w1, 8 * t4 + 4);
        const uint32_t dsb0 = (lane < 4) ? __byte_perm(wa, wb, 0x7632) : 0u;
        const uint32_t dsb1 = (lane < 4) ? __byte_perm(wc, wd, 0x7632) : 0u;
#pragma unroll
        for (int db = 0; db < 4; ++db) {
          uint32_t a[4];
          bm_ldmatrix_x4_trans(kbase + trans_lane_off + h * (D * 2) + db * 32, a);
          bm_mma<T>(acc[i][db], a, dsb0, dsb1);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->empty[slot]);
    }

    if (MODE == 2) {
      // the lanes with t4 == 0 hold the sums of their two keys per batch: add them up over g
#pragma unroll
      for (int i = 0; i < HPW; ++i) {
        float c = t4 == 0 ? corr[i] : 0.f;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) c += __shfl_xor_sync(0xffffffffu, c, d);
        if (lane == 0) p.delta_extra[qi * H + h0 + i] = c;
      }
      continue;
    }
    // lanes with t4 == 0 hold dims g and g+8 of every 16-dim block
    if (t4 == 0) {
#pragma unroll
      for (int i = 0; i < HPW; ++i) {
        T* dq = static_cast<T*>(p.dq) + qi * (H * D) + (h0 + i) * D;
#pragma unroll
        for (int db = 0; db < 4; ++db) {
          dq[db * 16 + g] = from_float<T>(acc[i][db][0]);
          dq[db * 16 + g + 8] = from_float<T>(acc[i][db][2]);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// key kernel: dK and dV
// ------------------------------------------------------------------------------------------------------------------
template <typename T, int HPW>
__global__ void __launch_bounds__(BM_THREADS, 1) attn_bwd_key_mma_kernel(const BwdMmaParams p) {
  constexpr int D = 64;
  constexpr int H = BM_WARPS * HPW;
  constexpr int ROW = H * D * 2;
  constexpr int RS = ROW + 16;
  constexpr int TENS = BM_BATCH * RS;
  constexpr int LINE = H * 4;                 // one pair's scratch words, all heads
  constexpr int SLOT = 2 * TENS + BM_BATCH * LINE;
  extern __shared__ __align__(128) unsigned char bm_smem[];
  BmShared* sh = reinterpret_cast<BmShared*>(bm_smem + BM_NB * SLOT);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = p.K;
  const long long nkeys = static_cast<long long>(p.B) * p.S;
  const long long TK = static_cast<long long>(p.T) * K;
  bm_init_barriers(sh);

  if (warp >= BM_WARPS) {
    // producers: each warp gathers 4 of a batch's 16 pairs: the q row, the dO row and the scratch line of each
    const int pw = warp - BM_WARPS;
    const int ent = pw * BM_KPP + (lane % BM_KPP), role = lane / BM_KPP;  // role 0: q, 1: dO, 2: scratch, others idle
    uint32_t it = 0;
    for (long long ki = blockIdx.x; ki < nkeys; ki += gridDim.x) {
      const long long b = ki / p.S, s = ki % p.S;
      const int e0 = p.key_start[b * (p.S + 1) + s], e1 = p.key_start[b * (p.S + 1) + s + 1];
      const int n = e1 - e0;
      if (n <= 0) continue;
      const int nb = (n + BM_BATCH - 1) / BM_BATCH;
      const int32_t* order = p.key_order + b * TK + e0;
      const int f_first = order[0];
      int f_next = (ent < n) ? order[ent] : f_first;
      for (int bt = 0; bt < nb; ++bt, ++it) {
        const int f = f_next;  // rows past the end of the list repeat the first pair (finite values, weight zero below)
        const int en = (bt + 1) * BM_BATCH + ent;
        f_next = (en < n) ? order[en] : f_first;
        const long long tq = f / K;
        const uint32_t slot = it % BM_NB;
        if (!mbar_wait_bounded(&sh->empty[slot], ((it / BM_NB) & 1u) ^ 1u)) {
          bm_drain(sh->full, it);
          report_status(p.status, GW_ERR_TIMEOUT);
          return;
        }
        if (lane == 0) mbar_arrive_expect_tx(&sh->full[slot], BM_KPP * (2 * ROW + LINE));
        __syncwarp();
        unsigned char* dst = bm_smem + slot * SLOT;
        if (role == 0)
          bulk_g2s(dst + ent * RS, static_cast<const unsigned char*>(p.q) + (b * p.T + tq) * ROW, ROW, &sh->full[slot]);
        else if (role == 1)
          bulk_g2s(dst + TENS + ent * RS, static_cast<const unsigned char*>(p.d_out) + (b * p.T + tq) * ROW, ROW, &sh->full[slot]);
        else if (role == 2)
          bulk_g2s(dst + 2 * TENS + ent * LINE, reinterpret_cast<const unsigned char*>(p.pds) + (b * TK + f) * LINE, LINE,
                   &sh->full[slot]);
      }
    }
    return;
  }

  // compute warps
  const int g = lane >> 2, t4 = lane & 3;
  const int h0 = warp * HPW;
  const uint32_t trans_lane_off = static_cast<uint32_t>(((lane & 7) + 8 * (lane >> 4)) * RS + ((lane >> 3) & 1) * 16);
  const uint32_t smem_base = smem_u32(bm_smem);
  uint32_t it = 0;

  for (long long ki = blockIdx.x; ki < nkeys; ki += gridDim.x) {
    const long long b = ki / p.S, s = ki % p.S;
    const int e0 = p.key_start[b * (p.S + 1) + s], e1 = p.key_start[b * (p.S + 1) + s + 1];
    const int n = e1 - e0;
    const int nb = n > 0 ? (n + BM_BATCH - 1) / BM_BATCH : 0;
    float accK[HPW][4][4], accV[HPW][4][4];
#pragma unroll
    for (int i = 0; i < HPW; ++i)
#pragma unroll
      for (int db = 0; db < 4; ++db)
#pragma unroll
        for (int r = 0; r < 4; ++r) accK[i][db][r] = accV[i][db][r] = 0.f;

    for (int bt = 0; bt < nb; ++bt, ++it) {
      const uint32_t slot = it % BM_NB;
      if (!mbar_wait_bounded(&sh->full[slot], (it / BM_NB) & 1u)) {
        report_status(p.status, GW_ERR_TIMEOUT);
        return;
      }
      const int left = n - bt * BM_BATCH;  // pairs of this batch that exist
      const uint32_t qbase = smem_base + slot * SLOT, dobase = qbase + TENS;
      const uint32_t* words = reinterpret_cast<const uint32_t*>(bm_smem + slot * SLOT + 2 * TENS);
#pragma unroll
      for (int i = 0; i < HPW; ++i) {
        const int h = h0 + i;
        // B fragments: lanes 0..3 hold pairs 2t,2t+1 (word 0) and 2t+8,2t+9 (word 1) of column 0
        uint32_t pb0 = 0u, pb1 = 0u, dsb0 = 0u, dsb1 = 0u;
        if (lane < 4) {
          const int r0 = 2 * t4, r1 = r0 + 1, r2 = r0 + 8, r3 = r0 + 9;
          const uint32_t wa = r0 < left ? words[r0 * H + h] : 0u;
          const uint32_t wb = r1 < left ? words[r1 * H + h] : 0u;
          const uint32_t wc = r2 < left ? words[r2 * H + h] : 0u;
          const uint32_t wd = r3 < left ? words[r3 * H + h] : 0u;
          pb0 = __byte_perm(wa, wb, 0x5410);
          pb1 = __byte_perm(wc, wd, 0x5410);
          dsb0 = __byte_perm(wa, wb, 0x7632);
          dsb1 = __byte_perm(wc, wd, 0x7632);
        }
#pragma unroll
        for (int db = 0; db < 4; ++db) {
          uint32_t a[4];
          bm_ldmatrix_x4_trans(qbase + trans_lane_off + h * (D * 2) + db * 32, a);
          bm_mma<T>(accK[i][db], a, dsb0, dsb1);
          bm_ldmatrix_x4_trans(dobase + trans_lane_off + h * (D * 2) + db * 32, a);
          bm_mma<T>(accV[i][db], a, pb0, pb1);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->empty[slot]);
    }

    if (t4 == 0) {
#pragma unroll
      for (int i = 0; i < HPW; ++i) {
        T* dk = static_cast<T*>(p.dk) + ki * (H * D) + (h0 + i) * D;
        T* dv = static_cast<T*>(p.dv) + ki * (H * D) + (h0 + i) * D;
#pragma unroll
        for (int db = 0; db < 4; ++db) {
          dk[db * 16 + g] = from_float<T>(accK[i][db][0]);
          dk[db * 16 + g + 8] = from_float<T>(accK[i][db][2]);
          dv[db * 16 + g] = from_float<T>(accV[i][db][0]);
          dv[db * 16 + g + 8] = from_float<T>(accV[i][db][2]);
        }
      }
    }
  }
}

template <typename T, int HPW, int MODE>
int launch_bwd_query_mma(const BwdMmaParams& p, int dev, int sms, cudaStream_t st) {
  constexpr int H = BM_WARPS * HPW;
  constexpr size_t SMEM_Q = BM_NB * static_cast<size_t>(2) * BM_BATCH * (H * 64 * 2 + 16) + sizeof(BmShared);
  static OncePerDevice once;
  int rc = ensure_dynamic_smem(attn_bwd_query_mma_kernel<T, HPW, MODE>, SMEM_Q, once, dev);
  if (rc != GW_OK) return rc;
  const long long nq = static_cast<long long>(p.B) * p.T;
  attn_bwd_query_mma_kernel<T, HPW, MODE><<<static_cast<int>(nq < sms ? nq : sms), BM_THREADS, SMEM_Q, st>>>(p);
  GW_LAUNCH_CHECK();
  return GW_OK;
}

template <typename T, int HPW>
int launch_bwd_mma(const BwdMmaParams& p, cudaStream_t st) {
  constexpr int H = BM_WARPS * HPW;
  constexpr size_t ROWS = static_cast<size_t>(2) * BM_BATCH * (H * 64 * 2 + 16);
  constexpr size_t SMEM_K = BM_NB * (ROWS + BM_BATCH * H * 4) + sizeof(BmShared);
  int dev = 0;
  DeviceFacts facts;
  int rc = device_facts(&dev, &facts);
  if (rc != GW_OK) return rc;
  if (p.d_attn_sum != nullptr) {
    rc = launch_bwd_query_mma<T, HPW, 2>(p, dev, facts.sms, st);
    if (rc != GW_OK) return rc;
    rc = launch_bwd_query_mma<T, HPW, 1>(p, dev, facts.sms, st);
  } else {
    rc = launch_bwd_query_mma<T, HPW, 0>(p, dev, facts.sms, st);
  }
  if (rc != GW_OK) return rc;
  static OncePerDevice once_k;
  rc = ensure_dynamic_smem(attn_bwd_key_mma_kernel<T, HPW>, SMEM_K, once_k, dev);
  if (rc != GW_OK) return rc;
  const long long nk = static_cast<long long>(p.B) * p.S;
  attn_bwd_key_mma_kernel<T, HPW><<<static_cast<int>(nk < facts.sms ? nk : facts.sms), BM_THREADS, SMEM_K, st>>>(p);
  GW_LAUNCH_CHECK();
  return GW_OK;
}

}  // namespace
}  // namespace gw
