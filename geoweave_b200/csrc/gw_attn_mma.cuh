// Stage 3, tensor-core form for 16-bit inputs with token-major K/V rows of at most 2 KB (e.g. 16 heads x 64).
// (Included by gw_attn.cu.)
//
// The scalar kernel spends most of its issue slots unpacking bf16 pairs on the half-rate integer pipe.  Here
// the two contractions run on mma.sync m16n8k16 (bf16/fp16 in, fp32 accumulate), fed by ldmatrix straight
// from the gathered rows, so no element is ever unpacked:
//   scores  S[key, 0]  = K_h[16 keys x 64] . q_h        A = key rows as they lie in shared memory, B = q_h in column 0
//   output  O^T[d, 0] += V_h^T[64 x 16 keys] . p_h      A = ldmatrix.trans of the value rows,     B = p_h in column 0
// Seven of the eight B columns are zero: all heads of a query contract with different K/V slices, so there is
// no second query to put there; the tensor pipe has that much to spare and the gather stays the bound.
//
// One persistent CTA per SM: eight compute warps split the heads of ONE query (H/8 heads each) and share its
// gathered rows; four more warps are producers (each gathers a quarter of every batch).  Keys arrive in batches of 16 (one bulk copy per K row and per
// V row, rows padded by 16 bytes so that ldmatrix hits eight different bank groups), three batches in flight,
// one full/empty mbarrier pair per batch slot, and the stream of batches runs on across queries without a
// bubble.  Padding entries of the index list are replaced by key 0 in the gather and masked in the softmax.
//
// SUM variant (attn_sum[t, j] = sum over heads of the softmax weight of key j, fp32): two batch slots instead of
// three, and the space of the third holds the scaled logits of the current query, [head][key] fp32 (K <= 1024).
// When a query's keys are through, the compute warps meet on an mbarrier, every thread sums
// exp2(logit - m_h) / l_h over the heads for its keys and writes them, and a second mbarrier hands the buffer to
// the next query -- K is gathered once, not twice as with a separate pass.
#pragma once

namespace gw {
namespace {

constexpr int AM_WARPS = 8;          // compute warps
constexpr int AM_PROD = 4;           // producer warps: one warp alone cannot issue bulk copies fast enough
                                     // (measured: 24 B/clk/SM from one issuing warp, 58 B/clk/SM from twelve;
                                     // this kernel at N = 33 312: 10.8 ms with 2, 9.4 ms with 4, 9.7 ms with 8)
constexpr int AM_THREADS = (AM_WARPS + AM_PROD) * 32;
constexpr int AM_BATCH = 16;         // keys per batch (the M of the score MMA, the K of the output MMA)
constexpr int AM_NB = 3;             // batch slots
constexpr int AM_NB_SUM = 2;         // batch slots of the variant that also produces attn_sum
constexpr int AM_SUM_MAXK = 1024;    // keys per query the variant's logit buffer holds

__device__ __forceinline__ void ldmatrix_x4(uint32_t saddr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t saddr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr));
}
template <typename T>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const T a = from_float<T>(lo), b = from_float<T>(hi);
  return static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&a)) |
         (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(&b)) << 16);
}

struct AmShared {
  uint64_t full[AM_NB], empty[AM_NB];
  uint64_t sum_ready, sum_done;   // SUM variant: logits and (m, 1/l) of a query complete / read by every warp
  uint32_t mask[AM_NB][AM_PROD];  // validity bits of each producer's four keys
  float2 ml[AM_WARPS * 2];        // SUM variant: per head (reference maximum, 1 / denominator)
};

// HPW = heads per compute warp (H = 8 * HPW), D = 64
template <typename T, int HPW, bool SUM>
__global__ void __launch_bounds__(AM_THREADS, 1) sparse_attn_mma_kernel(const AttnParams p) {
  constexpr int D = 64;
  constexpr int H = AM_WARPS * HPW;
  constexpr int NB = SUM ? AM_NB_SUM : AM_NB;
  constexpr int ROW = H * D * 2;            // bytes of one K (or V) token row
  constexpr int RS = ROW + 16;              // row pitch in shared memory
  constexpr int TENS = AM_BATCH * RS;       // one tensor's rows of a batch
  constexpr int SLOT = 2 * TENS;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  float* logits = reinterpret_cast<float*>(smem_raw + NB * SLOT);  // SUM: [H][AM_SUM_MAXK]
  AmShared* sh = reinterpret_cast<AmShared*>(smem_raw + NB * SLOT + (SUM ? H * AM_SUM_MAXK * sizeof(float) : 0));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = p.K;
  const int nbatch = (K + AM_BATCH - 1) / AM_BATCH;
  const long long nq = static_cast<long long>(p.B) * p.T;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NB; ++s) {
      mbar_init(&sh->full[s], AM_PROD);
      mbar_init(&sh->empty[s], AM_WARPS);
    }
    mbar_init(&sh->sum_ready, AM_WARPS);
    mbar_init(&sh->sum_done, AM_WARPS);
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  __syncthreads();

  if (warp >= AM_WARPS) {
    // ------------------------------ producers: each gathers 4 of a batch's 16 keys (K row and V row) ------------------------------
    const uint32_t S = static_cast<uint32_t>(p.S);
    const int pw = warp - AM_WARPS;
    constexpr int KPP = AM_BATCH / AM_PROD;  // keys per producer warp
    const int key = pw * KPP + (lane % KPP), tens = (lane / KPP) & 1;
    uint32_t it = 0;
    for (long long qi = blockIdx.x; qi < nq; qi += gridDim.x) {
      const int b = static_cast<int>(qi / p.T);
      const int32_t* pos = p.pos + qi * K;
      const unsigned char* src0 = static_cast<const unsigned char*>(tens ? p.v : p.k) + static_cast<int64_t>(b) * (tens ? p.vs_b : p.ks_b) * 2;
      const int64_t pitch = (tens ? p.vs_t : p.ks_t) * 2;
      int id_next = (key < K) ? pos[key] : -1;
      for (int bt = 0; bt < nbatch; ++bt, ++it) {
        const int id = id_next;
        const int kn = (bt + 1) * AM_BATCH + key;
        id_next = (bt + 1 < nbatch && kn < K) ? pos[kn] : -1;
        const bool valid = static_cast<uint32_t>(id) < S;
        const uint32_t mask = __ballot_sync(0xffffffffu, valid) & ((1u << KPP) - 1u);
        const uint32_t slot = it % NB;
        if (!mbar_wait_bounded(&sh->empty[slot], ((it / NB) & 1u) ^ 1u)) {
          report_status(p.status, GW_ERR_TIMEOUT);
          return;
        }
        if (lane == 0) {
          sh->mask[slot][pw] = mask;
          mbar_arrive_expect_tx(&sh->full[slot], 2 * (AM_BATCH / AM_PROD) * ROW);
        }
        __syncwarp();
        // a padding entry gathers key 0 (finite values) and is masked out of the softmax
        if (lane < 2 * (AM_BATCH / AM_PROD))
          bulk_g2s(smem_raw + slot * SLOT + tens * TENS + key * RS, src0 + static_cast<int64_t>(valid ? id : 0) * pitch, ROW,
                   &sh->full[slot]);
      }
    }
    return;
  }

  // ------------------------------ compute warps ------------------------------
  const int g = lane >> 2, t4 = lane & 3;
  const int h0 = warp * HPW;
  // ldmatrix row addresses (bytes inside a tensor's batch): scores use the rows as stored, outputs transposed
  const uint32_t k_lane_off = static_cast<uint32_t>(((lane & 7) + 8 * ((lane >> 3) & 1)) * RS + (lane >> 4) * 16);
  const uint32_t v_lane_off = static_cast<uint32_t>(((lane & 7) + 8 * (lane >> 4)) * RS + ((lane >> 3) & 1) * 16);
  const uint32_t smem_base = smem_u32(smem_raw);
  uint32_t it = 0, qn = 0;

  for (long long qi = blockIdx.x; qi < nq; qi += gridDim.x, ++qn) {
    const int b = static_cast<int>(qi / p.T);
    const int t = static_cast<int>(qi % p.T);
    // B fragments of q: column 0 only, i.e. lanes 0..3 hold 32-bit words (two elements) of the q row
    uint32_t qb[HPW][4][2];
    {
      const uint32_t* qrow = reinterpret_cast<const uint32_t*>(static_cast<const T*>(p.q) + b * p.qs_b + static_cast<int64_t>(t) * p.qs_t);
#pragma unroll
      for (int i = 0; i < HPW; ++i) {
        const uint32_t* qh = qrow + (static_cast<int64_t>(h0 + i) * p.qs_h) / 2;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          qb[i][ks][0] = (lane < 4) ? qh[ks * 8 + t4] : 0u;
          qb[i][ks][1] = (lane < 4) ? qh[ks * 8 + t4 + 4] : 0u;
        }
      }
    }
    float acc[HPW][4][4];
    float m_ref[HPW], l_part[HPW];
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
      m_ref[i] = -INFINITY;
      l_part[i] = 0.f;
#pragma unroll
      for (int db = 0; db < 4; ++db)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[i][db][r] = 0.f;
    }

    for (int bt = 0; bt < nbatch; ++bt, ++it) {
      const uint32_t slot = it % NB;
      if (!mbar_wait_bounded(&sh->full[slot], (it / NB) & 1u)) {
        report_status(p.status, GW_ERR_TIMEOUT);
        return;
      }
      if (SUM && bt == 0 && qn > 0) {  // the previous query's logits have been read by every warp
        if (!mbar_wait_bounded(&sh->sum_done, (qn - 1) & 1u)) {
          report_status(p.status, GW_ERR_TIMEOUT);
          return;
        }
      }
      uint32_t mask = 0;
#pragma unroll
      for (int pw = 0; pw < AM_PROD; ++pw) mask |= sh->mask[slot][pw] << (pw * (AM_BATCH / AM_PROD));
      const uint32_t kaddr = smem_base + slot * SLOT + k_lane_off;
      const uint32_t vaddr = smem_base + slot * SLOT + TENS + v_lane_off;
      const bool ok0 = (mask >> g) & 1u, ok1 = (mask >> (g + 8)) & 1u;  // keys g and g+8 of the batch
#pragma unroll
      for (int i = 0; i < HPW; ++i) {
        const int h = h0 + i;
        // ---- scores of 16 keys for head h ----
        float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          uint32_t a[4];
          ldmatrix_x4(kaddr + h * (D * 2) + ks * 32, a);
          mma_16816<T>(s, a, qb[i][ks][0], qb[i][ks][1]);
        }
        // column 0 lives in the lanes with t4 == 0: s[0] = key g, s[2] = key g + 8 (log2 domain after scaling)
        float s0 = ok0 ? s[0] * p.scale_log2 : -INFINITY;
        float s1 = ok1 ? s[2] * p.scale_log2 : -INFINITY;
        if (SUM && t4 == 0) {
          logits[h * AM_SUM_MAXK + bt * AM_BATCH + g] = s0;
          logits[h * AM_SUM_MAXK + bt * AM_BATCH + g + 8] = s1;
        }
        float bmax = fmaxf(s0, s1);
        bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 4));
        bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 8));
        bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 16));
        if (bmax > m_ref[i] + kRescaleSlack) {  // warp-uniform: bmax is the same in every lane with equal t4
          const float alpha = exp2f(m_ref[i] - bmax);
          l_part[i] *= alpha;
#pragma unroll
          for (int db = 0; db < 4; ++db)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[i][db][r] *= alpha;
          m_ref[i] = bmax;
        }
        // a masked key weighs nothing; written out because with nothing live yet m_ref is -inf and exp2f(-inf - -inf)
        // would be NaN (a row, or its first batches, may be all padding)
        const float p0 = ok0 ? exp2f(s0 - m_ref[i]) : 0.f, p1 = ok1 ? exp2f(s1 - m_ref[i]) : 0.f;
        if (t4 == 0) l_part[i] += p0 + p1;
        // ---- B fragment of p: lanes 0..3 need keys 2t,2t+1 (word 0) and 2t+8,2t+9 (word 1) ----
        const float pa = __shfl_sync(0xffffffffu, p0, 8 * t4);
        const float pb = __shfl_sync(0xffffffffu, p0, 8 * t4 + 4);
        const float pc = __shfl_sync(0xffffffffu, p1, 8 * t4);
        const float pd = __shfl_sync(0xffffffffu, p1, 8 * t4 + 4);
        const uint32_t pb0 = (lane < 4) ? pack2<T>(pa, pb) : 0u;
        const uint32_t pb1 = (lane < 4) ? pack2<T>(pc, pd) : 0u;
        // ---- O^T[16 dims x 1] += V^T . p for the four 16-dim blocks of head h ----
#pragma unroll
        for (int db = 0; db < 4; ++db) {
          uint32_t a[4];
          ldmatrix_x4_trans(vaddr + h * (D * 2) + db * 32, a);
          mma_16816<T>(acc[i][db], a, pb0, pb1);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->empty[slot]);
    }

    // ---- normalise and write: lanes with t4 == 0 hold dims g and g+8 of every 16-dim block ----
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
      float l = l_part[i];
      l += __shfl_xor_sync(0xffffffffu, l, 4);
      l += __shfl_xor_sync(0xffffffffu, l, 8);
      l += __shfl_xor_sync(0xffffffffu, l, 16);
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      if (SUM && lane == 0) sh->ml[h0 + i] = make_float2(l > 0.f ? m_ref[i] : 0.f, inv);
      if (t4 == 0) {
        T* op = static_cast<T*>(p.out) + b * p.os_b + static_cast<int64_t>(t) * p.os_t + static_cast<int64_t>(h0 + i) * p.os_h;
#pragma unroll
        for (int db = 0; db < 4; ++db) {
          op[db * 16 + g] = from_float<T>(acc[i][db][0] * inv);
          op[db * 16 + g + 8] = from_float<T>(acc[i][db][2] * inv);
        }
        if (p.lse != nullptr && lane == 0)
          p.lse[(static_cast<int64_t>(b) * p.H + h0 + i) * p.T + t] =
              l > 0.f ? (m_ref[i] + log2f(l)) * 0.6931471805599453f : -INFINITY;
      }
    }
    if (SUM) {
      // ---- attn_sum of this query: all warps' logits and (m, 1/l) must be in; then keys are split over the threads ----
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->sum_ready);
      if (!mbar_wait_bounded(&sh->sum_ready, qn & 1u)) {
        report_status(p.status, GW_ERR_TIMEOUT);
        return;
      }
      float* asum = p.attn_sum + qi * K;
      for (int j = threadIdx.x; j < K; j += AM_WARPS * 32) {
        float acc_j = 0.f;
#pragma unroll
        for (int h = 0; h < H; ++h) {
          const float2 ml = sh->ml[h];
          acc_j += exp2f(logits[h * AM_SUM_MAXK + j] - ml.x) * ml.y;  // a masked key holds -inf: contributes 0
        }
        asum[j] = acc_j;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->sum_done);
    }
  }
}

template <typename T, int HPW, bool SUM>
int launch_attn_mma(const AttnParams& p, cudaStream_t st) {
  constexpr int H = AM_WARPS * HPW;
  constexpr size_t SMEM = static_cast<size_t>(SUM ? AM_NB_SUM : AM_NB) * 2 * AM_BATCH * (H * 64 * 2 + 16) +
                          (SUM ? static_cast<size_t>(H) * AM_SUM_MAXK * sizeof(float) : 0) + sizeof(AmShared);
  auto kern = sparse_attn_mma_kernel<T, HPW, SUM>;
  int dev = 0;
  DeviceFacts facts;
  int rc = device_facts(&dev, &facts);
  if (rc != GW_OK) return rc;
  static OncePerDevice smem_once;
  rc = ensure_dynamic_smem(kern, SMEM, smem_once, dev);
  if (rc != GW_OK) return rc;
  const int sms = facts.sms;
  const long long nq = static_cast<long long>(p.B) * p.T;
  const int grid = static_cast<int>(nq < sms ? nq : sms);
  kern<<<grid, AM_THREADS, SMEM, st>>>(p);
  GW_LAUNCH_CHECK();
  return GW_OK;
}

}  // namespace
}  // namespace gw
