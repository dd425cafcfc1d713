// Fast form of the fused indexer for large key sets, where a sampled per-row threshold tau is available.
// (Included by gw_indexer.cu after IdxParams, the candidate sources/sinks and the tile constants.)
//
// Tile shape: tcgen05.mma has a floor of about 48 cycles per instruction on B200 whatever N <= 96 is (measured:
// 128x48, 128x64 and 128x96 steps all take 48 cycles, with the A operand in shared or in tensor memory), and
// the Hi separate accumulators of a tile must fit twice into the 512 TMEM columns for the tensor cores to run
// ahead of the epilogue, so N = 64 keys per tile with both operands in shared memory is the best available
// point: 16 instructions = 768 cycles per 64-key tile, two thirds of the tensor peak.
//
// The epilogue only filters: a thread (= one query row) appends (score, key) to a list in global memory when
// score >= tau, through predicated stores at a moving address (no divergent branch, no selection inside the
// kernel).  It is bound by instruction issue -- about 16 issued instructions per score in the epilogue alone: four
// FADD for 2*relu, two packed FMA, one shared-memory and half a tensor-memory load, and 6.6 for the compare, the
// pairing of score and key index, the predicated store and its bump -- so everything that costs issue slots
// without producing scores is kept out of the way: eight epilogue warps work on every tile (32 of its 64 columns
// for 32 rows each, so the per-tile barrier traffic is paid once per 32 columns; sixteen warps of 16 columns and
// two groups of eight on alternate tiles were both built and measured slower), TMEM reads are software-pipelined
// (the next 8 columns are in flight while 8 are reduced), tensor-memory addresses stay in uniform registers (the
// warp index is read through a shuffle, which the compiler treats as warp-uniform), and every wait of the
// producer and MMA threads sleeps between polls instead of spinning on issue slots the epilogue warps need.  The w*scale tile (stored head-major per tile) comes from a small shared-memory ring
// that the TMA producer fills alongside the keys.
//
// Work items are (row block, key split) pairs.  The first item of a CTA is its block index; every further item
// is drawn from a global counter by the producer thread and handed to the other roles through shared memory
// together with the query block's "loaded" barrier, so an SM that starts late or loses time (to a collective's
// CTAs, say) simply takes fewer items.
//
// The lists of all rows of a launch stay in the workspace and a second, occupancy-bound kernel
// (finalize_lists_kernel, one warp per row) turns each row's lists into the exact top-k.  A row whose list
// overflowed or holds fewer than k candidates is not resolved there: its row block is flagged and the robust
// kernel redoes that block from tau = -inf.  The result is therefore exact for any data; only the speed
// depends on the quality of tau.
#pragma once

#include "gw_select_tight.cuh"

namespace gw {
namespace {

constexpr int F_NQ = 2;                         // lists per (row, key split): one per column half of the tiles
constexpr int F_EPI = 4 * F_NQ;                 // epilogue warps: 4 lane quarters x 2 column halves
constexpr int F_THREADS = 64 + F_EPI * 32 + 32; // 352: producer, MMA issuer 0, 8 epilogue warps, MMA issuer 1
constexpr int FBN = 64;                         // keys per tile
constexpr int F_QCOLS = FBN / F_NQ;             // 32 columns per epilogue warp per tile
constexpr int FNSTG = 3;                        // key-tile ring depth
constexpr int FK_HEAD_BYTES = FBN * DI * 2;     // 8 KB
constexpr int F_ACC_COLS = 256;                 // TMEM columns per accumulator set (Hi * 64 <= 256)
constexpr int WSLOTS = 8;                       // w*scale tile ring
constexpr int W_TILE_FLOATS = 4 * FBN;          // [head][64] fp32
constexpr int W_TILE_BYTES = W_TILE_FLOATS * 4; // 1 KB

// Cycle counters for performance diagnosis (filled when IdxParams::profile is set, read back with
// gw_debug_indexer_profile): per CTA, per warp, eight 64-bit slots.
constexpr int PROF_SLOTS = 8;
__device__ unsigned long long g_idx_prof[MAX_SLOTS * (F_THREADS / 32) * PROF_SLOTS];  // [CTA][warp][slot]

// finalize statistics (always counted; 4 cheap atomics per row at most): rows whose lists overflowed, rows that
// came up short, rows that needed the general selection, rows finished by the lean selection
__device__ unsigned long long g_fin_stats[4];

struct ProfClock {
  unsigned long long acc[PROF_SLOTS] = {};
  long long t0 = 0;
  bool on;
  __device__ explicit ProfClock(bool enabled) : on(enabled) {}
  __device__ __forceinline__ void start() { if (on) t0 = clock64(); }
  __device__ __forceinline__ void stop(int slot) { if (on) { const long long t1 = clock64(); acc[slot] += t1 - t0; t0 = t1; } }
  __device__ void flush(int warp) const {
    if (!on) return;
    for (int i = 0; i < PROF_SLOTS; ++i) g_idx_prof[(blockIdx.x * (F_THREADS / 32) + warp) * PROF_SLOTS + i] = acc[i];
  }
};

struct alignas(8) FastShared {
  uint64_t q_full, q_empty;    // query block in shared memory: loaded / no longer read by any MMA
  uint64_t k_full[FNSTG], k_empty[FNSTG];
  uint64_t acc_full[2], acc_empty[2];
  uint64_t w_full[WSLOTS], w_empty[WSLOTS];
  uint32_t tmem_base;
  volatile int abort_flag;
  volatile int item[2];        // work item of the n-th query block of this CTA at [n & 1]; -1 = no more work
};

// Wait used by the producer and the MMA threads, which are far ahead of the epilogue and wait most of the time:
// between polls the thread sleeps, so its polling does not take issue slots from the epilogue warps that share
// its scheduler.  A wake-up that comes a few hundred cycles late is absorbed by the two accumulator sets and
// the three key stages.  Bounded like every other wait.
__device__ __forceinline__ bool mbar_wait_sleeping(uint64_t* bar, uint32_t parity, uint32_t max_sleep_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  uint32_t ns = 64;
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      __nanosleep(ns);
      if (mbar_try_wait_hint(bar, parity, max_sleep_ns)) return true;
      if (ns < max_sleep_ns) ns *= 2;  // back off: a poll costs eight issue slots of the scheduler it shares
    }
    if (global_timer_ns() - t0 > kWaitLimitNs) return false;
  }
}
constexpr uint32_t kMmaSleepNs = 512;        // the tensor cores are one accumulator set ahead: a late wake-up costs nothing
constexpr uint32_t kProducerSleepNs = 2048;  // the loads are three key stages ahead

// packed fp32 pairs (sm_100 f32x2 pipe): d = a * b + c on both halves
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %5};\n\t"
      "mov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

template <int HI>
__device__ __forceinline__ void fast_load_chunk(uint32_t taddr, uint32_t (&a)[HI][8]) {
#pragma unroll
  for (int h = 0; h < HI; ++h) tmem_ld_x8(taddr + h * FBN, a[h]);
}

// Append (score, col) at the list position {lo, hi} (the two halves of a 64-bit address) and advance it when
// score >= tau (and col < S if GUARD).  Only the low half ever moves -- the host lays the lists out so that none
// crosses a 4 GiB boundary -- which makes the bump one predicated 32-bit add: compare, predicated store,
// predicated add, no branch and no carry chain (the cheapest of the forms measured: 6.6 issued instructions per
// column including the pairing of score and key index, against 7.8 to 8.8 for 64-bit or counter-based forms).
template <bool GUARD>
__device__ __forceinline__ void append_if(uint32_t& lo, uint32_t hi, float s, float tau, uint32_t col, int S) {
  if (GUARD) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 a;\n\t"
        "mov.b64 a, {%0, %1};\n\t"
        "setp.ge.f32 p, %2, %3;\n\t"
        "setp.lt.and.s32 p, %5, %6, p;\n\t"
        "@p st.global.v2.b32 [a], {%4, %5};\n\t"
        "@p add.u32 %0, %0, 8;\n\t}"
        : "+r"(lo)
        : "r"(hi), "f"(s), "f"(tau), "r"(__float_as_uint(s)), "r"(col), "r"(S)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 a;\n\t"
        "mov.b64 a, {%0, %1};\n\t"
        "setp.ge.f32 p, %2, %3;\n\t"
        "@p st.global.v2.b32 [a], {%4, %5};\n\t"
        "@p add.u32 %0, %0, 8;\n\t}"
        : "+r"(lo)
        : "r"(hi), "f"(s), "f"(tau), "r"(__float_as_uint(s)), "r"(col)
        : "memory");
  }
}

// Reduce 8 columns held in `a` and append the ones that pass.  wt = this tile's w*scale, [head][FBN]; c0 = first
// column within the tile; col_g = its global key index.  All loads and arithmetic come first; the appends
// are predicated stores at a moving address.  The caller guarantees room for 8 more entries.
template <int HI, bool GUARD>
__device__ __forceinline__ void fast_reduce_chunk(const uint32_t (&a)[HI][8], const float* __restrict__ wt, int c0, int col_g,
                                                  int S, float tau, uint32_t& lo, uint32_t hi) {
  float2 acc[4];
#pragma unroll
  for (int h = 0; h < HI; ++h) {
    const float4 wa = *reinterpret_cast<const float4*>(wt + h * FBN + c0);
    const float4 wb = *reinterpret_cast<const float4*>(wt + h * FBN + c0 + 4);
    float r[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      // 2 * relu(x) = x + |x| is one full-rate FADD (max() runs on the half-rate ALU pipe); the factor 2 is
      // folded into the staged weights, which hold 0.5 * w * scale -- all exact powers of two
      const float x = __uint_as_float(a[h][c]);
      r[c] = x + fabsf(x);
    }
    const float2 w2[4] = {make_float2(wa.x, wa.y), make_float2(wa.z, wa.w), make_float2(wb.x, wb.y), make_float2(wb.z, wb.w)};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 r2 = make_float2(r[2 * q], r[2 * q + 1]);
      acc[q] = (h == 0) ? fmul2(r2, w2[q]) : ffma2(r2, w2[q], acc[q]);
    }
  }
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const float s = (c & 1) ? acc[c >> 1].y : acc[c >> 1].x;
    append_if<GUARD>(lo, hi, s, tau, static_cast<uint32_t>(col_g + c), S);
  }
}

// One warp's share of a tile: columns c_begin .. c_begin + 31 (taddr already points at column c_begin of head 0).
// With two epilogue warps per scheduler the TMEM round trip is hidden by software pipelining: the next 8 columns
// are in flight while 8 are reduced.
template <int HI, bool GUARD>
__device__ __forceinline__ void fast_reduce_tile(uint32_t taddr, const float* wt, int c_begin, int col_base, int S, float tau,
                                                 uint32_t& lo, uint32_t hi) {
  uint32_t a0[HI][8], a1[HI][8];
  fast_load_chunk<HI>(taddr, a0);
  tmem_wait_ld();
#pragma unroll
  for (int ch = 0; ch < F_QCOLS / 8; ch += 2) {
    fast_load_chunk<HI>(taddr + (ch + 1) * 8, a1);  // in flight while a0 is reduced
    fast_reduce_chunk<HI, GUARD>(a0, wt, c_begin + ch * 8, col_base + c_begin + ch * 8, S, tau, lo, hi);
    tmem_wait_ld();
    if (ch + 2 < F_QCOLS / 8) fast_load_chunk<HI>(taddr + (ch + 2) * 8, a0);
    fast_reduce_chunk<HI, GUARD>(a1, wt, c_begin + (ch + 1) * 8, col_base + c_begin + (ch + 1) * 8, S, tau, lo, hi);
    if (ch + 2 < F_QCOLS / 8) tmem_wait_ld();
  }
}

// key tiles of split `sp`: sp, sp + nsplit, sp + 2 nsplit, ... (`nt` of them; no split is empty while nsplit <= ntiles).
// Interleaved rather than contiguous ranges: where the high scores of a row crowd into one stretch of the key range
// (keys of unequal norm laid out in groups, as the pooled sources of the coarse-to-fine selection are), every split
// still gets its even share of them, and no single list overflows.
__device__ __forceinline__ void split_tiles(int sp, int nsplit, int ntiles, int& nt) {
  nt = (ntiles - sp + nsplit - 1) / nsplit;
}

template <int HI>
__global__ void __launch_bounds__(F_THREADS, 1)
indexer_fast_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const IdxParams p,
                    const uint32_t idesc) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* q_smem = smem;                                  // HI x 16 KB, 128-byte swizzled rows
  unsigned char* k_smem = q_smem + HI * Q_HEAD_BYTES;            // FNSTG x HI x 8 KB
  float* w_smem = reinterpret_cast<float*>(k_smem + FNSTG * HI * FK_HEAD_BYTES);
  FastShared* sh = reinterpret_cast<FastShared*>(reinterpret_cast<unsigned char*>(w_smem) + WSLOTS * W_TILE_BYTES);

  // read through a shuffle, the warp index is warp-uniform for the compiler: role dispatch and every
  // tensor-memory address derived from it stay in uniform registers
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const int blk_begin = p.row_begin / BM, blk_end = (p.row_end + BM - 1) / BM;  // this launch's row blocks
  const int ntiles = (p.S + FBN - 1) / FBN;
  // work item = (row block, key split): a launch with fewer row blocks than SMs, or a ragged last wave, is
  // evened out by cutting the key range of every row block into nsplit pieces that go to different CTAs
  const int nsplit = p.nsplit;
  const int nitems = (blk_end - blk_begin) * nsplit;

  if (threadIdx.x == 0) {
    mbar_init(&sh->q_full, 1);
    mbar_init(&sh->q_empty, 2);
    for (int s = 0; s < FNSTG; ++s) {
      mbar_init(&sh->k_full[s], 1);
      mbar_init(&sh->k_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->acc_full[b], 1);
      mbar_init(&sh->acc_empty[b], F_EPI);
    }
    for (int s = 0; s < WSLOTS; ++s) {
      mbar_init(&sh->w_full[s], 1);
      mbar_init(&sh->w_empty[s], F_EPI);
    }
    sh->abort_flag = 0;
    sh->item[0] = sh->item[1] = -1;
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) tmem_alloc(&sh->tmem_base, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, sh->tmem_base, 0);  // warp-uniform for the compiler, like `warp`

  if (warp == 0) {
    // ------------------------------ TMA producer: work items, Q block, key tiles, w*scale tiles ------------------------------
    if (lane == 0) {
      ProfClock pc(p.profile != 0);
      uint32_t tuse = 0, nblk = 0;
      int item = blockIdx.x;
      for (;; ++nblk) {
        if (item >= nitems) item = -1;
        pc.start();
        if (!mbar_wait_sleeping(&sh->q_empty, (nblk & 1u) ^ 1u, kProducerSleepNs)) { sh->abort_flag = 1; break; }
        pc.stop(0);
        if (sh->abort_flag) break;
        sh->item[nblk & 1u] = item;  // made visible to the other roles by the arrival on q_full below
        if (item < 0) {
          mbar_arrive(&sh->q_full);
          break;
        }
        const int rb = blk_begin + item / nsplit, sp = item % nsplit;
        int nt;
        split_tiles(sp, nsplit, ntiles, nt);
        mbar_arrive_expect_tx(&sh->q_full, HI * Q_HEAD_BYTES);
#pragma unroll
        for (int h = 0; h < HI; ++h) tma_load_2d(q_smem + h * Q_HEAD_BYTES, &tmQ, h * DI, rb * BM, &sh->q_full);
        for (int jl = 0; jl < nt; ++jl, ++tuse) {
          const int j = sp + jl * nsplit;
          const uint32_t s = tuse % FNSTG, n = tuse / FNSTG;
          const uint32_t ws = tuse % WSLOTS, wn = tuse / WSLOTS;
          pc.start();
          if (!mbar_wait_sleeping(&sh->k_empty[s], (n & 1u) ^ 1u, kProducerSleepNs)) { sh->abort_flag = 1; break; }
          pc.stop(1);
          if (!mbar_wait_sleeping(&sh->w_empty[ws], (wn & 1u) ^ 1u, kProducerSleepNs)) { sh->abort_flag = 1; break; }
          pc.stop(2);
          if (sh->abort_flag) break;
          mbar_arrive_expect_tx(&sh->w_full[ws], W_TILE_BYTES);
          bulk_g2s(w_smem + ws * W_TILE_FLOATS, p.wtile + static_cast<size_t>(j) * W_TILE_FLOATS, W_TILE_BYTES, &sh->w_full[ws]);
          mbar_arrive_expect_tx(&sh->k_full[s], HI * FK_HEAD_BYTES);
#pragma unroll
          for (int h = 0; h < HI; ++h)
            tma_load_2d(k_smem + (s * HI + h) * FK_HEAD_BYTES, &tmK, h * DI, j * FBN, &sh->k_full[s]);
          pc.stop(3);
        }
        if (sh->abort_flag) break;
        item = static_cast<int>(gridDim.x) + atomicAdd(p.item_counter, 1);
      }
      pc.flush(warp);
      if (sh->abort_flag) {
        // leaving early: let the copies this thread started land before the CTA's shared memory is given up,
        // and release the roles that may still be waiting for a work item
        if (nblk > 0) mbar_wait_limit(&sh->q_full, (nblk - 1u) & 1u, kDrainLimitNs);
        for (uint32_t u = tuse > FNSTG ? tuse - FNSTG : 0u; u < tuse; ++u)
          mbar_wait_limit(&sh->k_full[u % FNSTG], (u / FNSTG) & 1u, kDrainLimitNs);
        for (uint32_t u = tuse > WSLOTS ? tuse - WSLOTS : 0u; u < tuse; ++u)
          mbar_wait_limit(&sh->w_full[u % WSLOTS], (u / WSLOTS) & 1u, kDrainLimitNs);
        report_status(p.status, GW_ERR_TIMEOUT);
      }
    }
  } else if (warp == 1 || warp == 2 + F_EPI) {
    // ------------------------------ MMA issuers ------------------------------
    // Two issuing threads, one per accumulator set (even / odd key tiles).  A tcgen05.commit stalls the issuing
    // thread's next MMA until the committed ones have drained (measured: 63-73 instead of 48 cycles per MMA
    // with one issuer committing every tile); a second issuer fills those gaps.
    const uint32_t b = (warp == 1) ? 0u : 1u;
    if (lane == 0) {
      ProfClock pc(p.profile != 0);
      uint32_t nblk = 0, use = 0, tbase = 0;
      const uint64_t adesc0 = make_smem_desc(smem_u32(q_smem));
      const uint64_t bdesc00 = make_smem_desc(smem_u32(k_smem));
      const uint32_t d0 = tmem_base + b * F_ACC_COLS;
      for (;; ++nblk) {
        pc.start();
        if (!mbar_wait_sleeping(&sh->q_full, nblk & 1u, kMmaSleepNs)) { sh->abort_flag = 1; break; }
        pc.stop(0);
        const int item = sh->item[nblk & 1u];
        if (item < 0 || sh->abort_flag) break;
        int nt;
        split_tiles(item % nsplit, nsplit, ntiles, nt);
        for (int j = b; j < nt; j += 2, ++use) {
          const uint32_t tuse = tbase + j;
          pc.start();
          if (!mbar_wait_sleeping(&sh->acc_empty[b], (use & 1u) ^ 1u, kMmaSleepNs)) { sh->abort_flag = 1; break; }
          pc.stop(1);
          const uint32_t s = tuse % FNSTG;
          if (!mbar_wait_sleeping(&sh->k_full[s], (tuse / FNSTG) & 1u, kMmaSleepNs)) { sh->abort_flag = 1; break; }
          pc.stop(2);
          if (sh->abort_flag) break;
          tc_fence_after();
          const uint64_t bdesc0 = bdesc00 + s * ((HI * FK_HEAD_BYTES) >> 4);
#pragma unroll
          for (int h = 0; h < HI; ++h)
#pragma unroll
            for (int kk = 0; kk < DI / 16; ++kk)  // +32 bytes along K per step = +2 in the address field
              tc_mma_f16(d0 + h * FBN, adesc0 + h * (Q_HEAD_BYTES >> 4) + 2 * kk, bdesc0 + h * (FK_HEAD_BYTES >> 4) + 2 * kk, idesc,
                         kk > 0 ? 1u : 0u);
          tc_commit(&sh->k_empty[s]);
          tc_commit(&sh->acc_full[b]);
          pc.stop(3);
        }
        if (sh->abort_flag) break;
        tc_commit(&sh->q_empty);
        tbase += nt;
      }
      pc.flush(warp);
      if (sh->abort_flag) report_status(p.status, GW_ERR_TIMEOUT);
    }
  } else {
    // ------------------------------ epilogue: score, filter, append ------------------------------
    const int e = warp - 2;
    const int half = e >> 2;   // column half of every tile this warp reduces
    const int lq = warp & 3;   // TMEM lane quarter this warp may read
    const int row_in_tile = lq * 32 + lane;
    // every warp works on every tile, so both accumulator sets are drained by all eight warps and the tensor
    // cores never wait for half of them
    const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(lq * 32) << 16) + half * F_QCOLS;
    const bool last_partial = (p.S % FBN) != 0;
    const uint32_t list_bytes = static_cast<uint32_t>(p.caph) * 8u;
    uint32_t use0 = 0, use1 = 0, tbase = 0;
    ProfClock pc(p.profile != 0);
    for (uint32_t nblk = 0;; ++nblk) {
      pc.start();
      if (!mbar_wait_bounded(&sh->q_full, nblk & 1u)) { sh->abort_flag = 1; break; }
      pc.stop(0);
      // one value for the whole warp: through the shuffle the compiler also knows it, and keeps the tile loop and
      // the tensor-memory addresses in the uniform datapath
      const int item = __shfl_sync(0xffffffffu, sh->item[nblk & 1u], 0);
      if (item < 0 || __shfl_sync(0xffffffffu, sh->abort_flag, 0)) break;
      const int rb = blk_begin + item / nsplit, sp = item % nsplit;
      int nt;
      split_tiles(sp, nsplit, ntiles, nt);
      const int row = rb * BM + row_in_tile;
      const bool active = row < p.T;
      const float tau = active ? p.tau_in[row] : INFINITY;
      const size_t lrow = static_cast<size_t>(row - p.row_begin);
      const size_t seg = (lrow * nsplit + sp) * F_NQ + half;  // this thread's list
      const uintptr_t buf = reinterpret_cast<uintptr_t>(p.cand + seg * p.caph);
      const uint32_t lo0 = static_cast<uint32_t>(buf), hi = static_cast<uint32_t>(buf >> 32);
      uint32_t lo = lo0;
      // a list that wraps the low address word (the host places the lists so that none does) is not written at
      // all: the row goes to the robust kernel and the status word says so
      const bool wraps = lo0 + (list_bytes - 8u) < lo0;
      bool overflowed = wraps;
      const float tau_eff = wraps ? INFINITY : tau;
      if (wraps) report_status(p.status, GW_ERR_INTERNAL);
      for (int jl = 0; jl < nt; ++jl) {
        const int j = sp + jl * nsplit;
        const uint32_t b = jl & 1;
        const uint32_t n = b ? use1 : use0;
        const uint32_t ws = (tbase + jl) % WSLOTS, wn = (tbase + jl) / WSLOTS;
        pc.start();
        if (!mbar_wait_bounded(&sh->acc_full[b], n & 1u)) { sh->abort_flag = 1; break; }
        pc.stop(1);
        if (!mbar_wait_bounded(&sh->w_full[ws], wn & 1u)) { sh->abort_flag = 1; break; }
        pc.stop(2);
        tc_fence_after();
        // a list without room for this warp's whole share of a tile is given up (the row is redone by the robust
        // kernel): keep counting from the start of the list so that no store ever leaves it
        if (lo - lo0 > list_bytes - F_QCOLS * 8u) {  // compared as offsets: a list may end exactly where the low word wraps
          overflowed = true;
          lo = lo0;
        }
        const float* wt = w_smem + ws * W_TILE_FLOATS;
        if (last_partial && j == ntiles - 1)
          fast_reduce_tile<HI, true>(taddr_row + b * F_ACC_COLS, wt, half * F_QCOLS, j * FBN, p.S, tau_eff, lo, hi);
        else
          fast_reduce_tile<HI, false>(taddr_row + b * F_ACC_COLS, wt, half * F_QCOLS, j * FBN, p.S, tau_eff, lo, hi);
        tc_fence_before();
        __syncwarp();
        pc.stop(3);
        if (lane == 0) {
          mbar_arrive(&sh->acc_empty[b]);
          mbar_arrive(&sh->w_empty[ws]);
        }
        if (b) ++use1; else ++use0;
      }
      if (active) p.list_cnt[seg] = overflowed ? p.caph + 1 : static_cast<int>((lo - lo0) >> 3);
      tbase += nt;
      if (sh->abort_flag) break;
    }
    if (lane == 0) pc.flush(warp);
    if (sh->abort_flag) report_status(p.status, GW_ERR_TIMEOUT);
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// exact top-k of every row's lists (one warp per row, many warps per SM to hide the list reads)
// ---------------------------------------------------------------------------------------------
constexpr int FIN_WARPS = 8;

struct IdxOutSink {
  int32_t* oi;
  void* os;
  int dtype;
  __device__ __forceinline__ void operator()(int pos, uint32_t bits, uint32_t idx) const {
    oi[pos] = static_cast<int32_t>(idx);
    if (os != nullptr) {
      const float s = __uint_as_float(bits);
      if (dtype == GW_BF16) static_cast<__nv_bfloat16*>(os)[pos] = __float2bfloat16_rn(s);
      else if (dtype == GW_F16) static_cast<__half*>(os)[pos] = __float2half_rn(s);
      else static_cast<float*>(os)[pos] = s;
    }
  }
};

// flat view of a row's list segments for the general selection (rare path: the segment is found by a short scan)
struct SegListSrc {
  const uint2* base;
  const int* cnt;
  int cap;
  int nseg;
  __device__ __forceinline__ unsigned long long operator()(int i) const {
    int sgm = 0;
    while (sgm + 1 < nseg && i >= cnt[sgm]) {
      i -= cnt[sgm];
      ++sgm;
    }
    const uint2 e = base[static_cast<size_t>(sgm) * cap + i];
    return composite(score_key(__uint_as_float(e.x)), e.y);
  }
};

__global__ void __launch_bounds__(FIN_WARPS * 32) finalize_lists_kernel(const IdxParams p) {
  __shared__ TightSmem tsm[FIN_WARPS];
  __shared__ SelectSmem<SEL_BINS> gsm;  // general routine, used by one warp at a time (rare fall-back)
  __shared__ int gsm_lock;
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) gsm_lock = 0;
  __syncthreads();
  const int row = p.row_begin + blockIdx.x * FIN_WARPS + w;
  if (row >= p.row_end || row >= p.T) return;
  const size_t lrow = static_cast<size_t>(row - p.row_begin);
  const int nseg = F_NQ * p.nsplit;
  const int* cnt = p.list_cnt + lrow * nseg;
  int n = 0;
  bool over = false;
  for (int sgm = 0; sgm < nseg; ++sgm) {
    const int c = cnt[sgm];
    over = over || c > p.caph;
    n += c;
  }
  if (over || n < p.k) {  // a list overflowed, or tau was too high: redo from -inf
    if (lane == 0) {
      atomicAdd(&g_fin_stats[over ? 0 : 1], 1ull);
      p.tau_redo[row] = -INFINITY;
      p.block_flags[row / BM] = 1;
    }
    return;
  }
  if (lane == 0) p.tau_redo[row] = INFINITY;
  const uint2* b0 = p.cand + lrow * nseg * p.caph;
  IdxOutSink sink{p.out_idx + static_cast<int64_t>(row) * p.k,
                  p.out_scores ? static_cast<unsigned char*>(p.out_scores) +
                                     static_cast<int64_t>(row) * p.k * (p.out_dtype == GW_F32 ? 4 : 2)
                               : nullptr,
                  p.out_dtype};
  TightLists L{b0, cnt, p.caph, nseg};
  const uint32_t lo = score_key(p.tau_in[row]), hi = score_key(p.smax_in[row]);
  if (warp_select_tight(L, p.k, lo, hi, tsm[w], lane, sink, nullptr) == p.k) {
    if (lane == 0) atomicAdd(&g_fin_stats[3], 1ull);
    return;
  }
  if (lane == 0) atomicAdd(&g_fin_stats[2], 1ull);
  // boundary bin too crowded (heavy ties): general selection, serialised over the CTA's one scratch area
  bool got = false;
  for (int spin = 0; spin < (1 << 22) && !got; ++spin) {
    if (lane == 0) got = atomicCAS(&gsm_lock, 0, 1) == 0;
    got = __shfl_sync(0xffffffffu, got, 0);
    if (!got) __nanosleep(200);
  }
  if (!got) {
    report_status(p.status, GW_ERR_TIMEOUT);
    return;
  }
  SegListSrc src{b0, cnt, p.caph, nseg};
  FinalSink fsink{sink.oi, sink.os, sink.dtype};
  group_select_topk<32, SEL_BINS, SegListSrc, FinalSink, 8>(src, n, p.k, static_cast<unsigned long long>(lo) << 32,
                                                            (static_cast<unsigned long long>(hi) << 32) | 0xffffffffull, gsm, lane, 0,
                                                            fsink, nullptr, true);
  __threadfence_block();
  if (lane == 0) atomicExch(&gsm_lock, 0);
}

// tau = rank-th largest of each row of the sampled scores, smax = the row maximum (one warp per row)
__global__ void __launch_bounds__(FIN_WARPS * 32) sample_threshold_kernel(const float* sc, int m, int64_t stride, int T, int rank,
                                                                          float* tau, float* smax) {
  __shared__ TightSmem tsm[FIN_WARPS];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * FIN_WARPS + w;
  if (row >= T) return;
  const float* r = sc + static_cast<int64_t>(row) * stride;
  uint32_t kmin = 0xffffffffu, kmax = 0u;
  for (int i = lane; i < m; i += 32) {
    const uint32_t key = score_key(r[i]);
    kmin = min(kmin, key);
    kmax = max(kmax, key);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    kmin = min(kmin, __shfl_xor_sync(0xffffffffu, kmin, d));
    kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, d));
  }
  TightDenseRow L{r, m};
  uint32_t kth = 0;
  auto none = [](int, uint32_t, uint32_t) {};
  float t;
  if (warp_select_tight(L, rank, kmin, kmax, tsm[w], lane, none, &kth) == rank) {
    t = __uint_as_float(kth);
  } else {
    t = -INFINITY;  // pathological sample (a crowd of equal scores at the rank): no filtering for this row
  }
  if (lane == 0) {
    tau[row] = t;
    smax[row] = key_score(kmax);
  }
}

// 0.5 * w * scale as fp32 in the tile layout the fast kernel stages: [tile][head 0..3][64], zero beyond S and Hi
// (the epilogue multiplies it with 2 * relu(acc))
template <typename T>
__global__ void prep_w_tiled_kernel(const T* w, int S, int Hi, float scale, float* wtile, int ntiles) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= ntiles * W_TILE_FLOATS) return;
  const int tile = i / W_TILE_FLOATS, h = (i % W_TILE_FLOATS) / FBN, c = i % FBN;
  const int s = tile * FBN + c;
  wtile[i] = (s < S && h < Hi) ? to_float(w[static_cast<size_t>(s) * Hi + h]) * scale * 0.5f : 0.f;
}

inline size_t fast_smem_bytes(int Hi) {
  return 1024 + static_cast<size_t>(Hi) * Q_HEAD_BYTES + static_cast<size_t>(FNSTG) * Hi * FK_HEAD_BYTES +
         WSLOTS * W_TILE_BYTES + sizeof(FastShared);
}

}  // namespace
}  // namespace gw
