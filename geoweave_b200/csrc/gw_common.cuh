// Shared device/host helpers for the geoweave_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/geoweave_b200.h"

namespace gw {

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return GW_ERR_CUDA;
}

#define GW_CUDA_TRY(expr)                          \
  do {                                             \
    cudaError_t _e = (expr);                       \
    if (_e != cudaSuccess) return gw::cuda_fail(_e); \
  } while (0)

#define GW_LAUNCH_CHECK() GW_CUDA_TRY(cudaGetLastError())

// Per-device facts are read from the runtime once per device ordinal and kept for the life of the process
// (gw_device_cache_reset forgets them, e.g. after a cudaDeviceReset).  A launch path pays for
// cudaDeviceGetAttribute / cudaFuncSetAttribute only the first time it runs on a device.
constexpr int kMaxDevices = 64;
extern std::atomic<unsigned> g_cache_epoch;  // bumped by gw_device_cache_reset

struct DeviceFacts {
  int sms;
  int cc_major;
};
struct DeviceFactsSlot {
  std::atomic<unsigned> epoch_plus_one{0};  // 0 = never filled
  DeviceFacts facts{0, 0};
};
extern DeviceFactsSlot g_device_facts[kMaxDevices];

inline int device_facts(int* dev_out, DeviceFacts* out) {
  int dev = 0;
  GW_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return GW_ERR_UNSUPPORTED;
  DeviceFactsSlot& slot = g_device_facts[dev];
  const unsigned want = g_cache_epoch.load(std::memory_order_acquire) + 1u;
  if (slot.epoch_plus_one.load(std::memory_order_acquire) != want) {
    DeviceFacts f{0, 0};
    GW_CUDA_TRY(cudaDeviceGetAttribute(&f.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    GW_CUDA_TRY(cudaDeviceGetAttribute(&f.sms, cudaDevAttrMultiProcessorCount, dev));
    slot.facts = f;  // racing first calls write the same values
    slot.epoch_plus_one.store(want, std::memory_order_release);
  }
  if (dev_out) *dev_out = dev;
  *out = slot.facts;
  return GW_OK;
}

// "done once per device" marker for one kernel instantiation (one static object per launch site)
struct OncePerDevice {
  std::atomic<unsigned long long> mask{0};
  std::atomic<unsigned> epoch{0};
  bool needed(int dev) {
    const unsigned e = g_cache_epoch.load(std::memory_order_acquire);
    if (epoch.load(std::memory_order_acquire) != e) {
      mask.store(0, std::memory_order_relaxed);
      epoch.store(e, std::memory_order_release);
    }
    return ((mask.load(std::memory_order_acquire) >> dev) & 1ull) == 0;
  }
  void done(int dev) { mask.fetch_or(1ull << dev, std::memory_order_release); }
};

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) the first time `kern` is launched on device `dev`
template <typename Kern>
inline int ensure_dynamic_smem(Kern kern, size_t bytes, OncePerDevice& once, int dev) {
  if (once.needed(dev)) {
    GW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
    once.done(dev);
  }
  return GW_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t dtype_size(int dtype) { return dtype == GW_F32 ? 4 : 2; }
inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---------------------------------------------------------------------------------------------
// element conversion
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_float(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }

// two packed 16-bit elements -> two floats
template <typename T> __device__ __forceinline__ void unpack2(uint32_t u, float& lo, float& hi);
template <> __device__ __forceinline__ void unpack2<__nv_bfloat16>(uint32_t u, float& lo, float& hi) {
  lo = __uint_as_float(u << 16);
  hi = __uint_as_float(u & 0xffff0000u);
}
template <> __device__ __forceinline__ void unpack2<__half>(uint32_t u, float& lo, float& hi) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u));
  lo = f.x;
  hi = f.y;
}

// ---------------------------------------------------------------------------------------------
// ordering keys: larger score -> larger 32-bit key.  -0.0 is folded onto +0.0 so the two tie.
// A candidate is ranked by the 64-bit composite (key << 32 | ~index): descending composite order is
// (score descending, index ascending), which is the selection rule of the whole library.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t score_key(float f) {
  const uint32_t u = __float_as_uint(__fadd_rn(f, 0.0f));
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_score(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}
__device__ __forceinline__ unsigned long long composite(uint32_t key, uint32_t idx) {
  return (static_cast<unsigned long long>(key) << 32) | static_cast<unsigned long long>(~idx);
}
__device__ __forceinline__ uint32_t composite_key(unsigned long long c) { return static_cast<uint32_t>(c >> 32); }
__device__ __forceinline__ uint32_t composite_idx(unsigned long long c) { return ~static_cast<uint32_t>(c); }

// ---------------------------------------------------------------------------------------------
// PTX wrappers: shared-memory addresses, mbarriers, bulk (TMA) copies.  Every wait is bounded.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// try_wait that may stay suspended in hardware for up to `hint_ns` before it reports "not yet"
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Wait for a phase of an mbarrier, for at most `limit_ns` of wall time.  Returns false when the wait ran out;
// the caller records GW_ERR_TIMEOUT in the status word and leaves its loop (no trap, no endless spin).
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > limit_ns) return false;
  }
}
constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // ~2 s: every pipeline wait of the kernels
constexpr unsigned long long kDrainLimitNs = 50000000ull;    // 50 ms: waiting for copies still in flight on the way out
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) { return mbar_wait_limit(bar, parity, kWaitLimitNs); }

// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.  Both addresses 16-byte
// aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// ask for [src, src + bytes) to be brought into L2 (16-byte aligned address, size a multiple of 16)
__device__ __forceinline__ void bulk_prefetch_l2(const void* src_gmem, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src_gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// barrier `id` over `nthreads` threads that also ORs a predicate: every participant gets the same answer
__device__ __forceinline__ bool named_bar_or(int id, int nthreads, bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %3, 0;\n\t"
      "bar.red.or.pred p, %1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"(id), "r"(nthreads), "r"(static_cast<uint32_t>(pred))
      : "memory");
  return out != 0;
}

__device__ __forceinline__ void report_status(int* status_dev, int code) {
  if (status_dev != nullptr) atomicCAS(status_dev, 0, code);
}

}  // namespace gw
