// The exchange step of the sharded path over peer memory (GPUs of one node, one process per GPU): every rank's shard
// lies in a buffer all ranks have mapped; an exchange = copy my rows into my buffer, meet the other ranks at a barrier
// made of flags in peer memory, pull every peer's rows into the full tensors.  Two ways to pull:
//   * device-to-device copies spread over a few streams of this object -- the driver runs them on copy engines over
//     NVLink, so no SM is taken from the kernel that runs beside the exchange (K and V arrive while the indexer runs);
//   * one kernel that reads all peers with 16-byte loads -- for the small exchange in front of the indexer (K_idx, w),
//     where nothing runs beside it and the launch count is what costs.
// The reference has no counterpart: its multi-GPU inference all-gathers with NCCL around the same operators
// (easyvolcap/official_vggt/layers/dsa_attention.py:1138-1264).
//
// Barrier: flags[r] is rank r's flag array (uint32 [world]); slot s of it belongs to sender s.  For arrival number seq
// (1, 2, 3, ... the same on every rank for the same exchange) thread r of the one block writes seq into slot `rank` of
// rank r's array (release, system scope) and waits until slot r of this rank's own array has reached seq (acquire, system
// scope).  The numbers only grow, so nothing is ever reset and a rank that is already one exchange ahead does no harm.
// Every wait is bounded; on expiry the kernel reports GW_ERR_TIMEOUT in the status word and returns.
#include "gw_common.cuh"

namespace gw {
namespace {

constexpr int PX_MAX_STREAMS = 8;
constexpr int PX_MAX_COPIES = 64;   // (peers incl. self) x tensors of one exchange

__global__ void peer_barrier_kernel(uint32_t* const* flags, int rank, int world, uint32_t seq, unsigned long long limit_ns, int* status) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();  // what this rank wrote before the barrier is visible to whoever sees the flag
  uint32_t* theirs = flags[r] + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(seq) : "memory");
  const uint32_t* mine = flags[rank] + r;
  const unsigned long long t0 = global_timer_ns();
  uint32_t seen;
  for (;;) {
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if (static_cast<int32_t>(seen - seq) >= 0) break;
    if (global_timer_ns() - t0 > limit_ns) {
      report_status(status, GW_ERR_TIMEOUT);
      break;
    }
    __nanosleep(64);
  }
}

struct PullTable {
  const unsigned char* src[PX_MAX_COPIES];
  unsigned char* dst[PX_MAX_COPIES];
  unsigned long long bytes[PX_MAX_COPIES];
  int n;
};

// blockIdx.y = copy; the blocks of a row stride over it in 16-byte pieces where source, destination and size allow,
// in 4-byte or single-byte pieces otherwise
__global__ void __launch_bounds__(256) peer_pull_kernel(const PullTable t) {
  const int c = blockIdx.y;
  const unsigned char* src = t.src[c];
  unsigned char* dst = t.dst[c];
  const unsigned long long n = t.bytes[c];
  const unsigned long long tid = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x;
  const unsigned long long nthreads = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
  const uintptr_t both = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | static_cast<uintptr_t>(n);
  if ((both & 15u) == 0) {
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    const unsigned long long n16 = n / 16;
    unsigned long long i = tid;
    for (; i + 3 * nthreads < n16; i += 4 * nthreads) {  // four loads in flight per thread: the peer is microseconds away
      const uint4 a = s[i], b = s[i + nthreads], c2 = s[i + 2 * nthreads], e = s[i + 3 * nthreads];
      d[i] = a;
      d[i + nthreads] = b;
      d[i + 2 * nthreads] = c2;
      d[i + 3 * nthreads] = e;
    }
    for (; i < n16; i += nthreads) d[i] = s[i];
  } else if ((both & 3u) == 0) {
    const uint32_t* s = reinterpret_cast<const uint32_t*>(src);
    uint32_t* d = reinterpret_cast<uint32_t*>(dst);
    for (unsigned long long i = tid; i < n / 4; i += nthreads) d[i] = s[i];
  } else {
    for (unsigned long long i = tid; i < n; i += nthreads) dst[i] = src[i];
  }
}

}  // namespace
}  // namespace gw

using namespace gw;

struct GwPeerExchange {
  int device;
  int n_streams;
  cudaStream_t streams[PX_MAX_STREAMS];
  cudaEvent_t start, fanout, done[PX_MAX_STREAMS];
};

extern "C" int gw_peer_exchange_create(int n_copy_streams, GwPeerExchange** out) {
  if (!out || n_copy_streams < 1 || n_copy_streams > PX_MAX_STREAMS) return GW_ERR_INVALID_ARG;
  GwPeerExchange* ex = new GwPeerExchange();
  GW_CUDA_TRY(cudaGetDevice(&ex->device));
  ex->n_streams = n_copy_streams;
  for (int i = 0; i < n_copy_streams; ++i) {
    GW_CUDA_TRY(cudaStreamCreateWithFlags(&ex->streams[i], cudaStreamNonBlocking));
    GW_CUDA_TRY(cudaEventCreateWithFlags(&ex->done[i], cudaEventDisableTiming));
  }
  GW_CUDA_TRY(cudaEventCreateWithFlags(&ex->start, cudaEventDisableTiming));
  GW_CUDA_TRY(cudaEventCreateWithFlags(&ex->fanout, cudaEventDisableTiming));
  *out = ex;
  return GW_OK;
}

extern "C" void gw_peer_exchange_destroy(GwPeerExchange* ex) {
  if (!ex) return;
  for (int i = 0; i < ex->n_streams; ++i) {
    cudaStreamDestroy(ex->streams[i]);
    cudaEventDestroy(ex->done[i]);
  }
  cudaEventDestroy(ex->start);
  cudaEventDestroy(ex->fanout);
  delete ex;
}

extern "C" int gw_peer_barrier(const void* flag_ptrs_dev, int rank, int world, unsigned int seq, int limit_ms, int* status_dev,
                               gw_stream_t stream) {
  if (!flag_ptrs_dev || !status_dev || world < 1 || world > 64 || rank < 0 || rank >= world || limit_ms <= 0) return GW_ERR_INVALID_ARG;
  peer_barrier_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<uint32_t* const*>(flag_ptrs_dev), rank, world, seq,
                                                                          static_cast<unsigned long long>(limit_ms) * 1000000ull, status_dev);
  GW_LAUNCH_CHECK();
  return GW_OK;
}

extern "C" int gw_peer_exchange_run(GwPeerExchange* ex, gw_stream_t after, const void* flag_ptrs_dev, int rank, int world, unsigned int seq,
                                    int limit_ms, int* status_dev, int n_pack, const void* const* pack_src, void* const* pack_dst,
                                    const size_t* pack_bytes, int n_pull, const void* const* pull_src, void* const* pull_dst,
                                    const size_t* pull_bytes, int pull_with_kernel) {
  if (!ex || !flag_ptrs_dev || !status_dev || n_pack < 0 || n_pull < 0 || n_pull > PX_MAX_COPIES) return GW_ERR_INVALID_ARG;
  if ((n_pack && (!pack_src || !pack_dst || !pack_bytes)) || (n_pull && (!pull_src || !pull_dst || !pull_bytes))) return GW_ERR_INVALID_ARG;
  cudaStream_t s0 = ex->streams[0];
  // the exchange follows what the caller's stream has enqueued so far (the shard is complete, the outputs are free)
  GW_CUDA_TRY(cudaEventRecord(ex->start, reinterpret_cast<cudaStream_t>(after)));
  GW_CUDA_TRY(cudaStreamWaitEvent(s0, ex->start, 0));
  for (int i = 0; i < n_pack; ++i)
    if (pack_bytes[i]) GW_CUDA_TRY(cudaMemcpyAsync(pack_dst[i], pack_src[i], pack_bytes[i], cudaMemcpyDeviceToDevice, s0));
  int rc = gw_peer_barrier(flag_ptrs_dev, rank, world, seq, limit_ms, status_dev, s0);
  if (rc != GW_OK) return rc;
  if (pull_with_kernel) {
    PullTable t;
    t.n = n_pull;
    unsigned long long biggest = 0;
    for (int i = 0; i < n_pull; ++i) {
      t.src[i] = static_cast<const unsigned char*>(pull_src[i]);
      t.dst[i] = static_cast<unsigned char*>(pull_dst[i]);
      t.bytes[i] = pull_bytes[i];
      if (pull_bytes[i] > biggest) biggest = pull_bytes[i];
    }
    if (n_pull > 0 && biggest > 0) {
      unsigned long long blocks = (biggest / 16 + 1023) / 1024;      // at least four 16-byte pieces per thread
      const unsigned long long fill = (2ull * 148 + n_pull - 1) / n_pull;  // about two CTAs per SM over all copies
      if (blocks > fill) blocks = fill;
      if (blocks < 1) blocks = 1;
      peer_pull_kernel<<<dim3(static_cast<unsigned>(blocks), n_pull), 256, 0, s0>>>(t);
      GW_LAUNCH_CHECK();
    }
    GW_CUDA_TRY(cudaEventRecord(ex->done[0], s0));
    return GW_OK;
  }
  GW_CUDA_TRY(cudaEventRecord(ex->fanout, s0));
  for (int s = 1; s < ex->n_streams; ++s) GW_CUDA_TRY(cudaStreamWaitEvent(ex->streams[s], ex->fanout, 0));
  for (int i = 0; i < n_pull; ++i)
    if (pull_bytes[i])
      GW_CUDA_TRY(cudaMemcpyAsync(pull_dst[i], pull_src[i], pull_bytes[i], cudaMemcpyDeviceToDevice, ex->streams[i % ex->n_streams]));
  for (int s = 0; s < ex->n_streams; ++s) GW_CUDA_TRY(cudaEventRecord(ex->done[s], ex->streams[s]));
  // the next exchange of this object starts on stream 0: it must follow the copies of the other streams too
  for (int s = 1; s < ex->n_streams; ++s) GW_CUDA_TRY(cudaStreamWaitEvent(s0, ex->done[s], 0));
  return GW_OK;
}

extern "C" int gw_peer_exchange_join(GwPeerExchange* ex, gw_stream_t waiter, int last_was_kernel) {
  if (!ex) return GW_ERR_INVALID_ARG;
  const int n = last_was_kernel ? 1 : ex->n_streams;
  for (int s = 0; s < n; ++s) GW_CUDA_TRY(cudaStreamWaitEvent(reinterpret_cast<cudaStream_t>(waiter), ex->done[s], 0));
  return GW_OK;
}
