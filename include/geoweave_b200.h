/*
 * geoweave_b200 -- C ABI of the B200 (sm_100a) sparse top-k global-attention path.
 *
 * One shared library (libgeoweave_b200.so), plain pointers and sizes, no framework types.  Every pointer
 * argument is a DEVICE pointer unless said otherwise; every call enqueues work on `stream` and returns
 * without synchronising, allocates nothing and is safe to record into a CUDA graph (the exception is
 * documented on the function).  Return value: GW_OK or a negative GW_ERR_* (see gw_strerror).  Conditions
 * that can only be seen on the device (a bounded wait that ran out) are written to the caller's
 * `status_dev` word, which the caller reads after its next synchronisation.
 *
 * Each entry point names the interface of the reference project (zss171999645/GeoWeave, paths relative to
 * its root) that it replaces.
 */
#ifndef GEOWEAVE_B200_H
#define GEOWEAVE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* gw_stream_t; /* a cudaStream_t */

/* element types */
#define GW_F32 0
#define GW_BF16 1
#define GW_F16 2

/* status codes */
#define GW_OK 0
#define GW_ERR_INVALID_ARG (-1)  /* null pointer, non-positive size, misaligned pointer or stride */
#define GW_ERR_UNSUPPORTED (-2)  /* a shape or dtype this build has no kernel for (there is no fallback) */
#define GW_ERR_WORKSPACE (-3)    /* workspace smaller than gw_*_workspace_bytes() */
#define GW_ERR_CUDA (-4)         /* a CUDA runtime/driver call failed; see gw_last_cuda_error() */
#define GW_ERR_TIMEOUT (-5)      /* device side: a bounded wait inside a kernel ran out (status word) */
#define GW_ERR_NO_SM100 (-6)     /* the current device is not compute capability 10.x */
#define GW_ERR_TOO_LARGE (-7)    /* the problem exceeds the fixed capacity of a no-allocation entry point */
#define GW_ERR_INTERNAL (-8)     /* device side: a kernel found its own bookkeeping inconsistent and skipped the work (status word) */

const char* gw_strerror(int code);
int gw_last_cuda_error(void);   /* cudaError_t of the last GW_ERR_CUDA on this thread, else 0 */
int gw_abi_version(void);

/* The library remembers, per device ordinal, what it learned on its first call there: SM count, the raised
 * shared-memory limits of its kernels, the device address of the no-allocation scratch array, and (per host
 * thread) the last tensor maps it encoded.  A host that calls cudaDeviceReset, or destroys the context and
 * makes a new one on the same ordinal, must call this afterwards; the next call on each device looks
 * everything up again.  Host-only; no reference counterpart. */
int gw_device_cache_reset(void);

/* Diagnostics: a one-warp kernel waits on a barrier that nobody signals, for at most limit_us microseconds
 * (1..100000), then writes GW_ERR_TIMEOUT to *status_dev and returns -- the way every wait inside this
 * library's kernels ends when it cannot be satisfied.  waited_ns_dev (nullable) receives the time spent.
 * The context stays usable.  No reference counterpart. */
int gw_debug_bounded_wait_selftest(unsigned int limit_us, int* status_dev, unsigned long long* waited_ns_dev,
                                   gw_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Stage 1+2 fused: indexer score + exact top-k, the N x N score matrix never reaches memory.
 *
 *   score[t,s] = sum_h w[s,h] * relu(scale * <q_idx[t,h,:], k_idx[s,h,:]>)       (fp32)
 *   out_idx[t,:] = the k keys with the largest score, equal scores keep the LOWER key index.
 *
 * q_idx [B,T,Hi,Di], k_idx [B,S,Hi,Di], w [B,S,Hi], contiguous, all of `dtype` (GW_BF16 or GW_F16).
 * out_idx int32 [B,T,k] (order within a row unspecified), out_scores nullable, `dtype` [B,T,k].
 * Requirements: Di == 64 (one 128-byte tensor-core K block per head), 1 <= Hi <= 4, k <= S.
 * Replaces: easyvolcap/utils/custom_indexer/sparse_topk_indexer.py:2188 (sparse_topk_indexer_func),
 *           :1241-1776 (_blockwise_topk_scores_impl), and the k=512-only fused kernel
 *           easyvolcap/utils/custom_indexer/csrc/score_topk_fused_kernel.cu:52-224 (score_topk_fused_cuda).
 * ---------------------------------------------------------------------------------------------- */
size_t gw_indexer_topk_workspace_bytes(int B, int T, int S, int Hi, int Di, int k);
int gw_indexer_topk_fused(const void* q_idx, const void* k_idx, const void* w, int dtype, int B, int T, int S,
                          int Hi, int Di, float scale, int k, int32_t* out_idx, void* out_scores,
                          void* workspace, size_t workspace_bytes, int* status_dev, gw_stream_t stream);

/* Number of kernels one gw_indexer_topk_fused call enqueues (it depends on whether the key set is large
 * enough for the sampled threshold pass).  Host-only arithmetic; no reference counterpart. */
int gw_indexer_topk_launch_count(int B, int T, int S, int k);

/* Diagnostics: after gw_debug_indexer_profile_enable(1) the fused indexer kernel accumulates clock-cycle
 * counters per CTA and warp role (waiting on each hand-off, issuing, reducing, selecting); results are not
 * affected.  gw_debug_indexer_profile copies them to HOST memory (synchronising): four finalize counters (rows whose candidate lists overflowed, came up
 * short, needed the general selection, were finished by the lean selection; reset by this call), then
 * [CTA][11 warps][8 slots] of 64-bit cycle counts; returns the number of entries copied or a negative status.  No reference counterpart. */
int gw_debug_indexer_profile_enable(int on);
int gw_debug_indexer_profile(unsigned long long* host_out, int max_entries);

/* Dense score block (debug / verification / threshold sampling): out[t, j] = score[t, j*key_step] for
 * j < ceil(S/key_step), fp32, row stride `out_row_stride` elements.  Same tensor-core main loop as the
 * fused call.  Replaces: sparse_topk_indexer.py:935-951 (_compute_scores_block_einsum) and the Triton
 * _score_block_kernel (:981-1062). */
int gw_indexer_scores(const void* q_idx, const void* k_idx, const void* w, int dtype, int B, int T, int S, int Hi,
                      int Di, float scale, int key_step, float* out, int64_t out_row_stride, int* status_dev,
                      gw_stream_t stream);

/* Dense scores for fp32 operands (the arithmetic of the reference's `--backend torch` path, which forces
 * score_dtype=float32: geoweave/inference.py:56-58, easyvolcap/official_vggt/layers/indexer.py:321-326, :430-466).
 * q_idx [B,T,Hi,64], k_idx [B,S,Hi,64], w [B,S,Hi] fp32 contiguous; out[b, t - row_begin, s] for the query rows
 * [row_begin, row_begin + rows) of every batch, fp32 [B, rows, out_row_stride].  A plain FFMA kernel (fp32 operands
 * cannot use the 16-bit tensor-core path without changing the scores); the caller selects with gw_topk_exact. */
int gw_indexer_scores_f32(const float* q_idx, const float* k_idx, const float* w, int B, int T, int S, int Hi, int Di,
                          float scale, int64_t row_begin, int rows, float* out, int64_t out_row_stride,
                          gw_stream_t stream);

/* gw_indexer_scores for callers that must not allocate.  No counterpart in the reference.
 *
 * gw_indexer_scores needs a scratch table (w * scale as fp32, 16 bytes per key) and gets it from the stream-
 * ordered allocator.  Some hosts cannot do that: a plugin loaded into a serving runtime that owns the whole
 * device heap and forbids plugin-side allocation, or a latency-critical loop that cannot accept the
 * device-wide synchronisation an allocation may imply.  This variant keeps the table in a fixed 4 MiB array
 * that is part of the library image (every GPU that loads the library holds these 4 MiB until the process
 * exits) and calls no allocating routine.  Same arguments, same results.
 *
 * Limit: round_up(S, 64) + 64 * key_step + 64 <= GW_NOALLOC_MAX_KEYS, otherwise GW_ERR_TOO_LARGE and nothing
 * is launched.  The first call on each device looks up the array's device address (with that device
 * current); make that first call before any stream capture.  The address is remembered per device ordinal:
 * after cudaDeviceReset, or with a second context on the same device, call gw_device_cache_reset() first.  All calls on a device share the one array:
 * each call rewrites every entry it reads, so stale contents never matter, but two calls whose kernels may
 * overlap on the GPU (different streams) race on it -- serialise them. */
#define GW_NOALLOC_MAX_KEYS 262144
int gw_indexer_scores_noalloc(const void* q_idx, const void* k_idx, const void* w, int dtype, int B, int T, int S,
                              int Hi, int Di, float scale, int key_step, float* out, int64_t out_row_stride,
                              int* status_dev, gw_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Stage 2 alone: exact top-k of materialised rows (any k <= cols; ties keep the lower column).
 * scores [rows, cols] of `dtype` with row stride `row_stride` elements.  Either index output may be null:
 * out_idx32 int32 [rows,k], out_idx64 int64 [rows,k]; out_scores nullable, `dtype` [rows,k].
 * The order inside an output row is unspecified (the reference's torch.topk(sorted=False) leaves it open too).
 * Replaces: easyvolcap/utils/custom_indexer/csrc/topk_exact_kernel.cu:25-149 (topk_exact_cuda, k = 512 only).
 * ---------------------------------------------------------------------------------------------- */
int gw_topk_exact(const void* scores, int dtype, int64_t rows, int64_t cols, int64_t row_stride, int k,
                  int32_t* out_idx32, int64_t* out_idx64, void* out_scores, gw_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Merge a running top-k list with a pending list: keep the best k of the union by (score descending,
 * index ascending).  a_idx int32 [rows,ka]; b_pos int64 [rows,kb] with b_index = b_pos + b_start; negative
 * indices are empty slots.  Scores of `dtype`.  Outputs [rows,k] (may alias the `a` arrays).
 * Replaces: easyvolcap/utils/custom_indexer/csrc/merge_two_topk_kernel.cu:24-142 (merge_two_topk_cuda, k = 512 only).
 * ---------------------------------------------------------------------------------------------- */
int gw_merge_two_topk(const void* a_scores, const int32_t* a_idx, int ka, const void* b_scores,
                      const int64_t* b_pos, int kb, int64_t b_start, int dtype, int64_t rows, int k,
                      void* out_scores, int32_t* out_idx, gw_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Stage 3: attention of every query over only its selected keys (all heads of a query share one list).
 *
 *   out[t,h,:] = softmax_j(scale * <q[t,h,:], K[pos[t,j],h,:]>) . V[pos[t,j],h,:]
 *
 * q [B,T,H,D], k,v [B,S,H,D] given by element strides {batch, token, head} with a contiguous last
 * dimension (so both the reference's [B,T,H,D] and [B,H,T,D] layouts are passed as they are);
 * kv_pos int32 [B,T,K] contiguous, entries < 0 or >= S are padding.  out has strides out_strides and the
 * same dtype; lse (nullable) fp32 [B,H,T] natural-log sum-exp; attn_sum (nullable) fp32 [B,T,K] = sum over
 * heads of the softmax probabilities.  A row with only padding gives zeros and lse = -inf.
 * Requirements: D in {32,64,128}; 16-byte aligned pointers; strides multiples of 16 bytes.
 * Replaces: easyvolcap/utils/custom_flash_attn/sparse_index_flash_attn.py:122-259 (_fwd_kernel),
 *           :375-458 (_attn_sum_kernel) and :2001-2233 (_flash_attn_forward).
 * ---------------------------------------------------------------------------------------------- */
int gw_sparse_attn_fwd(const void* q, const void* k, const void* v, const int32_t* kv_pos, int dtype, int B, int T,
                       int S, int H, int D, int K, const int64_t q_strides[3], const int64_t k_strides[3],
                       const int64_t v_strides[3], float scale, void* out, const int64_t out_strides[3], float* lse,
                       float* attn_sum, int* status_dev, gw_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Stage 3 backward: dQ, dK, dV of gw_sparse_attn_fwd, including the gradient that arrives through attn_sum
 * (d_attn_sum fp32 [B,T,K], nullable).  q, out, d_out, dq [B,T,H,D]; k, v, dk, dv [B,S,H,D]; all contiguous and of `dtype`
 * (GW_F32, GW_BF16 or GW_F16); lse fp32 [B,H,T] as written by the forward.  No floating-point atomics: the sums over
 * the queries that selected a key run in the order given by the caller in key_order / key_start -- the positions
 * t*K + j of kv_pos (int32 [B, T*K]) stably sorted by key with padding entries last, and the first entry of every key
 * (int32 [B, S+1]) -- so results are reproducible.  workspace: gw_sparse_attn_bwd_workspace_bytes(B,T,H,K) bytes,
 * 256-byte aligned (p and dp per (query, head, slot)).  Requirements: D = 64, H <= 32, T*K < 2^31.  16-bit inputs with
 * 8 or 16 heads and a status word take tensor-core kernels (gathers by bulk copies, bounded waits that report
 * GW_ERR_TIMEOUT in status_dev; with d_attn_sum a pre-pass over the K rows first); every other case takes plain kernels
 * and status_dev may be null.
 * Replaces: easyvolcap/utils/custom_flash_attn/sparse_index_flash_attn.py:2442-2846 (_sparse_index_flash_attn_backward and
 *           its Triton kernels :535-1186, fp32 atomic adds) and csrc/sparse_bwd_grouped_kernel.cu:78-603 (sort-based).
 * ---------------------------------------------------------------------------------------------- */
/* The key_order / key_start arrays both backward passes take: the (query, slot) pairs of kv_pos (int32 [B,T,K]) stably sorted
 * by key -- key_order int32 [B, T*K] holds t*K + j, padding entries (outside [0,S)) last; key_start int32 [B, S+1] the first
 * entry of every key.  A radix sort over the bits a key can have.  workspace: gw_group_by_key_workspace_bytes(T,K,S),
 * 256-byte aligned.  (The reference sorts the same pairs with torch ops in its grouped backward,
 * easyvolcap/utils/custom_flash_attn/csrc/sparse_bwd_grouped_kernel.cu:78-180 and its Python caller.) */
size_t gw_group_by_key_workspace_bytes(int T, int K, int S);
int gw_group_by_key(const int32_t* kv_pos, int B, int T, int K, int S, int32_t* key_order, int32_t* key_start, void* workspace,
                    size_t workspace_bytes, gw_stream_t stream);
size_t gw_sparse_attn_bwd_workspace_bytes(int B, int T, int H, int K);
int gw_sparse_attn_bwd(const void* q, const void* k, const void* v, const int32_t* kv_pos, const void* out, const float* lse,
                       const void* d_out, const float* d_attn_sum, const int32_t* key_order, const int32_t* key_start,
                       int dtype, int B, int T, int S, int H, int D, int K, float scale, void* dq, void* dk, void* dv,
                       void* workspace, size_t workspace_bytes, int* status_dev, gw_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Backward of the indexer's selected scores
 *   score[t,j] = sum_h w[idx[t,j],h] * relu(scale * <q[t,h], k[idx[t,j],h]>)
 * given grad_scores fp32 [B,T,K]: dq [B,T,Hi,Di], dk [B,S,Hi,Di], dw [B,S,Hi] of the operands' type.  q, k, w contiguous,
 * GW_BF16 or GW_F16, Di = 64, Hi <= 4; topk_idx int32 [B,T,K], entries outside [0,S) carry no gradient.  key_order /
 * key_start as for gw_sparse_attn_bwd (the lists stably sorted by key): no floating-point atomics, reproducible sums.
 * workspace: gw_indexer_topk_bwd_workspace_bytes(B,T,S,K) bytes, 256-byte aligned.  Bounded waits report
 * GW_ERR_TIMEOUT in status_dev (required).
 * Replaces: easyvolcap/utils/custom_indexer/sparse_topk_indexer.py:757-895 (_backward_selected_topk_qkw) and its
 *           Triton kernels :1847-2044 (fp32 atomic adds into dk and dw).
 * ---------------------------------------------------------------------------------------------- */
size_t gw_indexer_topk_bwd_workspace_bytes(int B, int T, int S, int K);
int gw_indexer_topk_bwd(const void* q, const void* k, const void* w, const int32_t* topk_idx, const float* grad_scores,
                        const int32_t* key_order, const int32_t* key_start, int dtype, int B, int T, int S, int Hi, int Di,
                        int K, float scale, void* dq, void* dk, void* dw, void* workspace, size_t workspace_bytes,
                        int* status_dev, gw_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * The exchange step of the sharded path over peer memory (GPUs of one node, one process per GPU), in place of an NCCL
 * all-gather.  Every rank's shard lies in a buffer that all ranks have mapped; one exchange = copy my rows into my
 * buffer (pack), meet the other ranks at a barrier made of flags in peer memory, pull every peer's rows (pull).
 *
 * gw_peer_barrier: flag_ptrs_dev = device array of `world` pointers, entry r = rank r's flag array (uint32 [world], zero
 * before the first use, mapped by every rank); seq = 1, 2, 3, ... the same on every rank for the same barrier.  One
 * block; every wait is bounded by limit_ms and reports GW_ERR_TIMEOUT in status_dev.  Only with one process per GPU: ranks
 * that share a GPU would wait on kernels that cannot run beside them.
 *
 * gw_peer_exchange_create/destroy: an object that owns n_copy_streams streams (<= 8) and the events between them, on the
 * current device.  gw_peer_exchange_run enqueues, behind everything already enqueued on `after`: the n_pack pack copies,
 * the barrier, and the n_pull (<= 64) pulls -- as device-to-device copies dealt round-robin to the object's streams (copy
 * engines; no SM used) or, with pull_with_kernel != 0, as one kernel on its first stream.  All pointer arrays are host
 * arrays of device addresses.  gw_peer_exchange_join makes `waiter` wait for the last run; call it before the next run of
 * the same object.  Nothing synchronises the host.
 * No reference counterpart (its multi-GPU form of this path is NCCL all-gathers around the same operators,
 * easyvolcap/official_vggt/layers/dsa_attention.py:1138-1264).
 * ---------------------------------------------------------------------------------------------- */
typedef struct GwPeerExchange GwPeerExchange;
int gw_peer_barrier(const void* flag_ptrs_dev, int rank, int world, unsigned int seq, int limit_ms, int* status_dev,
                    gw_stream_t stream);
int gw_peer_exchange_create(int n_copy_streams, GwPeerExchange** out);
void gw_peer_exchange_destroy(GwPeerExchange* ex);
int gw_peer_exchange_run(GwPeerExchange* ex, gw_stream_t after, const void* flag_ptrs_dev, int rank, int world, unsigned int seq,
                         int limit_ms, int* status_dev, int n_pack, const void* const* pack_src, void* const* pack_dst,
                         const size_t* pack_bytes, int n_pull, const void* const* pull_src, void* const* pull_dst,
                         const size_t* pull_bytes, int pull_with_kernel);
int gw_peer_exchange_join(GwPeerExchange* ex, gw_stream_t waiter, int last_was_kernel);

/* ------------------------------------------------------------------------------------------------
 * Coarse-to-fine selection around the indexer (factor-2 pooled sources, round-robin expansion).
 * source_to_fine int32 [L, width] (width <= 4): the tokens of every source, -1 for a missing slot, slots filled from the
 * front.  gw_pool_sources: src_k [B,L,Hi,Di], src_w [B,L,Hi] = mean over a source's tokens of k [B,N,Hi,Di], w [B,N,Hi]
 * (fp32 accumulation, result in `dtype`; w and src_w may both be null: keys only, e.g. to pool queries the same way).
 * gw_expand_sources: per row (a query) a list of m kept sources and, optionally,
 * their scores -> out_k token indices: sources ordered by descending score (equal scores: lower source first; without
 * scores the given order is kept), then slot 0 of every source in that order, slot 1 of every source that has one, ...;
 * cut to out_k; a list that yields fewer tokens is padded by cycling over its last pad_window tokens.  m, out_k <= 4096.
 * Replaces: easyvolcap/official_vggt/layers/dsa_attention.py:3386-3543 (_prepare_source_downsample_projected, torch ops)
 *           and :4079-4128 (_expand_source_downsample_chunk, torch ops; the reference keeps the order its unsorted top-k
 *           returned).
 * ---------------------------------------------------------------------------------------------- */
int gw_pool_sources(const void* k, const void* w, const int32_t* source_to_fine, int dtype, int B, int N, int L, int Hi, int Di,
                    int width, void* src_k, void* src_w, gw_stream_t stream);
int gw_expand_sources(const int32_t* lists, const void* scores, int score_dtype, const int32_t* source_to_fine, int width, int L,
                      int n_tokens, long long rows, int m, int out_k, int pad_window, int32_t* out, gw_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Projection front-end (the step in front of stages 1-3): from the output of the layer's fused linear
 * projection to the six operator inputs, in one pass.
 *
 * fused [tokens, ld] of `dtype` holds per token [q | k | v | idx_q | idx_k | idx_w]
 * = 3*H*D + 2*Hi*Di + Hi values (qkv itself ordered [3][H][D]).  q, k: LayerNorm over D, then the 2-D rotary
 * embedding; v: copied; idx_q: rotary; idx_k: LayerNorm, rotary; idx_w: copied.  pos int64 [tokens, 2] = (y, x)
 * (null: no rotary embedding); cos_tab / sin_tab fp32 [table_rows, D/2], the tables of the reference's rotary
 * module (columns j and j + D/4 hold the same angle); a position outside the tables sets the status word.
 * Each LayerNorm is (weight, bias, eps) over 64 values, fp32, or null pointers for none.
 * Outputs, all of `dtype`, contiguous and token-major: q, k, v [tokens, H, D]; q_idx, k_idx [tokens, Hi, Di];
 * w [tokens, Hi] -- what gw_indexer_topk_fused and gw_sparse_attn_fwd read.
 * Requirements: D = Di = 64; rows of `fused` start on 8-byte boundaries (ld a multiple of 4 for 16-bit types, of 2
 *               for fp32); every pointer 16-byte aligned; Hi <= 32.
 * Replaces: easyvolcap/official_vggt/layers/dsa_attention.py:587-627 (_project_qkv_and_indexer_fused after its
 *           F.linear), :229-232 (_project_attention_qkv_from_flat), :4935-4941 (q_norm, k_norm, rope) and
 *           :5309-5315 (the .contiguous() transposes); easyvolcap/official_vggt/layers/indexer.py:302-328
 *           (LightningIndexer.project after its three linear layers); easyvolcap/official_vggt/layers/rope.py:134-188.
 * ---------------------------------------------------------------------------------------------- */
int gw_project_epilogue(const void* fused, int dtype, int64_t tokens, int64_t ld, int H, int D, int Hi, int Di,
                        const int64_t* pos, const float* cos_tab, const float* sin_tab, int table_rows,
                        const float* q_norm_w, const float* q_norm_b, float q_norm_eps, const float* k_norm_w,
                        const float* k_norm_b, float k_norm_eps, const float* idx_k_norm_w, const float* idx_k_norm_b,
                        float idx_k_norm_eps, void* q, void* k, void* v, void* q_idx, void* k_idx, void* w,
                        int* status_dev, gw_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * The projection itself, fused with gw_project_epilogue's work: [q | k | v | idx_q | idx_k | idx_w] = x . weight^T + bias
 * on the tcgen05 tensor cores (fp32 accumulation), then per head LayerNorm / rotary embedding as in
 * gw_project_epilogue on the fp32 accumulators, one rounding, token-major stores.  The raw product never reaches memory.
 * x [tokens, dim], weight [3*H*D + 2*Hi*Di + Hi, dim] (rows ordered qkv ([3][H][D]), idx_q, idx_k, idx_w), bias
 * [same rows] or null, all of `dtype` (GW_BF16 or GW_F16), contiguous.  Everything else as gw_project_epilogue.
 * Requirements: D = Di = 64, dim a multiple of 64, Hi <= 32, 16-byte aligned pointers.
 * Replaces: easyvolcap/official_vggt/layers/dsa_attention.py:545-627 (_project_qkv_and_indexer_fused: the F.linear
 *           over the concatenated weights and the split that follows), together with everything gw_project_epilogue replaces.
 * ---------------------------------------------------------------------------------------------- */
int gw_project_fused(const void* x, const void* weight, const void* bias, int dtype, int64_t tokens, int dim, int H, int D,
                     int Hi, int Di, const int64_t* pos, const float* cos_tab, const float* sin_tab, int table_rows,
                     const float* q_norm_w, const float* q_norm_b, float q_norm_eps, const float* k_norm_w,
                     const float* k_norm_b, float k_norm_eps, const float* idx_k_norm_w, const float* idx_k_norm_b,
                     float idx_k_norm_eps, void* q, void* k, void* v, void* q_idx, void* k_idx, void* w, int* status_dev,
                     gw_stream_t stream);

/* Diagnostics: the gather of gw_sparse_attn_fwd without its arithmetic -- for every query the K row and the V row
 * (row_bytes <= 2048, a multiple of 16; rows k_row_stride_bytes / v_row_stride_bytes apart) of each valid entry of
 * kv_pos int32 [T,K] is bulk-copied into shared memory and dropped.  Timed by the caller, it gives the rate this
 * copy method reaches on that index list: the ceiling for the attention kernel on the same list (L2-to-SM path
 * when K and V fit the L2, HBM otherwise).  Writes nothing to global memory.  No reference counterpart. */
int gw_debug_gather_rate(const void* k, const void* v, const int32_t* kv_pos, int64_t T, int S, int K, int row_bytes,
                         int64_t k_row_stride_bytes, int64_t v_row_stride_bytes, int* status_dev, gw_stream_t stream);
/* the same rows (contiguous, 2 KB each) fetched with plain 16-byte loads instead of bulk copies: the rate of the L2 -> SM path */
int gw_debug_gather_rate_ldg(const void* k, const void* v, const int32_t* kv_pos, int64_t T, int S, int K, int max_ctas,
                             gw_stream_t stream);
/* the same with at most max_ctas CTAs (0 = one per SM): how the gather rate depends on the number of SMs that gather */
int gw_debug_gather_rate_ctas(const void* k, const void* v, const int32_t* kv_pos, int64_t T, int S, int K, int row_bytes,
                              int64_t k_row_stride_bytes, int64_t v_row_stride_bytes, int max_ctas, int* status_dev,
                              gw_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* GEOWEAVE_B200_H */
