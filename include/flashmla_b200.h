/*
 * flashmla_b200 -- C ABI of the B200 (sm_100a) MLA attention library.
 *
 * This header is the whole boundary: plain pointers, sizes and strides, an
 * `int` status return, caller-owned outputs and scratch, and the CUDA stream
 * passed as an opaque pointer.  No torch / ATen type appears here.  Each entry
 * point names the function of the reference extension (csrc/pybind.cpp, bound
 * at :870-911) that it replaces.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer on the current device unless its name
 *     ends in `_host`;
 *   - strides are in ELEMENTS of the pointed-to type (bytes for the FP8 cache),
 *     as in the reference's parameter blocks (csrc/params.h:5-49, pybind.cpp:553);
 *   - functions only enqueue work on `stream` and return; they never call
 *     exit() or trap the device (the reference does both, csrc/utils.h:3-45);
 *   - return value 0 = FMLA_OK, otherwise an fmla_status code;
 *     fmla_status_string() gives a static description and
 *     fmla_last_error_message() a thread-local detailed message.
 *   - thread safety: entry points may be called concurrently from different
 *     host threads on different streams/devices; the library keeps no mutable
 *     global state besides per-device attribute caches guarded by a mutex.
 */
#ifndef FLASHMLA_B200_H_
#define FLASHMLA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum fmla_status {
  FMLA_OK = 0,
  FMLA_ERR_INVALID_ARGUMENT = 1,   /* shape / stride / pointer / alignment rejected */
  FMLA_ERR_UNSUPPORTED = 2,        /* valid request the kernels do not implement   */
  FMLA_ERR_CUDA = 3,               /* a CUDA runtime call failed (see message)      */
  FMLA_ERR_WRONG_ARCH = 4,         /* device is not compute capability 10.x         */
  FMLA_ERR_DEVICE_TIMEOUT = 5      /* a bounded device-side wait expired            */
} fmla_status;

enum { FMLA_TILE_SCHEDULER_METADATA_SIZE = 8 };  /* csrc/params.h:51 */
enum { FMLA_DTYPE_BF16 = 0, FMLA_DTYPE_FP16 = 1 };

const char* fmla_status_string(int status);
const char* fmla_last_error_message(void);
/* Library version "major.minor.patch" and the variant string the Python layer
 * reports as FLASH_MLA_LOADED_VARIANT (flash_mla/flash_mla_interface.py:54). */
const char* fmla_version(void);
const char* fmla_variant(void);

/* ------------------------------------------------------------------------- *
 * Split-KV tile scheduler.
 * Replaces get_mla_decoding_metadata (csrc/pybind.cpp:383-428), i.e.
 * get_attn_impl_meta (:288-380) + run_get_mla_metadata_kernel
 * (csrc/smxx/get_mla_metadata.cu:8-96).
 * ------------------------------------------------------------------------- */

/* Host query: how many partitions the schedule has for this problem on
 * `device` (so the caller can size tile_scheduler_metadata).
 *   num_q_tokens_per_head_k = s_q * h_q / h_k;  h_q is needed only when
 *   is_sparse != 0;  is_fp8_kvcache must equal is_sparse (dense FP8 and sparse
 *   BF16 caches are rejected, as in pybind.cpp:312-355). */
int fmla_get_num_sm_parts(int device, int num_q_tokens_per_head_k, int h_k, int h_q,
                          int is_fp8_kvcache, int is_sparse, int* num_sm_parts_host);

/* Enqueue the scheduler.  seqlens_k [batch] int32;  topk = -1 for dense
 * attention, otherwise every request is scheduled with length topk
 * (get_mla_metadata.cu:27).  Outputs:
 *   tile_scheduler_metadata [num_sm_parts][8] int32 =
 *     {begin_idx, begin_block_idx, end_idx (inclusive), end_block_idx
 *      (exclusive), begin_n_split_idx, 0, 0, 0}            (csrc/params.h:52)
 *   num_splits [batch+1] int32, exclusive prefix of per-request part counts. */
int fmla_get_mla_metadata(const int32_t* seqlens_k, int batch, int num_sm_parts, int topk,
                          int32_t* tile_scheduler_metadata, int32_t* num_splits, void* stream);

/* ------------------------------------------------------------------------- *
 * Decode attention over a paged KV cache (dense BF16, or sparse FP8 + top-k).
 * Replaces fwd_kvcache_mla (csrc/pybind.cpp:430-720): split-KV attention
 * kernel followed by the log-sum-exp combine (csrc/smxx/mla_combine.cu).
 * Mirrors DecodingParams (csrc/params.h:5-49); outputs and scratch are
 * caller-allocated (the reference allocates them at pybind.cpp:526-528, 574-581).
 * ------------------------------------------------------------------------- */
typedef struct fmla_decode_params {
  int32_t b, s_q, h_q, h_k;        /* batch, queries per request, q heads, kv heads */
  int32_t d, d_v;                  /* 576, 512                                       */
  int32_t num_blocks;              /* pages in the cache                             */
  int32_t page_block_size;         /* 64                                             */
  int32_t is_causal;               /* ignored when s_q == 1 (pybind.cpp:501)         */
  int32_t is_fp8;                  /* cache holds 656-byte FP8 token records         */
  int32_t topk;                    /* -1 = dense; else indices[...,topk] are used    */
  int32_t q_dtype;                 /* FMLA_DTYPE_BF16, or FMLA_DTYPE_FP16 (dense only) */
  float softmax_scale;

  const void* q;                   /* [b, s_q, h_q, d]; last dim contiguous          */
  int64_t q_stride_b, q_stride_s, q_stride_h;
  const void* kcache;              /* bf16 [num_blocks, 64, h_k, d]  or  bytes [num_blocks, 64, 1, 656] */
  int64_t k_stride_block, k_stride_row, k_stride_head;
  const int32_t* block_table;      /* [b, max_blocks]; dense only                    */
  int64_t block_table_stride_b;
  const int32_t* seqlens_k;        /* [b]                                            */
  const int32_t* indices;          /* [b, s_q, topk] physical slots page*64+off, <0 or >= num_blocks*64 = padding */
  int64_t indices_stride_b, indices_stride_s;

  const int32_t* tile_scheduler_metadata;  /* from fmla_get_mla_metadata             */
  int32_t num_sm_parts;
  const int32_t* num_splits;       /* [b+1]                                          */

  void* out;                       /* [b, s_q, h_q, d_v] q dtype; last dim contiguous */
  int64_t o_stride_b, o_stride_s, o_stride_h;
  float* softmax_lse;              /* [b, h_q, s_q] contiguous, natural log, +inf for empty rows */

  /* scratch for split requests: (b + num_sm_parts) partial slots, see
   * fmla_decode_scratch_bytes(); contents on entry are irrelevant. */
  float* lse_accum;                /* [b + num_sm_parts, h_k, s_q*h_q/h_k]           */
  float* o_accum;                  /* [b + num_sm_parts, h_k, s_q*h_q/h_k, d_v]      */

  /* optional cudaEvent_t pair recorded on `stream` immediately before and after
   * the attention kernel (the combine kernel follows the second); NULL = off. */
  void* profile_event_begin;
  void* profile_event_end;

  /* sparse decode only: when non-zero, `indices` hold LOGICAL token positions of the request (what a top-k
   * indexer produces); the kernel maps them through block_table itself (position p -> slot
   * block_table[b][p / 64] * 64 + p % 64; p < 0 or p >= seqlens_k[b] = padding).  No counterpart in the
   * reference, whose callers remap to physical slots first (README.md:176). */
  int32_t indices_logical;

  /* optional, dense decode: b * s_q * (h_q / 64) int32 counters, ZERO on entry and left zero on return.  When
   * given (and the heads per kv head are a multiple of 128), the CTA that writes the last partial of a split
   * request also merges that request's partials, so no separate merge kernel is launched: the whole step is
   * one kernel.  Calls that may overlap on the GPU need separate counter arrays.  NULL = the merge runs as a
   * second kernel (fmla's counterpart of csrc/smxx/mla_combine.cu).  No counterpart in the reference. */
  int32_t* arrival_counters;

  /* optional: non-zero = the caller knows that the schedule splits no request (num_splits[b] == b), so every
   * partition writes final outputs and the merge kernel has nothing to do: it is not launched.  A kernel that
   * meets a split request under this hint reports status 41 instead of leaving partials unmerged.  0 = unknown
   * (the merge kernel is launched and finds out by itself).  No counterpart in the reference. */
  int32_t no_split_hint;
} fmla_decode_params;

/* Bytes of lse_accum and o_accum for a problem (host-side arithmetic only). */
int fmla_decode_scratch_bytes(int b, int s_q, int h_q, int num_sm_parts, int d_v,
                              size_t* lse_accum_bytes_host, size_t* o_accum_bytes_host);

int fmla_fwd_kvcache_mla(const fmla_decode_params* params_host, void* stream);

/* Same computation as fmla_fwd_kvcache_mla for callers that must not allocate
 * (this entry point has no counterpart in the reference, whose extension always
 * allocates its accumulators with torch, csrc/pybind.cpp:574-581).
 *
 * Who needs it: a host that gives out device memory only at start-up (a fixed
 * arena, a plugin "enqueue" hook, a loop that is being recorded into a stream)
 * cannot size and allocate the split-KV scratch per call, and cudaMalloc there
 * would either be refused or stall the device.  Here the scratch lives in the
 * library image: params->lse_accum and params->o_accum are IGNORED and replaced
 * by two built-in device arrays; inputs and outputs are still the caller's.
 *
 *  - limit: (b + num_sm_parts) * s_q * h_q  <=  fmla_static_scratch_max_rows()
 *    (32768 rows, i.e. 64 MiB + 128 KiB held by every GPU that loads the library
 *    until the process exits); larger problems are rejected with
 *    FMLA_ERR_INVALID_ARGUMENT and a message naming both numbers;
 *  - the first call on each device looks up the arrays' device addresses
 *    (cudaGetSymbolAddress); make that first call before recording work into a
 *    stream, later calls only launch kernels;
 *  - every call on a GPU uses the same arrays: calls that overlap on the GPU
 *    (different streams or threads) race on them; serialise them.  Nothing has
 *    to be cleared between calls: each call overwrites every slot it later reads;
 *  - it performs no cudaMalloc / cudaFree and calls no allocating routine. */
int fmla_fwd_kvcache_mla_static_scratch(const fmla_decode_params* params_host, void* stream);
size_t fmla_static_scratch_max_rows(void);

/* ------------------------------------------------------------------------- *
 * Stand-alone log-sum-exp merge of normalised partial results.
 * Replaces run_flash_mla_combine_kernel (csrc/smxx/mla_combine.cu:170-195) and
 * lifts its 64-split limit (:156-167).  Also the merge step of a KV-sharded
 * decode across GPUs: partials written by peers into this GPU's memory are
 * merged exactly like local split-KV partials.
 *   lse_accum [num_parts, rows] base-2 (-inf = empty), o_accum [num_parts, rows, d_v] fp32
 *   out [rows, d_v] bf16 (row stride o_stride_row), lse [rows] natural log.
 * ------------------------------------------------------------------------- */
int fmla_combine_partials(const float* lse_accum, const float* o_accum, int num_parts, int rows,
                          int d_v, void* out, int64_t o_stride_row, float* lse, void* stream);

/* ------------------------------------------------------------------------- *
 * KV-sharded decode across GPUs (one long context whose cache pages are split
 * over N ranks).  No counterpart in the reference, which is single-GPU; the
 * math is its split-KV merge (csrc/smxx/mla_combine.cu:71-151) applied to
 * per-rank partials instead of per-SM partials.
 *
 * fmla_fwd_kvcache_mla_push_partial: runs the dense decode over this rank's
 * shard, merges the local splits and stores the normalised fp32 partial O
 * [b*h_q*s_q rows, 512] and its base-2 LSE into slot `slot` of every
 * destination's buffers (device pointers that may be peer-mapped memory of other
 * GPUs: plain stores over NVLink), then publishes `epoch` in dst_flag[d][slot]
 * with a system-scope release.  params->out / softmax_lse are not written.
 * `counter` is a zero-initialised device word owned by this rank.
 *
 * fmla_merge_peer_partials: waits (at most max_polls polls of ~200 ns per flag)
 * until flags[i] == epoch for all i < num_parts, then merges the parts like
 * fmla_combine_partials.  If a flag never arrives the kernel leaves the outputs
 * untouched and sets the device status word (fmla_device_status reports
 * FMLA_ERR_DEVICE_TIMEOUT); it does not hang.
 * ------------------------------------------------------------------------- */
typedef struct fmla_peer_push {
  int32_t slot;              /* this rank's slot in the destinations' buffers */
  int32_t num_dst;           /* 1..8                                          */
  float* dst_o[8];           /* [num_slots][rows][512] fp32                   */
  float* dst_lse[8];         /* [num_slots][rows] fp32, base 2                */
  uint32_t* dst_flag[8];     /* [num_slots]                                   */
  uint32_t epoch;            /* value published in the flags (change it every step) */
  uint32_t* counter;         /* local scratch word, zero before the first call */
} fmla_peer_push;

int fmla_fwd_kvcache_mla_push_partial(const fmla_decode_params* params_host, const fmla_peer_push* push_host, void* stream);
int fmla_merge_peer_partials(const float* part_lse, const float* part_o, int num_parts, int rows, int d_v,
                             const uint32_t* flags, uint32_t epoch, int max_polls, void* out, int64_t o_stride_row,
                             float* lse, void* stream);

/* ------------------------------------------------------------------------- *
 * Sparse MLA prefill forward.  Replaces sparse_prefill_fwd
 * (csrc/pybind.cpp:730-814) -> sm100::run_fwd_kernel
 * (csrc/sm100/prefill/sparse/fwd.cu:705-783).  Mirrors SparsePrefillParams
 * (csrc/params.h:65-84).  Requires h_kv == 1, d_qk == 576, d_v == 512,
 * h_q % 64 == 0, topk % 64 == 0.
 * ------------------------------------------------------------------------- */
typedef struct fmla_sparse_prefill_params {
  int32_t s_q, s_kv, h_q, h_kv, d_qk, d_v, topk;
  float sm_scale;
  const void* q;          int64_t q_stride_s, q_stride_h;        /* bf16 [s_q, h_q, d_qk]  */
  const void* kv;         int64_t kv_stride_s, kv_stride_h;      /* bf16 [s_kv, h_kv, d_qk] */
  const int32_t* indices; int64_t indices_stride_s, indices_stride_h;  /* [s_q, h_kv, topk]; <0 or >= s_kv = padding */
  void* out;              /* bf16 [s_q, h_q, d_v] contiguous */
  float* max_logits;      /* [s_q, h_q], base-2 logits' maximum, -inf for empty rows */
  float* lse;             /* [s_q, h_q], base-2 log-sum-exp, -inf for empty rows      */
} fmla_sparse_prefill_params;

int fmla_sparse_prefill_fwd(const fmla_sparse_prefill_params* params_host, void* stream);

/* ------------------------------------------------------------------------- *
 * Dense variable-length MHA forward / backward (bf16; head dims 192/128 or
 * 128/128).  Replace dense_prefill_fwd / dense_prefill_bwd
 * (csrc/pybind.cpp:817-867) -> FMHACutlassSM100FwdRun / BwdRun
 * (csrc/sm100/prefill/dense/fmha_cutlass_{fwd,bwd}_sm100.cu).  Unsupported head
 * dims return FMLA_ERR_UNSUPPORTED (the reference silently does nothing,
 * fmha_cutlass_fwd_sm100.cu:110-113).
 * ------------------------------------------------------------------------- */
typedef struct fmla_dense_params {
  int32_t batch;                     /* number of sequences                          */
  int32_t total_q, total_k;          /* packed token counts                          */
  int32_t h_q, h_k, d_qk, d_v;
  int32_t max_seqlen_q, max_seqlen_k;
  int32_t is_causal;                 /* mask_mode_code: 0 none, 1 causal (bottom-right aligned) */
  float softmax_scale;
  const void* q; int64_t q_stride_t, q_stride_h;     /* bf16 [total_q, h_q, d_qk] */
  const void* k; int64_t k_stride_t, k_stride_h;     /* bf16 [total_k, h_k, d_qk] */
  const void* v; int64_t v_stride_t, v_stride_h;     /* bf16 [total_k, h_k, d_v]  */
  const int32_t* cu_seqlens_q;       /* [batch+1] */
  const int32_t* cu_seqlens_k;       /* [batch+1] */
  void* o;       int64_t o_stride_t, o_stride_h;     /* bf16 [total_q, h_q, d_v]  */
  float* lse;    int64_t lse_stride_t, lse_stride_h; /* fp32 [total_q, h_q] natural log, -inf for empty rows */
  /* backward only */
  const void* d_o; int64_t do_stride_t, do_stride_h; /* bf16 [total_q, h_q, d_v]  */
  void* dq;      int64_t dq_stride_t, dq_stride_h;   /* bf16 [total_q, h_q, d_qk] */
  void* dk;      int64_t dk_stride_t, dk_stride_h;   /* bf16 [total_k, h_k, d_qk] */
  void* dv;      int64_t dv_stride_t, dv_stride_h;   /* bf16 [total_k, h_k, d_v]  */
  void* workspace; size_t workspace_bytes;           /* >= fmla_dense_bwd_workspace_bytes() */
} fmla_dense_params;

int fmla_dense_prefill_fwd(const fmla_dense_params* params_host, void* stream);
size_t fmla_dense_bwd_workspace_bytes(int total_q, int h_q, int d_qk);
int fmla_dense_prefill_bwd(const fmla_dense_params* params_host, void* stream);

/* ------------------------------------------------------------------------- *
 * FP8 KV-cache writer: bf16 [num_tokens, 576] rows -> 656-byte records
 * (README.md:162-170; the reference only has the torch helper
 * tests/quant.py:3-35).  dst_slots[i] = physical slot of token i, or NULL for
 * slot i = i.
 * ------------------------------------------------------------------------- */
int fmla_quantize_kv_fp8(const void* kv_bf16, int64_t kv_stride_row, int num_tokens,
                         const int32_t* dst_slots, void* cache_bytes, int64_t cache_stride_slot_bytes,
                         void* stream);

/* Synchronises the current device and reads the status word that the tcgen05
 * kernels set when one of their bounded waits (mbarrier polls) gives up instead
 * of hanging: 0 = no fault.  Returns FMLA_ERR_DEVICE_TIMEOUT when it is non-zero;
 * `reset` != 0 clears it.  The reference has no counterpart: its kernels wait
 * without bound and trap on failed asserts (csrc/utils.h:24-30).
 *
 * A kernel that gives up also stores the code into a page of host memory that the
 * library registers (page-locked, mapped) the first time a launching entry point
 * runs in the process; every launching entry point reads that word on entry,
 * without synchronising, and returns FMLA_ERR_DEVICE_TIMEOUT instead of launching
 * on top of a failed pipeline until the condition is cleared with `reset`.  That
 * first call does one-time set-up per device (a host-memory registration and a few
 * symbol updates) and therefore has to come before any stream capture. */
int fmla_device_status(int* status_host, int reset);

/* sizeof() of the parameter blocks as compiled into the library, so a foreign
 * binding (ctypes, cgo, JNI ...) can verify its own struct layout at load time. */
size_t fmla_sizeof_decode_params(void);
size_t fmla_sizeof_sparse_prefill_params(void);
size_t fmla_sizeof_dense_params(void);
size_t fmla_sizeof_peer_push(void);

#ifdef __cplusplus
}
#endif
#endif /* FLASHMLA_B200_H_ */
