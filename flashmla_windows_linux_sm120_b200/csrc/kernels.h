// Internal launcher declarations shared by the kernel translation units and the
// C-ABI layer (abi.cu).  Kernel parameter blocks are plain structs passed by
// value as __grid_constant__.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace fmla {

struct DecodeKernelParams {
  int b, s_q, h_q, h_k, hq_per_hk;
  int num_blocks;
  int is_causal;
  int topk;  // -1 dense
  float scale_log2;
  const void* q;
  int64_t q_stride_b, q_stride_s, q_stride_h;
  const void* kcache;
  int64_t k_stride_block, k_stride_row, k_stride_head;  // elements (dense) / bytes (fp8)
  const int* block_table;
  int64_t block_table_stride_b;
  const int* seqlens_k;
  const int* indices;
  int64_t indices_stride_b, indices_stride_s;
  const int* tile_scheduler_metadata;
  int num_sm_parts;
  const int* num_splits;
  void* out;
  int64_t o_stride_b, o_stride_s, o_stride_h;
  float* softmax_lse;
  float* lse_accum;
  float* o_accum;
  // KV-sharded decode across GPUs: every request goes through the accumulators (force_partial) and the
  // merge of the local splits is pushed, as a normalised fp32 partial, into slot `push_slot` of each
  // destination's partial buffers (peer-mapped device memory), followed by a flag store.
  int is_f16;                  // q, cache and out are fp16 instead of bf16 (dense decode only)
  int indices_logical;         // sparse decode: indices are token positions, mapped through block_table in the kernel
  int force_partial;
  int l2_prefetch_dist;        // pair kernel: cache pages this many blocks ahead are pulled into L2 (0 = off)
  int* arrival_counters;       // pair kernel: per (request, query token, 64-head tile) arrivals of split partials; zero on entry and exit
  int no_split_hint;           // the caller states that no request is split: no merge kernel follows; a split request is reported (status 41)
  int push_slot, push_num_dst;
  float* push_o[8];            // [num_slots][b * h_k * rows][512]
  float* push_lse[8];          // [num_slots][b * h_k * rows], base 2
  unsigned int* push_flag[8];  // [num_slots]
  unsigned int push_epoch;
  unsigned int* push_counter;  // local counter of finished CTAs (zero on entry, left zero)
};

struct SparsePrefillKernelParams {
  int s_q, s_kv, h_q, topk;
  float scale_log2;
  const void* q;
  int64_t q_stride_s, q_stride_h;
  const void* kv;
  int64_t kv_stride_s;
  const int* indices;
  int64_t indices_stride_s;
  void* out;
  float* max_logits;
  float* lse;
};

struct DenseKernelParams {
  int batch, h_q, h_k, d_qk, d_v, max_seqlen_q, max_seqlen_k, is_causal;
  int total_q, total_k;
  float scale, scale_log2;
  const void* q; int64_t q_stride_t, q_stride_h;
  const void* k; int64_t k_stride_t, k_stride_h;
  const void* v; int64_t v_stride_t, v_stride_h;
  const int* cu_q;
  const int* cu_k;
  void* o; int64_t o_stride_t, o_stride_h;
  float* lse; int64_t lse_stride_t, lse_stride_h;
  const void* d_o; int64_t do_stride_t, do_stride_h;
  void* dq; int64_t dq_stride_t, dq_stride_h;
  void* dk; int64_t dk_stride_t, dk_stride_h;
  void* dv; int64_t dv_stride_t, dv_stride_h;
  float* delta;      // workspace: [h_q, total_q] rowsum(dO * O)
  float* dq_acc;     // workspace (unused by the deterministic dQ pass)
};

// records `message` as the calling thread's last error and returns `code`
int set_error(int code, const char* message);

// Each kernel translation unit keeps a pointer to a host-mapped status word beside its device status word
// (tc_common.cuh); these set it for the current device.
cudaError_t set_status_mirror_mla(int* mapped_host_word);
cudaError_t set_status_mirror_pair(int* mapped_host_word);
cudaError_t set_status_mirror_merge(int* mapped_host_word);
cudaError_t set_status_mirror_dense_fwd(int* mapped_host_word);
cudaError_t set_status_mirror_dense_bwd(int* mapped_host_word);

cudaError_t launch_get_mla_metadata(const int* seqlens_k, int batch, int num_sm_parts, int topk, int* md,
                                    int* num_splits, cudaStream_t stream);
// tcgen05 / TMA / TMEM kernels (mla_tc.cu): dense decode, sparse FP8 decode, sparse prefill
cudaError_t launch_decode_dense_tc(const DecodeKernelParams& p, cudaStream_t stream);
cudaError_t launch_decode_sparse_tc(const DecodeKernelParams& p, cudaStream_t stream);
cudaError_t launch_sparse_prefill_tc(const SparsePrefillKernelParams& p, cudaStream_t stream);
// reads (and optionally clears) the status word the tcgen05 kernels set when a bounded wait expires
cudaError_t read_decode_tc_status(int* host_status, bool reset);
// dense decode as a CTA pair (mla_pair.cu): 128 heads per pair, tcgen05 cta_group::2; used by
// launch_decode_dense_tc whenever the heads per kv head are a multiple of 128
bool decode_dense_pair_applies(const DecodeKernelParams& p);
// true when launch_decode_dense_tc will merge the split partials inside the attention kernel (no merge launch needed)
bool decode_dense_merges_in_kernel(const DecodeKernelParams& p);
cudaError_t launch_decode_dense_pair(const DecodeKernelParams& p, cudaStream_t stream);
cudaError_t read_decode_pair_status(int* host_status, bool reset);
// sparse prefill forward as CTA pairs with TMA row gathers (mla_pair.cu); used by launch_sparse_prefill_tc for 128 heads
bool decode_sparse_pair_applies(const DecodeKernelParams& p);
cudaError_t launch_decode_sparse_pair(const DecodeKernelParams& p, cudaStream_t stream);
bool sparse_prefill_pair_applies(const SparsePrefillKernelParams& sp);
cudaError_t launch_sparse_prefill_pair(const SparsePrefillKernelParams& sp, cudaStream_t stream);
// Merge of split partials for a decode call (reads num_splits; skips unsplit requests).
cudaError_t launch_decode_combine(const DecodeKernelParams& p, cudaStream_t stream);
// Stand-alone merge of num_parts partial slots for `rows` rows.
cudaError_t launch_combine_partials(const float* lse_accum, const float* o_accum, int num_parts, int rows, void* out,
                                    int64_t o_stride_row, float* lse, cudaStream_t stream);
// merge of local splits + push of the result to peers (see DecodeKernelParams::push_*)
cudaError_t launch_decode_combine_push(const DecodeKernelParams& p, cudaStream_t stream);
// merge that first waits (bounded) until flags[i] == epoch for every part
cudaError_t launch_merge_peer_partials(const float* lse_accum, const float* o_accum, int num_parts, int rows, void* out,
                                       int64_t o_stride_row, float* lse, const unsigned int* flags, unsigned int epoch,
                                       int max_polls, cudaStream_t stream);
cudaError_t read_merge_status(int* host_status, bool reset);
// tcgen05 / TMA / TMEM forward (dense_fwd_tc.cu) and its status word
cudaError_t launch_dense_fwd_tc(const DenseKernelParams& p, cudaStream_t stream);
cudaError_t read_dense_tc_status(int* host_status, bool reset);
// tcgen05 / TMA / TMEM backward (dense_bwd_tc.cu) and its status word
cudaError_t launch_dense_bwd_tc(const DenseKernelParams& p, cudaStream_t stream);
cudaError_t read_dense_bwd_tc_status(int* host_status, bool reset);
cudaError_t launch_quantize_kv_fp8(const void* kv, int64_t kv_stride_row, int num_tokens, const int* dst_slots,
                                   void* cache, int64_t cache_stride_slot, cudaStream_t stream);

}  // namespace fmla
