// C-ABI entry points (include/flashmla_b200.h): argument validation,
// translation to kernel parameter blocks, launches.  No torch types, no
// allocation, no exit()/trap: every failure is a status code plus a
// thread-local message.
#include "../../include/flashmla_b200.h"
#include "kernels.h"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(FMLA_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define FMLA_REQUIRE(cond, ...) \
  do {                          \
    if (!(cond)) return fail(FMLA_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Per-device properties, cached (sm count, compute capability).
struct DevInfo {
  int sm_count = 0, major = 0, minor = 0;
  bool ok = false;
};
std::mutex g_dev_mutex;
DevInfo g_dev[64];

int device_info(int device, DevInfo* out) {
  if (device < 0 || device >= 64) return fail(FMLA_ERR_INVALID_ARGUMENT, "device index %d out of range", device);
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!g_dev[device].ok) {
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceProperties");
    g_dev[device].sm_count = prop.multiProcessorCount;
    g_dev[device].major = prop.major;
    g_dev[device].minor = prop.minor;
    g_dev[device].ok = true;
  }
  *out = g_dev[device];
  return FMLA_OK;
}

// ---- device-side timeouts, visible to the host without a synchronise ----------------------------------
// A bounded wait that expires inside a kernel records a code in a device status word AND stores it into a
// word of this page of host memory, which is registered (page-locked, mapped) once per process and whose
// device-side address every kernel translation unit learns once per device.  The next library call on that
// device reads the word with a plain load and refuses to launch on top of a failed pipeline.
constexpr int kStatusStride = 16;                       // ints: one 64-byte line per device
alignas(4096) int g_host_status[64 * kStatusStride];
std::mutex g_status_mutex;
bool g_status_registered = false, g_status_unavailable = false;
bool g_mirror_set[64] = {};

void ensure_status_mirror(int dev) {
  if (g_mirror_set[dev] || g_status_unavailable) return;
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (g_mirror_set[dev] || g_status_unavailable) return;
  if (!g_status_registered) {
    if (cudaHostRegister(g_host_status, sizeof(g_host_status), cudaHostRegisterMapped | cudaHostRegisterPortable) != cudaSuccess) {
      (void)cudaGetLastError();
      g_status_unavailable = true;      // the device status words and fmla_device_status() still work
      return;
    }
    g_status_registered = true;
  }
  void* dptr = nullptr;
  if (cudaHostGetDevicePointer(&dptr, &g_host_status[dev * kStatusStride], 0) != cudaSuccess) {
    (void)cudaGetLastError();
    g_status_unavailable = true;
    return;
  }
  int* w = static_cast<int*>(dptr);
  if (fmla::set_status_mirror_mla(w) != cudaSuccess || fmla::set_status_mirror_pair(w) != cudaSuccess ||
      fmla::set_status_mirror_merge(w) != cudaSuccess ||
      fmla::set_status_mirror_dense_fwd(w) != cudaSuccess || fmla::set_status_mirror_dense_bwd(w) != cudaSuccess) {
    (void)cudaGetLastError();
    g_status_unavailable = true;
    return;
  }
  g_mirror_set[dev] = true;
}

// Common prologue of every launching entry point: right architecture, status mirror in place, and no
// failure left behind by an earlier launch on this device.
int require_blackwell() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  DevInfo di;
  int rc = device_info(dev, &di);
  if (rc) return rc;
  if (di.major != 10) return fail(FMLA_ERR_WRONG_ARCH, "device %d is sm_%d%d; this library is built for sm_100a only", dev, di.major, di.minor);
  ensure_status_mirror(dev);
  const int code = *reinterpret_cast<volatile int*>(&g_host_status[dev * kStatusStride]);
  if (code != 0)
    return fail(FMLA_ERR_DEVICE_TIMEOUT,
                "an earlier launch on device %d gave up on a bounded device-side wait (code %d): its outputs are not valid; "
                "call fmla_device_status(&status, 1) to clear the condition", dev, code);
  return FMLA_OK;
}

}  // namespace

namespace fmla {
// lets other translation units of the library report through the same thread-local message
int set_error(int code, const char* message) { return fail(code, "%s", message); }
}  // namespace fmla

extern "C" {

const char* fmla_status_string(int status) {
  switch (status) {
    case FMLA_OK: return "ok";
    case FMLA_ERR_INVALID_ARGUMENT: return "invalid argument";
    case FMLA_ERR_UNSUPPORTED: return "unsupported configuration";
    case FMLA_ERR_CUDA: return "CUDA runtime error";
    case FMLA_ERR_WRONG_ARCH: return "wrong GPU architecture (needs compute capability 10.x)";
    case FMLA_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
    default: return "unknown status";
  }
}
const char* fmla_last_error_message(void) { return g_err; }
const char* fmla_version(void) { return "0.1.0"; }
const char* fmla_variant(void) { return "sm100a"; }
size_t fmla_sizeof_decode_params(void) { return sizeof(fmla_decode_params); }
size_t fmla_sizeof_sparse_prefill_params(void) { return sizeof(fmla_sparse_prefill_params); }
size_t fmla_sizeof_dense_params(void) { return sizeof(fmla_dense_params); }
size_t fmla_sizeof_peer_push(void) { return sizeof(fmla_peer_push); }

int fmla_get_num_sm_parts(int device, int num_q_tokens_per_head_k, int h_k, int h_q, int is_fp8_kvcache, int is_sparse,
                          int* num_sm_parts_host) {
  FMLA_REQUIRE(num_sm_parts_host != nullptr, "num_sm_parts_host is null");
  FMLA_REQUIRE(num_q_tokens_per_head_k > 0 && h_k > 0, "num_q_tokens_per_head_k and h_k must be positive");
  if (is_sparse && !is_fp8_kvcache) return fail(FMLA_ERR_UNSUPPORTED, "sparse attention over a BF16 cache is not supported");
  if (!is_sparse && is_fp8_kvcache) return fail(FMLA_ERR_UNSUPPORTED, "dense attention over an FP8 cache is not supported");
  DevInfo di;
  int rc = device_info(device, &di);
  if (rc) return rc;
  int parts;
  if (is_sparse) {
    FMLA_REQUIRE(h_q > 0 && h_q % h_k == 0, "h_q must be given and divisible by h_k for sparse attention");
    const int s_q = num_q_tokens_per_head_k * h_k / h_q;
    FMLA_REQUIRE(s_q > 0, "inconsistent num_q_tokens_per_head_k / h_q / h_k");
    parts = di.sm_count / h_k / (((h_q / h_k + 63) / 64) * s_q);
  } else {
    parts = di.sm_count / h_k / ((num_q_tokens_per_head_k + 63) / 64);
  }
  *num_sm_parts_host = parts > 1 ? parts : 1;
  return FMLA_OK;
}

int fmla_get_mla_metadata(const int32_t* seqlens_k, int batch, int num_sm_parts, int topk,
                          int32_t* tile_scheduler_metadata, int32_t* num_splits, void* stream) {
  FMLA_REQUIRE(seqlens_k && tile_scheduler_metadata && num_splits, "null pointer");
  FMLA_REQUIRE(batch > 0, "batch must be positive");
  FMLA_REQUIRE(num_sm_parts > 0 && num_sm_parts <= 1023, "num_sm_parts must be in 1..1023");
  FMLA_REQUIRE(topk == -1 || topk > 0, "topk must be -1 (dense) or positive");
  FMLA_REQUIRE(aligned16(tile_scheduler_metadata), "tile_scheduler_metadata must be 16-byte aligned");
  cudaError_t e = fmla::launch_get_mla_metadata(seqlens_k, batch, num_sm_parts, topk, tile_scheduler_metadata, num_splits,
                                               static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? FMLA_OK : cuda_fail(e, "get_mla_metadata launch");
}

int fmla_decode_scratch_bytes(int b, int s_q, int h_q, int num_sm_parts, int d_v, size_t* lse_bytes, size_t* o_bytes) {
  FMLA_REQUIRE(lse_bytes && o_bytes, "null pointer");
  FMLA_REQUIRE(b > 0 && s_q > 0 && h_q > 0 && num_sm_parts > 0 && d_v > 0, "sizes must be positive");
  const size_t rows = static_cast<size_t>(b + num_sm_parts) * s_q * h_q;
  *lse_bytes = rows * sizeof(float);
  *o_bytes = rows * d_v * sizeof(float);
  return FMLA_OK;
}

static int decode_impl(const fmla_decode_params* P, const fmla_peer_push* push, void* stream) {
  FMLA_REQUIRE(P != nullptr, "params is null");
  const fmla_decode_params& a = *P;
  const bool sparse = a.topk >= 0;
  FMLA_REQUIRE(a.b > 0, "batch size must be positive");
  FMLA_REQUIRE(a.s_q > 0 && a.h_q > 0 && a.h_k > 0, "s_q, h_q, h_k must be positive");
  FMLA_REQUIRE(a.d == 576, "Only head_size_k == 576 is supported");
  FMLA_REQUIRE(a.d_v == 512, "Only head_size_v == 512 is supported");
  FMLA_REQUIRE(a.page_block_size == 64, "Currently page_block_size must be 64");
  FMLA_REQUIRE(a.h_q % a.h_k == 0, "Number of heads in key/value must divide number of heads in query");
  if (a.q_dtype != FMLA_DTYPE_BF16 && a.q_dtype != FMLA_DTYPE_FP16) return fail(FMLA_ERR_INVALID_ARGUMENT, "q_dtype must be FMLA_DTYPE_BF16 or FMLA_DTYPE_FP16");
  if (a.q_dtype == FMLA_DTYPE_FP16 && (sparse || a.is_fp8)) return fail(FMLA_ERR_UNSUPPORTED, "float16 queries are supported for the dense (float16 cache) decode only");
  if (sparse != (a.is_fp8 != 0)) return fail(FMLA_ERR_UNSUPPORTED, "supported combinations: dense BF16 cache, or sparse (indices) FP8 cache");
  FMLA_REQUIRE(a.q && a.kcache && a.seqlens_k && a.tile_scheduler_metadata && a.num_splits && a.lse_accum && a.o_accum, "null pointer");
  FMLA_REQUIRE(push || (a.out && a.softmax_lse), "null output pointer");
  FMLA_REQUIRE(a.num_sm_parts > 0, "num_sm_parts must be positive");
  FMLA_REQUIRE(aligned16(a.q) && aligned16(a.kcache) && aligned16(a.out) && aligned16(a.o_accum) && aligned16(a.tile_scheduler_metadata), "q, kcache, out, o_accum and tile_scheduler_metadata must be 16-byte aligned");
  FMLA_REQUIRE(a.q_stride_b % 8 == 0 && a.q_stride_s % 8 == 0 && a.q_stride_h % 8 == 0, "q strides must be multiples of 8 elements");
  FMLA_REQUIRE(a.o_stride_b % 8 == 0 && a.o_stride_s % 8 == 0 && a.o_stride_h % 8 == 0, "out strides must be multiples of 8 elements");
  FMLA_REQUIRE(std::isfinite(a.softmax_scale) && a.softmax_scale > 0.f, "softmax_scale must be positive and finite");
  if (sparse) {
    FMLA_REQUIRE(a.h_k == 1, "Currently the number of k heads must be 1 when is_fp8_kvcache is True");
    FMLA_REQUIRE(a.indices != nullptr, "indices is null");
    FMLA_REQUIRE(a.topk > 0 && a.topk % 64 == 0, "topk must be a positive multiple of 64");
    FMLA_REQUIRE(a.k_stride_row == 656, "The whole block must be contiguous when is_fp8_cache is True");
    FMLA_REQUIRE(a.k_stride_block % 16 == 0, "FP8 cache block stride must be a multiple of 16 bytes");
    FMLA_REQUIRE(!a.is_causal, "causal must be false if sparse attention is enabled");
  } else {
    FMLA_REQUIRE(a.block_table != nullptr, "block_table is null");
    FMLA_REQUIRE(a.k_stride_block % 8 == 0 && a.k_stride_row % 8 == 0 && a.k_stride_head % 8 == 0, "kcache strides must be multiples of 8 elements");
  }
  FMLA_REQUIRE(!(push && sparse), "the peer push is implemented for the dense decode");
  int rc = require_blackwell();
  if (rc) return rc;

  fmla::DecodeKernelParams k = {};
  k.b = a.b; k.s_q = a.s_q; k.h_q = a.h_q; k.h_k = a.h_k; k.hq_per_hk = a.h_q / a.h_k;
  k.num_blocks = a.num_blocks;
  k.is_causal = (a.is_causal && a.s_q > 1) ? 1 : 0;   // s_q == 1 => causal is a no-op (pybind.cpp:501)
  k.topk = sparse ? a.topk : -1;
  k.scale_log2 = a.softmax_scale * 1.4426950408889634f;
  k.is_f16 = a.q_dtype == FMLA_DTYPE_FP16 ? 1 : 0;
  k.q = a.q; k.q_stride_b = a.q_stride_b; k.q_stride_s = a.q_stride_s; k.q_stride_h = a.q_stride_h;
  k.kcache = a.kcache; k.k_stride_block = a.k_stride_block; k.k_stride_row = a.k_stride_row; k.k_stride_head = a.k_stride_head;
  k.block_table = a.block_table; k.block_table_stride_b = a.block_table_stride_b;
  k.seqlens_k = a.seqlens_k;
  k.indices = a.indices; k.indices_stride_b = a.indices_stride_b; k.indices_stride_s = a.indices_stride_s;
  k.indices_logical = (sparse && a.indices_logical) ? 1 : 0;
  k.tile_scheduler_metadata = a.tile_scheduler_metadata; k.num_sm_parts = a.num_sm_parts; k.num_splits = a.num_splits;
  k.out = a.out; k.o_stride_b = a.o_stride_b; k.o_stride_s = a.o_stride_s; k.o_stride_h = a.o_stride_h;
  k.softmax_lse = a.softmax_lse; k.lse_accum = a.lse_accum; k.o_accum = a.o_accum;
  k.arrival_counters = (!push && !sparse) ? a.arrival_counters : nullptr;
  k.no_split_hint = (!push && a.no_split_hint) ? 1 : 0;
  if (push) {
    k.force_partial = 1;
    k.push_slot = push->slot; k.push_num_dst = push->num_dst; k.push_epoch = push->epoch; k.push_counter = push->counter;
    for (int d = 0; d < push->num_dst; ++d) { k.push_o[d] = push->dst_o[d]; k.push_lse[d] = push->dst_lse[d]; k.push_flag[d] = push->dst_flag[d]; }
  }

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (a.profile_event_begin) {
    e = cudaEventRecord(static_cast<cudaEvent_t>(a.profile_event_begin), s);
    if (e != cudaSuccess) return cuda_fail(e, "cudaEventRecord");
  }
  e = sparse ? fmla::launch_decode_sparse_tc(k, s) : fmla::launch_decode_dense_tc(k, s);
  if (e != cudaSuccess) return cuda_fail(e, "decode attention launch");
  if (a.profile_event_end) {
    e = cudaEventRecord(static_cast<cudaEvent_t>(a.profile_event_end), s);
    if (e != cudaSuccess) return cuda_fail(e, "cudaEventRecord");
  }
  if (push) {
    e = fmla::launch_decode_combine_push(k, s);
  } else if (!sparse && fmla::decode_dense_merges_in_kernel(k)) {
    e = cudaSuccess;      // the last CTA to deliver a partial of a request has merged it
  } else if (k.no_split_hint) {
    e = cudaSuccess;      // no request is split: every output is final already
  } else {
    e = fmla::launch_decode_combine(k, s);
  }
  if (e != cudaSuccess) return cuda_fail(e, "decode combine launch");
  return FMLA_OK;
}

int fmla_fwd_kvcache_mla(const fmla_decode_params* P, void* stream) { return decode_impl(P, nullptr, stream); }

int fmla_fwd_kvcache_mla_push_partial(const fmla_decode_params* P, const fmla_peer_push* push, void* stream) {
  FMLA_REQUIRE(push != nullptr, "push is null");
  FMLA_REQUIRE(push->num_dst >= 1 && push->num_dst <= 8, "num_dst must be in 1..8");
  FMLA_REQUIRE(push->slot >= 0 && push->counter != nullptr, "slot must be >= 0 and counter non-null");
  for (int d = 0; d < push->num_dst; ++d)
    FMLA_REQUIRE(push->dst_o[d] && push->dst_lse[d] && push->dst_flag[d] && aligned16(push->dst_o[d]), "destination pointers must be non-null, dst_o 16-byte aligned");
  return decode_impl(P, push, stream);
}

int fmla_merge_peer_partials(const float* part_lse, const float* part_o, int num_parts, int rows, int d_v, const uint32_t* flags,
                             uint32_t epoch, int max_polls, void* out, int64_t o_stride_row, float* lse, void* stream) {
  FMLA_REQUIRE(part_lse && part_o && flags && out && lse, "null pointer");
  FMLA_REQUIRE(num_parts > 0 && num_parts <= 4096 && rows > 0, "num_parts must be in 1..4096 and rows positive");
  FMLA_REQUIRE(d_v == 512, "Only head_size_v == 512 is supported");
  FMLA_REQUIRE(max_polls > 0, "max_polls must be positive");
  FMLA_REQUIRE(aligned16(part_o) && aligned16(out) && o_stride_row % 8 == 0, "part_o/out must be 16-byte aligned, stride a multiple of 8");
  if (int rc = require_blackwell()) return rc;
  cudaError_t e = fmla::launch_merge_peer_partials(part_lse, part_o, num_parts, rows, out, o_stride_row, lse, flags, epoch, max_polls,
                                                  static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? FMLA_OK : cuda_fail(e, "peer merge launch");
}

int fmla_combine_partials(const float* lse_accum, const float* o_accum, int num_parts, int rows, int d_v, void* out,
                          int64_t o_stride_row, float* lse, void* stream) {
  FMLA_REQUIRE(lse_accum && o_accum && out && lse, "null pointer");
  FMLA_REQUIRE(num_parts > 0 && rows > 0, "num_parts and rows must be positive");
  FMLA_REQUIRE(d_v == 512, "Only head_size_v == 512 is supported");
  FMLA_REQUIRE(num_parts <= 4096, "num_parts too large");
  FMLA_REQUIRE(aligned16(o_accum) && aligned16(out) && o_stride_row % 8 == 0, "o_accum/out must be 16-byte aligned, stride a multiple of 8");
  if (int rc = require_blackwell()) return rc;
  cudaError_t e = fmla::launch_combine_partials(lse_accum, o_accum, num_parts, rows, out, o_stride_row, lse,
                                               static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? FMLA_OK : cuda_fail(e, "combine launch");
}

int fmla_sparse_prefill_fwd(const fmla_sparse_prefill_params* P, void* stream) {
  FMLA_REQUIRE(P != nullptr, "params is null");
  const fmla_sparse_prefill_params& a = *P;
  FMLA_REQUIRE(a.s_q > 0 && a.s_kv > 0 && a.topk > 0, "s_q, s_kv, topk must be positive");
  FMLA_REQUIRE(a.h_kv == 1, "h_kv must be 1");
  FMLA_REQUIRE(a.d_qk == 576 && a.d_v == 512, "only d_qk == 576, d_v == 512 are supported");
  FMLA_REQUIRE(a.h_q % 64 == 0 && a.h_q > 0, "h_q must be a multiple of 64");
  FMLA_REQUIRE(a.topk % 64 == 0, "topk must be a multiple of 64");
  FMLA_REQUIRE(a.q && a.kv && a.indices && a.out && a.max_logits && a.lse, "null pointer");
  FMLA_REQUIRE(aligned16(a.q) && aligned16(a.kv) && aligned16(a.out), "q, kv, out must be 16-byte aligned");
  FMLA_REQUIRE(a.q_stride_s % 8 == 0 && a.q_stride_h % 8 == 0 && a.kv_stride_s % 8 == 0, "strides must be multiples of 8 elements");
  FMLA_REQUIRE(std::isfinite(a.sm_scale) && a.sm_scale > 0.f, "sm_scale must be positive and finite");
  int rc = require_blackwell();
  if (rc) return rc;
  fmla::SparsePrefillKernelParams k = {};
  k.s_q = a.s_q; k.s_kv = a.s_kv; k.h_q = a.h_q; k.topk = a.topk;
  k.scale_log2 = a.sm_scale * 1.4426950408889634f;
  k.q = a.q; k.q_stride_s = a.q_stride_s; k.q_stride_h = a.q_stride_h;
  k.kv = a.kv; k.kv_stride_s = a.kv_stride_s;
  k.indices = a.indices; k.indices_stride_s = a.indices_stride_s;
  k.out = a.out; k.max_logits = a.max_logits; k.lse = a.lse;
  cudaError_t e = fmla::launch_sparse_prefill_tc(k, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? FMLA_OK : cuda_fail(e, "sparse prefill launch");
}

static int fill_dense(const fmla_dense_params& a, bool bwd, fmla::DenseKernelParams* out) {
  FMLA_REQUIRE(a.batch > 0 && a.total_q > 0 && a.total_k > 0, "batch, total_q, total_k must be positive");
  FMLA_REQUIRE(a.h_q > 0 && a.h_k > 0 && a.h_q % a.h_k == 0, "h_q must be a positive multiple of h_k");
  if (!((a.d_qk == 192 || a.d_qk == 128) && a.d_v == 128))
    return fail(FMLA_ERR_UNSUPPORTED, "head dims (%d, %d) not supported; supported: (192,128), (128,128)", a.d_qk, a.d_v);
  FMLA_REQUIRE(a.max_seqlen_q > 0 && a.max_seqlen_k > 0, "max_seqlen must be positive");
  FMLA_REQUIRE(a.q && a.k && a.v && a.cu_seqlens_q && a.cu_seqlens_k && a.o && a.lse, "null pointer");
  FMLA_REQUIRE(aligned16(a.q) && aligned16(a.k) && aligned16(a.v) && aligned16(a.o), "q, k, v, o must be 16-byte aligned");
  FMLA_REQUIRE(a.q_stride_t % 8 == 0 && a.q_stride_h % 8 == 0 && a.k_stride_t % 8 == 0 && a.k_stride_h % 8 == 0 &&
               a.v_stride_t % 8 == 0 && a.v_stride_h % 8 == 0 && a.o_stride_t % 8 == 0 && a.o_stride_h % 8 == 0,
               "strides must be multiples of 8 elements");
  FMLA_REQUIRE(std::isfinite(a.softmax_scale) && a.softmax_scale > 0.f, "softmax_scale must be positive and finite");
  fmla::DenseKernelParams k = {};
  k.batch = a.batch; k.h_q = a.h_q; k.h_k = a.h_k; k.d_qk = a.d_qk; k.d_v = a.d_v;
  k.max_seqlen_q = a.max_seqlen_q; k.max_seqlen_k = a.max_seqlen_k; k.is_causal = a.is_causal ? 1 : 0;
  k.total_q = a.total_q; k.total_k = a.total_k;
  k.scale = a.softmax_scale; k.scale_log2 = a.softmax_scale * 1.4426950408889634f;
  k.q = a.q; k.q_stride_t = a.q_stride_t; k.q_stride_h = a.q_stride_h;
  k.k = a.k; k.k_stride_t = a.k_stride_t; k.k_stride_h = a.k_stride_h;
  k.v = a.v; k.v_stride_t = a.v_stride_t; k.v_stride_h = a.v_stride_h;
  k.cu_q = a.cu_seqlens_q; k.cu_k = a.cu_seqlens_k;
  k.o = a.o; k.o_stride_t = a.o_stride_t; k.o_stride_h = a.o_stride_h;
  k.lse = a.lse; k.lse_stride_t = a.lse_stride_t; k.lse_stride_h = a.lse_stride_h;
  if (bwd) {
    FMLA_REQUIRE(a.h_q == a.h_k, "backward does not support GQA (h_q must equal h_k)");
    FMLA_REQUIRE(a.d_o && a.dq && a.dk && a.dv && a.workspace, "null pointer");
    FMLA_REQUIRE(aligned16(a.d_o) && aligned16(a.dq) && aligned16(a.dk) && aligned16(a.dv) && aligned16(a.workspace), "backward tensors must be 16-byte aligned");
    FMLA_REQUIRE(a.do_stride_t % 8 == 0 && a.do_stride_h % 8 == 0 && a.dq_stride_t % 8 == 0 && a.dq_stride_h % 8 == 0 &&
                 a.dk_stride_t % 8 == 0 && a.dk_stride_h % 8 == 0 && a.dv_stride_t % 8 == 0 && a.dv_stride_h % 8 == 0,
                 "strides must be multiples of 8 elements");
    FMLA_REQUIRE(a.workspace_bytes >= fmla_dense_bwd_workspace_bytes(a.total_q, a.h_q, a.d_qk), "workspace too small");
    k.d_o = a.d_o; k.do_stride_t = a.do_stride_t; k.do_stride_h = a.do_stride_h;
    k.dq = a.dq; k.dq_stride_t = a.dq_stride_t; k.dq_stride_h = a.dq_stride_h;
    k.dk = a.dk; k.dk_stride_t = a.dk_stride_t; k.dk_stride_h = a.dk_stride_h;
    k.dv = a.dv; k.dv_stride_t = a.dv_stride_t; k.dv_stride_h = a.dv_stride_h;
    k.delta = reinterpret_cast<float*>(a.workspace);
  }
  *out = k;
  return FMLA_OK;
}

int fmla_dense_prefill_fwd(const fmla_dense_params* P, void* stream) {
  FMLA_REQUIRE(P != nullptr, "params is null");
  fmla::DenseKernelParams k;
  int rc = fill_dense(*P, false, &k);
  if (rc) return rc;
  rc = require_blackwell();
  if (rc) return rc;
  cudaError_t e = fmla::launch_dense_fwd_tc(k, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? FMLA_OK : cuda_fail(e, "dense forward launch");
}

size_t fmla_dense_bwd_workspace_bytes(int total_q, int h_q, int d_qk) {
  (void)d_qk;
  return (static_cast<size_t>(total_q) * h_q * sizeof(float) + 255) / 256 * 256;
}

int fmla_dense_prefill_bwd(const fmla_dense_params* P, void* stream) {
  FMLA_REQUIRE(P != nullptr, "params is null");
  fmla::DenseKernelParams k;
  int rc = fill_dense(*P, true, &k);
  if (rc) return rc;
  rc = require_blackwell();
  if (rc) return rc;
  cudaError_t e = fmla::launch_dense_bwd_tc(k, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? FMLA_OK : cuda_fail(e, "dense backward launch");
}

int fmla_device_status(int* status_host, int reset) {
  FMLA_REQUIRE(status_host != nullptr, "status_host is null");
  cudaError_t e = fmla::read_decode_tc_status(status_host, reset != 0);
  if (e != cudaSuccess) return cuda_fail(e, "reading the device status word");
  int pair_status = 0;
  e = fmla::read_decode_pair_status(&pair_status, reset != 0);
  if (e != cudaSuccess) return cuda_fail(e, "reading the device status word");
  if (*status_host == 0) *status_host = pair_status;
  int merge_status = 0;
  e = fmla::read_merge_status(&merge_status, reset != 0);
  if (e != cudaSuccess) return cuda_fail(e, "reading the device status word");
  if (*status_host == 0) *status_host = merge_status;
  int dense_status = 0;
  e = fmla::read_dense_tc_status(&dense_status, reset != 0);
  if (e != cudaSuccess) return cuda_fail(e, "reading the device status word");
  if (*status_host == 0) *status_host = dense_status;
  e = fmla::read_dense_bwd_tc_status(&dense_status, reset != 0);
  if (e != cudaSuccess) return cuda_fail(e, "reading the device status word");
  if (*status_host == 0) *status_host = dense_status;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
    volatile int* w = reinterpret_cast<volatile int*>(&g_host_status[dev * kStatusStride]);
    if (*status_host == 0) *status_host = *w;
    if (reset) *w = 0;
  }
  return *status_host == 0 ? FMLA_OK : fail(FMLA_ERR_DEVICE_TIMEOUT, "a bounded device-side wait expired (code %d)", *status_host);
}

int fmla_quantize_kv_fp8(const void* kv_bf16, int64_t kv_stride_row, int num_tokens, const int32_t* dst_slots,
                         void* cache_bytes, int64_t cache_stride_slot_bytes, void* stream) {
  FMLA_REQUIRE(kv_bf16 && cache_bytes, "null pointer");
  FMLA_REQUIRE(num_tokens >= 0, "num_tokens must be non-negative");
  FMLA_REQUIRE(aligned16(kv_bf16) && aligned16(cache_bytes) && kv_stride_row % 8 == 0 && cache_stride_slot_bytes % 16 == 0,
               "kv and cache must be 16-byte aligned with 16-byte-multiple row pitches");
  FMLA_REQUIRE(cache_stride_slot_bytes >= 656, "cache slot pitch must be at least 656 bytes");
  cudaError_t e = fmla::launch_quantize_kv_fp8(kv_bf16, kv_stride_row, num_tokens, dst_slots, cache_bytes,
                                              cache_stride_slot_bytes, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? FMLA_OK : cuda_fail(e, "quantize launch");
}

}  // extern "C"
