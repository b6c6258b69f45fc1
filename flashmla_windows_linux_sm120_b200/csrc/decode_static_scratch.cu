// Decode entry point for callers that are not allowed to allocate device memory.
//
// The split-KV decode needs scratch for the partial results of requests that the
// schedule cut into several parts.  fmla_fwd_kvcache_mla() takes that scratch from
// the caller.  Some callers have nowhere to get it from at call time: an inference
// server that hands the library a fixed arena at start-up and forbids cudaMalloc
// afterwards, a plugin whose "enqueue" hook may only launch work, code that runs
// while a stream is being recorded.  For them this file keeps the scratch inside
// the library image, as two file-scope __device__ arrays of fixed size, and offers
// one more entry point that uses them.  It calls no cudaMalloc / cudaFree and no
// allocating library routine.
//
// The arrays exist once per GPU that loads the library (about 64 MiB, held until the
// process exits) and are shared by every call: two calls that overlap on one GPU
// (different streams, different host threads) would write the same slots and race.
// Nothing in them has to be zero on entry: every slot that the merge kernel reads
// was written by the attention kernel of the same call, so stale contents of an
// earlier call are never observed and no clearing pass is needed.
#include "../../include/flashmla_b200.h"
#include "kernels.h"

#include <cstdio>
#include <mutex>

namespace {

// Largest (batch + num_sm_parts) * s_q * h_q the entry point accepts.
constexpr size_t kMaxPartialRows = 32768;
constexpr int kHeadDimV = 512;

static __device__ __align__(256) float g_static_o_accum[kMaxPartialRows * kHeadDimV];   // 64 MiB
static __device__ __align__(256) float g_static_lse_accum[kMaxPartialRows];             // 128 KiB

// In host code the array names above are host-side stand-ins, not device addresses.  The device
// addresses are looked up once per device, with that device current, and cached here.
struct ScratchPtrs {
  float* o_accum = nullptr;
  float* lse_accum = nullptr;
  bool ready = false;
};
std::mutex g_scratch_mutex;
ScratchPtrs g_scratch[64];

int scratch_for_current_device(ScratchPtrs* out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fmla::set_error(FMLA_ERR_CUDA, cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fmla::set_error(FMLA_ERR_INVALID_ARGUMENT, "device index out of range");
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  ScratchPtrs& s = g_scratch[dev];
  if (!s.ready) {
    void* po = nullptr;
    void* pl = nullptr;
    e = cudaGetSymbolAddress(&po, g_static_o_accum);
    if (e != cudaSuccess) return fmla::set_error(FMLA_ERR_CUDA, cudaGetErrorString(e));
    e = cudaGetSymbolAddress(&pl, g_static_lse_accum);
    if (e != cudaSuccess) return fmla::set_error(FMLA_ERR_CUDA, cudaGetErrorString(e));
    s.o_accum = static_cast<float*>(po);
    s.lse_accum = static_cast<float*>(pl);
    s.ready = true;
  }
  *out = s;
  return FMLA_OK;
}

}  // namespace

extern "C" int fmla_fwd_kvcache_mla_static_scratch(const fmla_decode_params* params_host, void* stream) {
  if (params_host == nullptr) return fmla::set_error(FMLA_ERR_INVALID_ARGUMENT, "params is null");
  const fmla_decode_params& a = *params_host;
  if (a.b <= 0 || a.s_q <= 0 || a.h_q <= 0 || a.num_sm_parts <= 0)
    return fmla::set_error(FMLA_ERR_INVALID_ARGUMENT, "b, s_q, h_q and num_sm_parts must be positive");
  if (a.d_v != kHeadDimV) return fmla::set_error(FMLA_ERR_INVALID_ARGUMENT, "Only head_size_v == 512 is supported");
  const size_t rows = (static_cast<size_t>(a.b) + static_cast<size_t>(a.num_sm_parts)) * static_cast<size_t>(a.s_q) *
                      static_cast<size_t>(a.h_q);
  if (rows > kMaxPartialRows) {
    char msg[256];
    snprintf(msg, sizeof(msg),
             "problem needs %zu partial rows ((b + num_sm_parts) * s_q * h_q) but the built-in scratch holds %zu; "
             "use fmla_fwd_kvcache_mla with caller-provided scratch",
             rows, kMaxPartialRows);
    return fmla::set_error(FMLA_ERR_INVALID_ARGUMENT, msg);
  }
  ScratchPtrs s;
  const int rc = scratch_for_current_device(&s);
  if (rc != FMLA_OK) return rc;
  fmla_decode_params p = a;       // the caller's block is not modified
  p.o_accum = s.o_accum;
  p.lse_accum = s.lse_accum;
  return fmla_fwd_kvcache_mla(&p, stream);
}

extern "C" size_t fmla_static_scratch_max_rows(void) { return kMaxPartialRows; }
