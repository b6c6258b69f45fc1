// Log-sum-exp merge of split-KV partial results.
//
// Math of csrc/smxx/mla_combine.cu:71-107, 128-151: with base-2 partial LSEs
// lse_i and normalised partial outputs o_i,
//   lse = log2(sum_i 2^lse_i)  (computed max-shifted; all -inf -> +inf),
//   o   = sum_i 2^(lse_i - lse) * o_i,
// written as natural-log LSE and bf16 O.  One warp per output row, any number of
// parts (the reference is limited to 64, mla_combine.cu:156-167).  Each lane
// owns 16 of the 512 output columns as 4 float4 so a warp reads 512 B
// contiguous per load instruction.
#include "fmla_common.cuh"
#include "kernels.h"
#include "tc_common.cuh"

namespace fmla {

constexpr int kCombineWarps = 8;

// lse_part(i) / o_part(i) address part i of this row.  COHERENT: the partial outputs may have been written by
// another GPU while this kernel was already resident (peer merge), so they are read with ld.global.cv
// instead of the non-coherent path, which is undefined for memory modified during the kernel's lifetime.
template <bool COHERENT = false, class LseAt, class OAt>
__device__ __forceinline__ void combine_row(int nparts, LseAt lse_at, OAt o_at, float* s_w, __nv_bfloat16* out_row,
                                            float* lse_out, bool f16 = false) {
  const int lane = threadIdx.x & 31;
  float mx = neg_inf();
  for (int i = lane; i < nparts; i += 32) mx = fmaxf(mx, lse_at(i));
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  if (mx == neg_inf()) mx = 0.f;
  float sum = 0.f;
  for (int i = lane; i < nparts; i += 32) sum += exp2f(lse_at(i) - mx);
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  const float glse = (sum == 0.f || sum != sum) ? pos_inf() : log2f(sum) + mx;
  if (lane == 0) *lse_out = glse * kLn2;
  for (int i = lane; i < nparts; i += 32) s_w[i] = exp2f(lse_at(i) - glse);
  __syncwarp();

  float4 acc[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i = 0; i < nparts; ++i) {
    const float w = s_w[i];
    if (w == 0.f) continue;
    const float4* src = reinterpret_cast<const float4*>(o_at(i));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 v = COHERENT ? __ldcv(src + j * 32 + lane) : __ldg(src + j * 32 + lane);
      acc[j].x += w * v.x;
      acc[j].y += w * v.y;
      acc[j].z += w * v.z;
      acc[j].w += w * v.w;
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    // out_row addresses 16-bit elements: bf16, or fp16 when the queries were fp16
    uint2 packed = f16 ? make_uint2(pack_f16x2(acc[j].x, acc[j].y), pack_f16x2(acc[j].z, acc[j].w))
                       : make_uint2(pack_bf16x2(acc[j].x, acc[j].y), pack_bf16x2(acc[j].z, acc[j].w));
    *reinterpret_cast<uint2*>(out_row + (j * 32 + lane) * 4) = packed;
  }
}

// grid (b, ceil(h_k*q_seq_per_hk / 8)); requests with a single part were written
// in final form by the attention kernel and are skipped (mla_combine.cu:30-32).
__global__ void __launch_bounds__(kCombineWarps * 32) decode_combine_kernel(const __grid_constant__ DecodeKernelParams p) {
  extern __shared__ float s_weights[];  // [8][num_sm_parts]
  pdl_wait();                           // launched as a programmatic dependent of the attention kernel
  const int batch = blockIdx.x;
  const int lo = __ldg(p.num_splits + batch), hi = __ldg(p.num_splits + batch + 1);
  const int nparts = hi - lo;
  if (nparts <= 1) return;
  const int q_seq_per_hk = p.s_q * p.hq_per_hk;
  const int rows = p.h_k * q_seq_per_hk;
  const int warp = threadIdx.x >> 5;
  const int r = blockIdx.y * kCombineWarps + warp;
  if (r >= rows) return;
  const int kh = r / q_seq_per_hk, row = r % q_seq_per_hk;
  const int sq = row / p.hq_per_hk, head = kh * p.hq_per_hk + row % p.hq_per_hk;
  const float* lse_base = p.lse_accum + (int64_t)lo * rows + r;
  const float* o_base = p.o_accum + ((int64_t)lo * rows + r) * 512;
  const int64_t part_stride = rows;
  combine_row(
      nparts, [&](int i) { return __ldg(lse_base + i * part_stride); },
      [&](int i) { return o_base + i * part_stride * 512; }, s_weights + warp * p.num_sm_parts,
      reinterpret_cast<__nv_bfloat16*>(p.out) + batch * p.o_stride_b + sq * p.o_stride_s + head * p.o_stride_h,
      p.softmax_lse + ((int64_t)batch * p.h_q + head) * p.s_q + sq, p.is_f16 != 0);
}

__global__ void __launch_bounds__(kCombineWarps * 32)
combine_partials_kernel(const float* __restrict__ lse_accum, const float* __restrict__ o_accum, int nparts, int rows,
                        __nv_bfloat16* __restrict__ out, int64_t o_stride_row, float* __restrict__ lse) {
  extern __shared__ float s_weights[];  // [8][nparts]
  const int warp = threadIdx.x >> 5;
  const int r = blockIdx.x * kCombineWarps + warp;
  if (r >= rows) return;
  combine_row(
      nparts, [&](int i) { return __ldg(lse_accum + (int64_t)i * rows + r); },
      [&](int i) { return o_accum + ((int64_t)i * rows + r) * 512; }, s_weights + warp * nparts, out + r * o_stride_row,
      lse + r);
}

// ---- KV-sharded decode across GPUs ---------------------------------------------------------------
// Each rank merges its local splits per row and stores the normalised fp32 result + base-2 LSE
// into its slot of every destination's partial buffers with plain (peer) stores; the last CTA to
// finish publishes the epoch in the destinations' flag words (release, system scope).
__device__ __forceinline__ void st_release_sys(unsigned int* addr, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* addr) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

__global__ void __launch_bounds__(kCombineWarps * 32) decode_combine_push_kernel(const __grid_constant__ DecodeKernelParams p) {
  extern __shared__ float s_weights[];  // [8][num_sm_parts]
  const int batch = blockIdx.x;
  const int lo = __ldg(p.num_splits + batch), hi = __ldg(p.num_splits + batch + 1);
  const int nparts = hi - lo;
  const int q_seq_per_hk = p.s_q * p.hq_per_hk;
  const int rows = p.h_k * q_seq_per_hk;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.y * kCombineWarps + warp;
  if (r < rows) {
    const float* lse_base = p.lse_accum + (int64_t)lo * rows + r;
    const float* o_base = p.o_accum + ((int64_t)lo * rows + r) * 512;
    float* w = s_weights + warp * p.num_sm_parts;
    float mx = neg_inf();
    for (int i = lane; i < nparts; i += 32) mx = fmaxf(mx, __ldg(lse_base + (int64_t)i * rows));
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    const float mref = mx == neg_inf() ? 0.f : mx;
    float sum = 0.f;
    for (int i = lane; i < nparts; i += 32) sum += exp2f(__ldg(lse_base + (int64_t)i * rows) - mref);
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float glse = (sum == 0.f || sum != sum) ? neg_inf() : log2f(sum) + mref;   // base 2, -inf = empty shard
    for (int i = lane; i < nparts; i += 32) w[i] = glse == neg_inf() ? 0.f : exp2f(__ldg(lse_base + (int64_t)i * rows) - glse);
    __syncwarp();
    float4 acc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = 0; i < nparts; ++i) {
      const float wi = w[i];
      if (wi == 0.f) continue;
      const float4* src = reinterpret_cast<const float4*>(o_base + (int64_t)i * rows * 512);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 v = __ldg(src + j * 32 + lane);
        acc[j].x += wi * v.x; acc[j].y += wi * v.y; acc[j].z += wi * v.z; acc[j].w += wi * v.w;
      }
    }
    const int64_t total_rows = (int64_t)p.b * rows;
    const int64_t grow = (int64_t)p.push_slot * total_rows + (int64_t)batch * rows + r;
    for (int d = 0; d < p.push_num_dst; ++d) {
      float4* dst = reinterpret_cast<float4*>(p.push_o[d] + grow * 512);
#pragma unroll
      for (int j = 0; j < 4; ++j) dst[j * 32 + lane] = acc[j];
      if (lane == 0) p.push_lse[d][grow] = glse;
    }
  }
  // publish: every thread's peer stores are ordered before the flag by fence + barrier + release
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int total = gridDim.x * gridDim.y;
    const unsigned int done = atomicAdd(p.push_counter, 1u) + 1u;
    if (done == total) {
      __threadfence_system();
      for (int d = 0; d < p.push_num_dst; ++d) st_release_sys(p.push_flag[d] + p.push_slot, p.push_epoch);
      *p.push_counter = 0u;
    }
  }
}

// Merge of per-rank partials that arrive through peer stores: wait (bounded) for every rank's flag.
__global__ void __launch_bounds__(kCombineWarps * 32)
merge_peer_partials_kernel(const float* __restrict__ lse_accum, const float* __restrict__ o_accum, int nparts, int rows,
                           __nv_bfloat16* __restrict__ out, int64_t o_stride_row, float* __restrict__ lse,
                           const unsigned int* __restrict__ flags, unsigned int epoch, int max_polls, int* status) {
  extern __shared__ float s_weights[];  // [8][nparts]
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int i = 0; i < nparts && ok; ++i) {
      int polls = 0;
      while (ld_acquire_sys(flags + i) != epoch) {
        if (++polls > max_polls) { ok = 0; break; }
        __nanosleep(200);
      }
    }
    if (!ok) tc::report_status(status, 20);
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;     // the caller reads the status word; outputs are left untouched
  const int warp = threadIdx.x >> 5;
  const int r = blockIdx.x * kCombineWarps + warp;
  if (r >= rows) return;
  combine_row<true>(
      nparts, [&](int i) { return __ldcv(lse_accum + (int64_t)i * rows + r); },
      [&](int i) { return o_accum + ((int64_t)i * rows + r) * 512; }, s_weights + warp * nparts, out + r * o_stride_row,
      lse + r);
}

__device__ int g_merge_status = 0;

cudaError_t set_status_mirror_merge(int* mapped_host_word) { return tc::set_status_mirror(mapped_host_word); }

// The merge kernels keep one weight per (warp, part) in dynamic shared memory; above 48 KB the limit of the
// kernel has to be raised first.
template <class Kernel>
static cudaError_t allow_dynamic_smem(Kernel kernel, size_t bytes) {
  if (bytes <= 48 * 1024) return cudaSuccess;
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
}

cudaError_t launch_decode_combine_push(const DecodeKernelParams& p, cudaStream_t stream) {
  const int rows = p.h_k * p.s_q * p.hq_per_hk;
  dim3 grid(p.b, (rows + kCombineWarps - 1) / kCombineWarps);
  const size_t smem = sizeof(float) * kCombineWarps * p.num_sm_parts;
  if (cudaError_t e = allow_dynamic_smem(decode_combine_push_kernel, smem); e != cudaSuccess) return e;
  decode_combine_push_kernel<<<grid, kCombineWarps * 32, smem, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_merge_peer_partials(const float* lse_accum, const float* o_accum, int num_parts, int rows, void* out,
                                       int64_t o_stride_row, float* lse, const unsigned int* flags, unsigned int epoch,
                                       int max_polls, cudaStream_t stream) {
  int* status = nullptr;
  cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_merge_status);
  if (e != cudaSuccess) return e;
  const size_t smem = sizeof(float) * kCombineWarps * num_parts;
  e = allow_dynamic_smem(merge_peer_partials_kernel, smem);
  if (e != cudaSuccess) return e;
  merge_peer_partials_kernel<<<(rows + kCombineWarps - 1) / kCombineWarps, kCombineWarps * 32, smem, stream>>>(
      lse_accum, o_accum, num_parts, rows, reinterpret_cast<__nv_bfloat16*>(out), o_stride_row, lse, flags, epoch, max_polls,
      status);
  return cudaGetLastError();
}

cudaError_t read_merge_status(int* host_status, bool reset) {
  cudaError_t e = cudaMemcpyFromSymbol(host_status, g_merge_status, sizeof(int));
  if (e != cudaSuccess) return e;
  if (reset && *host_status != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_merge_status, &zero, sizeof(int));
  }
  return e;
}

cudaError_t launch_decode_combine(const DecodeKernelParams& p, cudaStream_t stream) {
  const int rows = p.h_k * p.s_q * p.hq_per_hk;
  dim3 grid(p.b, (rows + kCombineWarps - 1) / kCombineWarps);
  const size_t smem = sizeof(float) * kCombineWarps * p.num_sm_parts;
  if (cudaError_t e = allow_dynamic_smem(decode_combine_kernel, smem); e != cudaSuccess) return e;
  // programmatic dependent launch: the blocks may become resident while the attention kernel drains and start
  // the moment it has completed (they wait in pdl_wait()), instead of being launched after it
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kCombineWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, decode_combine_kernel, p);
}

cudaError_t launch_combine_partials(const float* lse_accum, const float* o_accum, int num_parts, int rows, void* out,
                                    int64_t o_stride_row, float* lse, cudaStream_t stream) {
  const size_t smem = sizeof(float) * kCombineWarps * num_parts;
  if (cudaError_t e = allow_dynamic_smem(combine_partials_kernel, smem); e != cudaSuccess) return e;
  combine_partials_kernel<<<(rows + kCombineWarps - 1) / kCombineWarps, kCombineWarps * 32, smem, stream>>>(
      lse_accum, o_accum, num_parts, rows, reinterpret_cast<__nv_bfloat16*>(out), o_stride_row, lse);
  return cudaGetLastError();
}

}  // namespace fmla
