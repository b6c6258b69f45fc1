// FP8 KV-cache writer: bf16 [num_tokens, 576] -> 656-byte token records
// (512 x e4m3 | 4 x fp32 scale | 64 x bf16 rope; README.md:162-170).
// Arithmetic of tests/quant.py:3-35: per 128-wide tile, scale = bf16(amax/448)
// widened to fp32, q = e4m3_rn(fp32(x) / scale).  One warp per token.
#include "fmla_common.cuh"
#include "kernels.h"

#include <cuda_fp8.h>

namespace fmla {

__global__ void __launch_bounds__(256) quantize_kv_fp8_kernel(const __nv_bfloat16* __restrict__ kv, int64_t kv_stride_row,
                                                             int num_tokens, const int* __restrict__ dst_slots,
                                                             unsigned char* __restrict__ cache, int64_t cache_stride_slot) {
  const int tok = (blockIdx.x * 256 + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (tok >= num_tokens) return;
  const int slot = dst_slots ? dst_slots[tok] : tok;
  if (slot < 0) return;
  const __nv_bfloat16* src = kv + (int64_t)tok * kv_stride_row;
  unsigned char* rec = cache + (int64_t)slot * cache_stride_slot;

  uint4 raw[2];
  raw[0] = *reinterpret_cast<const uint4*>(src + lane * 16);
  raw[1] = *reinterpret_cast<const uint4*>(src + lane * 16 + 8);
  float x[16];
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(raw);
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float2 f = __bfloat1622float2(h2[i]);
    x[2 * i] = f.x;
    x[2 * i + 1] = f.y;
    amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
  }
#pragma unroll
  for (int off = 1; off <= 4; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  const float scale = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(amax, 448.0f)));
  uint32_t q[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t w = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __nv_fp8_storage_t b = __nv_cvt_float_to_fp8(__fdiv_rn(x[i * 4 + k], scale), __NV_SATFINITE, __NV_E4M3);
      w |= static_cast<uint32_t>(b) << (8 * k);
    }
    q[i] = w;
  }
  *reinterpret_cast<uint4*>(rec + lane * 16) = make_uint4(q[0], q[1], q[2], q[3]);
  const float s_tile = __shfl_sync(0xffffffffu, scale, (lane & 3) * 8);
  if (lane < 4) reinterpret_cast<float*>(rec + 512)[lane] = s_tile;
  if (lane < 8) *reinterpret_cast<uint4*>(rec + 528 + lane * 16) = *reinterpret_cast<const uint4*>(src + 512 + lane * 8);
}

cudaError_t launch_quantize_kv_fp8(const void* kv, int64_t kv_stride_row, int num_tokens, const int* dst_slots, void* cache,
                                   int64_t cache_stride_slot, cudaStream_t stream) {
  if (num_tokens == 0) return cudaSuccess;
  quantize_kv_fp8_kernel<<<(num_tokens + 7) / 8, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(kv), kv_stride_row,
                                                                  num_tokens, dst_slots,
                                                                  reinterpret_cast<unsigned char*>(cache), cache_stride_slot);
  return cudaGetLastError();
}

}  // namespace fmla
