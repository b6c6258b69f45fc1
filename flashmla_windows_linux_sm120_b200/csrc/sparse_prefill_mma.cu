// Sparse MLA prefill forward on the shared 64-row attention tile.
//
// One CTA = 64 heads of one query token; its KV "sequence" is the token's top-k
// index list, gathered row by row from kv[s_kv, 576].  Outputs follow
// csrc/sm100/prefill/sparse/fwd.cu:399-417, 438-445 and README.md:201-217:
// out = softmax-weighted sum of kv[idx][:512]; max_logits and lse in base 2 of
// q.k*sm_scale*log2(e); an index < 0 or >= s_kv is skipped (fwd.cu:677-679);
// rows without any valid index give out = 0, max_logits = lse = -inf.
#include "attn_tile.cuh"
#include "kernels.h"

namespace fmla {

using PrefillCfg = TileCfg<576, 512, true>;

struct SparsePrefillProb {
  const SparsePrefillKernelParams& p;
  int s, head_base;
  const int* idx_row;
  __device__ __forceinline__ SparsePrefillProb(const SparsePrefillKernelParams& p_) : p(p_) {}

  __device__ __forceinline__ void load_q(uint32_t sQ) {
    const int r = threadIdx.x >> 2;
    const __nv_bfloat16* src =
        reinterpret_cast<const __nv_bfloat16*>(p.q) + (int64_t)s * p.q_stride_s + (head_base + r) * p.q_stride_h;
    load_rows_async<576>(sQ, src, p.q);
  }
  __device__ __forceinline__ void load_kv_begin(int blk, int, uint32_t sK, uint32_t, int* sValid) {
    const int r = threadIdx.x >> 2;
    const int idx = __ldg(idx_row + blk * 64 + r);
    const bool ok = idx >= 0 && idx < p.s_kv;
    if ((threadIdx.x & 3) == 0) sValid[r] = ok ? 1 : 0;
    const __nv_bfloat16* src = ok ? reinterpret_cast<const __nv_bfloat16*>(p.kv) + (int64_t)idx * p.kv_stride_s : nullptr;
    load_rows_async<576>(sK, src, p.kv);
  }
  __device__ __forceinline__ void load_kv_end(int, uint32_t, uint32_t) {}
  __device__ __forceinline__ bool needs_mask(int) const { return true; }
  __device__ __forceinline__ bool valid(int, int, int tok, const int* sValid) const { return sValid[tok] != 0; }
};

// grid (h_q/64, s_q)
__global__ void __launch_bounds__(256, 1) sparse_prefill_kernel(const __grid_constant__ SparsePrefillKernelParams p) {
  extern __shared__ __align__(1024) char smem[];
  SparsePrefillProb prob(p);
  prob.s = blockIdx.y;
  prob.head_base = blockIdx.x * 64;
  prob.idx_row = p.indices + (int64_t)prob.s * p.indices_stride_s;

  TileAcc<PrefillCfg> acc;
  run_tile<PrefillCfg>(prob, smem, 0, p.topk / 64, p.scale_log2, acc);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rg = warp & 3, th = warp >> 2, g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int head = prob.head_base + rg * 16 + g + h * 8;
    const float l = acc.l[h];
    const float inv = l == 0.f ? 0.f : 1.f / l;
    __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + ((int64_t)prob.s * p.h_q + head) * 512;
#pragma unroll
    for (int nt = 0; nt < PrefillCfg::NT_O; ++nt) {
      const int col = th * 256 + nt * 8 + 2 * t4;
      *reinterpret_cast<uint32_t*>(orow + col) = pack_bf16x2(acc.o[nt][h * 2] * inv, acc.o[nt][h * 2 + 1] * inv);
    }
    if (th == 0 && t4 == 0) {
      p.max_logits[(int64_t)prob.s * p.h_q + head] = acc.m[h];
      p.lse[(int64_t)prob.s * p.h_q + head] = l == 0.f ? neg_inf() : log2f(l) + acc.m[h];
    }
  }
}

cudaError_t launch_sparse_prefill_mma(const SparsePrefillKernelParams& p, cudaStream_t stream) {
  auto kern = sparse_prefill_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PrefillCfg::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  dim3 grid(p.h_q / 64, p.s_q);
  kern<<<grid, 256, PrefillCfg::SMEM_BYTES, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace fmla
