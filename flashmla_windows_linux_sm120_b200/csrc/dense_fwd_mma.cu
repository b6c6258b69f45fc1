// Dense variable-length MHA forward (bf16, head dims 192/128 and 128/128) on the
// shared 64-row attention tile.
//
// Semantics of the reference forward (csrc/sm100/prefill/dense/
// fmha_cutlass_fwd_sm100.cu:67-119 and its mainloop): packed varlen q/k/v with
// cu_seqlens; GQA maps q head h to kv head h / (h_q/h_k); causal masking is
// bottom-right aligned (query i sees keys j <= i + s_k - s_q,
// collective/fmha_fusion.hpp:266-274); LSE is the natural log of the row sum;
// rows with no visible key give O = 0, LSE = -inf.
#include "attn_tile.cuh"
#include "kernels.h"

namespace fmla {

template <int D_QK>
struct DenseFwdProb {
  using Cfg = TileCfg<D_QK, 128, false>;
  const DenseKernelParams& p;
  int q0, lq, k0, lk, m_base, head, kv_head;
  __device__ __forceinline__ DenseFwdProb(const DenseKernelParams& p_) : p(p_) {}

  __device__ __forceinline__ void load_q(uint32_t sQ) {
    const int r = threadIdx.x >> 2;
    const __nv_bfloat16* src = nullptr;
    if (m_base + r < lq)
      src = reinterpret_cast<const __nv_bfloat16*>(p.q) + (int64_t)(q0 + m_base + r) * p.q_stride_t + head * p.q_stride_h;
    load_rows_async<D_QK>(sQ, src, p.q);
  }
  __device__ __forceinline__ void load_kv_begin(int blk, int, uint32_t sK, uint32_t sV, int*) {
    const int r = threadIdx.x >> 2;
    const int tok = blk * 64 + r;
    const __nv_bfloat16 *ks = nullptr, *vs = nullptr;
    if (tok < lk) {
      ks = reinterpret_cast<const __nv_bfloat16*>(p.k) + (int64_t)(k0 + tok) * p.k_stride_t + kv_head * p.k_stride_h;
      vs = reinterpret_cast<const __nv_bfloat16*>(p.v) + (int64_t)(k0 + tok) * p.v_stride_t + kv_head * p.v_stride_h;
    }
    load_rows_async<D_QK>(sK, ks, p.k);
    load_rows_async<128>(sV, vs, p.v);
  }
  __device__ __forceinline__ void load_kv_end(int, uint32_t, uint32_t) {}
  __device__ __forceinline__ bool needs_mask(int blk) const {
    const int last = (blk + 1) * 64 - 1;
    return last >= lk || (p.is_causal && last > m_base + (lk - lq));
  }
  __device__ __forceinline__ bool valid(int row, int blk, int tok, const int*) const {
    const int j = blk * 64 + tok;
    return j < lk && (!p.is_causal || j <= m_base + row + (lk - lq));
  }
};

// grid (ceil(max_seqlen_q/64), h_q, batch)
template <int D_QK>
__global__ void __launch_bounds__(256, 2) dense_fwd_kernel(const __grid_constant__ DenseKernelParams p) {
  extern __shared__ __align__(1024) char smem[];
  using Prob = DenseFwdProb<D_QK>;
  using Cfg = typename Prob::Cfg;
  Prob prob(p);
  const int b = blockIdx.z;
  prob.q0 = __ldg(p.cu_q + b);
  prob.lq = __ldg(p.cu_q + b + 1) - prob.q0;
  prob.k0 = __ldg(p.cu_k + b);
  prob.lk = __ldg(p.cu_k + b + 1) - prob.k0;
  prob.m_base = blockIdx.x * 64;
  prob.head = blockIdx.y;
  prob.kv_head = blockIdx.y / (p.h_q / p.h_k);
  if (prob.m_base >= prob.lq) return;

  int nblk = (prob.lk + 63) / 64;
  if (p.is_causal) {
    const int last_key = min(prob.m_base + 63, prob.lq - 1) + (prob.lk - prob.lq);  // inclusive
    nblk = last_key < 0 ? 0 : min(nblk, last_key / 64 + 1);
  }
  TileAcc<Cfg> acc;
  run_tile<Cfg>(prob, smem, 0, nblk, p.scale_log2, acc);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rg = warp & 3, th = warp >> 2, g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = prob.m_base + rg * 16 + g + h * 8;
    if (r >= prob.lq) continue;
    const float l = acc.l[h];
    const float inv = l == 0.f ? 0.f : 1.f / l;
    __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.o) + (int64_t)(prob.q0 + r) * p.o_stride_t + prob.head * p.o_stride_h;
#pragma unroll
    for (int nt = 0; nt < Cfg::NT_O; ++nt) {
      const int col = th * 64 + nt * 8 + 2 * t4;
      *reinterpret_cast<uint32_t*>(orow + col) = pack_bf16x2(acc.o[nt][h * 2] * inv, acc.o[nt][h * 2 + 1] * inv);
    }
    if (th == 0 && t4 == 0)
      p.lse[(int64_t)(prob.q0 + r) * p.lse_stride_t + prob.head * p.lse_stride_h] =
          l == 0.f ? neg_inf() : (log2f(l) + acc.m[h]) * kLn2;
  }
}

template <int D_QK>
static cudaError_t launch_fwd(const DenseKernelParams& p, cudaStream_t stream) {
  using Cfg = typename DenseFwdProb<D_QK>::Cfg;
  auto kern = dense_fwd_kernel<D_QK>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  dim3 grid((p.max_seqlen_q + 63) / 64, p.h_q, p.batch);
  kern<<<grid, 256, Cfg::SMEM_BYTES, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_dense_fwd_mma(const DenseKernelParams& p, cudaStream_t stream) {
  if (p.d_qk == 192) return launch_fwd<192>(p, stream);
  return launch_fwd<128>(p, stream);
}

}  // namespace fmla
