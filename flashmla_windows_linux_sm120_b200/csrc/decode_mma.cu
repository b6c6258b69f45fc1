// Split-KV MLA decode kernels (dense BF16 paged cache, sparse FP8 cache with
// top-k slot indices) on the shared 64-row attention tile (attn_tile.cuh).
//
// Semantics follow the reference decode kernels:
//   - schedule rows [begin_idx, begin_block, end_idx, end_block, n_split_idx]
//     (csrc/params.h:52) are consumed as in
//     csrc/sm90/decode/dense/splitkv_mla.cu:1022-1042 and
//     csrc/sm100/decode/sparse_fp8/splitkv_mla.cu:168-186;
//   - causal border: query s_q_idx sees tokens < seqlen_k - (s_q-1-s_q_idx)
//     (csrc/sm90/decode/dense/splitkv_mla.cu:948-957);
//   - unsplit requests write bf16 O and natural-log LSE (+inf for rows with no
//     key); split requests write normalised fp32 partial O and base-2 LSE (-inf
//     when empty) at slot num_splits[b] + n_split_idx (:1237-1269);
//   - FP8 records: 512 e4m3 + 4 fp32 scales + 64 bf16 (README.md:162-170);
//     de-quantisation is bf16(fp32(e4m3) * scale) as tests/quant.py:60-63.
#include "attn_tile.cuh"
#include "kernels.h"

#include <cuda_fp8.h>

namespace fmla {

using DecodeCfg = TileCfg<576, 512, true>;

struct DecodeRowMap {
  // regrouped row r (0 .. s_q*hq_per_hk) of kv head kh -> (s_q_idx, head)
  int hq_per_hk;
  __device__ __forceinline__ int sq_idx(int row) const { return row / hq_per_hk; }
  __device__ __forceinline__ int head(int kh, int row) const { return kh * hq_per_hk + row % hq_per_hk; }
};

template <bool SPARSE>
struct DecodeProb {
  const DecodeKernelParams& p;
  int batch, kh, row_base, nvalid_rows;
  int seqlen;       // dense: cache_seqlens[batch]
  int min_border;   // smallest causal border over the tile's rows
  const int* idx_row;  // sparse: indices[batch, s_q_idx, :]
  uint4 pre[10];       // sparse: raw bytes of the next token quarter (8x16 B fp8 + 2x16 B rope)
  float pre_scale;
  bool pre_ok;

  __device__ __forceinline__ DecodeProb(const DecodeKernelParams& p_) : p(p_) {}

  __device__ __forceinline__ void load_q(uint32_t sQ) {
    const int r = threadIdx.x >> 2;
    const __nv_bfloat16* src = nullptr;
    if (r < nvalid_rows) {
      const int row = row_base + r;
      const int sq = row / p.hq_per_hk, head = kh * p.hq_per_hk + row % p.hq_per_hk;
      src = reinterpret_cast<const __nv_bfloat16*>(p.q) + batch * p.q_stride_b + sq * p.q_stride_s + head * p.q_stride_h;
    }
    load_rows_async<576>(sQ, src, p.q);
  }

  __device__ __forceinline__ void load_kv_begin(int blk, int stage, uint32_t sK, uint32_t, int* sValid) {
    const int r = threadIdx.x >> 2;
    if constexpr (!SPARSE) {
      const int tok = blk * 64 + r;
      const __nv_bfloat16* src = nullptr;
      if (tok < seqlen) {
        const int page = __ldg(p.block_table + batch * p.block_table_stride_b + blk);
        src = reinterpret_cast<const __nv_bfloat16*>(p.kcache) + (int64_t)page * p.k_stride_block + r * p.k_stride_row +
              kh * p.k_stride_head;
      }
      load_rows_async<576>(sK, src, p.kcache);
    } else {
      const int quarter = threadIdx.x & 3;
      const int slot = __ldg(idx_row + blk * 64 + r);
      pre_ok = slot >= 0 && slot < p.num_blocks * 64;
      if (quarter == 0) sValid[r] = pre_ok ? 1 : 0;
      if (pre_ok) {
        const unsigned char* rec = reinterpret_cast<const unsigned char*>(p.kcache) + (int64_t)(slot >> 6) * p.k_stride_block +
                                   (slot & 63) * p.k_stride_row;
        const uint4* nope = reinterpret_cast<const uint4*>(rec + quarter * 128);
#pragma unroll
        for (int i = 0; i < 8; ++i) pre[i] = __ldg(nope + i);
        pre_scale = __ldg(reinterpret_cast<const float*>(rec + 512) + quarter);
        const uint4* rope = reinterpret_cast<const uint4*>(rec + 528 + quarter * 32);
        pre[8] = __ldg(rope);
        pre[9] = __ldg(rope + 1);
      }
    }
  }

  __device__ __forceinline__ void load_kv_end(int, uint32_t sK, uint32_t) {
    if constexpr (SPARSE) {
      const int r = threadIdx.x >> 2, quarter = threadIdx.x & 3;
      // 128 nope values -> chunks quarter*16 .. +15 ; 16 rope values -> chunks 64 + quarter*2 .. +1
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
        if (pre_ok) {
          const uint32_t w[4] = {pre[i].x, pre[i].y, pre[i].z, pre[i].w};
          uint32_t o[8];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // 4 e4m3 bytes -> 4 floats (exact), * scale in fp32, round to bf16
            const __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[k] & 0xffffu), __NV_E4M3);
            const __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[k] >> 16), __NV_E4M3);
            const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
            const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
            o[k * 2] = pack_bf16x2(f01.x * pre_scale, f01.y * pre_scale);
            o[k * 2 + 1] = pack_bf16x2(f23.x * pre_scale, f23.y * pre_scale);
          }
          lo = make_uint4(o[0], o[1], o[2], o[3]);
          hi = make_uint4(o[4], o[5], o[6], o[7]);
        }
        const int ch = quarter * 16 + i * 2;
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(sK + swz_off(r, ch, 1152)), "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w));
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(sK + swz_off(r, ch + 1, 1152)), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w));
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const uint4 v = pre_ok ? pre[8 + i] : make_uint4(0, 0, 0, 0);
        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(sK + swz_off(r, 64 + quarter * 2 + i, 1152)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w));
      }
    }
  }

  __device__ __forceinline__ bool needs_mask(int blk) const {
    if constexpr (SPARSE) return true;
    return (blk + 1) * 64 > min_border;
  }
  __device__ __forceinline__ bool valid(int row, int blk, int tok, const int* sValid) const {
    if constexpr (SPARSE) return sValid[tok] != 0;
    const int sq = (row_base + row) / p.hq_per_hk;
    const int border = p.is_causal ? seqlen - (p.s_q - 1 - sq) : seqlen;
    return blk * 64 + tok < border;
  }
};

template <bool SPARSE>
__global__ void __launch_bounds__(256, 1) decode_splitkv_kernel(const __grid_constant__ DecodeKernelParams p) {
  extern __shared__ __align__(1024) char smem[];
  const int part = blockIdx.z;
  const int4 md = __ldg(reinterpret_cast<const int4*>(p.tile_scheduler_metadata + part * 8));
  const int begin_idx = md.x, begin_block = md.y, end_idx = md.z, end_block = md.w;
  const int begin_split = __ldg(p.tile_scheduler_metadata + part * 8 + 4);
  if (begin_idx >= p.b) return;

  const int q_seq_per_hk = p.s_q * p.hq_per_hk;
  DecodeProb<SPARSE> prob(p);
  int sq_fixed = 0;
  if constexpr (SPARSE) {
    // grid (head blocks, s_q, parts): the tile is 64 heads of one query token
    sq_fixed = blockIdx.y;
    prob.kh = 0;
    prob.row_base = sq_fixed * p.hq_per_hk + blockIdx.x * 64;
    prob.nvalid_rows = min(64, p.hq_per_hk - blockIdx.x * 64);
  } else {
    // grid (row blocks, h_k, parts): 64 consecutive regrouped rows of one kv head
    prob.kh = blockIdx.y;
    prob.row_base = blockIdx.x * 64;
    prob.nvalid_rows = min(64, q_seq_per_hk - blockIdx.x * 64);
  }

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp & 3, th = warp >> 2, g = lane >> 2, t4 = lane & 3;

  for (int batch = begin_idx; batch <= end_idx; ++batch) {
    prob.batch = batch;
    int nblk_total;
    if constexpr (SPARSE) {
      nblk_total = p.topk / 64;
      prob.seqlen = p.topk;
      prob.min_border = 0;
      prob.idx_row = p.indices + batch * p.indices_stride_b + sq_fixed * p.indices_stride_s;
    } else {
      prob.seqlen = __ldg(p.seqlens_k + batch);
      nblk_total = (prob.seqlen + 63) / 64;
      prob.min_border = p.is_causal ? prob.seqlen - (p.s_q - 1) : prob.seqlen;
    }
    const int blk_lo = batch == begin_idx ? begin_block : 0;
    const int blk_hi = min(batch == end_idx ? end_block : nblk_total, nblk_total);
    const int n_split_idx = batch == begin_idx ? begin_split : 0;
    const int split_lo = __ldg(p.num_splits + batch);
    const bool no_split = !p.force_partial && __ldg(p.num_splits + batch + 1) - split_lo == 1;

    TileAcc<DecodeCfg> acc;
    run_tile<DecodeCfg>(prob, smem, blk_lo, blk_hi, p.scale_log2, acc);

#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = rg * 16 + g + h * 8;
      if (r >= prob.nvalid_rows) continue;
      const int row = prob.row_base + r;
      const int sq = row / p.hq_per_hk, head = prob.kh * p.hq_per_hk + row % p.hq_per_hk;
      const float l = acc.l[h];
      const float inv = l == 0.f ? 0.f : 1.f / l;
      if (no_split) {
        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + batch * p.o_stride_b + sq * p.o_stride_s + head * p.o_stride_h;
#pragma unroll
        for (int nt = 0; nt < DecodeCfg::NT_O; ++nt) {
          const int col = th * 256 + nt * 8 + 2 * t4;
          *reinterpret_cast<uint32_t*>(orow + col) = pack_bf16x2(acc.o[nt][h * 2] * inv, acc.o[nt][h * 2 + 1] * inv);
        }
        if (th == 0 && t4 == 0)
          p.softmax_lse[((int64_t)batch * p.h_q + head) * p.s_q + sq] = l == 0.f ? pos_inf() : (log2f(l) + acc.m[h]) * kLn2;
      } else {
        const int64_t arow = ((int64_t)(split_lo + n_split_idx) * p.h_k + prob.kh) * q_seq_per_hk + row;
        float* orow = p.o_accum + arow * 512;
#pragma unroll
        for (int nt = 0; nt < DecodeCfg::NT_O; ++nt) {
          const int col = th * 256 + nt * 8 + 2 * t4;
          *reinterpret_cast<float2*>(orow + col) = make_float2(acc.o[nt][h * 2] * inv, acc.o[nt][h * 2 + 1] * inv);
        }
        if (th == 0 && t4 == 0) p.lse_accum[arow] = l == 0.f ? neg_inf() : log2f(l) + acc.m[h];
      }
    }
    __syncthreads();
  }
}

cudaError_t launch_decode_mma(const DecodeKernelParams& p, cudaStream_t stream) {
  const int q_seq_per_hk = p.s_q * p.hq_per_hk;
  cudaError_t e;
  if (p.topk >= 0) {
    auto kern = decode_splitkv_kernel<true>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeCfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    dim3 grid((p.hq_per_hk + 63) / 64, p.s_q, p.num_sm_parts);
    kern<<<grid, 256, DecodeCfg::SMEM_BYTES, stream>>>(p);
  } else {
    auto kern = decode_splitkv_kernel<false>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeCfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    dim3 grid((q_seq_per_hk + 63) / 64, p.h_k, p.num_sm_parts);
    kern<<<grid, 256, DecodeCfg::SMEM_BYTES, stream>>>(p);
  }
  return cudaGetLastError();
}

}  // namespace fmla
