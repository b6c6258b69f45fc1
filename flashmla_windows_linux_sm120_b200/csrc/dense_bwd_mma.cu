// Dense variable-length MHA backward (bf16, head dims 192/128 and 128/128).
//
// Math of the reference backward (csrc/sm100/prefill/dense/device/
// fmha_device_bwd.hpp:290-316 and kernel/sm100_fmha_bwd_mla_kernel_tma_
// warpspecialized.hpp:1308-1324): with P = exp(S*scale - lse),
//   delta = rowsum(dO * O),  dP = dO V^T,  dS = P * (dP - delta),
//   dV = P^T dO,  dK = scale * dS^T Q,  dQ = scale * dS K,
// P and dS rounded to bf16 before the second GEMMs.  Unlike the reference, whose
// dQ is accumulated with floating-point reduce-adds in a launch-dependent order,
// every output here is produced by exactly one CTA in a fixed order, so dQ, dK
// and dV are bitwise reproducible.  Three kernels:
//   1. delta pre-pass                        (FmhaKernelBwdSumOdO's job)
//   2. dK/dV: one CTA per (64-key tile, head, sequence), loops over query tiles
//   3. dQ:    one CTA per (64-query tile, head, sequence), loops over key tiles
// Requires h_q == h_k (as flash_mla/flash_mla_interface.py:413-415).
#include "fmla_common.cuh"
#include "kernels.h"

namespace fmla {

// acc[n][4] (16 x 8*NT) += A[a_row0.., 0..KDIM) * B[b_row0.., 0..KDIM)^T, both
// row-major swizzled bf16 tiles in shared memory.
template <int KDIM, int NT>
__device__ __forceinline__ void gemm_nt(float (&acc)[NT][4], uint32_t sA, int a_pitch, int a_row0, uint32_t sB, int b_pitch,
                                        int b_row0) {
  const int lane = threadIdx.x & 31;
  const int a_row = a_row0 + (lane & 7) + ((lane >> 3) & 1) * 8, a_ch = lane >> 4;
  const int b_row = b_row0 + (lane & 7) + (lane >> 4) * 8, b_ch = (lane >> 3) & 1;
#pragma unroll 4
  for (int ks = 0; ks < KDIM / 16; ++ks) {
    uint32_t a[4];
    ldmatrix_x4(sA + swz_off(a_row, ks * 2 + a_ch, a_pitch), a);
#pragma unroll
    for (int n2 = 0; n2 < NT / 2; ++n2) {
      uint32_t b[4];
      ldmatrix_x4(sB + swz_off(b_row + n2 * 16, ks * 2 + b_ch, b_pitch), b);
      mma_bf16_16816(acc[n2 * 2], a, b[0], b[1]);
      mma_bf16_16816(acc[n2 * 2 + 1], a, b[2], b[3]);
    }
  }
}

// acc (16 x 8*NT) += A[a_row0.., 0..64) * B[0..64, 8*b_ch0 ..), A and B row-major
// swizzled bf16 tiles (B is read transposed).
template <int NT>
__device__ __forceinline__ void gemm_nn64(float (&acc)[NT][4], uint32_t sA, int a_pitch, int a_row0, uint32_t sB, int b_pitch,
                                          int b_ch0) {
  const int lane = threadIdx.x & 31;
  const int a_row = a_row0 + (lane & 7) + ((lane >> 3) & 1) * 8, a_ch = lane >> 4;
  const int v_row = ((lane >> 3) & 1) * 8 + (lane & 7), v_ch = b_ch0 + (lane >> 4);
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    uint32_t a[4];
    ldmatrix_x4(sA + swz_off(a_row, kk * 2 + a_ch, a_pitch), a);
#pragma unroll
    for (int n2 = 0; n2 < NT / 2; ++n2) {
      uint32_t b[4];
      ldmatrix_x4_trans(sB + swz_off(kk * 16 + v_row, v_ch + n2 * 2, b_pitch), b);
      mma_bf16_16816(acc[n2 * 2], a, b[0], b[1]);
      mma_bf16_16816(acc[n2 * 2 + 1], a, b[2], b[3]);
    }
  }
}

template <int ROW_ELEMS>
__device__ __forceinline__ void load_rows64(uint32_t sdst, const __nv_bfloat16* src_row, const void* safe) {
  constexpr int CHUNKS = ROW_ELEMS / 8;
  const int row = threadIdx.x >> 2, c0 = threadIdx.x & 3;
  const bool ok = src_row != nullptr;
  const char* base = ok ? reinterpret_cast<const char*>(src_row) : reinterpret_cast<const char*>(safe);
#pragma unroll
  for (int i = 0; i < CHUNKS / 4; ++i) {
    const int c = c0 + 4 * i;
    cp_async16(sdst + swz_off(row, c, ROW_ELEMS * 2), ok ? base + c * 16 : base, ok);
  }
}

// ---- 1. delta[t, h] = sum_d dO * O -------------------------------------------
__global__ void __launch_bounds__(256) dense_bwd_delta_kernel(const __grid_constant__ DenseKernelParams p) {
  const int warp = (blockIdx.x * 256 + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= p.total_q * p.h_q) return;
  const int t = warp / p.h_q, h = warp % p.h_q;
  const __nv_bfloat16* o = reinterpret_cast<const __nv_bfloat16*>(p.o) + (int64_t)t * p.o_stride_t + h * p.o_stride_h;
  const __nv_bfloat16* d = reinterpret_cast<const __nv_bfloat16*>(p.d_o) + (int64_t)t * p.do_stride_t + h * p.do_stride_h;
  const uint2 ov = *reinterpret_cast<const uint2*>(o + lane * 4);
  const uint2 dv = *reinterpret_cast<const uint2*>(d + lane * 4);
  const float2 o0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ov.x));
  const float2 o1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ov.y));
  const float2 d0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dv.x));
  const float2 d1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dv.y));
  float s = o0.x * d0.x + o0.y * d0.y + o1.x * d1.x + o1.y * d1.y;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) p.delta[(int64_t)h * p.total_q + t] = s;
}

template <int D_QK>
struct BwdSmem {
  static constexpr int QK_PITCH = D_QK * 2, V_PITCH = 256;
  static constexpr int RES_QK = 0;                            // resident [64 x D_QK]
  static constexpr int RES_V = RES_QK + 64 * QK_PITCH;        // resident [64 x 128]
  static constexpr int STG_QK = RES_V + 64 * V_PITCH;         // 2 stages [64 x D_QK]
  static constexpr int STG_V = STG_QK + 2 * 64 * QK_PITCH;    // 2 stages [64 x 128]
  static constexpr int PT = STG_V + 2 * 64 * V_PITCH;         // [64 x 64] bf16
  static constexpr int DST = PT + 8192;                       // [64 x 64] bf16
  static constexpr int STATS = DST + 8192;                    // float [2 stages][2][64] (lse*log2e, delta)
  static constexpr int BYTES = STATS + 2 * 2 * 64 * 4;
};

// ---- 2. dK, dV ----------------------------------------------------------------
// grid (ceil(max_seqlen_k/64), h, batch).  Warp (rg, th): keys rg*16.., queries
// th*32.. of each 64-query tile for S^T / dP^T; output columns th*half.. for dK, dV.
template <int D_QK>
__global__ void __launch_bounds__(256, 1) dense_bwd_dkdv_kernel(const __grid_constant__ DenseKernelParams p) {
  extern __shared__ __align__(1024) char smem[];
  using L = BwdSmem<D_QK>;
  const int b = blockIdx.z, head = blockIdx.y, n_base = blockIdx.x * 64;
  const int q0 = __ldg(p.cu_q + b), lq = __ldg(p.cu_q + b + 1) - q0;
  const int k0 = __ldg(p.cu_k + b), lk = __ldg(p.cu_k + b + 1) - k0;
  if (n_base >= lk) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp & 3, th = warp >> 2, g = lane >> 2, t4 = lane & 3;
  const uint32_t sK = smem_u32(smem + L::RES_QK), sV = smem_u32(smem + L::RES_V);
  const uint32_t sQ0 = smem_u32(smem + L::STG_QK), sDO0 = smem_u32(smem + L::STG_V);
  const uint32_t sPT = smem_u32(smem + L::PT), sDST = smem_u32(smem + L::DST);
  float* sStats = reinterpret_cast<float*>(smem + L::STATS);
  const __nv_bfloat16* Q = reinterpret_cast<const __nv_bfloat16*>(p.q);
  const __nv_bfloat16* K = reinterpret_cast<const __nv_bfloat16*>(p.k);
  const __nv_bfloat16* V = reinterpret_cast<const __nv_bfloat16*>(p.v);
  const __nv_bfloat16* DO = reinterpret_cast<const __nv_bfloat16*>(p.d_o);

  // first query tile that can see this key tile: causal => i >= j - (lk - lq)
  int m_lo = 0;
  if (p.is_causal) m_lo = max(0, n_base - (lk - lq)) / 64;
  const int m_hi = (lq + 63) / 64;

  auto load_q_tile = [&](int mt, int st) {
    const int r = tid >> 2, i = mt * 64 + r;
    const bool ok = i < lq;
    load_rows64<D_QK>(sQ0 + st * 64 * L::QK_PITCH, ok ? Q + (int64_t)(q0 + i) * p.q_stride_t + head * p.q_stride_h : nullptr, Q);
    load_rows64<128>(sDO0 + st * 64 * L::V_PITCH, ok ? DO + (int64_t)(q0 + i) * p.do_stride_t + head * p.do_stride_h : nullptr, DO);
    if (tid < 64) {
      const int ii = mt * 64 + tid;
      float l2 = 0.f, dl = 0.f;
      if (ii < lq) {
        l2 = p.lse[(int64_t)(q0 + ii) * p.lse_stride_t + head * p.lse_stride_h] * kLog2e;
        dl = p.delta[(int64_t)head * p.total_q + q0 + ii];
      }
      sStats[st * 128 + tid] = l2;
      sStats[st * 128 + 64 + tid] = dl;
    }
  };

  {
    const int r = tid >> 2, j = n_base + r;
    const bool ok = j < lk;
    load_rows64<D_QK>(sK, ok ? K + (int64_t)(k0 + j) * p.k_stride_t + head * p.k_stride_h : nullptr, K);
    load_rows64<128>(sV, ok ? V + (int64_t)(k0 + j) * p.v_stride_t + head * p.v_stride_h : nullptr, V);
  }
  if (m_lo < m_hi) load_q_tile(m_lo, 0);
  cp_async_commit();

  constexpr int NT_DK = (D_QK / 2) / 8, NT_DV = 64 / 8;
  float dk[NT_DK][4], dv[NT_DV][4];
#pragma unroll
  for (int i = 0; i < NT_DK; ++i) dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
#pragma unroll
  for (int i = 0; i < NT_DV; ++i) dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f;

  for (int mt = m_lo; mt < m_hi; ++mt) {
    const int st = (mt - m_lo) & 1;
    const uint32_t sQ = sQ0 + st * 64 * L::QK_PITCH, sDO = sDO0 + st * 64 * L::V_PITCH;
    cp_async_wait<0>();
    __syncthreads();
    if (mt + 1 < m_hi) load_q_tile(mt + 1, st ^ 1);
    cp_async_commit();

    float s[4][4], dp[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      dp[j][0] = dp[j][1] = dp[j][2] = dp[j][3] = 0.f;
    }
    gemm_nt<D_QK, 4>(s, sK, L::QK_PITCH, rg * 16, sQ, L::QK_PITCH, th * 32);   // S^T  [keys x queries]
    gemm_nt<128, 4>(dp, sV, L::V_PITCH, rg * 16, sDO, L::V_PITCH, th * 32);    // dP^T
    const float* lse2 = sStats + st * 128;
    const float* dlt = lse2 + 64;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t pk[2], dk_[2];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float pv[2], dsv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = n_base + rg * 16 + g + hh * 8;
          const int ql = th * 32 + j * 8 + 2 * t4 + e;
          const int qi = mt * 64 + ql;
          const float l2 = lse2[ql];
          const bool ok = qi < lq && key < lk && (!p.is_causal || key <= qi + (lk - lq)) && l2 != neg_inf();
          const float pr = ok ? exp2f(s[j][hh * 2 + e] * p.scale_log2 - l2) : 0.f;
          pv[e] = pr;
          dsv[e] = pr * (dp[j][hh * 2 + e] - dlt[ql]);
        }
        pk[hh] = pack_bf16x2(pv[0], pv[1]);
        dk_[hh] = pack_bf16x2(dsv[0], dsv[1]);
      }
      const int ch = th * 4 + j;
      *reinterpret_cast<uint32_t*>(smem + L::PT + swz_off(rg * 16 + g, ch, 128) + t4 * 4) = pk[0];
      *reinterpret_cast<uint32_t*>(smem + L::PT + swz_off(rg * 16 + g + 8, ch, 128) + t4 * 4) = pk[1];
      *reinterpret_cast<uint32_t*>(smem + L::DST + swz_off(rg * 16 + g, ch, 128) + t4 * 4) = dk_[0];
      *reinterpret_cast<uint32_t*>(smem + L::DST + swz_off(rg * 16 + g + 8, ch, 128) + t4 * 4) = dk_[1];
    }
    bar_sync(1 + rg, 64);
    gemm_nn64<NT_DV>(dv, sPT, 128, rg * 16, sDO, L::V_PITCH, th * 8);               // dV += P^T dO
    gemm_nn64<NT_DK>(dk, sDST, 128, rg * 16, sQ, L::QK_PITCH, th * (D_QK / 16));   // dK += dS^T Q
  }
  cp_async_wait<0>();

#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int j = n_base + rg * 16 + g + hh * 8;
    if (j >= lk) continue;
    __nv_bfloat16* dkrow = reinterpret_cast<__nv_bfloat16*>(p.dk) + (int64_t)(k0 + j) * p.dk_stride_t + head * p.dk_stride_h;
    __nv_bfloat16* dvrow = reinterpret_cast<__nv_bfloat16*>(p.dv) + (int64_t)(k0 + j) * p.dv_stride_t + head * p.dv_stride_h;
#pragma unroll
    for (int nt = 0; nt < NT_DK; ++nt)
      *reinterpret_cast<uint32_t*>(dkrow + th * (D_QK / 2) + nt * 8 + 2 * t4) =
          pack_bf16x2(dk[nt][hh * 2] * p.scale, dk[nt][hh * 2 + 1] * p.scale);
#pragma unroll
    for (int nt = 0; nt < NT_DV; ++nt)
      *reinterpret_cast<uint32_t*>(dvrow + th * 64 + nt * 8 + 2 * t4) = pack_bf16x2(dv[nt][hh * 2], dv[nt][hh * 2 + 1]);
  }
}

// ---- 3. dQ ----------------------------------------------------------------------
// grid (ceil(max_seqlen_q/64), h, batch).  Warp (rg, th): queries rg*16.., keys
// th*32.. of each key tile for S / dP; dQ columns th*D_QK/2.. .
template <int D_QK>
__global__ void __launch_bounds__(256, 1) dense_bwd_dq_kernel(const __grid_constant__ DenseKernelParams p) {
  extern __shared__ __align__(1024) char smem[];
  using L = BwdSmem<D_QK>;
  const int b = blockIdx.z, head = blockIdx.y, m_base = blockIdx.x * 64;
  const int q0 = __ldg(p.cu_q + b), lq = __ldg(p.cu_q + b + 1) - q0;
  const int k0 = __ldg(p.cu_k + b), lk = __ldg(p.cu_k + b + 1) - k0;
  if (m_base >= lq) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp & 3, th = warp >> 2, g = lane >> 2, t4 = lane & 3;
  const uint32_t sQ = smem_u32(smem + L::RES_QK), sDO = smem_u32(smem + L::RES_V);
  const uint32_t sK0 = smem_u32(smem + L::STG_QK), sV0 = smem_u32(smem + L::STG_V);
  const uint32_t sDS = smem_u32(smem + L::DST);
  const __nv_bfloat16* Q = reinterpret_cast<const __nv_bfloat16*>(p.q);
  const __nv_bfloat16* K = reinterpret_cast<const __nv_bfloat16*>(p.k);
  const __nv_bfloat16* V = reinterpret_cast<const __nv_bfloat16*>(p.v);
  const __nv_bfloat16* DO = reinterpret_cast<const __nv_bfloat16*>(p.d_o);

  int n_hi = (lk + 63) / 64;
  if (p.is_causal) {
    const int last_key = min(m_base + 63, lq - 1) + (lk - lq);
    n_hi = last_key < 0 ? 0 : min(n_hi, last_key / 64 + 1);
  }
  auto load_k_tile = [&](int nt, int st) {
    const int r = tid >> 2, j = nt * 64 + r;
    const bool ok = j < lk;
    load_rows64<D_QK>(sK0 + st * 64 * L::QK_PITCH, ok ? K + (int64_t)(k0 + j) * p.k_stride_t + head * p.k_stride_h : nullptr, K);
    load_rows64<128>(sV0 + st * 64 * L::V_PITCH, ok ? V + (int64_t)(k0 + j) * p.v_stride_t + head * p.v_stride_h : nullptr, V);
  };
  {
    const int r = tid >> 2, i = m_base + r;
    const bool ok = i < lq;
    load_rows64<D_QK>(sQ, ok ? Q + (int64_t)(q0 + i) * p.q_stride_t + head * p.q_stride_h : nullptr, Q);
    load_rows64<128>(sDO, ok ? DO + (int64_t)(q0 + i) * p.do_stride_t + head * p.do_stride_h : nullptr, DO);
  }
  if (n_hi > 0) load_k_tile(0, 0);
  cp_async_commit();

  float lse2[2], dlt[2];
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int i = m_base + rg * 16 + g + hh * 8;
    lse2[hh] = i < lq ? p.lse[(int64_t)(q0 + i) * p.lse_stride_t + head * p.lse_stride_h] * kLog2e : neg_inf();
    dlt[hh] = i < lq ? p.delta[(int64_t)head * p.total_q + q0 + i] : 0.f;
  }

  constexpr int NT_DQ = (D_QK / 2) / 8;
  float dq[NT_DQ][4];
#pragma unroll
  for (int i = 0; i < NT_DQ; ++i) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;

  for (int nt = 0; nt < n_hi; ++nt) {
    const int st = nt & 1;
    const uint32_t sK = sK0 + st * 64 * L::QK_PITCH, sV = sV0 + st * 64 * L::V_PITCH;
    cp_async_wait<0>();
    __syncthreads();
    if (nt + 1 < n_hi) load_k_tile(nt + 1, st ^ 1);
    cp_async_commit();

    float s[4][4], dp[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      dp[j][0] = dp[j][1] = dp[j][2] = dp[j][3] = 0.f;
    }
    gemm_nt<D_QK, 4>(s, sQ, L::QK_PITCH, rg * 16, sK, L::QK_PITCH, th * 32);
    gemm_nt<128, 4>(dp, sDO, L::V_PITCH, rg * 16, sV, L::V_PITCH, th * 32);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t pk[2];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float dsv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int qi = m_base + rg * 16 + g + hh * 8;
          const int key = nt * 64 + th * 32 + j * 8 + 2 * t4 + e;
          const bool ok = qi < lq && key < lk && (!p.is_causal || key <= qi + (lk - lq)) && lse2[hh] != neg_inf();
          const float pr = ok ? exp2f(s[j][hh * 2 + e] * p.scale_log2 - lse2[hh]) : 0.f;
          dsv[e] = pr * (dp[j][hh * 2 + e] - dlt[hh]);
        }
        pk[hh] = pack_bf16x2(dsv[0], dsv[1]);
      }
      const int ch = th * 4 + j;
      *reinterpret_cast<uint32_t*>(smem + L::DST + swz_off(rg * 16 + g, ch, 128) + t4 * 4) = pk[0];
      *reinterpret_cast<uint32_t*>(smem + L::DST + swz_off(rg * 16 + g + 8, ch, 128) + t4 * 4) = pk[1];
    }
    bar_sync(1 + rg, 64);
    gemm_nn64<NT_DQ>(dq, sDS, 128, rg * 16, sK, L::QK_PITCH, th * (D_QK / 16));   // dQ += dS K
  }
  cp_async_wait<0>();

#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int i = m_base + rg * 16 + g + hh * 8;
    if (i >= lq) continue;
    __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(p.dq) + (int64_t)(q0 + i) * p.dq_stride_t + head * p.dq_stride_h;
#pragma unroll
    for (int nt = 0; nt < NT_DQ; ++nt)
      *reinterpret_cast<uint32_t*>(row + th * (D_QK / 2) + nt * 8 + 2 * t4) =
          pack_bf16x2(dq[nt][hh * 2] * p.scale, dq[nt][hh * 2 + 1] * p.scale);
  }
}

template <int D_QK>
static cudaError_t launch_bwd(const DenseKernelParams& p, cudaStream_t stream) {
  using L = BwdSmem<D_QK>;
  auto k1 = dense_bwd_dkdv_kernel<D_QK>;
  auto k2 = dense_bwd_dq_kernel<D_QK>;
  cudaError_t e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, L::BYTES);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, L::BYTES);
  if (e != cudaSuccess) return e;
  const int rows = p.total_q * p.h_q;
  dense_bwd_delta_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(p);
  k1<<<dim3((p.max_seqlen_k + 63) / 64, p.h_q, p.batch), 256, L::BYTES, stream>>>(p);
  k2<<<dim3((p.max_seqlen_q + 63) / 64, p.h_q, p.batch), 256, L::BYTES, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_dense_bwd_mma(const DenseKernelParams& p, cudaStream_t stream) {
  if (p.d_qk == 192) return launch_bwd<192>(p, stream);
  return launch_bwd<128>(p, stream);
}

}  // namespace fmla
