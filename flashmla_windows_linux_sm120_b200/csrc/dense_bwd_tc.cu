// Dense variable-length MHA backward (bf16, head dims 192/128 and 128/128) for sm_100a on
// tcgen05 / TMA / tensor memory.
//
// Math of the reference backward (csrc/sm100/prefill/dense/device/fmha_device_bwd.hpp:290-316 and
// kernel/sm100_fmha_bwd_mla_kernel_tma_warpspecialized.hpp:1308-1324): with P = exp(S*scale - lse),
//   delta = rowsum(dO * O),  dP = dO V^T,  dS = P * (dP - delta),
//   dV = P^T dO,  dK = scale * dS^T Q,  dQ = scale * dS K,
// P and dS rounded to bf16 before the second GEMMs.  Unlike the reference, whose dQ is accumulated
// with floating-point reduce-adds in a launch-dependent order, every output here is produced by
// exactly one CTA in a fixed order, so dQ, dK and dV are bitwise reproducible.  Three kernels:
//   1. delta pre-pass                         (FmhaKernelBwdSumOdO's job)
//   2. dQ:    one CTA per (128-query tile, head, sequence), walks the keys in blocks of 64
//   3. dK/dV: one CTA per (128-key tile, head, sequence), walks the queries in blocks of 64
// Requires h_q == h_k (as flash_mla/flash_mla_interface.py:413-415).
//
// Both main kernels use the same roles as the forward: warps 0-3 element-wise (one thread per row of
// the resident tile = one TMEM lane), warp 4 TMA, warp 5 MMA.  The two first GEMMs of a step write
// fp32 tiles [128 x 64] into tensor memory; the element-wise warps turn them into bf16 P / dS in the
// same columns; the second GEMMs read those as their A operand straight from tensor memory and the
// streamed tile, read MN-major, as B.
// Every mbarrier wait is bounded (tc_common.cuh); a pipeline fault sets a status word and lets the
// CTA drain and free its tensor memory.
#include "kernels.h"
#include "tc_common.cuh"
#include "tma_host.cuh"

namespace fmla {

namespace dbt {
constexpr int kResChunk = 128 * 128;              // resident tiles: [128 rows x 64 bf16] chunks
constexpr int kStgChunk = 64 * 128;               // streamed tiles: [64 rows x 64 bf16] chunks
constexpr int kStages = 3;                        // ring of streamed tiles (the TMEM buffers alternate independently)
template <int V> struct IC { static constexpr int value = V; };
// calls f(IC<stage>, IC<buffer>) with compile-time stage (0..2) and buffer (0..1): every combination gets
// its own straight-line code, so that all descriptors stay a warp-uniform base plus an immediate
template <typename F>
__device__ __forceinline__ void dispatch_stage_buffer(int st, int b, F&& f) {
  if (st == 0) { if (b == 0) f(IC<0>{}, IC<0>{}); else f(IC<0>{}, IC<1>{}); }
  else if (st == 1) { if (b == 0) f(IC<1>{}, IC<0>{}); else f(IC<1>{}, IC<1>{}); }
  else { if (b == 0) f(IC<2>{}, IC<0>{}); else f(IC<2>{}, IC<1>{}); }
}
template <int D_QK>
struct Layout {
  static constexpr int NCH = D_QK / 64;
  static constexpr int kResA = NCH * kResChunk;   // resident [128 x D_QK]   (Q or K)
  static constexpr int kResB = 2 * kResChunk;     // resident [128 x 128]    (dO or V)
  static constexpr int kStgA = NCH * kStgChunk;   // streamed [64 x D_QK]    (K or Q)
  static constexpr int kStgB = 2 * kStgChunk;     // streamed [64 x 128]     (V or dO)
  static constexpr int kStage = kStgA + kStgB;
  static constexpr int RES_OFF = 0;
  static constexpr int STG_OFF = kResA + kResB;
  static constexpr int BAR_OFF = STG_OFF + kStages * kStage;
  static constexpr int VEC_OFF = BAR_OFF + 128;   // float [2][2][64]: per-query lse*log2(e) and delta (dK/dV kernel)
  static constexpr int MISC_OFF = VEC_OFF + 1024;
  static constexpr int SMEM_BYTES = MISC_OFF + 16;
  static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared memory limit per CTA");
};
}  // namespace dbt

__device__ int g_dense_bwd_tc_status = 0;

// Optional timeline of the first steps of CTA (0,0,0) of the dQ kernel, compiled in with -DFMLA_TRACE only.
#ifdef FMLA_TRACE
__device__ long long g_dense_bwd_trace[64 * 16];
#define DBT_TRACE_AT(blk, slot)                                                          \
  do {                                                                                     \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (blk) < 64) g_dense_bwd_trace[(blk) * 16 + (slot)] = clock64(); \
  } while (0)
#else
#define DBT_TRACE_AT(blk, slot) do {} while (0)
#endif

// ---- 1. delta[h, t] = sum_d dO * O --------------------------------------------------------------
__global__ void __launch_bounds__(256) dense_bwd_delta_tc_kernel(const __grid_constant__ DenseKernelParams p) {
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

// Zeroes rows [rows_valid, 64) of a streamed tile of NCHUNK 64-column chunks (whole warp).  Rows past
// the end of a sequence hold the next sequence's data or the TMA zero fill; they meet exact zeros of
// P / dS in the second GEMMs, and 0 * (Inf or NaN) must not reach the accumulators.
__device__ __forceinline__ void zero_stage_tail(unsigned char* tile, int nchunk, int rows_valid, int lane) {
  const int nrows = 64 - rows_valid;
  for (int i = lane; i < nrows * nchunk * 8; i += 32) {
    const int row = rows_valid + i / (nchunk * 8), c16 = i % (nchunk * 8);
    *reinterpret_cast<uint4*>(tile + (c16 >> 3) * dbt::kStgChunk + row * 128 + (c16 & 7) * 16) = make_uint4(0, 0, 0, 0);
  }
  tc::fence_proxy_async_smem();
  __syncwarp();
}

// D[128 x 64] (TMEM column d_col) = A[128 x 64*NCH] (resident, K-major) * B[64 x 64*NCH]^T (streamed, K-major)
template <int NCH>
__device__ __forceinline__ void mma_res_stg(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc) {
#pragma unroll
  for (int c = 0; c < NCH; ++c)
#pragma unroll
    for (int s = 0; s < 4; ++s)
      tc::mma_ss(d_tmem, tc::desc_advance(desc_a, c * dbt::kResChunk + s * 32), tc::desc_advance(desc_b, c * dbt::kStgChunk + s * 32), idesc,
                 (c | s) ? 1u : 0u);
}
// D[128 x N] += A[128 x 64] (bf16 in TMEM, 8 columns per 16-row step) * B[64 x N] (streamed tile read MN-major)
__device__ __forceinline__ void mma_tmem_stg(uint32_t d_tmem, uint32_t a_tmem, uint64_t desc_b, uint32_t idesc, bool first) {
#pragma unroll
  for (int s = 0; s < 4; ++s) tc::mma_ts(d_tmem, a_tmem + s * 8, tc::desc_advance(desc_b, s * 2048), idesc, (first && s == 0) ? 0u : 1u);
}

// ---- 2. dQ ------------------------------------------------------------------------------------------
// grid (ceil(max_seqlen_q/128), h_q, batch), 224 threads (warps 0-3 element-wise, 4 TMA, 5 and 6 MMA).
// Resident: Q, dO tiles of 128 queries.
// Per step (64 keys): S = Q K^T and dP = dO V^T into one of two TMEM buffer pairs, dS (bf16) into one of two
// slots, then dQ += dS K.  TMEM: dQ = [0, D_QK), buffer b: S = [192 + 128 b, +64), dP = [256 + 128 b, +64),
// dS slot b = [448 + 32 b, +32).
namespace dbt {
enum BarQ { Q_RES_FULL = 0, Q_KV_FULL0, Q_KV_EMPTY0 = Q_KV_FULL0 + kStages, Q_SD_FULL0 = Q_KV_EMPTY0 + kStages, Q_SD_FULL1, Q_DS_FULL0, Q_DS_FULL1, Q_BUF_FREE0, Q_BUF_FREE1, Q_DONE, Q_NUM_BARS };
}

template <int D_QK>
__global__ void __launch_bounds__(224, 1)
dense_bwd_dq_tc_kernel(const __grid_constant__ DenseKernelParams p, const __grid_constant__ CUtensorMap tmap_q,
                       const __grid_constant__ CUtensorMap tmap_do, const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v) {
  using namespace dbt;
  using L = Layout<D_QK>;
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase + L::RES_OFF, sDO = sQ + L::kResA, sStg = sbase + L::STG_OFF;
  auto bar = [&](int i) { return sbase + L::BAR_OFF + i * 8; };
  volatile uint32_t* sTmem = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFF);
  int* status = &g_dense_bwd_tc_status;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z, head = blockIdx.y;
  const int q0 = __ldg(p.cu_q + b), lq = __ldg(p.cu_q + b + 1) - q0;
  const int k0 = __ldg(p.cu_k + b), lk = __ldg(p.cu_k + b + 1) - k0;
  const int m_base = (gridDim.x - 1 - blockIdx.x) * 128;    // the tiles with the most keys first
  if (m_base >= lq) return;
  if ((sbase & 1023u) != 0) {
    if (tid == 0) tc::report_status(status, 30);
    return;
  }
  int nblk = (lk + 63) >> 6;
  if (p.is_causal) {
    const int last_key = min(m_base + 127, lq - 1) + (lk - lq);   // inclusive
    nblk = last_key < 0 ? 0 : min(nblk, (last_key >> 6) + 1);
  }

  if (tid == 0) {
    for (int i = 0; i < Q_NUM_BARS; ++i) tc::mbar_init(bar(i), (i == Q_DS_FULL0 || i == Q_DS_FULL1) ? 128 : 1);
    tc::fence_mbar_init();
  }
  if (warp == 5) tc::tmem_alloc(sbase + L::MISC_OFF, 512);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *sTmem;
  constexpr int TM_DQ = 0, TM_SD = 192, TM_DS = 448;

  if (warp == 4) {
    // ================================ TMA producer =====================================
    if (tc::elect_one() && nblk > 0) {
      tc::mbar_arrive_expect_tx(bar(Q_RES_FULL), L::kResA + L::kResB);
#pragma unroll
      for (int c = 0; c < L::NCH; ++c) tc::tma_load_3d(sQ + c * kResChunk, &tmap_q, c * 64, head, q0 + m_base, bar(Q_RES_FULL));
#pragma unroll
      for (int c = 0; c < 2; ++c) tc::tma_load_3d(sDO + c * kResChunk, &tmap_do, c * 64, head, q0 + m_base, bar(Q_RES_FULL));
      bool alive = true;
      for (int j = 0; j < nblk && alive; ++j) {
        const int st = j % kStages;
        const uint32_t stage = sStg + st * L::kStage;
        const int tok = k0 + j * 64;
        alive = tc::mbar_wait(bar(Q_KV_EMPTY0 + st), ((j / kStages) & 1) ^ 1, status, 51);
        if (!alive) break;
        DBT_TRACE_AT(j, 0);
        tc::mbar_arrive_expect_tx(bar(Q_KV_FULL0 + st), L::kStage);
#pragma unroll
        for (int c = 0; c < L::NCH; ++c) tc::tma_load_3d(stage + c * kStgChunk, &tmap_k, c * 64, head, tok, bar(Q_KV_FULL0 + st));
#pragma unroll
        for (int c = 0; c < 2; ++c) tc::tma_load_3d(stage + L::kStgA + c * kStgChunk, &tmap_v, c * 64, head, tok, bar(Q_KV_FULL0 + st));
      }
    }
  } else if (warp == 5 || warp == 6) {
    // ================================ MMA issuers =======================================
    constexpr uint32_t idesc_sd = tc::idesc_bf16_f32(128, 64, 0, 0);
    constexpr uint32_t idesc_dq = tc::idesc_bf16_f32(128, D_QK, 0, 1);
    const uint64_t desc_q = tc::smem_desc_sw128(sQ, 16, 1024);
    const uint64_t desc_do = tc::smem_desc_sw128(sDO, 16, 1024);
    const uint64_t desc_k = tc::smem_desc_sw128(sStg, 16, 1024);                      // K tile of stage 0, K-major (B of S)
    const uint64_t desc_v = tc::smem_desc_sw128(sStg + L::kStgA, 16, 1024);           // V tile of stage 0, K-major (B of dP)
    const uint64_t desc_kt = tc::smem_desc_sw128(sStg, kStgChunk, 1024);              // K tile of stage 0, MN-major (B of dQ)
    bool alive = nblk > 0;
    if (alive) alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(Q_RES_FULL), 0, status, 52));
    // Two issuing warps: warp 5 the first GEMMs of a step (S, dP), warp 6 the second one (dQ).  Each
    // wait on an mbarrier costs the issuing warp a few hundred cycles in which the tensor pipe would
    // otherwise idle; with two warps the waits of one overlap the instructions of the other.
    if (warp == 5) {
      for (int j = 0; j < nblk && alive; ++j) {
        const int st = j % kStages, bf = j & 1;
        // the tile has landed, and the S / dP buffer pair bf is free (the element-wise warps have read step
        // j-2 out of it)
        alive = tc::mbar_wait2(bar(Q_KV_FULL0 + st), (j / kStages) & 1, bar(Q_DS_FULL0 + bf), ((j >> 1) & 1) ^ 1, status, 54);
        if (!alive) break;
        // K rows past the end of the sequence must be exact zeros for dQ += dS K
        if (lk - j * 64 < 64) zero_stage_tail(smem + L::STG_OFF + st * L::kStage, L::NCH, lk - j * 64, lane);
        tc::tc_fence_after();
        if (lane == 0) DBT_TRACE_AT(j, 2);
        if (tc::elect_one()) {
          dispatch_stage_buffer(st, bf, [&](auto ST, auto BF) {
            constexpr int kOff = decltype(ST)::value * L::kStage, kCol = TM_SD + decltype(BF)::value * 128;
            mma_res_stg<L::NCH>(tmem + kCol, desc_q, tc::desc_advance(desc_k, kOff), idesc_sd);
            mma_res_stg<2>(tmem + kCol + 64, desc_do, tc::desc_advance(desc_v, kOff), idesc_sd);
          });
          tc::tc_commit(bar(Q_SD_FULL0 + bf));
          DBT_TRACE_AT(j, 3);
        }
        __syncwarp();
      }
    } else {
      for (int j = 0; j < nblk && alive; ++j) {
        const int st = j % kStages, bf = j & 1;
        if (lane == 0) DBT_TRACE_AT(j, 10);
        alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(Q_DS_FULL0 + bf), (j >> 1) & 1, status, 53));
        if (!alive) break;
        if (lane == 0) DBT_TRACE_AT(j, 11);
        tc::tc_fence_after();
        if (lane == 0) DBT_TRACE_AT(j, 4);
        if (tc::elect_one()) {
          dispatch_stage_buffer(st, bf, [&](auto ST, auto BF) {
            mma_tmem_stg(tmem + TM_DQ, tmem + TM_DS + decltype(BF)::value * 32, tc::desc_advance(desc_kt, decltype(ST)::value * L::kStage),
                         idesc_dq, j == 0);
          });
          tc::tc_commit(bar(Q_KV_EMPTY0 + st));
          tc::tc_commit(bar(Q_BUF_FREE0 + bf));
          if (j == nblk - 1) tc::tc_commit(bar(Q_DONE));
          DBT_TRACE_AT(j, 5);
        }
        __syncwarp();
      }
    }
  } else {
    // ================================ element-wise / epilogue ==========================
    const int row = m_base + tid;
    const bool row_ok = row < lq;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const float lse2 = row_ok ? __ldg(p.lse + (int64_t)(q0 + row) * p.lse_stride_t + head * p.lse_stride_h) * kLog2e : 0.f;
    const float dl = row_ok ? __ldg(p.delta + (int64_t)head * p.total_q + q0 + row) : 0.f;
    const int limit = !row_ok ? 0 : (p.is_causal ? max(0, min(lk, row + (lk - lq) + 1)) : lk);
    bool alive = true;
    for (int j = 0; j < nblk && alive; ++j) {
      const int st = j & 1;
      const uint32_t sd_addr = tmem + lane_addr + TM_SD + st * 128;
      // S and dP of this step are there, and the dS slot st is free (it was last read by the dQ
      // instructions of step j-2; dS has slots of its own so that the fp32 buffers are free again as
      // soon as they have been read)
      alive = tc::mbar_wait2(bar(Q_SD_FULL0 + st), (j >> 1) & 1, bar(Q_BUF_FREE0 + st), ((j >> 1) & 1) ^ 1, status, 55);
      if (!alive) break;
      if (tid == 0) DBT_TRACE_AT(j, 6);
      tc::tc_fence_after();
      uint32_t sv[2][32], dp[2][32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        tc::tmem_ld32(sd_addr + c * 32, sv[c]);
        tc::tmem_ld32(sd_addr + 64 + c * 32, dp[c]);
      }
      tc::tmem_wait_ld();
      if (tid == 0) DBT_TRACE_AT(j, 7);
      const int cnt = limit - j * 64;                          // visible keys of this block: [0, cnt)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = exp2f(fmaf(__uint_as_float(sv[c][2 * i]), p.scale_log2, -lse2));
          const float p1 = exp2f(fmaf(__uint_as_float(sv[c][2 * i + 1]), p.scale_log2, -lse2));
          // a select, not a product: masked entries may hold Inf or NaN
          const float d0 = (c * 32 + 2 * i < cnt) ? p0 * (__uint_as_float(dp[c][2 * i]) - dl) : 0.f;
          const float d1 = (c * 32 + 2 * i + 1 < cnt) ? p1 * (__uint_as_float(dp[c][2 * i + 1]) - dl) : 0.f;
          pk[i] = pack_bf16x2(d0, d1);
        }
        tc::tmem_st16(tmem + lane_addr + TM_DS + st * 32 + c * 16, pk);
      }
      if (tid == 0) DBT_TRACE_AT(j, 8);
      tc::tmem_wait_st();
      tc::tc_fence_before();
      tc::mbar_arrive(bar(Q_DS_FULL0 + st));
      if (tid == 0) DBT_TRACE_AT(j, 9);
    }
    bool have = nblk > 0 && alive;
    if (have) {
      have = __all_sync(0xffffffffu, tc::mbar_wait(bar(Q_DONE), 0, status, 56));
      tc::tc_fence_after();
    }
    __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.dq) + (int64_t)(q0 + row) * p.dq_stride_t + head * p.dq_stride_h;
#pragma unroll 1
    for (int c = 0; c < D_QK / 32; ++c) {
      uint32_t ov[32];
      if (have) {
        tc::tmem_ld32(tmem + lane_addr + TM_DQ + c * 32, ov);
        tc::tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) ov[i] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(ov[q4 * 8 + 0]) * p.scale, __uint_as_float(ov[q4 * 8 + 1]) * p.scale);
          v.y = pack_bf16x2(__uint_as_float(ov[q4 * 8 + 2]) * p.scale, __uint_as_float(ov[q4 * 8 + 3]) * p.scale);
          v.z = pack_bf16x2(__uint_as_float(ov[q4 * 8 + 4]) * p.scale, __uint_as_float(ov[q4 * 8 + 5]) * p.scale);
          v.w = pack_bf16x2(__uint_as_float(ov[q4 * 8 + 6]) * p.scale, __uint_as_float(ov[q4 * 8 + 7]) * p.scale);
          *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = v;
        }
      }
    }
  }

  tc::tc_fence_before();
  __syncthreads();
  if (warp == 5) tc::tmem_dealloc(tmem, 512);
}

// ---- 3. dK, dV ----------------------------------------------------------------------------------
// grid (ceil(max_seqlen_k/128), h, batch), 192 threads.  Resident: K, V tiles of 128 keys.
// Per step (64 queries): S^T = K Q^T into one of two buffers, dP^T = V dO^T into a single buffer
// (tensor memory has no room for a second one beside dK and dV), P^T over S^T and dS^T over dP^T,
// then dV += P^T dO and dK += dS^T Q.
// TMEM: dV = [0,128), dK = [128, 128 + D_QK), S^T buffer b = [320 + 64 b, +64), dP^T = [448, 512).
namespace dbt {
enum BarK { K_RES_FULL = 0, K_QD_FULL0, K_QD_EMPTY0 = K_QD_FULL0 + kStages, K_SD_FULL = K_QD_EMPTY0 + kStages, K_PD_FULL, K_DONE, K_NUM_BARS };
}

template <int D_QK>
__global__ void __launch_bounds__(192, 1)
dense_bwd_dkdv_tc_kernel(const __grid_constant__ DenseKernelParams p, const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_q,
                         const __grid_constant__ CUtensorMap tmap_do) {
  using namespace dbt;
  using L = Layout<D_QK>;
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sK = sbase + L::RES_OFF, sV = sK + L::kResA, sStg = sbase + L::STG_OFF;
  auto bar = [&](int i) { return sbase + L::BAR_OFF + i * 8; };
  float* sVec = reinterpret_cast<float*>(smem + L::VEC_OFF);
  volatile uint32_t* sTmem = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFF);
  volatile int* sAbort = reinterpret_cast<volatile int*>(smem + L::MISC_OFF + 8);   // set by an element-wise thread whose wait expired
  int* status = &g_dense_bwd_tc_status;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z, head = blockIdx.y;
  const int q0 = __ldg(p.cu_q + b), lq = __ldg(p.cu_q + b + 1) - q0;
  const int k0 = __ldg(p.cu_k + b), lk = __ldg(p.cu_k + b + 1) - k0;
  const int n_base = blockIdx.x * 128;                       // with a causal mask the first key tiles see the most queries
  if (n_base >= lk) return;
  if ((sbase & 1023u) != 0) {
    if (tid == 0) tc::report_status(status, 30);
    return;
  }
  // query blocks [jb_lo, jb_hi) of 64 rows that see at least one key of this tile
  const int jb_hi = (lq + 63) >> 6;
  const int jb_lo = p.is_causal ? min(jb_hi, max(0, n_base - (lk - lq)) >> 6) : 0;
  const int nstep = jb_hi - jb_lo;

  if (tid == 0) {
    for (int i = 0; i < K_NUM_BARS; ++i) tc::mbar_init(bar(i), i == K_PD_FULL ? 128 : 1);
    tc::fence_mbar_init();
    *sAbort = 0;
  }
  if (warp == 5) tc::tmem_alloc(sbase + L::MISC_OFF, 512);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *sTmem;
  constexpr int TM_DV = 0, TM_DK = 128, TM_ST = 320, TM_DPT = 448;

  if (warp == 4) {
    // ================================ TMA producer =====================================
    if (tc::elect_one() && nstep > 0) {
      tc::mbar_arrive_expect_tx(bar(K_RES_FULL), L::kResA + L::kResB);
#pragma unroll
      for (int c = 0; c < L::NCH; ++c) tc::tma_load_3d(sK + c * kResChunk, &tmap_k, c * 64, head, k0 + n_base, bar(K_RES_FULL));
#pragma unroll
      for (int c = 0; c < 2; ++c) tc::tma_load_3d(sV + c * kResChunk, &tmap_v, c * 64, head, k0 + n_base, bar(K_RES_FULL));
      bool alive = true;
      for (int j = 0; j < nstep && alive; ++j) {
        const int st = j % kStages;
        const uint32_t stage = sStg + st * L::kStage;
        const int tok = q0 + (jb_lo + j) * 64;
        alive = tc::mbar_wait(bar(K_QD_EMPTY0 + st), ((j / kStages) & 1) ^ 1, status, 61);
        if (!alive) break;
        tc::mbar_arrive_expect_tx(bar(K_QD_FULL0 + st), L::kStage);
#pragma unroll
        for (int c = 0; c < L::NCH; ++c) tc::tma_load_3d(stage + c * kStgChunk, &tmap_q, c * 64, head, tok, bar(K_QD_FULL0 + st));
#pragma unroll
        for (int c = 0; c < 2; ++c) tc::tma_load_3d(stage + L::kStgA + c * kStgChunk, &tmap_do, c * 64, head, tok, bar(K_QD_FULL0 + st));
      }
    }
  } else if (warp == 5) {
    // ================================ MMA issuer =======================================
    constexpr uint32_t idesc_sd = tc::idesc_bf16_f32(128, 64, 0, 0);
    constexpr uint32_t idesc_dv = tc::idesc_bf16_f32(128, 128, 0, 1);
    constexpr uint32_t idesc_dk = tc::idesc_bf16_f32(128, D_QK, 0, 1);
    const uint64_t desc_k = tc::smem_desc_sw128(sK, 16, 1024);
    const uint64_t desc_v = tc::smem_desc_sw128(sV, 16, 1024);
    const uint64_t desc_q = tc::smem_desc_sw128(sStg, 16, 1024);                      // Q tile of stage 0, K-major (B of S^T)
    const uint64_t desc_do = tc::smem_desc_sw128(sStg + L::kStgA, 16, 1024);          // dO tile of stage 0, K-major (B of dP^T)
    const uint64_t desc_qt = tc::smem_desc_sw128(sStg, kStgChunk, 1024);              // Q tile, MN-major (B of dK)
    const uint64_t desc_dot = tc::smem_desc_sw128(sStg + L::kStgA, kStgChunk, 1024);  // dO tile, MN-major (B of dV)
    bool alive = nstep > 0;
    if (alive) alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(K_RES_FULL), 0, status, 62));
    // waits for the tile of step j, clears its rows past the end of the sequence, issues S^T(j)
    auto issue_st = [&](int j) {
      const int st = j % kStages, bf = j & 1;
      alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(K_QD_FULL0 + st), (j / kStages) & 1, status, 63));
      if (!alive) return;
      const int rows_valid = lq - (jb_lo + j) * 64;
      if (rows_valid < 64) zero_stage_tail(smem + L::STG_OFF + st * L::kStage, L::NCH + 2, rows_valid, lane);
      tc::tc_fence_after();
      if (tc::elect_one()) {
        dispatch_stage_buffer(st, bf, [&](auto ST, auto BF) {
          mma_res_stg<L::NCH>(tmem + TM_ST + decltype(BF)::value * 64, desc_k, tc::desc_advance(desc_q, decltype(ST)::value * L::kStage), idesc_sd);
        });
      }
      __syncwarp();
    };
    auto issue_dpt = [&](int j) {
      const int st = j % kStages;
      if (tc::elect_one()) {
        dispatch_stage_buffer(st, 0, [&](auto ST, auto) {
          mma_res_stg<2>(tmem + TM_DPT, desc_v, tc::desc_advance(desc_do, decltype(ST)::value * L::kStage), idesc_sd);
        });
        tc::tc_commit(bar(K_SD_FULL));
      }
      __syncwarp();
    };
    if (alive) issue_st(0);
    if (alive) issue_dpt(0);
    for (int j = 0; j < nstep && alive; ++j) {
      const int st = j % kStages, bf = j & 1;
      if (j + 1 < nstep) issue_st(j + 1);
      if (alive) alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(K_PD_FULL), j & 1, status, 64));
      if (!alive) break;
      tc::tc_fence_after();
      if (tc::elect_one()) {
        dispatch_stage_buffer(st, bf, [&](auto ST, auto BF) {
          constexpr int kOff = decltype(ST)::value * L::kStage;
          mma_tmem_stg(tmem + TM_DV, tmem + TM_ST + decltype(BF)::value * 64, tc::desc_advance(desc_dot, kOff), idesc_dv, j == 0);
          mma_tmem_stg(tmem + TM_DK, tmem + TM_DPT, tc::desc_advance(desc_qt, kOff), idesc_dk, j == 0);
        });
        if (j + 1 >= nstep) tc::tc_commit(bar(K_DONE));
      }
      __syncwarp();
      // dP^T of the next step goes into the buffer that the dK instructions above read (the tensor
      // pipe runs them in order); the stage of step j is handed back right after its last readers
      if (tc::elect_one()) tc::tc_commit(bar(K_QD_EMPTY0 + st));
      __syncwarp();
      if (j + 1 < nstep) issue_dpt(j + 1);
    }
  } else {
    // ================================ element-wise / epilogue ==========================
    const int key = n_base + tid;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const int shift = lk - lq;                                 // query i sees keys <= i + shift
    bool alive = true;
    for (int j = 0; j < nstep && alive; ++j) {
      const int jb = jb_lo + j, st = j & 1;
      // per-query vectors of this step: lse * log2(e) (threads 0-63) and delta (threads 64-127)
      {
        const int i = jb * 64 + (tid & 63);
        float v = 0.f;
        if (i < lq) {
          v = tid < 64 ? __ldg(p.lse + (int64_t)(q0 + i) * p.lse_stride_t + head * p.lse_stride_h) * kLog2e
                       : __ldg(p.delta + (int64_t)head * p.total_q + q0 + i);
        }
        sVec[st * 128 + tid] = v;
      }
      if (!tc::mbar_wait(bar(K_SD_FULL), j & 1, status, 65)) *sAbort = 1;
      bar_sync(1, 128);                                        // vectors visible; also keeps the two buffers of sVec apart
      if (*sAbort) { alive = false; break; }                   // read right after the barrier: the same for all 128 threads
      tc::tc_fence_after();
      uint32_t sv[2][32], dp[2][32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        tc::tmem_ld32(tmem + lane_addr + TM_ST + st * 64 + c * 32, sv[c]);
        tc::tmem_ld32(tmem + lane_addr + TM_DPT + c * 32, dp[c]);
      }
      tc::tmem_wait_ld();
      const int c_max = lq - jb * 64;                          // columns (queries) [c_min, c_max) see this key
      const int c_min = p.is_causal ? key - shift - jb * 64 : 0;
      const float4* vl = reinterpret_cast<const float4*>(sVec + st * 128);
      const float4* vd = reinterpret_cast<const float4*>(sVec + st * 128 + 64);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t pp[16], pd[16];
#pragma unroll
        for (int i4 = 0; i4 < 8; ++i4) {
          const float4 l4 = vl[c * 8 + i4], d4 = vd[c * 8 + i4];
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, ds[4] = {d4.x, d4.y, d4.z, d4.w};
          float pv[4], dv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int col = c * 32 + i4 * 4 + e;
            const bool vis = col >= c_min && col < c_max;
            const float pe = exp2f(fmaf(__uint_as_float(sv[c][i4 * 4 + e]), p.scale_log2, -ls[e]));
            // selects, not products: masked entries may hold Inf or NaN
            pv[e] = vis ? pe : 0.f;
            dv[e] = vis ? pe * (__uint_as_float(dp[c][i4 * 4 + e]) - ds[e]) : 0.f;
          }
          pp[i4 * 2] = pack_bf16x2(pv[0], pv[1]);
          pp[i4 * 2 + 1] = pack_bf16x2(pv[2], pv[3]);
          pd[i4 * 2] = pack_bf16x2(dv[0], dv[1]);
          pd[i4 * 2 + 1] = pack_bf16x2(dv[2], dv[3]);
        }
        tc::tmem_st16(tmem + lane_addr + TM_ST + st * 64 + c * 16, pp);
        tc::tmem_st16(tmem + lane_addr + TM_DPT + c * 16, pd);
      }
      tc::tmem_wait_st();
      tc::tc_fence_before();
      tc::mbar_arrive(bar(K_PD_FULL));
    }
    bool have = nstep > 0 && alive;
    if (have) {
      have = __all_sync(0xffffffffu, tc::mbar_wait(bar(K_DONE), 0, status, 66));
      tc::tc_fence_after();
    }
    const bool row_ok = key < lk;
    __nv_bfloat16* dv_row = reinterpret_cast<__nv_bfloat16*>(p.dv) + (int64_t)(k0 + key) * p.dv_stride_t + head * p.dv_stride_h;
    __nv_bfloat16* dk_row = reinterpret_cast<__nv_bfloat16*>(p.dk) + (int64_t)(k0 + key) * p.dk_stride_t + head * p.dk_stride_h;
#pragma unroll 1
    for (int c = 0; c < (128 + D_QK) / 32; ++c) {
      uint32_t ov[32];
      if (have) {
        tc::tmem_ld32(tmem + lane_addr + c * 32, ov);          // dV columns first, then dK
        tc::tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) ov[i] = 0u;
      }
      const float mul = c < 4 ? 1.f : p.scale;
      __nv_bfloat16* dst = c < 4 ? dv_row + c * 32 : dk_row + (c - 4) * 32;
      if (row_ok) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(ov[q4 * 8 + 0]) * mul, __uint_as_float(ov[q4 * 8 + 1]) * mul);
          v.y = pack_bf16x2(__uint_as_float(ov[q4 * 8 + 2]) * mul, __uint_as_float(ov[q4 * 8 + 3]) * mul);
          v.z = pack_bf16x2(__uint_as_float(ov[q4 * 8 + 4]) * mul, __uint_as_float(ov[q4 * 8 + 5]) * mul);
          v.w = pack_bf16x2(__uint_as_float(ov[q4 * 8 + 6]) * mul, __uint_as_float(ov[q4 * 8 + 7]) * mul);
          *reinterpret_cast<uint4*>(dst + q4 * 8) = v;
        }
      }
    }
  }

  tc::tc_fence_before();
  __syncthreads();
  if (warp == 5) tc::tmem_dealloc(tmem, 512);
}

// ---- host side ----------------------------------------------------------------------------------
template <int D_QK>
static cudaError_t launch_bwd_tc(const DenseKernelParams& p, cudaStream_t stream) {
  using L = dbt::Layout<D_QK>;
  CUtensorMap q128, do128, k64, v64, k128, v128, q64, do64;
  bool ok = tmah::make_map_thd(&q128, p.q, p.d_qk, p.h_q, p.total_q, p.q_stride_h, p.q_stride_t, 128) &&
            tmah::make_map_thd(&q64, p.q, p.d_qk, p.h_q, p.total_q, p.q_stride_h, p.q_stride_t, 64) &&
            tmah::make_map_thd(&do128, p.d_o, p.d_v, p.h_q, p.total_q, p.do_stride_h, p.do_stride_t, 128) &&
            tmah::make_map_thd(&do64, p.d_o, p.d_v, p.h_q, p.total_q, p.do_stride_h, p.do_stride_t, 64) &&
            tmah::make_map_thd(&k128, p.k, p.d_qk, p.h_k, p.total_k, p.k_stride_h, p.k_stride_t, 128) &&
            tmah::make_map_thd(&k64, p.k, p.d_qk, p.h_k, p.total_k, p.k_stride_h, p.k_stride_t, 64) &&
            tmah::make_map_thd(&v128, p.v, p.d_v, p.h_k, p.total_k, p.v_stride_h, p.v_stride_t, 128) &&
            tmah::make_map_thd(&v64, p.v, p.d_v, p.h_k, p.total_k, p.v_stride_h, p.v_stride_t, 64);
  if (!ok) return cudaErrorInvalidValue;
  auto kq = dense_bwd_dq_tc_kernel<D_QK>;
  auto kk = dense_bwd_dkdv_tc_kernel<D_QK>;
  cudaError_t e = cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(kk, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  const int rows = p.total_q * p.h_q;
  dense_bwd_delta_tc_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(p);
  kk<<<dim3((p.max_seqlen_k + 127) / 128, p.h_q, p.batch), 192, L::SMEM_BYTES, stream>>>(p, k128, v128, q64, do64);
  kq<<<dim3((p.max_seqlen_q + 127) / 128, p.h_q, p.batch), 224, L::SMEM_BYTES, stream>>>(p, q128, do128, k64, v64);
  return cudaGetLastError();
}

cudaError_t launch_dense_bwd_tc(const DenseKernelParams& p, cudaStream_t stream) {
  if (p.d_qk == 192) return launch_bwd_tc<192>(p, stream);
  return launch_bwd_tc<128>(p, stream);
}

#ifdef FMLA_TRACE
extern "C" int fmla_debug_read_dense_bwd_trace(long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_dense_bwd_trace, sizeof(long long) * n);
}
#endif

cudaError_t set_status_mirror_dense_bwd(int* mapped_host_word) { return tc::set_status_mirror(mapped_host_word); }

cudaError_t read_dense_bwd_tc_status(int* host_status, bool reset) {
  cudaError_t e = cudaMemcpyFromSymbol(host_status, g_dense_bwd_tc_status, sizeof(int));
  if (e != cudaSuccess) return e;
  if (reset && *host_status != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_dense_bwd_tc_status, &zero, sizeof(int));
  }
  return e;
}

}  // namespace fmla
