// Dense variable-length MHA forward (bf16, head dims 192/128 and 128/128) for sm_100a on
// tcgen05 / TMA / tensor memory.
//
// One CTA = 256 query rows (two tiles of 128) of one (sequence, head); keys are walked in blocks of 128.
//   warps 0-3  softmax of tile 0, warps 6-9 softmax of tile 1: one thread per query row (TMEM lane =
//              row, so no exchange between threads): S -> registers, mask, running max / sum (base 2),
//              P (bf16) written back into the columns S came from, lazy rescale of O, final 1/l
//              normalisation and stores
//   warp 4     TMA: both Q tiles once; K blocks into a 2-stage ring, V blocks into a single stage
//              (64-column chunks of [128 rows x 128 bytes], 128-byte swizzle)
//   warp 5     MMA: S_t = Q_t K^T (tcgen05.mma m128n128k16, both operands from shared memory),
//              O_t += P_t V (m128n128k16, P from tensor memory, V from shared memory MN-major), in the
//              order  P V of tile 0, S of tile 0 for the next block, P V of tile 1, S of tile 1 for the
//              next block: while the softmax of one tile runs, the tensor pipe works for the other
//              tile, and the exponentials of the two tiles (the SFU does 16 per clock and SM, about as
//              long as the two GEMMs of a tile) overlap with the GEMMs instead of alternating with them
// TMEM map (all 512 columns): S/P of tile 0 = [0,128), of tile 1 = [128,256), O of tile 0 = [256,384),
// of tile 1 = [384,512).  For M = 128 element (row r, col c) of a result sits in lane r, column c;
// the bf16 A operand in tensor memory holds k values (2c, 2c+1) of row r in the 32-bit column c of lane r.
//
// Semantics of the reference forward (csrc/sm100/prefill/dense/fmha_cutlass_fwd_sm100.cu:67-119
// and its mainloop): packed varlen q/k/v with cu_seqlens; GQA maps q head h to kv head
// h / (h_q/h_k); causal masking is bottom-right aligned (query i sees keys j <= i + s_k - s_q,
// collective/fmha_fusion.hpp:266-274); LSE is the natural log of the row sum; rows with no
// visible key give O = 0, LSE = -inf.
// Every mbarrier wait is bounded (tc_common.cuh); a pipeline fault sets a status word and lets the
// CTA drain and free its tensor memory.
#include "kernels.h"
#include "tc_common.cuh"
#include "tma_host.cuh"

namespace fmla {

namespace dft {
constexpr int kChunkBytes = 128 * 128;            // [128 rows x 64 bf16], 128-byte rows
constexpr int kVBytes = 2 * kChunkBytes;          // 128 x 128 bf16
enum Bar { Q_FULL = 0, K_FULL0, K_FULL1, K_EMPTY0, K_EMPTY1, V_FULL, V_EMPTY, S_FULL0, S_FULL1, P_FULL0, P_FULL1, PV_DONE0, PV_DONE1, NUM_BARS };
constexpr int TMEM_S = 0, TMEM_O = 256;
constexpr float kRescaleThreshold = 8.0f;         // log2 units; below it O keeps its stale scale
template <int D_QK>
struct Layout {
  static constexpr int NCH = D_QK / 64;           // 64-column chunks of Q and K
  static constexpr int kTileBytes = NCH * kChunkBytes;    // one Q tile / one K block
  static constexpr int Q_OFF = 0;                 // 2 tiles
  static constexpr int K_OFF = 2 * kTileBytes;    // 2 stages
  static constexpr int V_OFF = K_OFF + 2 * kTileBytes;
  static constexpr int BAR_OFF = V_OFF + kVBytes;
  static constexpr int MISC_OFF = BAR_OFF + 128;
  static constexpr int SMEM_BYTES = MISC_OFF + 16;
  static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared memory limit per CTA");
};
static_assert(NUM_BARS * 8 <= 128, "barrier area too small");
}  // namespace dft

__device__ int g_dense_tc_status = 0;

// The S = Q K^T instructions of tile T for the key block in K stage ST, as straight-line code whose
// descriptors are a warp-uniform base plus an immediate.
template <int T, int ST, int D_QK>
__device__ __forceinline__ void dense_s_block(uint32_t tmem, uint64_t desc_q, uint64_t desc_k, uint32_t idesc) {
  using L = dft::Layout<D_QK>;
#pragma unroll
  for (int c = 0; c < L::NCH; ++c)
#pragma unroll
    for (int s = 0; s < 4; ++s)
      tc::mma_ss(tmem + dft::TMEM_S + T * 128, tc::desc_advance(desc_q, T * L::kTileBytes + c * dft::kChunkBytes + s * 32),
                 tc::desc_advance(desc_k, ST * L::kTileBytes + c * dft::kChunkBytes + s * 32), idesc, (c | s) ? 1u : 0u);
}
// O_T += P_T V of one key block: P from the S columns of tile T (8 columns per 16-token step).
template <int T>
__device__ __forceinline__ void dense_pv_block(uint32_t tmem, uint64_t desc_v, uint32_t idesc, bool first) {
#pragma unroll
  for (int s = 0; s < 8; ++s)
    tc::mma_ts(tmem + dft::TMEM_O + T * 128, tmem + dft::TMEM_S + T * 128 + s * 8, tc::desc_advance(desc_v, s * 2048), idesc,
               (first && s == 0) ? 0u : 1u);
}

// grid (ceil(max_seqlen_q/256), h_q, batch), 320 threads
template <int D_QK>
__global__ void __launch_bounds__(320, 1)
dense_fwd_tc_kernel(const __grid_constant__ DenseKernelParams p, const __grid_constant__ CUtensorMap tmap_q,
                    const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v) {
  using namespace dft;
  using L = Layout<D_QK>;
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase + L::Q_OFF, sK = sbase + L::K_OFF, sV = sbase + L::V_OFF;
  auto bar = [&](int i) { return sbase + L::BAR_OFF + i * 8; };
  volatile uint32_t* sTmem = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFF);
  int* status = &g_dense_tc_status;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z, head = blockIdx.y, kv_head = head / (p.h_q / p.h_k);
  const int q0 = __ldg(p.cu_q + b), lq = __ldg(p.cu_q + b + 1) - q0;
  const int k0 = __ldg(p.cu_k + b), lk = __ldg(p.cu_k + b + 1) - k0;
  // with a causal mask the last tiles have the most keys: they are started first
  const int m_base = (gridDim.x - 1 - blockIdx.x) * 256;
  if (m_base >= lq) return;
  if ((sbase & 1023u) != 0) {   // the swizzled tiles need a 1024-byte aligned base
    if (tid == 0) tc::report_status(status, 30);
    return;
  }
  // both tiles walk the key blocks the last row of the CTA needs; blocks a row cannot see are masked
  int nblk = (lk + 127) >> 7;
  if (p.is_causal) {
    const int last_key = min(m_base + 255, lq - 1) + (lk - lq);   // inclusive
    nblk = last_key < 0 ? 0 : min(nblk, (last_key >> 7) + 1);
  }

  if (tid == 0) {
    for (int i = 0; i < NUM_BARS; ++i) tc::mbar_init(bar(i), (i == P_FULL0 || i == P_FULL1) ? 128 : 1);
    tc::fence_mbar_init();
  }
  if (warp == 5) tc::tmem_alloc(sbase + L::MISC_OFF, 512);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *sTmem;

  if (warp == 4) {
    // ================================ TMA producer =====================================
    if (tc::elect_one() && nblk > 0) {
      tc::prefetch_tensormap(&tmap_q);
      tc::prefetch_tensormap(&tmap_k);
      tc::prefetch_tensormap(&tmap_v);
      tc::mbar_arrive_expect_tx(bar(Q_FULL), 2 * L::kTileBytes);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int c = 0; c < L::NCH; ++c)
          tc::tma_load_3d(sQ + t * L::kTileBytes + c * kChunkBytes, &tmap_q, c * 64, head, q0 + m_base + t * 128, bar(Q_FULL));
      bool alive = true;
      for (int j = 0; j < nblk && alive; ++j) {
        const int st = j & 1;
        const int tok = k0 + j * 128;
        alive = tc::mbar_wait(bar(K_EMPTY0 + st), ((j >> 1) & 1) ^ 1, status, 41);
        if (!alive) break;
        tc::mbar_arrive_expect_tx(bar(K_FULL0 + st), L::kTileBytes);
#pragma unroll
        for (int c = 0; c < L::NCH; ++c) tc::tma_load_3d(sK + st * L::kTileBytes + c * kChunkBytes, &tmap_k, c * 64, kv_head, tok, bar(K_FULL0 + st));
        alive = tc::mbar_wait(bar(V_EMPTY), (j & 1) ^ 1, status, 42);
        if (!alive) break;
        tc::mbar_arrive_expect_tx(bar(V_FULL), kVBytes);
#pragma unroll
        for (int c = 0; c < 2; ++c) tc::tma_load_3d(sV + c * kChunkBytes, &tmap_v, c * 64, kv_head, tok, bar(V_FULL));
      }
    }
  } else if (warp == 5) {
    // ================================ MMA issuer =======================================
    constexpr uint32_t idesc_s = tc::idesc_bf16_f32(128, 128, 0, 0);
    constexpr uint32_t idesc_o = tc::idesc_bf16_f32(128, 128, 0, 1);
    const uint64_t desc_q = tc::smem_desc_sw128(sQ, 16, 1024);               // A of S: K-major (tile 0)
    const uint64_t desc_k = tc::smem_desc_sw128(sK, 16, 1024);               // B of S: K-major (stage 0)
    const uint64_t desc_v = tc::smem_desc_sw128(sV, kChunkBytes, 1024);      // B of PV: MN-major, 64-wide column groups 16 KB apart
    bool alive = nblk > 0;
    if (alive) alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(Q_FULL), 0, status, 43));
    // S of tile t for block j (whole warp; K(j) must have been waited for)
    auto issue_s = [&](int t, int j) {
      const int st = j & 1;
      tc::tc_fence_after();
      if (tc::elect_one()) {
        if (t == 0) {
          if (st == 0) dense_s_block<0, 0, D_QK>(tmem, desc_q, desc_k, idesc_s);
          else dense_s_block<0, 1, D_QK>(tmem, desc_q, desc_k, idesc_s);
          tc::tc_commit(bar(S_FULL0));
        } else {
          if (st == 0) dense_s_block<1, 0, D_QK>(tmem, desc_q, desc_k, idesc_s);
          else dense_s_block<1, 1, D_QK>(tmem, desc_q, desc_k, idesc_s);
          tc::tc_commit(bar(S_FULL1));
          tc::tc_commit(bar(K_EMPTY0 + st));     // both tiles have read this K block
        }
      }
      __syncwarp();
    };
    // P V of tile t for block j
    auto issue_pv = [&](int t, int j) {
      alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(P_FULL0 + t), j & 1, status, 45));
      if (!alive) return;
      tc::tc_fence_after();
      if (tc::elect_one()) {
        if (t == 0) {
          dense_pv_block<0>(tmem, desc_v, idesc_o, j == 0);
          tc::tc_commit(bar(PV_DONE0));
        } else {
          dense_pv_block<1>(tmem, desc_v, idesc_o, j == 0);
          tc::tc_commit(bar(PV_DONE1));
          tc::tc_commit(bar(V_EMPTY));           // both tiles have read this V block
        }
      }
      __syncwarp();
    };
    if (alive) alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(K_FULL0), 0, status, 46));
    if (alive) { issue_s(0, 0); issue_s(1, 0); }
    for (int j = 0; j < nblk && alive; ++j) {
      alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(V_FULL), j & 1, status, 44));
      if (!alive) break;
      // V rows past the end of the sequence belong to the next sequence (or are the zero fill) and are
      // cleared first, so that 0 * (Inf or NaN) cannot reach O
      const int rows_valid = lk - j * 128;
      if (rows_valid < 128) {
        unsigned char* v = smem + L::V_OFF;
        const int nrows = 128 - rows_valid;
        for (int i = lane; i < nrows * 16; i += 32) {
          const int row = rows_valid + (i >> 4), c16 = i & 15;
          *reinterpret_cast<uint4*>(v + (c16 >> 3) * kChunkBytes + row * 128 + (c16 & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
        tc::fence_proxy_async_smem();
        __syncwarp();
      }
      const bool more = j + 1 < nblk;
      issue_pv(0, j);
      if (!alive) break;
      if (more) {
        alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(K_FULL0 + ((j + 1) & 1)), ((j + 1) >> 1) & 1, status, 46));
        if (!alive) break;
        issue_s(0, j + 1);        // overwrites the columns P of tile 0 was just read from: the tensor pipe runs in order
      }
      issue_pv(1, j);
      if (!alive) break;
      if (more) issue_s(1, j + 1);
    }
  } else {
    // ================================ softmax / epilogue ================================
    const int t = warp >= 6 ? 1 : 0;                            // the tile this warp works for
    const int rl = (warp & 3) * 32 + lane;                     // row within the tile = TMEM lane
    const int row = m_base + t * 128 + rl;                     // query row within its sequence
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_addr = tmem + lane_addr + TMEM_S + t * 128;
    const uint32_t o_addr = tmem + lane_addr + TMEM_O + t * 128;
    // number of keys this row may see: bottom-right aligned causal mask, clipped to the sequence
    const int limit = p.is_causal ? max(0, min(lk, row + (lk - lq) + 1)) : lk;
    float m_run = neg_inf();     // running maximum (base-2 scaled logits)
    float m_used = 0.f;          // the maximum O and l are currently scaled with
    float l_run = 0.f;
    bool alive = true;
    for (int j = 0; j < nblk && alive; ++j) {
      alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(S_FULL0 + t), j & 1, status, 47));
      if (!alive) break;
      tc::tc_fence_after();
      uint32_t sv[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tc::tmem_ld32(s_addr + c * 32, sv[c]);
      tc::tmem_wait_ld();
      const int cnt = limit - j * 128;                         // visible keys of this block: [0, cnt)
      const bool full = __all_sync(0xffffffffu, cnt >= 128);
      float mx4[4] = {neg_inf(), neg_inf(), neg_inf(), neg_inf()};   // independent chains
      if (full) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[c][i]));
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < cnt) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[c][i]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m_run, mx * p.scale_log2);
      // O and l carry the scale 2^-m_used; it is moved only when the maximum grew by more than the
      // threshold (or when the first real value arrives after fully masked blocks)
      bool need = false;
      if (j == 0) {
        m_used = (m_new == neg_inf()) ? 0.f : m_new;
      } else {
        need = (m_new - m_used) > kRescaleThreshold || (m_run == neg_inf() && m_new != neg_inf());
      }
      m_run = m_new;
      if (__any_sync(0xffffffffu, need)) {
        // the previous P V of this tile must be complete before O is rescaled
        alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(PV_DONE0 + t), (j - 1) & 1, status, 48));
        if (!alive) break;
        const float m_next = need ? m_new : m_used;
        const float alpha = exp2f(m_used - m_next);
        m_used = m_next;
        l_run *= alpha;
        tc::tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t ov[32];
          tc::tmem_ld32(o_addr + c * 32, ov);
          tc::tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tc::tmem_st32(o_addr + c * 32, ov);
        }
      }
      // P = 2^(s * scale - m_used), written as bf16 pairs over the first 64 columns S came from
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = exp2f(fmaf(__uint_as_float(sv[c][2 * i]), p.scale_log2, -m_used));
          float p1 = exp2f(fmaf(__uint_as_float(sv[c][2 * i + 1]), p.scale_log2, -m_used));
          if (!full) {
            if (c * 32 + 2 * i >= cnt) p0 = 0.f;
            if (c * 32 + 2 * i + 1 >= cnt) p1 = 0.f;
          }
          rs4[i & 3] += p0 + p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
        tc::tmem_st16(s_addr + c * 16, pk);
      }
      l_run += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      tc::tmem_wait_st();
      tc::tc_fence_before();
      tc::mbar_arrive(bar(P_FULL0 + t));
    }

    // ---- epilogue ---------------------------------------------------------------------------
    bool have_o = nblk > 0 && alive;
    if (have_o) {
      have_o = __all_sync(0xffffffffu, tc::mbar_wait(bar(PV_DONE0 + t), (nblk - 1) & 1, status, 49));
      tc::tc_fence_after();
    }
    const bool row_ok = row < lq;
    const float inv = (l_run == 0.f || !have_o) ? 0.f : 1.f / l_run;
    __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.o) + (int64_t)(q0 + row) * p.o_stride_t + head * p.o_stride_h;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t ov[32];
      if (have_o) {
        tc::tmem_ld32(o_addr + c * 32, ov);
        tc::tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) ov[i] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(ov[q4 * 8 + 0]) * inv, __uint_as_float(ov[q4 * 8 + 1]) * inv);
          v.y = pack_bf16x2(__uint_as_float(ov[q4 * 8 + 2]) * inv, __uint_as_float(ov[q4 * 8 + 3]) * inv);
          v.z = pack_bf16x2(__uint_as_float(ov[q4 * 8 + 4]) * inv, __uint_as_float(ov[q4 * 8 + 5]) * inv);
          v.w = pack_bf16x2(__uint_as_float(ov[q4 * 8 + 6]) * inv, __uint_as_float(ov[q4 * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = v;
        }
      }
    }
    if (row_ok)
      p.lse[(int64_t)(q0 + row) * p.lse_stride_t + head * p.lse_stride_h] = inv == 0.f ? neg_inf() : (log2f(l_run) + m_used) * kLn2;
  }

  tc::tc_fence_before();
  __syncthreads();
  if (warp == 5) tc::tmem_dealloc(tmem, 512);
}

// ---- host side ----------------------------------------------------------------------------------
template <int D_QK>
static cudaError_t launch_fwd_tc(const DenseKernelParams& p, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                                 cudaStream_t stream) {
  using L = dft::Layout<D_QK>;
  auto kern = dense_fwd_tc_kernel<D_QK>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  dim3 grid((p.max_seqlen_q + 255) / 256, p.h_q, p.batch);
  kern<<<grid, 320, L::SMEM_BYTES, stream>>>(p, tq, tk, tv);
  return cudaGetLastError();
}

cudaError_t launch_dense_fwd_tc(const DenseKernelParams& p, cudaStream_t stream) {
  CUtensorMap tq, tk, tv;
  if (!tmah::make_map_thd(&tq, p.q, p.d_qk, p.h_q, p.total_q, p.q_stride_h, p.q_stride_t, 128)) return cudaErrorInvalidValue;
  if (!tmah::make_map_thd(&tk, p.k, p.d_qk, p.h_k, p.total_k, p.k_stride_h, p.k_stride_t, 128)) return cudaErrorInvalidValue;
  if (!tmah::make_map_thd(&tv, p.v, p.d_v, p.h_k, p.total_k, p.v_stride_h, p.v_stride_t, 128)) return cudaErrorInvalidValue;
  if (p.d_qk == 192) return launch_fwd_tc<192>(p, tq, tk, tv, stream);
  return launch_fwd_tc<128>(p, tq, tk, tv, stream);
}

cudaError_t set_status_mirror_dense_fwd(int* mapped_host_word) { return tc::set_status_mirror(mapped_host_word); }

cudaError_t read_dense_tc_status(int* host_status, bool reset) {
  cudaError_t e = cudaMemcpyFromSymbol(host_status, g_dense_tc_status, sizeof(int));
  if (e != cudaSuccess) return e;
  if (reset && *host_status != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_dense_tc_status, &zero, sizeof(int));
  }
  return e;
}

}  // namespace fmla
