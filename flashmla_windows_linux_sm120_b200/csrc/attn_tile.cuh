// One 64-row query tile of flash attention against a stream of 64-token KV
// blocks, shared by every forward kernel of the library.
//
// CTA = 256 threads = 8 warps.  Warp w owns query rows 16*(w&3) .. +15 and the
// half th = w>>2 of (a) the 64 tokens of a block for S = Q K^T and (b) the D_V
// output columns for O += P V.  The two warps of a row group exchange their row
// maxima and the bf16 probabilities through shared memory, so QK^T is computed
// once per row group.  K/V blocks are double-buffered with cp.async; tiles are
// XOR-swizzled (fmla_common.cuh).  Tensor-core work is mma.sync m16n8k16 bf16
// with fp32 accumulation; probabilities are rounded to bf16 before P V and the
// row sums are taken from the fp32 values, as the reference kernels do
// (csrc/sm90/decode/dense/splitkv_mla.cu:383-389).
//
// A `Prob` type supplies the addressing and masking of one use case:
//   void load_q(uint32_t sQ)                          issue cp.async for the Q tile
//   void load_kv_begin(int blk, int stage, uint32_t sK, uint32_t sV, int* sValid)
//   void load_kv_end(int stage, uint32_t sK, uint32_t sV)   (after the block's math)
//   bool needs_mask(int blk)
//   bool valid(int row, int blk, int tok, const int* sValid)  may (row, token tok of blk) attend?
#pragma once

#include "fmla_common.cuh"

namespace fmla {

template <int D_QK_, int D_V_, bool V_IS_K_>
struct TileCfg {
  static constexpr int D_QK = D_QK_;
  static constexpr int D_V = D_V_;
  static constexpr bool V_IS_K = V_IS_K_;
  static constexpr int BLOCK_M = 64;
  static constexpr int BLOCK_N = 64;
  static constexpr int NTHREADS = 256;
  static constexpr int QK_ROW_BYTES = D_QK * 2;
  static constexpr int V_ROW_BYTES = V_IS_K ? QK_ROW_BYTES : D_V * 2;
  static constexpr int Q_BYTES = BLOCK_M * QK_ROW_BYTES;
  static constexpr int K_BYTES = BLOCK_N * QK_ROW_BYTES;
  static constexpr int V_BYTES = V_IS_K ? 0 : BLOCK_N * D_V * 2;
  static constexpr int P_BYTES = BLOCK_M * BLOCK_N * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + Q_BYTES;          // 2 stages
  static constexpr int V_OFF = K_OFF + 2 * K_BYTES;      // 2 stages (absent when V aliases K)
  static constexpr int P_OFF = V_OFF + 2 * V_BYTES;
  static constexpr int MX_OFF = P_OFF + P_BYTES;         // float [2][64] row maxima / row sums exchange
  static constexpr int VALID_OFF = MX_OFF + 2 * 64 * 4;  // int [2][64] per-stage token validity
  static constexpr int SMEM_BYTES = VALID_OFF + 2 * 64 * 4;
  static constexpr int NT_O = (D_V / 2) / 8;             // 8-wide output n-tiles per warp
  static_assert(D_QK % 64 == 0 && D_V % 64 == 0, "row pitch must be a multiple of 128 bytes");
};

// Per-thread result of a tile: rows r0 = 16*(warp&3) + lane/4 and r0+8;
// o[nt][0..1] -> row r0, o[nt][2..3] -> row r0+8, columns
// (warp>>2)*(D_V/2) + nt*8 + 2*(lane&3) + {0,1}.  m is in base-2 scaled units,
// l is the full row sum (both token halves).
template <class Cfg>
struct TileAcc {
  float o[Cfg::NT_O][4];
  float m[2];
  float l[2];
};

template <class Cfg, class Prob>
__device__ __forceinline__ void run_tile(Prob& prob, char* smem, int blk_begin, int blk_end, float scale_log2,
                                         TileAcc<Cfg>& acc) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp & 3, th = warp >> 2;
  const int g = lane >> 2, t4 = lane & 3;
  const int r0 = rg * 16 + g;
  const uint32_t sQ = smem_u32(smem + Cfg::Q_OFF);
  const uint32_t sK0 = smem_u32(smem + Cfg::K_OFF);
  const uint32_t sV0 = Cfg::V_IS_K ? sK0 : smem_u32(smem + Cfg::V_OFF);
  const uint32_t sP = smem_u32(smem + Cfg::P_OFF);
  float* sMx = reinterpret_cast<float*>(smem + Cfg::MX_OFF);
  int* sValid = reinterpret_cast<int*>(smem + Cfg::VALID_OFF);
  constexpr int V_STAGE = Cfg::V_IS_K ? Cfg::K_BYTES : Cfg::V_BYTES;

#pragma unroll
  for (int i = 0; i < Cfg::NT_O; ++i) acc.o[i][0] = acc.o[i][1] = acc.o[i][2] = acc.o[i][3] = 0.f;
  acc.m[0] = acc.m[1] = neg_inf();
  acc.l[0] = acc.l[1] = 0.f;

  prob.load_q(sQ);
  if (blk_begin < blk_end) {
    prob.load_kv_begin(blk_begin, 0, sK0, sV0, sValid);
    prob.load_kv_end(0, sK0, sV0);
  }
  cp_async_commit();

  for (int blk = blk_begin; blk < blk_end; ++blk) {
    const int st = (blk - blk_begin) & 1;
    const uint32_t sK = sK0 + st * Cfg::K_BYTES;
    const uint32_t sV = sV0 + st * V_STAGE;
    cp_async_wait<0>();
    __syncthreads();
    const bool has_next = blk + 1 < blk_end;
    if (has_next) prob.load_kv_begin(blk + 1, st ^ 1, sK0 + (st ^ 1) * Cfg::K_BYTES, sV0 + (st ^ 1) * V_STAGE, sValid + (st ^ 1) * 64);
    cp_async_commit();

    // ---- S = Q K^T for rows rg*16.., tokens th*32.. ------------------------
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    {
      const int a_row = rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const int a_ch = lane >> 4;
      const int b_row = th * 32 + (lane & 7) + (lane >> 4) * 8;
      const int b_ch = (lane >> 3) & 1;
#pragma unroll 4
      for (int ks = 0; ks < Cfg::D_QK / 16; ++ks) {
        uint32_t a[4], b[4];
        ldmatrix_x4(sQ + swz_off(a_row, ks * 2 + a_ch, Cfg::QK_ROW_BYTES), a);
        ldmatrix_x4(sK + swz_off(b_row, ks * 2 + b_ch, Cfg::QK_ROW_BYTES), b);
        mma_bf16_16816(s[0], a, b[0], b[1]);
        mma_bf16_16816(s[1], a, b[2], b[3]);
        ldmatrix_x4(sK + swz_off(b_row + 16, ks * 2 + b_ch, Cfg::QK_ROW_BYTES), b);
        mma_bf16_16816(s[2], a, b[0], b[1]);
        mma_bf16_16816(s[3], a, b[2], b[3]);
      }
    }

    // ---- mask, online softmax ----------------------------------------------
    if (prob.needs_mask(blk)) {
      const int* vflags = sValid + st * 64;
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = th * 32 + j * 8 + 2 * t4 + (e & 1);
          const int row = r0 + (e >> 1) * 8;
          if (!prob.valid(row, blk, tok, vflags)) s[j][e] = neg_inf();
        }
    }
    float mx[2] = {neg_inf(), neg_inf()};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    if (t4 == 0) {
      sMx[th * 64 + r0] = mx[0];
      sMx[th * 64 + r0 + 8] = mx[1];
    }
    bar_sync(1 + rg, 64);
    float alpha[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float other = sMx[(th ^ 1) * 64 + r0 + h * 8];
      const float m_new = fmaxf(acc.m[h], fmaxf(mx[h], other) * scale_log2);
      m_use[h] = (m_new == neg_inf()) ? 0.f : m_new;
      alpha[h] = exp2f(acc.m[h] - m_use[h]);
      acc.m[h] = m_new;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float p0 = exp2f(s[j][0] * scale_log2 - m_use[0]);
      const float p1 = exp2f(s[j][1] * scale_log2 - m_use[0]);
      const float p2 = exp2f(s[j][2] * scale_log2 - m_use[1]);
      const float p3 = exp2f(s[j][3] * scale_log2 - m_use[1]);
      rs[0] += p0 + p1;
      rs[1] += p2 + p3;
      const int ch = th * 4 + j;
      uint32_t* d0 = reinterpret_cast<uint32_t*>(smem + Cfg::P_OFF + swz_off(r0, ch, 128) + t4 * 4);
      uint32_t* d1 = reinterpret_cast<uint32_t*>(smem + Cfg::P_OFF + swz_off(r0 + 8, ch, 128) + t4 * 4);
      *d0 = pack_bf16x2(p0, p1);
      *d1 = pack_bf16x2(p2, p3);
    }
    acc.l[0] = acc.l[0] * alpha[0] + rs[0];
    acc.l[1] = acc.l[1] * alpha[1] + rs[1];
#pragma unroll
    for (int i = 0; i < Cfg::NT_O; ++i) {
      acc.o[i][0] *= alpha[0];
      acc.o[i][1] *= alpha[0];
      acc.o[i][2] *= alpha[1];
      acc.o[i][3] *= alpha[1];
    }
    bar_sync(1 + rg, 64);

    // ---- O += P V for rows rg*16.., output columns th*D_V/2.. ----------------
    {
      const int a_row = rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const int a_ch = lane >> 4;
      const int v_row = ((lane >> 3) & 1) * 8 + (lane & 7);
      const int v_ch = th * (Cfg::D_V / 16) + (lane >> 4);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(sP + swz_off(a_row, kk * 2 + a_ch, 128), a);
#pragma unroll
        for (int n2 = 0; n2 < Cfg::NT_O / 2; ++n2) {
          uint32_t b[4];
          ldmatrix_x4_trans(sV + swz_off(kk * 16 + v_row, v_ch + n2 * 2, Cfg::V_ROW_BYTES), b);
          mma_bf16_16816(acc.o[n2 * 2], a, b[0], b[1]);
          mma_bf16_16816(acc.o[n2 * 2 + 1], a, b[2], b[3]);
        }
      }
    }
    if (has_next) prob.load_kv_end(st ^ 1, sK0 + (st ^ 1) * Cfg::K_BYTES, sV0 + (st ^ 1) * V_STAGE);
  }
  cp_async_wait<0>();

  // Row sums were accumulated per token half: add the partner's.
  __syncthreads();
  // the per-thread partial sums differ between the 4 lanes of a quad (each saw
  // different tokens): reduce over the quad first
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    acc.l[h] += __shfl_xor_sync(0xffffffffu, acc.l[h], 1);
    acc.l[h] += __shfl_xor_sync(0xffffffffu, acc.l[h], 2);
  }
  if (t4 == 0) {
    sMx[th * 64 + r0] = acc.l[0];
    sMx[th * 64 + r0 + 8] = acc.l[1];
  }
  __syncthreads();
  acc.l[0] += sMx[(th ^ 1) * 64 + r0];
  acc.l[1] += sMx[(th ^ 1) * 64 + r0 + 8];
  __syncthreads();
}

// Cooperative cp.async of a [64 x ROW_ELEMS] bf16 tile: thread -> row tid/4,
// 16-byte chunks (tid&3) + 4*i.  `src_row` is the global address of the row or
// nullptr (zero fill).
template <int ROW_ELEMS>
__device__ __forceinline__ void load_rows_async(uint32_t sdst, const __nv_bfloat16* src_row, const void* safe_ptr) {
  constexpr int CHUNKS = ROW_ELEMS / 8;
  static_assert(CHUNKS % 4 == 0, "");
  const int row = threadIdx.x >> 2, c0 = threadIdx.x & 3;
  const bool ok = src_row != nullptr;
  const char* base = ok ? reinterpret_cast<const char*>(src_row) : reinterpret_cast<const char*>(safe_ptr);
#pragma unroll
  for (int i = 0; i < CHUNKS / 4; ++i) {
    const int c = c0 + 4 * i;
    cp_async16(sdst + swz_off(row, c, ROW_ELEMS * 2), ok ? base + c * 16 : base, ok);
  }
}

}  // namespace fmla
