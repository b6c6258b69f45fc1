// Dense variable-length MHA forward (bf16, head dims 192/128 and 128/128) for sm_100a on
// tcgen05 / TMA / tensor memory.
//
// One CTA = 128 query rows of one (sequence, head); keys are walked in blocks of 128.
//   warps 0-3, 6-9 softmax : two threads per query row (TMEM lane = row, 64 key columns each):
//                       S -> registers, mask, running max / sum (base 2), P (bf16) written back into
//                       the columns S came from, lazy rescale of O, final 1/l normalisation and stores
//   warp 4   TMA      : Q tile once; K and V blocks into a 2-stage ring (64-column chunks of
//                       [128 rows x 128 bytes], 128-byte swizzle), K and V with barriers of their own
//                       so that K is refilled right after S and V right after P V
//   warp 5   MMA      : S = Q K^T  (tcgen05.mma m128n128k16, both operands from shared memory)
//                       O += P V   (m128n128k16, P from tensor memory, V from shared memory MN-major)
// TMEM map (512 columns allocated): S/P buffer 0 = [0,128), buffer 1 = [128,256), O = [256,384).
// For M = 128 element (row r, col c) of a result sits in lane r, column c; the bf16 A operand in
// tensor memory holds k values (2c, 2c+1) of row r in the 32-bit column c of lane r.
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
enum Bar { Q_FULL = 0, K_FULL0, K_FULL1, K_EMPTY0, K_EMPTY1, V_FULL0, V_FULL1, V_EMPTY0, V_EMPTY1, S_FULL0, S_FULL1, P_FULL0, P_FULL1, PV_DONE, NUM_BARS };
constexpr int TMEM_S = 0, TMEM_O = 256;
constexpr float kRescaleThreshold = 8.0f;         // log2 units; below it O keeps its stale scale
template <int D_QK>
struct Layout {
  static constexpr int NCH = D_QK / 64;           // 64-column chunks of Q and K
  static constexpr int kQBytes = NCH * kChunkBytes;
  static constexpr int kStageBytes = kQBytes + kVBytes;   // K then V
  static constexpr int Q_OFF = 0;
  static constexpr int KV_OFF = kQBytes;
  static constexpr int BAR_OFF = KV_OFF + 2 * kStageBytes;
  static constexpr int XCH_OFF = BAR_OFF + 128;    // float [2][256]: row maxima / sums exchanged between the two threads of a row
  static constexpr int MISC_OFF = XCH_OFF + 2048;
  static constexpr int SMEM_BYTES = MISC_OFF + 16;
  static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared memory limit per CTA");
};
static_assert(NUM_BARS * 8 <= 128, "barrier area too small");
}  // namespace dft

__device__ int g_dense_tc_status = 0;

// Optional timeline of the first blocks of CTA (0,0,0), compiled in with -DFMLA_TRACE only.
#ifdef FMLA_TRACE
__device__ long long g_dense_trace[64 * 16];
#define DFT_TRACE_AT(blk, slot)                                                          \
  do {                                                                                     \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (blk) < 64) g_dense_trace[(blk) * 16 + (slot)] = clock64(); \
  } while (0)
#else
#define DFT_TRACE_AT(blk, slot) do {} while (0)
#endif

// The S = Q K^T instructions of one key block in stage ST (result into S buffer ST), as straight-line
// code whose descriptors are a warp-uniform base plus an immediate.
template <int ST, int D_QK>
__device__ __forceinline__ void dense_s_block(uint32_t tmem, uint64_t desc_q, uint64_t desc_k, uint32_t idesc) {
  using L = dft::Layout<D_QK>;
#pragma unroll
  for (int c = 0; c < L::NCH; ++c)
#pragma unroll
    for (int s = 0; s < 4; ++s)
      tc::mma_ss(tmem + dft::TMEM_S + ST * 128, tc::desc_advance(desc_q, c * dft::kChunkBytes + s * 32),
                 tc::desc_advance(desc_k, ST * L::kStageBytes + c * dft::kChunkBytes + s * 32), idesc, (c | s) ? 1u : 0u);
}
// O += P V of one key block: P from S buffer ST (8 columns per 16-token step), V from stage ST.
template <int ST, int D_QK>
__device__ __forceinline__ void dense_pv_block(uint32_t tmem, uint64_t desc_v, uint32_t idesc, bool first) {
  using L = dft::Layout<D_QK>;
#pragma unroll
  for (int s = 0; s < 8; ++s)
    tc::mma_ts(tmem + dft::TMEM_O, tmem + dft::TMEM_S + ST * 128 + s * 8, tc::desc_advance(desc_v, ST * L::kStageBytes + s * 2048), idesc,
               (first && s == 0) ? 0u : 1u);
}

// grid (ceil(max_seqlen_q/128), h_q, batch), 320 threads
template <int D_QK>
__global__ void __launch_bounds__(320, 1)
dense_fwd_tc_kernel(const __grid_constant__ DenseKernelParams p, const __grid_constant__ CUtensorMap tmap_q,
                    const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v) {
  using namespace dft;
  using L = Layout<D_QK>;
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase + L::Q_OFF, sKV = sbase + L::KV_OFF;
  auto bar = [&](int i) { return sbase + L::BAR_OFF + i * 8; };
  volatile uint32_t* sTmem = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFF);
  volatile int* sAbort = reinterpret_cast<volatile int*>(smem + L::MISC_OFF + 8);   // set by a softmax thread whose wait expired
  float* sXch = reinterpret_cast<float*>(smem + L::XCH_OFF);
  int* status = &g_dense_tc_status;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z, head = blockIdx.y, kv_head = head / (p.h_q / p.h_k);
  const int q0 = __ldg(p.cu_q + b), lq = __ldg(p.cu_q + b + 1) - q0;
  const int k0 = __ldg(p.cu_k + b), lk = __ldg(p.cu_k + b + 1) - k0;
  // with a causal mask the last tiles have the most keys: they are started first
  const int m_base = (gridDim.x - 1 - blockIdx.x) * 128;
  if (m_base >= lq) return;
  if ((sbase & 1023u) != 0) {   // the swizzled tiles need a 1024-byte aligned base
    if (tid == 0) atomicCAS(status, 0, 30);
    return;
  }
  int nblk = (lk + 127) >> 7;
  if (p.is_causal) {
    const int last_key = min(m_base + 127, lq - 1) + (lk - lq);   // inclusive
    nblk = last_key < 0 ? 0 : min(nblk, (last_key >> 7) + 1);
  }

  if (tid == 0) {
    tc::mbar_init(bar(Q_FULL), 1);
    for (int i = K_FULL0; i <= S_FULL1; ++i) tc::mbar_init(bar(i), 1);
    tc::mbar_init(bar(P_FULL0), 256);
    tc::mbar_init(bar(P_FULL1), 256);
    tc::mbar_init(bar(PV_DONE), 1);
    tc::fence_mbar_init();
    *sAbort = 0;
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
      tc::mbar_arrive_expect_tx(bar(Q_FULL), L::kQBytes);
#pragma unroll
      for (int c = 0; c < L::NCH; ++c) tc::tma_load_3d(sQ + c * kChunkBytes, &tmap_q, c * 64, head, q0 + m_base, bar(Q_FULL));
      bool alive = true;
      for (int j = 0; j < nblk && alive; ++j) {
        const int st = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        const uint32_t stage = sKV + st * L::kStageBytes;
        const int tok = k0 + j * 128;
        alive = tc::mbar_wait(bar(K_EMPTY0 + st), ph, status, 41);
        if (!alive) break;
        DFT_TRACE_AT(j, 0);
        tc::mbar_arrive_expect_tx(bar(K_FULL0 + st), L::kQBytes);
#pragma unroll
        for (int c = 0; c < L::NCH; ++c) tc::tma_load_3d(stage + c * kChunkBytes, &tmap_k, c * 64, kv_head, tok, bar(K_FULL0 + st));
        alive = tc::mbar_wait(bar(V_EMPTY0 + st), ph, status, 42);
        if (!alive) break;
        DFT_TRACE_AT(j, 1);
        tc::mbar_arrive_expect_tx(bar(V_FULL0 + st), kVBytes);
#pragma unroll
        for (int c = 0; c < 2; ++c) tc::tma_load_3d(stage + L::kQBytes + c * kChunkBytes, &tmap_v, c * 64, kv_head, tok, bar(V_FULL0 + st));
      }
    }
  } else if (warp == 5) {
    // ================================ MMA issuer =======================================
    constexpr uint32_t idesc_s = tc::idesc_bf16_f32(128, 128, 0, 0);
    constexpr uint32_t idesc_o = tc::idesc_bf16_f32(128, 128, 0, 1);
    const uint64_t desc_q = tc::smem_desc_sw128(sQ, 16, 1024);                          // A of S: K-major
    const uint64_t desc_k = tc::smem_desc_sw128(sKV, 16, 1024);                         // B of S: K-major (stage 0)
    const uint64_t desc_v = tc::smem_desc_sw128(sKV + L::kQBytes, kChunkBytes, 1024);   // B of PV: MN-major, 64-wide column groups 16 KB apart
    bool alive = nblk > 0;
    if (alive) alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(Q_FULL), 0, status, 43));
    // P V of one block; V rows past the end of the sequence belong to the next sequence (or are
    // the zero fill) and are cleared first, so that 0 * (Inf or NaN) cannot reach O
    auto issue_pv = [&](int j) {
      const int st = j & 1;
      alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(V_FULL0 + st), (j >> 1) & 1, status, 44));
      if (alive) alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(P_FULL0 + st), (j >> 1) & 1, status, 45));
      if (!alive) return;
      const int rows_valid = lk - j * 128;
      if (rows_valid < 128) {
        unsigned char* v = smem + L::KV_OFF + st * L::kStageBytes + L::kQBytes;
        const int nrows = 128 - rows_valid;
        for (int i = lane; i < nrows * 16; i += 32) {
          const int row = rows_valid + (i >> 4), c16 = i & 15;
          *reinterpret_cast<uint4*>(v + (c16 >> 3) * kChunkBytes + row * 128 + (c16 & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
        tc::fence_proxy_async_smem();
        __syncwarp();
      }
      tc::tc_fence_after();
      if (lane == 0) DFT_TRACE_AT(j, 4);
      if (tc::elect_one()) {
        if (st == 0) dense_pv_block<0, D_QK>(tmem, desc_v, idesc_o, j == 0);
        else dense_pv_block<1, D_QK>(tmem, desc_v, idesc_o, j == 0);
        tc::tc_commit(bar(V_EMPTY0 + st));
        tc::tc_commit(bar(PV_DONE));
        DFT_TRACE_AT(j, 5);
      }
      __syncwarp();
    };
    for (int j = 0; j < nblk && alive; ++j) {
      const int st = j & 1;
      alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(K_FULL0 + st), (j >> 1) & 1, status, 46));
      if (!alive) break;
      // the S buffer of this stage was last read as P by the P V of block j-2, issued earlier by
      // this thread: the tensor pipe runs them in order
      tc::tc_fence_after();
      if (lane == 0) DFT_TRACE_AT(j, 2);
      if (tc::elect_one()) {
        if (st == 0) dense_s_block<0, D_QK>(tmem, desc_q, desc_k, idesc_s);
        else dense_s_block<1, D_QK>(tmem, desc_q, desc_k, idesc_s);
        tc::tc_commit(bar(S_FULL0 + st));
        tc::tc_commit(bar(K_EMPTY0 + st));
        DFT_TRACE_AT(j, 3);
      }
      __syncwarp();
      if (j > 0) issue_pv(j - 1);
    }
    if (alive && nblk > 0) issue_pv(nblk - 1);
  } else {
    // ================================ softmax / epilogue ================================
    // Eight warps: warp w reads the TMEM lane quarter w % 4 (rows 32 (w % 4) ..), warps 0-3 the key
    // columns [0,64) of a block and warps 6-9 the columns [64,128).  The two threads of a row exchange
    // their maxima (and at the end their sums) through shared memory.
    const int ch = warp >= 6 ? 1 : 0;                          // column half
    const int rl = (warp & 3) * 32 + lane;                     // row within the tile = TMEM lane
    const int row = m_base + rl;                               // query row within its sequence
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    // number of keys this row may see: bottom-right aligned causal mask, clipped to the sequence
    const int limit = p.is_causal ? max(0, min(lk, row + (lk - lq) + 1)) : lk;
    float m_run = neg_inf();     // running maximum (base-2 scaled logits)
    float m_used = 0.f;          // the maximum O and l are currently scaled with
    float l_run = 0.f;           // this thread's share of the row sum
    bool aborted = false;        // uniform over the softmax threads: only read right after a bar_sync
    for (int j = 0; j < nblk && !aborted; ++j) {
      const int st = j & 1;
      const uint32_t s_addr = tmem + lane_addr + TMEM_S + st * 128;
      uint32_t sv[2][32];
      if (tc::mbar_wait(bar(S_FULL0 + st), (j >> 1) & 1, status, 47)) {
        if (tid == 0) DFT_TRACE_AT(j, 6);
        tc::tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; ++c) tc::tmem_ld32(s_addr + ch * 64 + c * 32, sv[c]);
        tc::tmem_wait_ld();
      } else {
        *sAbort = 1;
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) sv[c][i] = 0u;
      }
      if (tid == 0) DFT_TRACE_AT(j, 7);
      const int cnt = limit - j * 128 - ch * 64;               // visible keys among this thread's 64: [0, cnt)
      const bool full = __all_sync(0xffffffffu, cnt >= 64);
      float mx4[4] = {neg_inf(), neg_inf(), neg_inf(), neg_inf()};   // independent chains
      if (full) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[c][i]));
      } else {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < cnt) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[c][i]));
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      float* xch = sXch + (j & 1) * 256;
      xch[ch * 128 + rl] = mx;
      // after this barrier both threads of a row also hold all their S values in registers, so P may
      // overwrite the columns S came from
      bar_sync(1, 256);
      if (*sAbort) { aborted = true; break; }
      if (tid == 0) DFT_TRACE_AT(j, 8);
      mx = fmaxf(mx, xch[(ch ^ 1) * 128 + rl]);
      const float m_new = fmaxf(m_run, mx);
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
        // the previous P V must be complete before O is rescaled
        if (!tc::mbar_wait(bar(PV_DONE), (j - 1) & 1, status, 48)) *sAbort = 1;
        const float m_next = need ? m_new : m_used;
        const float alpha = exp2f(m_used - m_next);
        m_used = m_next;
        l_run *= alpha;
        tc::tc_fence_after();
        // each of the two warps of a lane quarter rescales its half of the O columns
#pragma unroll 1
        for (int c = ch * 2; c < ch * 2 + 2; ++c) {
          uint32_t ov[32];
          tc::tmem_ld32(tmem + lane_addr + TMEM_O + c * 32, ov);
          tc::tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tc::tmem_st32(tmem + lane_addr + TMEM_O + c * 32, ov);
        }
      }
      if (tid == 0) DFT_TRACE_AT(j, 9);
      // P = 2^(s * scale - m_used), written as bf16 pairs: key 64 ch + e of the block -> column 32 ch + e / 2
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 2; ++c) {
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
        tc::tmem_st16(s_addr + ch * 32 + c * 16, pk);
      }
      l_run += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      if (tid == 0) DFT_TRACE_AT(j, 10);
      tc::tmem_wait_st();
      tc::tc_fence_before();
      tc::mbar_arrive(bar(P_FULL0 + st));
      if (tid == 0) DFT_TRACE_AT(j, 11);
    }

    // ---- epilogue ---------------------------------------------------------------------------
    // row sum over the two threads of a row (the barriers on both sides keep this use of the
    // exchange buffer apart from the block loop)
    bar_sync(1, 256);
    sXch[ch * 128 + rl] = l_run;
    bar_sync(1, 256);
    if (*sAbort) aborted = true;
    const float l = l_run + sXch[(ch ^ 1) * 128 + rl];
    bool have_o = nblk > 0 && !aborted;
    if (have_o) {
      have_o = tc::mbar_wait(bar(PV_DONE), (nblk - 1) & 1, status, 49);
      tc::tc_fence_after();
    }
    have_o = __all_sync(0xffffffffu, have_o);
    const bool row_ok = row < lq;
    const float inv = (l == 0.f || !have_o) ? 0.f : 1.f / l;
    __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.o) + (int64_t)(q0 + row) * p.o_stride_t + head * p.o_stride_h;
#pragma unroll 1
    for (int c = ch * 2; c < ch * 2 + 2; ++c) {
      uint32_t ov[32];
      if (have_o) {
        tc::tmem_ld32(tmem + lane_addr + TMEM_O + c * 32, ov);
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
    if (row_ok && ch == 0)
      p.lse[(int64_t)(q0 + row) * p.lse_stride_t + head * p.lse_stride_h] = inv == 0.f ? neg_inf() : (log2f(l) + m_used) * kLn2;
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
  dim3 grid((p.max_seqlen_q + 127) / 128, p.h_q, p.batch);
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

#ifdef FMLA_TRACE
extern "C" int fmla_debug_read_dense_trace(long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_dense_trace, sizeof(long long) * n);
}
#endif

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
