// MLA attention for sm_100a on tcgen05 / TMA / tensor memory: one kernel skeleton, three uses
//   kDense         dense BF16 split-KV decode over a paged cache (pages loaded by TMA)
//   kSparseDecode  sparse FP8 split-KV decode: top-k slot indices, 656-byte records gathered and
//                  de-quantised to bf16 in shared memory by eight producer warps
//   kSparsePrefill sparse prefill forward: top-k row indices into kv[s_kv, 576], rows gathered with
//                  cp.async by eight producer warps
//
// One CTA = the 64-head tile of one query token.
//   warps 0-3 softmax : TMEM S -> registers, mask, running max / sum (base 2), P (bf16) -> shared
//                       memory, lazy rescale of O in TMEM, final 1/l normalisation and stores
//   warp 4   TMA      : Q tile (9 boxes of 64 rows x 64 cols); in kDense also one 64-token page per
//                       step (9 boxes) into a 2-stage ring, plus L2 prefetch of later pages
//   warp 5   MMA      : S = Q K^T  (36 x tcgen05.mma.ws m64n64k16)  -> TMEM S[stage]
//                       O += P V   ( 8 x tcgen05.mma.ws m64n256k16) -> TMEM O
//                       V is the first 512 columns of the same K tile, read MN-major
//   warps 6-13 gather : sparse modes only; write K rows in exactly the layout TMA produces
//                       (64-column chunks of 128-byte rows, 128-byte swizzle), so the MMA side is
//                       the same for all three uses
// TMEM map (512 columns allocated): O = [0,256) (two N=256 halves of 128 columns),
// S[0] = [256,288), S[1] = [288,320).  In the M=64 weight-stationary layout element
// (row r, col c) of an N-wide result sits in lane r + 64*(c >= N/2), column c % (N/2).
//
// Semantics follow the reference kernels: decode borders / split outputs / LSE conventions
// csrc/sm90/decode/dense/splitkv_mla.cu:948-957, 1022-1042, 1237-1269; sparse decode
// csrc/sm100/decode/sparse_fp8/splitkv_mla.cu:168-186, 217-256; sparse prefill
// csrc/sm100/prefill/sparse/fwd.cu:399-417, 438-445, 677-679; FP8 record README.md:162-170 with
// de-quantisation bf16(fp32(e4m3) * scale) as tests/quant.py:60-63.
// Every mbarrier wait is bounded (tc_common.cuh); a pipeline fault sets a status word and lets the
// CTA drain and free its tensor memory.
#include "kernels.h"
#include "mla_work.cuh"
#include "tc_common.cuh"

#include <cuda.h>
#include <cuda_fp8.h>

#include <cstdlib>

namespace fmla {

namespace dtc {
constexpr int kChunkBytes = 64 * 128;             // [64 rows x 64 bf16], 128-byte rows
constexpr int kTileBytes = 9 * kChunkBytes;       // 64 x 576 bf16
constexpr int Q_OFF = 0;
constexpr int KV_OFF = kTileBytes;                // 2 stages
constexpr int P_OFF = 3 * kTileBytes;             // [64 x 64] bf16
constexpr int BAR_OFF = P_OFF + kChunkBytes;      // mbarriers
constexpr int MX_OFF = BAR_OFF + 128;             // float [3][128] exchange (2 for row maxima, 1 for row sums)
constexpr int MISC_OFF = MX_OFF + 1536;           // tmem base, abort flag, token validity masks
constexpr int SMEM_BYTES = MISC_OFF + 64;         // misc words
enum Bar { Q_FULL = 0, Q_EMPTY, KV_FULL0, KV_FULL1, KV_EMPTY0, KV_EMPTY1, S_FULL0, S_FULL1, S_EMPTY0, S_EMPTY1, P_FULL, P_EMPTY, O_FULL, O_EMPTY, NUM_BARS };
constexpr int TMEM_O = 0, TMEM_S = 256;
static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared memory limit per CTA");
static_assert(NUM_BARS * 8 <= 128, "barrier area too small");
#ifndef FMLA_PREFETCH_DIST
#define FMLA_PREFETCH_DIST 6
#endif
constexpr int kPrefetchDist = FMLA_PREFETCH_DIST; // cache pages prefetched into L2 ahead of the stage loads
constexpr float kRescaleThreshold = 8.0f;         // log2 units; below it O keeps its stale scale
constexpr int kGatherThreadsDecode = 256;         // sparse decode: 8 gather warps
constexpr int kGatherThreadsPrefill = 256;        // sparse prefill: 8 gather warps
}  // namespace dtc

__device__ int g_decode_tc_status = 0;

// Optional timeline of the first blocks of CTA (0,0,0), compiled in with -DFMLA_TRACE only.
#ifdef FMLA_TRACE
__device__ long long g_decode_trace[64 * 16];
#define FMLA_TRACE_AT(blk, slot)                                                          \
  do {                                                                                     \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (blk) < 64) g_decode_trace[(blk) * 16 + (slot)] = clock64(); \
  } while (0)
#else
#define FMLA_TRACE_AT(blk, slot) do {} while (0)
#endif

// 16-byte chunk c16 (0..71) of row r of a stage -> byte offset in the TMA-compatible layout
__device__ __forceinline__ uint32_t stage_off(int r, int c16) {
  return static_cast<uint32_t>((c16 >> 3) * dtc::kChunkBytes + r * 128 + (((c16 & 7) ^ (r & 7)) << 4));
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// even-lane bits of a ballot (lanes 0,2,..,30) packed into 16 bits
__device__ __forceinline__ uint32_t compress_even_bits(uint32_t m) {
  m &= 0x55555555u;
  m = (m | (m >> 1)) & 0x33333333u;
  m = (m | (m >> 2)) & 0x0f0f0f0fu;
  m = (m | (m >> 4)) & 0x00ff00ffu;
  m = (m | (m >> 8)) & 0x0000ffffu;
  return m;
}

// The 36 S = Q K^T instructions of one block in stage ST, as straight-line code whose descriptors are
// a warp-uniform base plus an immediate.  (Two unrolled copies, one per stage, still fit the instruction cache
// here and were measured faster than one copy with a run-time stage base: 686 vs 641 TFLOP/s on the sparse prefill.)
template <int ST>
__device__ __forceinline__ void s_block(uint32_t tmem, uint64_t desc_q, uint64_t desc_k, uint32_t idesc) {
  using namespace dtc;
#pragma unroll
  for (int c = 0; c < 9; ++c)
#pragma unroll
    for (int s = 0; s < 4; ++s)
      tc::mma_ws_ss(tmem + TMEM_S + ST * 32, tc::desc_advance(desc_q, c * kChunkBytes + s * 32),
                    tc::desc_advance(desc_k, ST * kTileBytes + c * kChunkBytes + s * 32), idesc, (c | s) ? 1u : 0u);
}

// grid: kDense (s_q*ceil(hq_per_hk/64), h_k, parts), 192 threads;
//       kSparseDecode (ceil(h_q/64), s_q, parts), 448 threads; kSparsePrefill (h_q/64, min(s_q, SMs / (h_q/64))) persistent over the query tokens, 448 threads
template <int MODE, bool F16>
__global__ void __launch_bounds__(MODE == kDense ? 192 : 448, 1)
mla_tc_kernel(const __grid_constant__ TcParams P, const __grid_constant__ CUtensorMap tmap_q,
              const __grid_constant__ CUtensorMap tmap_kv) {
  using namespace dtc;
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase + Q_OFF, sKV = sbase + KV_OFF, sP = sbase + P_OFF;
  auto bar = [&](int i) { return sbase + BAR_OFF + i * 8; };
  float* sMx = reinterpret_cast<float*>(smem + MX_OFF);
  volatile uint32_t* sTmem = reinterpret_cast<volatile uint32_t*>(smem + MISC_OFF);
  volatile int* sAbort = reinterpret_cast<volatile int*>(smem + MISC_OFF + 8);   // set by a softmax thread whose wait expired
  volatile uint32_t* sValid = reinterpret_cast<volatile uint32_t*>(smem + MISC_OFF + 16);   // [stage][token half]: 32 validity bits
  int* status = &g_decode_tc_status;
  const DecodeKernelParams& p = P.d;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const Tile tile = make_tile<MODE>(P);
  if (tile.n_work == 0) return;
  if ((sbase & 1023u) != 0) {   // the swizzled tiles need a 1024-byte aligned base
    if (tid == 0) tc::report_status(status, 30);
    return;
  }
  const float scale_log2 = MODE == kSparsePrefill ? P.sp.scale_log2 : p.scale_log2;
  // arrivals per filled stage: one (with a byte count) from the TMA thread, or one per gather thread
  constexpr int kKvFullCount = MODE == kDense ? 1 : (MODE == kSparseDecode ? kGatherThreadsDecode : kGatherThreadsPrefill + kGatherThreadsPrefill / 32);

  if (tid == 0) {
    tc::mbar_init(bar(Q_FULL), 1);
    tc::mbar_init(bar(Q_EMPTY), 1);
    tc::mbar_init(bar(KV_FULL0), kKvFullCount);
    tc::mbar_init(bar(KV_FULL1), kKvFullCount);
    tc::mbar_init(bar(KV_EMPTY0), 1);
    tc::mbar_init(bar(KV_EMPTY1), 1);
    tc::mbar_init(bar(S_FULL0), 1);
    tc::mbar_init(bar(S_FULL1), 1);
    tc::mbar_init(bar(S_EMPTY0), 128);
    tc::mbar_init(bar(S_EMPTY1), 128);
    tc::mbar_init(bar(P_FULL), 128);
    tc::mbar_init(bar(P_EMPTY), 1);
    tc::mbar_init(bar(O_FULL), 1);
    tc::mbar_init(bar(O_EMPTY), 128);
    tc::fence_mbar_init();
    *sAbort = 0;
  }
  if (warp == 5) tc::tmem_alloc(sbase + MISC_OFF, 512);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *sTmem;
  if constexpr (MODE != kSparsePrefill) pdl_allow_dependents();   // the merge kernel may become resident now

  if (warp == 4) {
    // ================================ TMA producer =====================================
    if (tc::elect_one()) {
      tc::prefetch_tensormap(&tmap_q);
      if constexpr (MODE == kDense) tc::prefetch_tensormap(&tmap_kv);
      int g = 0, req = 0;
      bool alive = true;
#ifdef FMLA_STAGGER_NS
      if constexpr (MODE == kDense) {
        if (blockIdx.z & 1) { const long long t0 = clock64(); while (clock64() - t0 < FMLA_STAGGER_NS) {} }
      }
#endif
      for (int wi = 0; wi < tile.n_work && alive; ++wi) {
        const Work r = get_work<MODE>(P, tile, wi);
        if (r.blk_hi == r.blk_lo) continue;
        alive = tc::mbar_wait(bar(Q_EMPTY), (req & 1) ^ 1, status, 1);
        if (!alive) break;
        tc::mbar_arrive_expect_tx(bar(Q_FULL), kTileBytes);
#pragma unroll
        for (int c = 0; c < 9; ++c)
          tc::tma_load_4d(sQ + c * kChunkBytes, &tmap_q, c * 64, tile.head0, MODE == kSparsePrefill ? r.batch : tile.sq, MODE == kSparsePrefill ? 0 : r.batch, bar(Q_FULL));
        if constexpr (MODE == kDense) {
          const int* bt = p.block_table + r.batch * p.block_table_stride_b;
          // pages kPrefetchDist steps ahead are pulled into L2 while the two shared-memory stages are
          // busy, so that the load that later fills a stage sees L2 latency instead of HBM latency
          for (int blk = r.blk_lo; blk < min(r.blk_lo + kPrefetchDist, r.blk_hi); ++blk) {
            const int pg = __ldg(bt + blk);
#pragma unroll
            for (int c = 0; c < 9; ++c) tc::tma_prefetch_l2_4d(&tmap_kv, c * 64, tile.kh, 0, pg);
          }
          int page_next = __ldg(bt + r.blk_lo);
          for (int blk = r.blk_lo; blk < r.blk_hi; ++blk, ++g) {
            const int st = g & 1;
            const int page = page_next;
            if (blk + 1 < r.blk_hi) page_next = __ldg(bt + blk + 1);
            if (blk + kPrefetchDist < r.blk_hi) {
              const int pg = __ldg(bt + blk + kPrefetchDist);
#pragma unroll
              for (int c = 0; c < 9; ++c) tc::tma_prefetch_l2_4d(&tmap_kv, c * 64, tile.kh, 0, pg);
            }
            alive = tc::mbar_wait(bar(KV_EMPTY0 + st), ((g >> 1) & 1) ^ 1, status, 2);
            if (!alive) break;
            FMLA_TRACE_AT(g, 0);
            tc::mbar_arrive_expect_tx(bar(KV_FULL0 + st), kTileBytes);
#pragma unroll
            for (int c = 0; c < 9; ++c)
              tc::tma_load_4d(sKV + st * kTileBytes + c * kChunkBytes, &tmap_kv, c * 64, tile.kh, 0, page, bar(KV_FULL0 + st));
            FMLA_TRACE_AT(g, 1);
          }
        }
        ++req;
      }
    }
  } else if (warp >= 6) {
    // ================================ gather producers (sparse modes) ==================
    if constexpr (MODE == kSparsePrefill) {
      // Eight gather warps, eight rows each, all on the same block.  For each row the 32 lanes copy
      // consecutive 16-byte pieces (pieces lane, lane+32 and, for 8 lanes, lane+64 of the 72):
      // coalesced cp.async with a handful of address instructions per row.
      const int gw = warp - 6;
      const char* kv = reinterpret_cast<const char*>(P.sp.kv);
      const int64_t row_bytes = P.sp.kv_stride_s * 2;
      const uint32_t lane_base = static_cast<uint32_t>((lane >> 3) * kChunkBytes);
      const int sw = lane & 7;
      int g = 0;
      bool alive = true;
      for (int wi = 0; wi < tile.n_work && alive; ++wi) {
        const Work r = get_work<MODE>(P, tile, wi);
        for (int blk = r.blk_lo; blk < r.blk_hi && alive; ++blk, ++g) {
          const int st = g & 1;
          int my_idx = __ldg(r.idx + blk * 64 + gw * 8 + (lane & 7));
          if (my_idx < 0 || my_idx >= P.sp.s_kv) my_idx = -1;
          alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(KV_EMPTY0 + st), ((g >> 1) & 1) ^ 1, status, 11));
          if (!alive) break;
          if (lane == 0 && gw == 0) FMLA_TRACE_AT(g, 0);
          const uint32_t bal = __ballot_sync(0xffffffffu, my_idx >= 0) & 0xffu;
          if (lane == 0) reinterpret_cast<volatile uint8_t*>(sValid)[st * 8 + gw] = static_cast<uint8_t>(bal);   // tokens 8*gw ..
          const uint32_t stage = sKV + st * kTileBytes + lane_base;
#pragma unroll
          for (int rr = 0; rr < 8; ++rr) {
            const int idx = __shfl_sync(0xffffffffu, my_idx, rr);
            const bool ok = idx >= 0;
            const int row = gw * 8 + rr;                  // row & 7 == rr
            const char* src = kv + (ok ? (int64_t)idx * row_bytes + lane * 16 : 0);
            const uint32_t dst = stage + row * 128 + ((sw ^ rr) << 4);
            cp_async16(dst, src, ok);
            cp_async16(dst + 4 * kChunkBytes, src + (ok ? 512 : 0), ok);
            if (lane < 8) cp_async16(dst + 8 * kChunkBytes, src + (ok ? 1024 : 0), ok);
          }
          // No thread waits for its own copies: the stage barrier counts one arrival per gather thread that the
          // hardware performs when that thread's copies have landed, so the warp goes on to the next block at once
          // and the L2 round trips of several blocks overlap.  Lane 0 adds one ordinary arrival after its store of
          // the validity bits.  The issuing thread makes the landed data visible to the tensor pipe (proxy fence).
#ifdef FMLA_PREFILL_SYNC_GATHER
          cp_async_commit();
          cp_async_wait<0>();
          tc::fence_proxy_async_smem();
          tc::mbar_arrive(bar(KV_FULL0 + st));
          if (lane == 0) tc::mbar_arrive(bar(KV_FULL0 + st));
#else
          asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar(KV_FULL0 + st)) : "memory");
          if (lane == 0) tc::mbar_arrive(bar(KV_FULL0 + st));
#endif
          if (lane == 0 && gw == 0) FMLA_TRACE_AT(g, 1);
        }
      }
    } else if constexpr (MODE == kSparseDecode) {
      // Eight gather warps, eight records each.  For one record the 32 lanes read the 32 chunks of
      // e4m3 values (512 contiguous bytes), their tile's scale, and 8 lanes the bf16 rope part.  The
      // raw bytes of the next block are fetched into registers before the wait for the stage to
      // drain, so their latency overlaps that wait.
      const int gw = warp - 6;
      const unsigned char* cache = reinterpret_cast<const unsigned char*>(p.kcache);
      uint4 nope[8], rope[8];
      float scl[8];
      int my_slot = -1;             // lanes 0..7: slot of row 8*gw + lane of the fetched block
      auto fetch = [&](const Work& r, int blk) {
        my_slot = __ldg(r.idx + blk * 64 + gw * 8 + (lane & 7));
        if (p.indices_logical) {
          // token position of the request -> physical slot through its block table
          const int pos = my_slot;
          my_slot = -1;
          if (pos >= 0 && pos < __ldg(p.seqlens_k + r.batch))
            my_slot = __ldg(p.block_table + r.batch * p.block_table_stride_b + (pos >> 6)) * 64 + (pos & 63);
        }
        if (my_slot < 0 || my_slot >= p.num_blocks * 64) my_slot = -1;
#pragma unroll
        for (int rr = 0; rr < 8; ++rr) {
          const int slot = __shfl_sync(0xffffffffu, my_slot, rr);
          nope[rr] = make_uint4(0, 0, 0, 0);
          rope[rr] = make_uint4(0, 0, 0, 0);
          scl[rr] = 0.f;
          if (slot >= 0) {
            const unsigned char* rec = cache + (int64_t)(slot >> 6) * p.k_stride_block + (slot & 63) * p.k_stride_row;
            nope[rr] = __ldg(reinterpret_cast<const uint4*>(rec) + lane);
            scl[rr] = __ldg(reinterpret_cast<const float*>(rec + 512) + (lane >> 3));
            if (lane < 8) rope[rr] = __ldg(reinterpret_cast<const uint4*>(rec + 528) + lane);
          }
        }
      };
      int g = 0;
      bool alive = true;
      int wi = 0;
      Work r = get_work<MODE>(P, tile, 0);
      while (wi < tile.n_work && r.blk_hi == r.blk_lo) { ++wi; if (wi < tile.n_work) r = get_work<MODE>(P, tile, wi); }
      int blk = r.blk_lo;
      if (wi < tile.n_work) fetch(r, blk);
      while (wi < tile.n_work && alive) {
        const int st = g & 1;
        alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(KV_EMPTY0 + st), ((g >> 1) & 1) ^ 1, status, 12));
        if (!alive) break;
        if (gw == 0 && lane == 0) FMLA_TRACE_AT(g, 0);
        const uint32_t stage = sKV + st * kTileBytes;
#pragma unroll
        for (int rr = 0; rr < 8; ++rr) {
          const int row = gw * 8 + rr;
          const float scale = scl[rr];
          const uint32_t w[4] = {nope[rr].x, nope[rr].y, nope[rr].z, nope[rr].w};
          uint32_t o[8];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // 4 e4m3 bytes -> 4 floats (exact), * scale in fp32, round to bf16
            const __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[k] & 0xffffu), __NV_E4M3);
            const __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[k] >> 16), __NV_E4M3);
            const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
            const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
            o[k * 2] = pack_bf16x2(f01.x * scale, f01.y * scale);
            o[k * 2 + 1] = pack_bf16x2(f23.x * scale, f23.y * scale);
          }
          st_shared_v4(stage + stage_off(row, lane * 2), make_uint4(o[0], o[1], o[2], o[3]));
          st_shared_v4(stage + stage_off(row, lane * 2 + 1), make_uint4(o[4], o[5], o[6], o[7]));
          if (lane < 8) st_shared_v4(stage + stage_off(row, 64 + lane), rope[rr]);
        }
        const uint32_t bal = __ballot_sync(0xffffffffu, my_slot >= 0) & 0xffu;
        if (lane == 0) reinterpret_cast<volatile uint8_t*>(sValid)[st * 8 + gw] = static_cast<uint8_t>(bal);   // tokens 8*gw ..
        tc::fence_proxy_async_smem();
        tc::mbar_arrive(bar(KV_FULL0 + st));
        if (gw == 0 && lane == 0) FMLA_TRACE_AT(g, 1);
        ++g;
        // advance to the next block (possibly of the next work item) and fetch it
        ++blk;
        while (wi < tile.n_work && blk >= r.blk_hi) {
          ++wi;
          if (wi < tile.n_work) { r = get_work<MODE>(P, tile, wi); blk = r.blk_lo; }
        }
        if (wi < tile.n_work) fetch(r, blk);
      }
    }
  } else if (warp == 5) {
    // ================================ MMA issuer =======================================
    constexpr uint32_t idesc_s = tc::idesc_bf16_f32(64, 64, 0, 0, F16);
    constexpr uint32_t idesc_o = tc::idesc_bf16_f32(64, 256, 0, 1, F16);
    // descriptors of the operand bases; per-MMA addresses are constant offsets added to the low word
    const uint64_t desc_q = tc::smem_desc_sw128(sQ, 16, 1024);             // A of S: K-major
    const uint64_t desc_k = tc::smem_desc_sw128(sKV, 16, 1024);            // B of S: K-major (stage 0)
    const uint64_t desc_p = tc::smem_desc_sw128(sP, 16, 1024);             // A of PV: K-major
    const uint64_t desc_v = tc::smem_desc_sw128(sKV, kChunkBytes, 1024);   // B of PV: MN-major, 64-wide column groups 8 KB apart
    int g = 0, req = 0;
    bool alive = true;
    // both issue helpers are called by the whole warp; one elected thread issues
    auto issue_pv = [&](int gi, bool first_of_request) {
      const int st = gi & 1;
      tc::tc_fence_after();
      if (lane == 0) FMLA_TRACE_AT(gi, 4);
      // elect.sync (not a lane-id test) selects the issuing thread: only then does the compiler keep
      // the descriptors in uniform registers, which halves the per-instruction issue cost
      if (tc::elect_one()) {
        // the stage index is resolved by a branch so that every descriptor below is a warp-uniform
        // base plus an immediate
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (st == 0) {
#pragma unroll
            for (int s = 0; s < 4; ++s)
              tc::mma_ws_ss(tmem + TMEM_O + h * 128, tc::desc_advance(desc_p, s * 32),
                            tc::desc_advance(desc_v, h * 4 * kChunkBytes + s * 2048), idesc_o, (first_of_request && s == 0) ? 0u : 1u);
          } else {
#pragma unroll
            for (int s = 0; s < 4; ++s)
              tc::mma_ws_ss(tmem + TMEM_O + h * 128, tc::desc_advance(desc_p, s * 32),
                            tc::desc_advance(desc_v, kTileBytes + h * 4 * kChunkBytes + s * 2048), idesc_o, (first_of_request && s == 0) ? 0u : 1u);
          }
        }
        tc::tc_commit(bar(KV_EMPTY0 + st));
        tc::tc_commit(bar(P_EMPTY));
        FMLA_TRACE_AT(gi, 5);
      }
      __syncwarp();
    };
    // rows of the last page beyond the sequence may hold anything (NaN included): zero them so
    // that 0 * garbage cannot reach O through P V
    auto zero_tail_rows = [&](int st, int rows_valid) {
      if (rows_valid < 64) {
        unsigned char* stage = smem + KV_OFF + st * kTileBytes;
        const int nrows = 64 - rows_valid;
        for (int i = lane; i < nrows * 72; i += 32) {
          const int row = rows_valid + i / 72, c16 = i % 72;
          *reinterpret_cast<uint4*>(stage + (c16 >> 3) * kChunkBytes + row * 128 + (c16 & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
        tc::fence_proxy_async_smem();
        __syncwarp();
      }
    };
    for (int wi = 0; wi < tile.n_work && alive; ++wi) {
      const Work r = get_work<MODE>(P, tile, wi);
      const int nblk = r.blk_hi - r.blk_lo;
      if (nblk == 0) continue;
      alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(Q_FULL), req & 1, status, 5));
      // S of block js and P V of block jp < js are issued in whichever order their inputs become
      // ready; P V goes first when both are possible: it releases a cache stage and the next load
      // depends on that.  One poll reads all barriers of interest at once, one per lane, and a ballot
      // shares the result:  lane 0 P_FULL(jp)   lane 1 O_EMPTY   lane 2 S_EMPTY(js)   lane 3 KV_FULL(js)
      // The S instructions of a block are issued from one straight-line site per stage (splitting
      // them into several separately issued groups more than doubled the time of S: the tensor
      // pipe drains in every gap).
      int js = 0, jp = 0, idle = 0;
      while (jp < nblk && alive) {
        const int gi = g + min(js, nblk - 1), st = gi & 1;
        const uint32_t ph = (gi >> 1) & 1;
        int pb = P_FULL;
        uint32_t pp = (g + jp) & 1;
        if (lane == 1) { pb = O_EMPTY; pp = (req & 1) ^ 1; }
        if (lane == 2) { pb = S_EMPTY0 + st; pp = ph ^ 1; }
        if (lane >= 3) { pb = KV_FULL0 + st; pp = ph; }
        const bool hit = lane < 4 && tc::mbar_test_wait(bar(pb), pp);
        const uint32_t m = __ballot_sync(0xffffffffu, hit);
        bool did = false;
        if (jp < js && (m & 1u) && (jp > 0 || (m & 2u))) {
          issue_pv(g + jp, jp == 0);
          ++jp;
          did = true;
        } else if (js < nblk && (m & 0xcu) == 0xcu) {
          if constexpr (MODE == kDense) zero_tail_rows(st, r.seqlen - (r.blk_lo + js) * 64);
          if constexpr (MODE == kSparsePrefill) tc::fence_proxy_async_smem();   // rows written by cp.async -> tensor pipe
          tc::tc_fence_after();
          if (lane == 0) FMLA_TRACE_AT(gi, 2);
          if (tc::elect_one()) {
            if (st == 0) s_block<0>(tmem, desc_q, desc_k, idesc_s);
            else s_block<1>(tmem, desc_q, desc_k, idesc_s);
            tc::tc_commit(bar(S_FULL0 + st));
            FMLA_TRACE_AT(gi, 3);
            if (js == nblk - 1) tc::tc_commit(bar(Q_EMPTY));
          }
          __syncwarp();
          ++js;
          did = true;
        }
        if (did) {
          idle = 0;
        } else if (++idle > tc::kSpinLimit) {
          if (lane == 0) tc::report_status(status, 6);
          alive = false;
        } else {
          __nanosleep(20);   // a tight poll would take issue slots from the softmax warp on this scheduler
        }
      }
      g += nblk;
      if (alive && tc::elect_one()) tc::tc_commit(bar(O_FULL));
      __syncwarp();
      ++req;
    }
  } else if (warp < 4) {
    // ================================ softmax / epilogue ================================
    const int r_row = tid & 63, th = tid >> 6;           // TMEM lane tid: row tid%64, token/column half tid/64
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    int g = 0, req = 0;
    bool aborted = false;        // uniform over the 128 softmax threads: only read right after a bar_sync
    for (int wi = 0; wi < tile.n_work; ++wi) {
      const Work r = get_work<MODE>(P, tile, wi);
      const int nblk = r.blk_hi - r.blk_lo;
      float m_run = neg_inf();     // running maximum (base-2 scaled logits)
      float m_used = 0.f;          // the maximum O and l are currently scaled with
      float l_part = 0.f;          // this thread's share of the row sum
      for (int j = 0; j < nblk && !aborted; ++j, ++g) {
        const int st = g & 1;
        uint32_t sv[32];
        uint32_t vbits = 0xffffffffu;
        if (tc::mbar_wait(bar(S_FULL0 + st), (g >> 1) & 1, status, 8)) {
          if (tid == 0) FMLA_TRACE_AT(g, 6);
          tc::tc_fence_after();
          tc::tmem_ld32(tmem + lane_addr + TMEM_S + st * 32, sv);
          if constexpr (MODE != kDense) vbits = sValid[st * 2 + th];
          tc::tmem_wait_ld();
          tc::tc_fence_before();
        } else {
          *sAbort = 1;
#pragma unroll
          for (int i = 0; i < 32; ++i) sv[i] = 0u;
        }
        tc::mbar_arrive(bar(S_EMPTY0 + st));
        if (tid == 0) FMLA_TRACE_AT(g, 7);

        if constexpr (MODE == kDense) {
          const int tok0 = (r.blk_lo + j) * 64 + th * 32;
          if (tok0 + 32 > r.border) vbits = tok0 >= r.border ? 0u : (0xffffffffu >> (32 - (r.border - tok0)));
        }
        // masked logits become -inf (a select: they may hold anything); the maximum is taken over the raw
        // logits in four independent chains and scaled once (the scale is positive)
        if (vbits != 0xffffffffu) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (!((vbits >> i) & 1u)) sv[i] = 0xff800000u;
        }
        float mx4[4] = {neg_inf(), neg_inf(), neg_inf(), neg_inf()};
#pragma unroll
        for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
        float* xch = sMx + (j & 1) * 128;
        xch[tid] = mx;
        bar_sync(1, 128);
        if (*sAbort) { aborted = true; break; }
        if (tid == 0) FMLA_TRACE_AT(g, 8);
        mx = fmaxf(mx, xch[tid ^ 64]);
        const float m_new = fmaxf(m_run, mx);

        // O and l carry the scale 2^-m_used; it is moved only when the maximum grew by more than the
        // threshold (or when the first real value arrives after fully masked blocks)
        bool need = false;
        if (j == 0 || (m_run == neg_inf() && m_new != neg_inf())) {
          // first block, or the first visible key after fully masked blocks: O and l are exactly zero, so the
          // reference scale is simply set (multiplying 0 by 2^(0 - m_new) would give NaN for m_new < -128)
          m_used = (m_new == neg_inf()) ? 0.f : m_new;
        } else {
          need = (m_new - m_used) > kRescaleThreshold;
        }
        m_run = m_new;
        const bool any_need = __any_sync(0xffffffffu, need);
        bool pv_done = false;    // the previous P V must be complete before O is rescaled and before P is overwritten
        if (any_need) {
          if (!tc::mbar_wait(bar(P_EMPTY), (g & 1) ^ 1, status, 9)) *sAbort = 1;
          pv_done = true;
          const float m_next = need ? m_new : m_used;
          const float alpha = exp2f(m_used - m_next);
          m_used = m_next;
          l_part *= alpha;
          tc::tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            uint32_t ov[32];
            tc::tmem_ld32(tmem + lane_addr + TMEM_O + c * 32, ov);
            tc::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tc::tmem_st32(tmem + lane_addr + TMEM_O + c * 32, ov);
          }
          tc::tmem_wait_st();
          tc::tc_fence_before();
        }
        if (tid == 0) FMLA_TRACE_AT(g, 10);
        float rs4[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = exp2f(fmaf(__uint_as_float(sv[2 * i]), scale_log2, -m_used));
          const float p1 = exp2f(fmaf(__uint_as_float(sv[2 * i + 1]), scale_log2, -m_used));
          rs4[i & 3] += p0 + p1;
          pk[i] = pack_16x2<F16>(p0, p1);
        }
        l_part += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
        if (!pv_done && !tc::mbar_wait(bar(P_EMPTY), (g & 1) ^ 1, status, 9)) *sAbort = 1;
        if (tid == 0) FMLA_TRACE_AT(g, 9);
        // P[row][th*32 .. +32) -> K-major 128B-swizzled A operand: 16-byte chunk (th*4 + q) ^ (row & 7)
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4)
          st_shared_v4(sP + r_row * 128 + ((((th * 4 + q4) ^ (r_row & 7))) << 4),
                       make_uint4(pk[q4 * 4], pk[q4 * 4 + 1], pk[q4 * 4 + 2], pk[q4 * 4 + 3]));
        tc::fence_proxy_async_smem();
        tc::mbar_arrive(bar(P_FULL));
        if (tid == 0) FMLA_TRACE_AT(g, 11);
      }

      // ---- epilogue of this work item ---------------------------------------------------
      float* xch = sMx + 256;
      bar_sync(1, 128);
      xch[tid] = l_part;
      bar_sync(1, 128);
      if (*sAbort) aborted = true;
      if (aborted) break;
      const float l = l_part + xch[tid ^ 64];
      const bool row_ok = r_row < tile.nvalid;
      const int head = tile.head0 + r_row;
      const float inv = (l == 0.f || nblk == 0) ? 0.f : 1.f / l;
      bool have_o = nblk > 0;
      if (have_o) {
        if (!tc::mbar_wait(bar(O_FULL), req & 1, status, 10)) { *sAbort = 1; have_o = false; }
        tc::tc_fence_after();
      }
      // destination rows: final bf16 output, or the fp32 partial slot of a split request
      __nv_bfloat16* o_final;
      float* o_part = nullptr;
      int64_t part_row = 0;
      if constexpr (MODE == kSparsePrefill) {
        o_final = reinterpret_cast<__nv_bfloat16*>(P.sp.out) + ((int64_t)r.batch * P.sp.h_q + head) * 512;
      } else {
        const int q_seq_per_hk = p.s_q * p.hq_per_hk;
        const int row_in_group = tile.sq * p.hq_per_hk + tile.hb * 64 + r_row;   // regrouped row index within the kv head
        o_final = reinterpret_cast<__nv_bfloat16*>(p.out) + r.batch * p.o_stride_b + tile.sq * p.o_stride_s + head * p.o_stride_h;
        part_row = ((int64_t)r.split_slot * p.h_k + tile.kh) * q_seq_per_hk + row_in_group;
        o_part = p.o_accum + part_row * 512;
      }
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        uint32_t ov[32];
        if (have_o) {
          tc::tmem_ld32(tmem + lane_addr + TMEM_O + c * 32, ov);
          tc::tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = 0u;
        }
        const int col = (c >> 2) * 256 + th * 128 + (c & 3) * 32;
        if (row_ok) {
          if (r.no_split) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 v;
              v.x = pack_16x2<F16>(__uint_as_float(ov[q4 * 8 + 0]) * inv, __uint_as_float(ov[q4 * 8 + 1]) * inv);
              v.y = pack_16x2<F16>(__uint_as_float(ov[q4 * 8 + 2]) * inv, __uint_as_float(ov[q4 * 8 + 3]) * inv);
              v.z = pack_16x2<F16>(__uint_as_float(ov[q4 * 8 + 4]) * inv, __uint_as_float(ov[q4 * 8 + 5]) * inv);
              v.w = pack_16x2<F16>(__uint_as_float(ov[q4 * 8 + 6]) * inv, __uint_as_float(ov[q4 * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(o_final + col + q4 * 8) = v;
            }
          } else {
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4) {
              float4 v = make_float4(__uint_as_float(ov[q4 * 4 + 0]) * inv, __uint_as_float(ov[q4 * 4 + 1]) * inv,
                                     __uint_as_float(ov[q4 * 4 + 2]) * inv, __uint_as_float(ov[q4 * 4 + 3]) * inv);
              *reinterpret_cast<float4*>(o_part + col + q4 * 4) = v;
            }
          }
        }
      }
      if (nblk > 0) {
        tc::tc_fence_before();
        tc::mbar_arrive(bar(O_EMPTY));
        ++req;
      }
      if (row_ok && th == 0) {
        if constexpr (MODE == kSparsePrefill) {
          const int64_t o = (int64_t)r.batch * P.sp.h_q + head;
          P.sp.max_logits[o] = inv == 0.f ? neg_inf() : m_run;
          P.sp.lse[o] = inv == 0.f ? neg_inf() : log2f(l) + m_used;
        } else if (r.no_split) {
          p.softmax_lse[((int64_t)r.batch * p.h_q + head) * p.s_q + tile.sq] = inv == 0.f ? pos_inf() : (log2f(l) + m_used) * kLn2;
        } else {
          p.lse_accum[part_row] = inv == 0.f ? neg_inf() : log2f(l) + m_used;
          if (p.no_split_hint && tid == 0) tc::report_status(status, 41);     // a split request although the caller ruled it out
        }
      }
    }
  }

  tc::tc_fence_before();
  __syncthreads();
  if (warp == 5) tc::tmem_dealloc(tmem, 512);
}

// ---- host side ----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess) f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// bf16 tensor [d3][d2][d1][d0=576] with element strides s1,s2,s3 ; box {64, b1, b2, 1}
static bool make_map_4d(CUtensorMap* m, const void* base, uint64_t d1, uint64_t d2, uint64_t d3, int64_t s1, int64_t s2, int64_t s3,
                        uint32_t b1, uint32_t b2) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return false;
  cuuint64_t dims[4] = {576, d1, d2, d3};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(s1) * 2, static_cast<cuuint64_t>(s2) * 2, static_cast<cuuint64_t>(s3) * 2};
  cuuint32_t box[4] = {64, b1, b2, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int MODE, bool F16 = false>
static cudaError_t launch_tc(const TcParams& P, const CUtensorMap& tq, const CUtensorMap& tkv, dim3 grid, cudaStream_t stream) {
  auto kern = mla_tc_kernel<MODE, F16>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, dtc::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  kern<<<grid, MODE == kDense ? 192 : 448, dtc::SMEM_BYTES, stream>>>(P, tq, tkv);
  return cudaGetLastError();
}

// FMLA_DISABLE_PAIR=1 in the environment keeps the one-CTA-per-64-heads kernel for every shape (A/B runs)
static bool pair_kernel_enabled() {
  static const bool on = [] {
    const char* v = getenv("FMLA_DISABLE_PAIR");
    return !(v && v[0] == '1');
  }();
  return on;
}

bool decode_dense_merges_in_kernel(const DecodeKernelParams& p) {
  return p.topk < 0 && decode_dense_pair_applies(p) && pair_kernel_enabled() && p.arrival_counters != nullptr && !p.force_partial;
}

cudaError_t launch_decode_dense_tc(const DecodeKernelParams& p, cudaStream_t stream) {
  if (decode_dense_pair_applies(p) && pair_kernel_enabled()) return launch_decode_dense_pair(p, stream);
  TcParams P = {};
  P.d = p;
  CUtensorMap tq, tkv;
  // q [b][s_q][h_q][576] ; box = 64 heads x 64 columns (heads past h_q read as zero)
  if (!make_map_4d(&tq, p.q, p.h_q, p.s_q, p.b, p.q_stride_h, p.q_stride_s, p.q_stride_b, 64, 1)) return cudaErrorInvalidValue;
  // cache [num_blocks][64][h_k][576] addressed as (col, head, row-in-page, page) ; box = 64 rows x 64 columns of one head
  if (!make_map_4d(&tkv, p.kcache, p.h_k, 64, p.num_blocks, p.k_stride_head, p.k_stride_row, p.k_stride_block, 1, 64))
    return cudaErrorInvalidValue;
  const int n_hb = (p.hq_per_hk + 63) / 64;
  // the tensor maps only move 16-bit elements: one map type serves bf16 and fp16
  if (p.is_f16) return launch_tc<kDense, true>(P, tq, tkv, dim3(p.s_q * n_hb, p.h_k, p.num_sm_parts), stream);
  return launch_tc<kDense>(P, tq, tkv, dim3(p.s_q * n_hb, p.h_k, p.num_sm_parts), stream);
}

cudaError_t launch_decode_sparse_tc(const DecodeKernelParams& p, cudaStream_t stream) {
  if (decode_sparse_pair_applies(p) && pair_kernel_enabled()) return launch_decode_sparse_pair(p, stream);
  TcParams P = {};
  P.d = p;
  CUtensorMap tq;
  if (!make_map_4d(&tq, p.q, p.h_q, p.s_q, p.b, p.q_stride_h, p.q_stride_s, p.q_stride_b, 64, 1)) return cudaErrorInvalidValue;
  return launch_tc<kSparseDecode>(P, tq, tq, dim3((p.hq_per_hk + 63) / 64, p.s_q, p.num_sm_parts), stream);
}

cudaError_t launch_sparse_prefill_tc(const SparsePrefillKernelParams& sp, cudaStream_t stream) {
  if (sparse_prefill_pair_applies(sp) && pair_kernel_enabled()) return launch_sparse_prefill_pair(sp, stream);
  TcParams P = {};
  P.sp = sp;
  CUtensorMap tq;
  // q [s_q][h_q][576] as (col, head, token, 1)
  if (!make_map_4d(&tq, sp.q, sp.h_q, sp.s_q, 1, sp.q_stride_h, sp.q_stride_s, sp.q_stride_s * sp.s_q, 64, 1)) return cudaErrorInvalidValue;
  // one CTA per SM (and head tile) walks the query tokens
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 148;
  const int n_hb = sp.h_q / 64;
  const int lanes = max(1, min(sp.s_q, sms / n_hb));
  return launch_tc<kSparsePrefill>(P, tq, tq, dim3(n_hb, lanes, 1), stream);
}

#ifdef FMLA_TRACE
extern "C" int fmla_debug_read_trace(long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_decode_trace, sizeof(long long) * n);
}
#endif

cudaError_t set_status_mirror_mla(int* mapped_host_word) { return tc::set_status_mirror(mapped_host_word); }

cudaError_t read_decode_tc_status(int* host_status, bool reset) {
  cudaError_t e = cudaMemcpyFromSymbol(host_status, g_decode_tc_status, sizeof(int));
  if (e != cudaSuccess) return e;
  if (reset && *host_status != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_decode_tc_status, &zero, sizeof(int));
  }
  return e;
}

}  // namespace fmla
