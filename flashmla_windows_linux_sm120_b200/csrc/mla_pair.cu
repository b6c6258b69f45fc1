// MLA attention for 128 heads on sm_100a as a CTA pair (cluster of two CTAs, tcgen05 cta_group::2): dense BF16 /
// FP16 split-KV decode, sparse FP8 split-KV decode and sparse prefill.  The dense mode is described first; the two
// gathering modes differ in how the K rows reach shared memory and where the V operand comes from (further down).
//
// The pair owns 128 query heads of one (query token, kv head, partition): CTA r of the pair (cluster rank r)
// owns heads 64r .. 64r+63, i.e. the Q tile, the S tile, the P tile and the O accumulator of those heads.
// One thread of the leader (rank 0) issues every MMA for both SMs:
//   S = Q K^T   36 x tcgen05.mma.cta_group::2 m128n64k16: the B operand (64 tokens x 576) is split along N, so
//               each CTA stages only ITS 32 token rows of a page (36 KB) -- the pair reads a page for S once
//   O += P V    8 x tcgen05.mma.cta_group::2 m128n256k16: B = V, split along N = value columns, so each CTA
//               stages 64 tokens x 256 value columns (32 KB): chunks {2r, 2r+1, 4+2r, 5+2r} of the page
// What this buys over one CTA per 64 heads with a 72 KB page stage that is held from its load until the end
// of its P V: the K part is released right after S and the V part is loaded independently of it, so two
// small rings (3 x 36 KB + 2 x 32 KB) keep more loads in flight per SM than two 72 KB stages, and the paired
// instructions run at 25 / 65 clocks (S / P V) instead of 32 / 81.
// Two thirds of Q live in tensor memory: the 192 columns that O and S leave idle hold column chunks 0..5 of
// the CTA's Q tile (tcgen05.cp from shared memory, rows duplicated into both lane halves as an M=64-per-CTA
// A operand wants them), so only chunks 6..8 (24 KB) stay in shared memory -- that is what makes room for
// the third K stage -- and the S instructions that take A from tensor memory run at 18 instead of 25 clocks.
// The six chunks pass through the V ring on their way (free between the last P V of a request and the first of
// the next); the K loads depend on nothing but the K ring and run ahead into the next request.
//
//   warps 0-3 softmax : as in mla_tc.cu (TMEM lane = row + 64 * (token >= 32)); arrivals that the issuing
//                       thread waits for go to the leader's barriers (remote arrive from rank 1)
//   warp 4   K loader : per 64-token block the CTA's 32 token rows.  The leader's copies complete on
//                       the barrier its MMA warp waits on; the peer's copies complete on a barrier of the peer
//                       and one thread there passes each completion on with a single remote arrive (letting the
//                       peer's copies count their bytes on the leader's barrier directly -- cp.async.bulk.tensor
//                       ... cta_group::2 -- made a 36 KB part take about 3 us to be seen as landed)
//   warp 5   MMA      : rank 0: issues every MMA; rank 1: the relay of the Q / K completions just described
//   warp 6   V loader : the Q tile of a request, then per block 4 boxes of 64 rows x 64 columns, completing on a local barrier
//   warp 7   V relay  : waits for the local V part, clears the rows of the last page that lie beyond the
//                       sequence (they may hold NaN and 0 * NaN must not reach O), tells the leader
// TMEM (512 columns per CTA, allocated as a pair): O = [0,256), S[0] = [256,288), S[1] = [288,320), Q chunks
// 0..5 = [320,512) (32 columns each); O / S layouts as in mla_tc.cu (the 64-row halves of an M=128 pair
// instruction have the layout of the M=64 .ws form).
//
// Gathering modes (sparse FP8 decode: 480 threads, sparse prefill: 320 threads).  Each CTA brings only its 32 token
// rows of a 64-index block into the K ring -- prefill: three warps of 16-byte cp.async copies that arrive on the
// landing barrier by hardware; FP8 decode: two groups of four warps that read the 656-byte records into registers,
// de-quantise them once per pair and store them in the layout TMA would produce.  The V operand (64 tokens x 256
// columns per CTA) is not read from global memory at all: the thread of warp 6 forwards it out of the landed K rows
// with eight 4 KB cp.async.bulk shared-memory copies, four into its own V stage and four into the peer's
// (distributed shared memory).  That thread also relays K landings to the leader and loads Q.  Invalid indices
// leave zero rows and reach the softmax as validity bits.
//
// Semantics follow csrc/sm90/decode/dense/splitkv_mla.cu:948-957, 1022-1042, 1237-1269 of the reference
// (borders, split outputs, LSE conventions), csrc/sm100/decode/sparse_fp8 and csrc/sm100/prefill/sparse for the
// index handling of the sparse modes.  Every wait is bounded; on expiry the pair drains and frees
// its tensor memory.
#include "kernels.h"
#include "mla_work.cuh"
#include "tc_common.cuh"

#include <cuda.h>
#include <cuda_fp8.h>

#include <cstdlib>

namespace fmla {

namespace ptc {
constexpr int kChunkBytes = 64 * 128;             // Q / P / V chunk: [64 rows x 64 x 16-bit], 128-byte rows
constexpr int kQBytes = 9 * kChunkBytes;          // 64 heads x 576
constexpr int kQTmemChunks = 6;                   // column chunks 0..5 of Q are kept in tensor memory
constexpr int kQSmemChunks = 9 - kQTmemChunks;    // chunks 6..8 stay in shared memory
constexpr int kKChunkBytes = 32 * 128;            // K chunk of this CTA: [32 token rows x 64 columns]
constexpr int kKStageBytes = 9 * kKChunkBytes;    // 36 864
constexpr int kKStages = 3;
constexpr int kVStageBytes = 4 * kChunkBytes;     // 32 768: 64 tokens x 256 value columns
constexpr int Q_OFF = 0;                          // kQSmemChunks chunks
constexpr int K_OFF = Q_OFF + kQSmemChunks * kChunkBytes;   // kKStages stages; also the staging area of Q chunks 0..5
constexpr int V_OFF = K_OFF + kKStages * kKStageBytes;      // 2 stages
constexpr int P_OFF = V_OFF + 2 * kVStageBytes;   // 2 x [64 x 64]
constexpr int BAR_OFF = P_OFF + 2 * kChunkBytes;
constexpr int MX_OFF = BAR_OFF + 256;             // float [3][128] exchange
constexpr int MISC_OFF = MX_OFF + 1536;
constexpr int SMEM_BYTES = MISC_OFF + 128;
static_assert(kQTmemChunks * kChunkBytes <= 2 * kVStageBytes, "Q staging must fit into the V ring (sparse prefill)");
// leader-side barriers (waited on by the MMA warp of rank 0; arrivals come from both CTAs)
// and per-CTA barriers (each CTA waits on its own copy; the leader's commits arrive on both copies)
enum Bar { Q_FULL = 0, K_FULL0, K_FULL1, K_FULL2, V_FULL0, V_FULL1, S_EMPTY0, S_EMPTY1, P_FULL0, P_FULL1, O_EMPTY,
           Q_EMPTY, QT_DONE, K_EMPTY0, K_EMPTY1, K_EMPTY2, V_EMPTY0, V_EMPTY1, V_LAND0, V_LAND1, S_FULL0, S_FULL1,
           P_EMPTY0, P_EMPTY1, O_FULL, Q_LAND, K_LAND0, K_LAND1, K_LAND2, NUM_BARS };
constexpr int TMEM_O = 0, TMEM_S = 256, TMEM_Q = 320;
static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared memory limit per CTA");
static_assert(NUM_BARS * 8 <= 256, "barrier area too small");
constexpr float kRescaleThreshold = 8.0f;
constexpr int kThreads = 256;
#ifndef FMLA_GATHER_WARPS
#define FMLA_GATHER_WARPS 3
#endif
constexpr int kGatherWarps = FMLA_GATHER_WARPS;                 // sparse prefill: warp 4 and warps 8 .. 6 + kGatherWarps (measured: 3 -> 993, 4 -> 983, 5 -> 935, 2 -> 452 TFLOP/s)
constexpr int kPrefillThreads = (7 + kGatherWarps) * 32;
#ifndef FMLA_DECODE_GROUPS
#define FMLA_DECODE_GROUPS 2
#endif
constexpr int kDecodeGatherGroups = FMLA_DECODE_GROUPS;            // sparse FP8 decode: groups of four gather warps that take alternate blocks
constexpr int kSparseDecodeThreads = (7 + 4 * kDecodeGatherGroups) * 32;
}  // namespace ptc

__device__ int g_decode_pair_status = 0;

#ifdef FMLA_TRACE
__device__ long long g_pair_trace[160 * 16];
__device__ long long g_pair_span[512 * 2];       // per CTA: first and last clock (globaltimer would be comparable across SMs)
#define FMLA_PTRACE_AT(blk, slot)                                                          \
  do {                                                                                      \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == FMLA_TRACE_PART && (blk) < 160) g_pair_trace[(blk) * 16 + (slot)] = clock64(); \
  } while (0)
#ifndef FMLA_TRACE_PART
#define FMLA_TRACE_PART 0
#endif
// cross-CTA timeline in nanoseconds (globaltimer): [block][rank][slot]
__device__ long long g_pair_gt[160 * 2 * 8];
__device__ long long g_pair_head[256][2];
__device__ __forceinline__ long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return (long long)t; }
#define FMLA_GTRACE_AT(blk, rk, slot)                                                       \
  do {                                                                                       \
    if (blockIdx.y == 0 && blockIdx.z == FMLA_TRACE_PART && blockIdx.x < 2 && (blk) < 160) g_pair_gt[((blk) * 2 + (rk)) * 8 + (slot)] = gtime(); \
  } while (0)
#else
#define FMLA_PTRACE_AT(blk, slot) do {} while (0)
#define FMLA_GTRACE_AT(blk, rk, slot) do {} while (0)
#endif

__device__ __forceinline__ void pst_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// 32 bytes to global memory: one 256-bit store when the address allows it, else two 128-bit stores
__device__ __forceinline__ void st_global_32B(void* p, const uint32_t (&w)[8]) {
  if ((reinterpret_cast<uintptr_t>(p) & 31u) == 0) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]),
                 "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
  } else {
    reinterpret_cast<uint4*>(p)[0] = make_uint4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<uint4*>(p)[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

__device__ __forceinline__ void mma_pair_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
// shared memory -> tensor memory, 64 rows x 16 bytes per instruction, rows 0..31 into lanes 0..31 and 64..95,
// rows 32..63 into lanes 32..63 and 96..127, in both CTAs of the pair (each from its own shared memory)
__device__ __forceinline__ void tmem_cp_pair_64x128b(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::2.64x128b.warpx2::02_13 [%0], %1;\n" ::"r"(taddr), "l"(desc) : "memory");
}

// The 36 S instructions of one block: descriptors and tensor memory addresses are a warp-uniform base (which
// carries the ring stage, chosen at run time) plus an immediate.  One copy of this code serves every stage:
// with one unrolled copy per (K stage, S buffer) the issuing thread ran out of instruction cache -- each copy
// came around once in six blocks and cost about 300 ns of instruction fetch before its first MMA.
__device__ __forceinline__ void s_block_pair(uint32_t tmem_s, uint32_t tmem_q, uint64_t desc_q, uint64_t desc_k_stage, uint32_t idesc) {
  using namespace ptc;
#pragma unroll
  for (int c = 0; c < 9; ++c)
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const uint64_t db = tc::desc_advance(desc_k_stage, c * kKChunkBytes + s * 32);
      if (c < kQTmemChunks) mma_pair_ts(tmem_s, tmem_q + c * 32 + s * 8, db, idesc, (c | s) ? 1u : 0u);
      else tc::mma_pair_ss(tmem_s, tc::desc_advance(desc_q, (c - kQTmemChunks) * kChunkBytes + s * 32), db, idesc, 1u);
    }
}
__device__ __forceinline__ void pv_block_pair(uint32_t tmem_o, uint64_t desc_p_stage, uint64_t desc_v_stage, uint32_t idesc, bool first) {
  using namespace ptc;
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int s = 0; s < 4; ++s)
      tc::mma_pair_ss(tmem_o + h * 128, tc::desc_advance(desc_p_stage, s * 32),
                      tc::desc_advance(desc_v_stage, h * 2 * kChunkBytes + s * 2048), idesc, (first && s == 0) ? 0u : 1u);
}

// Decode: grid (s_q * hq_per_hk / 64, h_k, parts), clusters of two CTAs along x; 256 threads.
// kSparseDecode (FP8 cache, 128 heads): grid (2, s_q, parts); token rows gathered by index and de-quantised by two
// groups of four warps (480 threads), everything else as in the prefill mode below, outputs as in the dense mode.
// kSparsePrefill (sparse prefill forward, 128 heads): grid (2, lanes), every pair walks the query tokens lane, lane + lanes, ..;
// each CTA gathers its 32 token rows of a 64-index block from kv[s_kv, 576] with cp.async and the value operand is
// forwarded from those rows (tmap_k32 / tmap_v64 unused); invalid indices leave zero rows and are masked through
// validity bits.
template <bool F16, int WM>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(WM == kDense ? ptc::kThreads : WM == kSparsePrefill ? ptc::kPrefillThreads : ptc::kSparseDecodeThreads, 1)
mla_pair_kernel(const __grid_constant__ TcParams P, const __grid_constant__ CUtensorMap tmap_q,
                const __grid_constant__ CUtensorMap tmap_k32, const __grid_constant__ CUtensorMap tmap_v64) {
  using namespace ptc;
  constexpr bool PREFILL = WM == kSparsePrefill;     // output / scale / work list of the prefill interface
  constexpr bool SPARSE = WM != kDense;              // token rows gathered by index, value operand forwarded from them
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase + Q_OFF, sK = sbase + K_OFF, sV = sbase + V_OFF, sP = sbase + P_OFF;
  auto bar = [&](int i) { return sbase + BAR_OFF + i * 8; };
  float* sMx = reinterpret_cast<float*>(smem + MX_OFF);
  volatile uint32_t* sTmem = reinterpret_cast<volatile uint32_t*>(smem + MISC_OFF);
  volatile int* sAbort = reinterpret_cast<volatile int*>(smem + MISC_OFF + 8);
  int* status = &g_decode_pair_status;
  const DecodeKernelParams& p = P.d;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = tc::cluster_rank();
#ifdef FMLA_TRACE
  if (tid == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_pair_span[(blockIdx.z * gridDim.x + blockIdx.x) * 2] = (long long)t;
  }
#endif
  const Tile tile = make_tile<WM>(P);
  if (tile.n_work == 0) return;                 // both CTAs of a pair see the same schedule row
  const bool misaligned = (sbase & 1023u) != 0;  // the swizzled tiles need a 1024-byte aligned base
  auto lbar = [&](int i) { return tc::mapa(bar(i), 0); };    // the leader's copy of barrier i
  const float scale_log2 = PREFILL ? P.sp.scale_log2 : p.scale_log2;
  // prefill: validity bits of the 64 tokens of a block, ring of 6 blocks x 2 words (the K loader runs at most three
  // blocks ahead of S, and S of block g+3 is only issued after the softmax has read block g+1)
  volatile uint32_t* sValid = reinterpret_cast<volatile uint32_t*>(smem + MISC_OFF + 32);

  if (tid == 0) {
    tc::mbar_init(bar(Q_FULL), 2);
    tc::mbar_init(bar(K_FULL0), 2);
    tc::mbar_init(bar(K_FULL1), 2);
    tc::mbar_init(bar(K_FULL2), 2);
    tc::mbar_init(bar(V_FULL0), 2);
    tc::mbar_init(bar(V_FULL1), 2);
    // one arrival per softmax warp of either CTA (lane 0, after the warp has synchronised): 128 remote arrivals per
    // barrier phase took the peer's P ~700 ns to reach the leader
    tc::mbar_init(bar(S_EMPTY0), 8);
    tc::mbar_init(bar(S_EMPTY1), 8);
    tc::mbar_init(bar(P_FULL0), 8);
    tc::mbar_init(bar(P_FULL1), 8);
    tc::mbar_init(bar(O_EMPTY), 8);
    // prefill: a K stage is free again once its S has completed (one commit) and the value columns forwarded out of
    // it have landed in both CTAs (one arrival from the V relay of each CTA)
    // and a K stage has landed when every lane of the gather warps has arrived by hardware, plus the thread that
    // published the validity bits (prefill), or when every gather warp has stored its rows (FP8 decode)
    for (int i = Q_EMPTY; i < NUM_BARS; ++i)
      tc::mbar_init(bar(i), !SPARSE ? 1 : (i >= K_EMPTY0 && i <= K_EMPTY2) ? 3 : (i >= K_LAND0 && i <= K_LAND2) ? (PREFILL ? kGatherWarps * 32 + 1 : 4 /* FP8 decode: the four gather warps of a group */) : 1);
    tc::fence_mbar_init();
    *sAbort = 0;
    if (misaligned) tc::report_status(status, 30);
  }
  if (warp == 5) tc::tmem_alloc_pair(sbase + MISC_OFF, 512);
  tc::tc_fence_before();
  __syncthreads();
  tc::cluster_sync_all();      // barriers of both CTAs exist before anything is sent to them
  tc::tc_fence_after();
  pdl_allow_dependents();      // a merge kernel launched as a programmatic dependent may become resident now
  const uint32_t tmem = *sTmem;

  if (misaligned) {
    // nothing was issued; fall through to the common exit
  } else if ((warp == 4 || warp >= 8) && WM == kSparsePrefill) {
    // ================================ Q and K loader, sparse prefill ===================
    // The CTA's 32 token rows of a block (32 x 1152 bytes) are gathered with 16-byte cp.async copies by three warps
    // (4, 8, 9): 72 warp instructions per block, dealt out round robin, consecutive lanes on consecutive pieces of a row.
    // Measured at the benchmark shape: with each warp taking a contiguous third of the instructions 751 TFLOP/s; with
    // the round-robin deal two warps 452, three 979-1009, four 964-982, five 935-957.  The TMA engine (tile::gather4, 4 rows x 64
    // columns per copy) gathers no faster than ~11 bytes per clock and SM, and mixing the two paths was slower
    // than either (8 of the 32 rows by TMA: 545 TFLOP/s; 16: 466), because the gathers queue behind the forwarding
    // copies in the TMA engine.  Each lane's copies arrive on the landing barrier by hardware (arrive.noinc).
    // Nothing else of the block is read from global memory: the value operand of both CTAs is put together from
    // these rows by shared-memory copies (warp 6), which also loads Q: the gather runs ahead into the next query
    // token while the current one drains.  Warp 4 publishes the validity bits of the 64 indices.  An index outside
    // the tensor (negative or >= s_kv) leaves a zero row.
    int g = 0;
    bool alive = true;
    const int s_kv = P.sp.s_kv;
    const int gw = warp == 4 ? 0 : warp - 7;                 // 0..3
    const char* kvb = reinterpret_cast<const char*>(P.sp.kv);
    const int64_t row_bytes = P.sp.kv_stride_s * 2;
    for (int wi = 0; wi < tile.n_work && alive; ++wi) {
      const Work r = get_work<WM>(P, tile, wi);
      // the indices of a block are read one block ahead of their use: their latency would otherwise be paid in
      // every turn of this loop
      const int* my_idx = r.idx + 32 * static_cast<int>(rank) + lane;
      int mine_next = r.blk_lo < r.blk_hi ? __ldg(my_idx + r.blk_lo * 64) : -1, i0_next = -1, i1_next = -1;
      if (warp == 4 && r.blk_lo < r.blk_hi) {
        i0_next = __ldg(r.idx + r.blk_lo * 64 + lane);
        i1_next = __ldg(r.idx + r.blk_lo * 64 + 32 + lane);
      }
      for (int blk = r.blk_lo; blk < r.blk_hi && alive; ++blk, ++g) {
        const int st = g % kKStages;
        int mine = mine_next;                                                          // row `lane` of this CTA's part
        const int i0 = i0_next, i1 = i1_next;
        if (blk + 1 < r.blk_hi) {
          mine_next = __ldg(my_idx + (blk + 1) * 64);
          if (warp == 4) {
            i0_next = __ldg(r.idx + (blk + 1) * 64 + lane);
            i1_next = __ldg(r.idx + (blk + 1) * 64 + 32 + lane);
          }
        }
        if (mine < 0 || mine >= s_kv) mine = -1;
        uint32_t b0 = 0, b1 = 0;
        if (warp == 4) {
          b0 = __ballot_sync(0xffffffffu, i0 >= 0 && i0 < s_kv);
          b1 = __ballot_sync(0xffffffffu, i1 >= 0 && i1 < s_kv);
        }
        alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(K_EMPTY0 + st), ((g / kKStages) & 1) ^ 1, status, 102));
        if (!alive) break;
        if (warp == 4 && lane == 0) FMLA_PTRACE_AT(g, 0);
        const uint32_t dst = sK + st * kKStageBytes;
        if (warp == 4 && lane == 0) {
          sValid[(g % 6) * 2] = b0;
          sValid[(g % 6) * 2 + 1] = b1;
          tc::mbar_arrive(bar(K_LAND0 + st));
        }
        constexpr int kInstr = 32 * 72 / 32;                      // warp instructions per block, dealt out round robin
#pragma unroll
        for (int inst = 0; inst < kInstr; inst += kGatherWarps) {
          if (inst + gw >= kInstr) break;
          const int e = (inst + gw) * 32 + lane;                 // piece e of 32 rows x 72 pieces of 16 bytes
          const int row = e / 72, piece = e % 72;
          const int idx = __shfl_sync(0xffffffffu, mine, row);
          const bool ok = idx >= 0;
          const char* src = kvb + (ok ? (int64_t)idx * row_bytes + piece * 16 : 0);
          cp_async16(dst + (piece >> 3) * kKChunkBytes + row * 128 + (((piece & 7) ^ (row & 7)) << 4), src, ok);
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar(K_LAND0 + st)) : "memory");
      }
    }
  } else if ((warp == 4 || warp >= 8) && WM == kSparseDecode) {
    // ================================ K loader, sparse FP8 decode ======================
    // Groups of four gather warps, eight of the CTA's 32 token rows per warp.  For one 656-byte record the 32 lanes read the 32
    // 16-byte pieces of e4m3 values (512 contiguous bytes), their tile's scale, and 8 lanes the bf16 rope part;
    // bf16(fp32(e4m3) * scale) goes into the K stage in the layout TMA would produce.  Every record is de-quantised
    // once per pair: the value operand of both CTAs is forwarded from these rows (warp 6).  The raw bytes of the
    // next block are fetched into registers before the wait for the stage, across requests.  Warp 4 also
    // publishes the validity bits of all 64 indices of a block.
    const int gi = warp == 4 ? 0 : warp - 7;                 // gather warp 0 .. 4 * kDecodeGatherGroups - 1
    const int gw = gi & 3, grp = gi >> 2;                    // rows 8*gw .. of the blocks grp, grp + groups, ..
    const bool publisher = gw == 0;                          // this warp also publishes the validity bits of its blocks
    const unsigned char* cache = reinterpret_cast<const unsigned char*>(p.kcache);
    uint4 nope[8], rope[8];
    float scl[8];
    auto to_slot = [&](int v, int batch) {
      if (p.indices_logical) {       // token position of the request -> physical slot through its block table
        const int pos = v;
        v = -1;
        if (pos >= 0 && pos < __ldg(p.seqlens_k + batch)) v = __ldg(p.block_table + batch * p.block_table_stride_b + (pos >> 6)) * 64 + (pos & 63);
      }
      return (v < 0 || v >= p.num_blocks * 64) ? -1 : v;
    };
    // Within a group the index reader runs two of its blocks ahead of the stores and the record reader one: the
    // index -> record chain of loads would otherwise be paid, end to end, once per block.  The groups take
    // alternate blocks, so that the record reads of consecutive blocks are in flight together.
    int c_wi = 0, c_blk = 0;         // position of the index reader in the CTA's block list
    Work c_r = get_work<WM>(P, tile, 0);
    while (c_wi < tile.n_work && c_r.blk_hi == c_r.blk_lo) { ++c_wi; if (c_wi < tile.n_work) c_r = get_work<WM>(P, tile, c_wi); }
    c_blk = c_r.blk_lo;
    auto advance = [&] {
      if (c_wi >= tile.n_work) return;
      ++c_blk;
      while (c_wi < tile.n_work && c_blk >= c_r.blk_hi) {
        ++c_wi;
        if (c_wi < tile.n_work) { c_r = get_work<WM>(P, tile, c_wi); c_blk = c_r.blk_lo; }
      }
    };
    for (int i = 0; i < grp; ++i) advance();
    // Raw index words of the group's next unread block, and the request they belong to: lanes 0..7 the row
    // 8*gw + lane of this CTA's part; publisher: tokens lane and 32 + lane.  The words are only looked at one turn
    // later (an instruction that consumes a load waits for it, in program order).
    struct Raw { int mine, t0, t1, batch; };
    auto read_indices = [&](Raw& w) -> bool {
      if (c_wi >= tile.n_work) return false;
      w.mine = __ldg(c_r.idx + c_blk * 64 + 32 * static_cast<int>(rank) + gw * 8 + (lane & 7));
      if (publisher) {
        w.t0 = __ldg(c_r.idx + c_blk * 64 + lane);
        w.t1 = __ldg(c_r.idx + c_blk * 64 + 32 + lane);
      }
      w.batch = c_r.batch;
      for (int i = 0; i < kDecodeGatherGroups; ++i) advance();
      return true;
    };
    auto read_records = [&](int my_slot) {
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
    // byte offset of 16-byte piece `piece` (0..71) of row `row` (0..31) in a K stage: 4 KB chunks of 64 columns, 128-byte swizzle
    auto stage_off = [](int row, int piece) { return (piece >> 3) * kKChunkBytes + row * 128 + (((piece & 7) ^ (row & 7)) << 4); };
    int g = grp;
    bool alive = true;
    uint32_t b0 = 0, b1 = 0;
    Raw raw = {-1, -1, -1, 0};
    auto use_indices = [&] {       // validity bits and record reads of the block whose index words are in `raw`
      if (publisher) {
        b0 = __ballot_sync(0xffffffffu, to_slot(raw.t0, raw.batch) >= 0);
        b1 = __ballot_sync(0xffffffffu, to_slot(raw.t1, raw.batch) >= 0);
      }
      read_records(to_slot(raw.mine, raw.batch));
    };
    bool have = read_indices(raw);
    if (have) use_indices();
    bool have_n = have && read_indices(raw);
    while (have && alive) {
      const int st = g % kKStages;
      alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(K_EMPTY0 + st), ((g / kKStages) & 1) ^ 1, status, 102));
      if (!alive) break;
      if (publisher && lane == 0) FMLA_PTRACE_AT(g, 0);
      const uint32_t stage = sK + st * kKStageBytes;
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
        pst_shared_v4(stage + stage_off(row, lane * 2), make_uint4(o[0], o[1], o[2], o[3]));
        pst_shared_v4(stage + stage_off(row, lane * 2 + 1), make_uint4(o[4], o[5], o[6], o[7]));
        if (lane < 8) pst_shared_v4(stage + stage_off(row, 64 + lane), rope[rr]);
      }
      if (publisher && lane == 0) {
        sValid[(g % 6) * 2] = b0;
        sValid[(g % 6) * 2 + 1] = b1;
        FMLA_PTRACE_AT(g, 1);
      }
      if (gw == 3 && lane == 0) FMLA_PTRACE_AT(g, 10);
      tc::fence_proxy_async_smem();      // these stores -> the forwarding copies and the tensor pipe
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(bar(K_LAND0 + st));
      g += kDecodeGatherGroups;
      // the records of the next block (its indices are here already), then the indices of the one after
      have = have_n;
      if (have) {
        use_indices();
        have_n = read_indices(raw);
      }
    }
  } else if (warp == 4) {
    // ================================ K loader =========================================
    // depends on nothing but the K ring: it runs ahead into the next request while the current one drains (Q is
    // staged through the V ring and loaded by warp 6)
    if (tc::elect_one()) {
      tc::prefetch_tensormap(&tmap_k32);
      int g = 0;
      bool alive = true;
      for (int wi = 0; wi < tile.n_work && alive; ++wi) {
        const Work r = get_work<WM>(P, tile, wi);
        if (r.blk_hi == r.blk_lo) continue;
        const int* bt = p.block_table + r.batch * p.block_table_stride_b;
        const int pf = p.l2_prefetch_dist;
        // the leader pulls whole pages into L2 `pf` blocks ahead of the loads of both CTAs (the V parts use the
        // 64-row map, whose boxes cover a page in 9 pieces)
        if (pf > 0 && rank == 0) {
          for (int blk = r.blk_lo; blk < min(r.blk_lo + pf, r.blk_hi); ++blk) {
            const int pg = __ldg(bt + blk);
#pragma unroll
            for (int c = 0; c < 9; ++c) tc::tma_prefetch_l2_4d(&tmap_v64, c * 64, tile.kh, 0, pg);
          }
        }
        int page_next = __ldg(bt + r.blk_lo);
        for (int blk = r.blk_lo; blk < r.blk_hi; ++blk, ++g) {
          const int st = g % kKStages;
          const int page = page_next;
          if (blk + 1 < r.blk_hi) page_next = __ldg(bt + blk + 1);
          if (pf > 0 && rank == 0 && blk + pf < r.blk_hi) {
            const int pg = __ldg(bt + blk + pf);
#pragma unroll
            for (int c = 0; c < 9; ++c) tc::tma_prefetch_l2_4d(&tmap_v64, c * 64, tile.kh, 0, pg);
          }
          alive = tc::mbar_wait(bar(K_EMPTY0 + st), ((g / kKStages) & 1) ^ 1, status, 102);
          if (!alive) break;
          FMLA_PTRACE_AT(g, 0);
          FMLA_GTRACE_AT(g, rank, 7);
          const uint32_t full = rank == 0 ? bar(K_FULL0 + st) : bar(K_LAND0 + st);
          tc::mbar_arrive_expect_tx(full, kKStageBytes);
#pragma unroll
          for (int c = 0; c < 9; ++c)
            tc::tma_load_4d(sK + st * kKStageBytes + c * kKChunkBytes, &tmap_k32, c * 64, tile.kh, 32 * static_cast<int>(rank), page, full);
        }
      }
    }
  } else if (warp == 6 && SPARSE) {
    // ================================ K relay and V forwarder, sparse prefill ==========
    // The gathered rows of this CTA (32 tokens x 576 columns) hold the value columns of those tokens for both CTAs.
    // Once they have landed, each 64-column chunk of the value part goes, as one 4 KB shared-memory copy, to the
    // V stage of the CTA whose output columns it belongs to (its own or, over the cluster's shared-memory network,
    // the peer's): rows [32 * rank, 32 * rank + 32) of that stage's chunk.  The 128-byte swizzle pattern repeats every
    // 1024 bytes, so a chunk moves as it is.  Global memory and L2 are read once per pair and block.
    // Q of a query token: chunks 6..8 go to their place, chunks 0..5 are staged in the V ring (48 of its 64 KB) until
    // the leader has copied them into tensor memory.  Loaded once every S of the previous token has completed (Q in
    // shared and tensor memory free) and its last two P V have released the V stages.
    // One thread does all of it without ever blocking on one condition while another could be served: the relay of
    // a landed K stage to the leader (the next S must not wait behind a V stage that is still in use), the Q load
    // of the next request, the forwarding copies.
    if (tc::elect_one()) {
      tc::prefetch_tensormap(&tmap_q);
      int total = 0;
      for (int wi = 0; wi < tile.n_work; ++wi) {
        const Work r = get_work<WM>(P, tile, wi);
        total += max(r.blk_hi - r.blk_lo, 0);
      }
      int kg = 0;                       // next block whose landing is relayed
      int vg = 0, v_end = 0, req = 0;   // next block to forward, end of the current request's blocks, requests started
      int wi = 0;
      Work r = get_work<WM>(P, tile, 0);
      auto skip_empty = [&] {
        while (wi < tile.n_work && r.blk_hi <= r.blk_lo) { ++wi; if (wi < tile.n_work) r = get_work<WM>(P, tile, wi); }
        if (wi < tile.n_work) v_end = vg + (r.blk_hi - r.blk_lo);
      };
      skip_empty();
      enum { kNeedQ, kWaitQt, kForward };
      int state = kNeedQ, idle = 0;
      bool alive = true;
      auto v_empty_after = [&](int gg) { return tc::mbar_test_wait(bar(V_EMPTY0 + (gg & 1)), (gg >> 1) & 1); };   // P V of block gg has completed
      while (alive && (kg < total || wi < tile.n_work)) {
        bool did = false;
        if (kg < total && tc::mbar_test_wait(bar(K_LAND0 + kg % kKStages), (kg / kKStages) & 1)) {
          tc::fence_proxy_async_smem();        // rows written by cp.async / plain stores -> bulk copies and the tensor pipe
          tc::mbar_arrive_cluster(lbar(K_FULL0 + kg % kKStages));
          FMLA_PTRACE_AT(kg, 15);
          ++kg;
          did = true;
        }
        if (wi < tile.n_work) {
          if (state == kNeedQ) {
            // every S of the previous request has completed (Q in shared and tensor memory free) and its last two
            // P V have released the V stages the new Q is staged in
            if (tc::mbar_test_wait(bar(Q_EMPTY), (req & 1) ^ 1) && (vg < 1 || v_empty_after(vg - 1)) && (vg < 2 || v_empty_after(vg - 2))) {
              const uint32_t q_bar = rank == 0 ? bar(Q_FULL) : bar(Q_LAND);
              tc::mbar_arrive_expect_tx(q_bar, kQBytes);
#pragma unroll
              for (int c = 0; c < 9; ++c)
                tc::tma_load_4d(c < kQTmemChunks ? sV + c * kChunkBytes : sQ + (c - kQTmemChunks) * kChunkBytes, &tmap_q, c * 64, tile.head0,
                                PREFILL ? r.batch : tile.sq, PREFILL ? 0 : r.batch, q_bar);
              state = kWaitQt;
              did = true;
            }
          } else if (state == kWaitQt) {
            if (tc::mbar_test_wait(bar(QT_DONE), req & 1)) {       // in both CTAs: the commit goes to both
              ++req;
              state = kForward;
              did = true;
            }
          } else if (vg < kg && (vg < 2 || v_empty_after(vg - 2))) {
            // the rows of block vg have landed (and were fenced above); P V of block vg-2 has completed in both CTAs
            // (its commit goes to both): both V stages are free
            const int kst = vg % kKStages, vst = vg & 1;
            FMLA_PTRACE_AT(vg, 12);
#ifdef FMLA_EXP_NO_FWD          // timing experiment only: results are wrong
            tc::mbar_arrive(bar(V_LAND0 + vst));
#else
            tc::mbar_arrive_expect_tx(bar(V_LAND0 + vst), kVStageBytes);      // 16 KB from this CTA, 16 KB from the peer
#pragma unroll
            for (int d = 0; d < 2; ++d) {
              const uint32_t dest = rank ^ static_cast<uint32_t>(d);
              const uint32_t dst_bar = tc::mapa(bar(V_LAND0 + vst), dest);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int chunk = (i >> 1) * 4 + 2 * static_cast<int>(dest) + (i & 1);     // value columns 64*chunk ..
                const uint32_t src = sK + kst * kKStageBytes + chunk * kKChunkBytes;
                const uint32_t dst = tc::mapa(sV + vst * kVStageBytes + i * kChunkBytes + rank * kKChunkBytes, dest);
                asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
                             "r"(src), "r"(kKChunkBytes), "r"(dst_bar)
                             : "memory");
              }
            }
#endif
            ++vg;
            did = true;
            if (vg == v_end) {
              ++wi;
              if (wi < tile.n_work) r = get_work<WM>(P, tile, wi);
              skip_empty();
              state = kNeedQ;
            }
          }
        }
        if (did) {
          idle = 0;
        } else if (++idle > tc::kSpinLimit) {
          tc::report_status(status, 112);
          alive = false;
        }
      }
    }
  } else if (warp == 6) {
    // ================================ V loader =========================================
    // Also loads Q: chunks 6..8 go to their place, chunks 0..5 are staged in the V ring (48 of its 64 KB) until the
    // leader has copied them into tensor memory -- once every S of the previous request has completed (Q in shared
    // and tensor memory free) and its last two P V have released the V stages.
    if (tc::elect_one()) {
      tc::prefetch_tensormap(&tmap_q);
      tc::prefetch_tensormap(&tmap_v64);
      int g = 0, req = 0;
      bool alive = true;
      for (int wi = 0; wi < tile.n_work && alive; ++wi) {
        const Work r = get_work<WM>(P, tile, wi);
        if (r.blk_hi == r.blk_lo) continue;
        alive = tc::mbar_wait(bar(Q_EMPTY), (req & 1) ^ 1, status, 101);
        for (int gg = max(0, g - 2); gg < g && alive; ++gg) alive = tc::mbar_wait(bar(V_EMPTY0 + (gg & 1)), (gg >> 1) & 1, status, 103);
        if (!alive) break;
        {
          const uint32_t q_bar = rank == 0 ? bar(Q_FULL) : bar(Q_LAND);
          tc::mbar_arrive_expect_tx(q_bar, kQBytes);
#pragma unroll
          for (int c = 0; c < 9; ++c)
            tc::tma_load_4d(c < kQTmemChunks ? sV + c * kChunkBytes : sQ + (c - kQTmemChunks) * kChunkBytes, &tmap_q, c * 64, tile.head0,
                            tile.sq, r.batch, q_bar);
        }
        alive = tc::mbar_wait(bar(QT_DONE), req & 1, status, 107);       // the V ring may be refilled
        if (!alive) break;
        ++req;
        const int* bt = p.block_table + r.batch * p.block_table_stride_b;
        for (int blk = r.blk_lo; blk < r.blk_hi; ++blk, ++g) {
          const int st = g & 1;
          const int page = __ldg(bt + blk);
          alive = tc::mbar_wait(bar(V_EMPTY0 + st), ((g >> 1) & 1) ^ 1, status, 103);
          if (!alive) break;
          FMLA_PTRACE_AT(g, 12);
#ifdef FMLA_EXP_NO_V_LOAD      // timing experiment only: results are wrong
          tc::mbar_arrive(bar(V_LAND0 + st));
          (void)page;
#else
          tc::mbar_arrive_expect_tx(bar(V_LAND0 + st), kVStageBytes);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int chunk = (i >> 1) * 4 + 2 * static_cast<int>(rank) + (i & 1);     // value columns 64*chunk ..
            tc::tma_load_4d(sV + st * kVStageBytes + i * kChunkBytes, &tmap_v64, chunk * 64, tile.kh, 0, page, bar(V_LAND0 + st));
          }
#endif
        }
      }
    }
  } else if (warp == 7) {
    // ================================ V relay ==========================================
    int g = 0;
    bool alive = true;
    for (int wi = 0; wi < tile.n_work && alive; ++wi) {
      const Work r = get_work<WM>(P, tile, wi);
      for (int blk = r.blk_lo; blk < r.blk_hi && alive; ++blk, ++g) {
        const int st = g & 1;
        alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(V_LAND0 + st), (g >> 1) & 1, status, 104));
        if (!alive) break;
        const int rows_valid = SPARSE ? 64 : r.seqlen - blk * 64;
        if (rows_valid < 64) {
          unsigned char* stage = smem + V_OFF + st * kVStageBytes;
          const int nrows = 64 - rows_valid;
          for (int i = lane; i < nrows * 32; i += 32) {
            const int row = rows_valid + (i >> 5), c16 = i & 31;            // 4 chunks x 8 pieces of 16 bytes per row
            *reinterpret_cast<uint4*>(stage + (c16 >> 3) * kChunkBytes + row * 128 + (c16 & 7) * 16) = make_uint4(0, 0, 0, 0);
          }
          tc::fence_proxy_async_smem();
          __syncwarp();
        }
        if (lane == 0) {
          FMLA_PTRACE_AT(g, 13);
          tc::mbar_arrive_cluster(lbar(V_FULL0 + st));
          if constexpr (SPARSE) {       // every copy out of K stage g % 3 of either CTA into this V stage has completed
            tc::mbar_arrive_cluster(tc::mapa(bar(K_EMPTY0 + g % kKStages), 0));
            tc::mbar_arrive_cluster(tc::mapa(bar(K_EMPTY0 + g % kKStages), 1));
          }
        }
      }
    }
  } else if (warp == 5 && rank != 0) {
    // ================================ Q / K relay (peer only) ==========================
    int g = 0, req = 0;
    bool alive = true;
    for (int wi = 0; wi < tile.n_work && alive; ++wi) {
      const Work r = get_work<WM>(P, tile, wi);
      if (r.blk_hi == r.blk_lo) continue;
      alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(Q_LAND), req & 1, status, 111));
      if (!alive) break;
      if (lane == 0) tc::mbar_arrive_cluster(lbar(Q_FULL));
      for (int blk = r.blk_lo; blk < r.blk_hi && alive && !SPARSE; ++blk, ++g) {      // sparse modes: warp 6 relays K
        const int st = g % kKStages;
        alive = __all_sync(0xffffffffu, tc::mbar_wait(bar(K_LAND0 + st), (g / kKStages) & 1, status, 112));
        if (alive && lane == 0) tc::mbar_arrive_cluster(lbar(K_FULL0 + st));
      }
      ++req;
    }
  } else if (warp == 5) {
    // ================================ MMA issuer (leader only) =========================
    if (rank == 0) {
      constexpr uint32_t idesc_s = tc::idesc_bf16_f32(128, 64, 0, 0, F16);
      constexpr uint32_t idesc_o = tc::idesc_bf16_f32(128, 256, 0, 1, F16);
      const uint64_t desc_q = tc::smem_desc_sw128(sQ, 16, 1024);             // A of S, chunks 6..8: K-major
      const uint64_t desc_qstage = tc::smem_desc_sw128(sV, 16, 1024);                  // chunks 0..5 of Q where the loader stages them (the V ring)
      const uint64_t desc_k = tc::smem_desc_sw128(sK, 16, 1024);             // B of S: K-major, 32 rows per CTA (stage 0)
      const uint64_t desc_p = tc::smem_desc_sw128(sP, 16, 1024);             // A of PV: K-major
      const uint64_t desc_v = tc::smem_desc_sw128(sV, kChunkBytes, 1024);    // B of PV: MN-major, 64-wide column groups 8 KB apart
      // every commit goes to the barrier copy of each CTA (two plain commits, each naming one barrier)
      auto commit_both = [&](int b) {
        tc::tc_commit_pair(bar(b));
        tc::tc_commit_pair(tc::mapa(bar(b), 1));
      };
      int g = 0, req = 0;
      bool alive = true;
#ifdef FMLA_TRACE
      int seen_k = -1, seen_s = -1, seen_p = -1, seen_v = -1, after_issue = 0;
#endif
      for (int wi = 0; wi < tile.n_work && alive; ++wi) {
        const Work r = get_work<WM>(P, tile, wi);
        const int nblk = r.blk_hi - r.blk_lo;
        if (nblk == 0) continue;
        alive = __all_sync(0xffffffffu, tc::mbar_wait_cluster(bar(Q_FULL), req & 1, status, 105));
        if (!alive) break;
        // Q chunks 0..5: shared memory -> tensor memory of both CTAs (8 copies of 64 rows x 16 bytes per chunk)
        tc::tc_fence_after();
        if (tc::elect_one()) {
#pragma unroll
          for (int c = 0; c < kQTmemChunks; ++c)
#pragma unroll
            for (int sub = 0; sub < 8; ++sub)
              tmem_cp_pair_64x128b(tmem + TMEM_Q + c * 32 + sub * 4, tc::desc_advance(desc_qstage, c * kChunkBytes + sub * 16));
          commit_both(QT_DONE);
        }
        __syncwarp();
        // One poll reads every barrier of interest, one per lane:
        //   lane 0 P_FULL(jp)  lane 1 O_EMPTY  lane 2 V_FULL(jp)  lane 3 S_EMPTY(js)  lane 4 K_FULL(js)
        int js = 0, jp = 0, idle = 0;
        while (jp < nblk && alive) {
#ifdef FMLA_TRACE
          if (lane == 0 && after_issue && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == FMLA_TRACE_PART) {   // first pass through the loop head after an issue: rank-0 slots 1 / 10 hold ns
            if (after_issue == 1) g_pair_head[(g + js - 1) & 255][0] = gtime(); else g_pair_head[(g + jp - 1) & 255][1] = gtime();
          }
          after_issue = 0;
#endif
          const int gs = g + min(js, nblk - 1), sbs = gs & 1, kst = gs % kKStages;
          const uint32_t phs = (gs >> 1) & 1, phk = (gs / kKStages) & 1;
          const int gp = g + jp, stp = gp & 1;
          const uint32_t php = (gp >> 1) & 1;
          int pb = P_FULL0 + stp;
          uint32_t pp = php;
          if (lane == 1) { pb = O_EMPTY; pp = (req & 1) ^ 1; }
          if (lane == 2) { pb = V_FULL0 + stp; pp = php; }
          if (lane == 3) { pb = S_EMPTY0 + sbs; pp = phs ^ 1; }
          if (lane >= 4) { pb = K_FULL0 + kst; pp = phk; }
          const bool hit = lane < 5 && tc::mbar_test_wait_cluster(bar(pb), pp);
          const uint32_t m = __ballot_sync(0xffffffffu, hit);
#ifdef FMLA_TRACE
          if (lane == 0) {     // first time each input of the next S / P V is seen ready (rank-1 slots 3..6 of the timeline)
            if ((m & 0x10u) && js < nblk && seen_k != gs) { seen_k = gs; FMLA_GTRACE_AT(gs, 1, 3); }
            if ((m & 0x8u) && js < nblk && seen_s != gs) { seen_s = gs; FMLA_GTRACE_AT(gs, 1, 4); }
            if ((m & 0x1u) && jp < js && seen_p != gp) { seen_p = gp; FMLA_GTRACE_AT(gp, 1, 5); }
            if ((m & 0x4u) && jp < js && seen_v != gp) { seen_v = gp; FMLA_GTRACE_AT(gp, 1, 6); }
          }
#endif
          bool did = false;
          if (jp < js && (m & 5u) == 5u && (jp > 0 || (m & 2u))) {
            tc::tc_fence_after();
            if (lane == 0) { FMLA_PTRACE_AT(gp, 4); FMLA_GTRACE_AT(gp, 0, 5); }
            if (tc::elect_one()) {
#ifndef FMLA_EXP_NO_PV         // timing experiment only: results are wrong
              pv_block_pair(tmem + TMEM_O, tc::desc_advance(desc_p, stp * kChunkBytes), tc::desc_advance(desc_v, stp * kVStageBytes), idesc_o, jp == 0);
#endif
              commit_both(V_EMPTY0 + stp);
              commit_both(P_EMPTY0 + stp);
              FMLA_PTRACE_AT(gp, 5);
              FMLA_GTRACE_AT(gp, 0, 6);
            }
            __syncwarp();
            ++jp;
            did = true;
#ifdef FMLA_TRACE
            after_issue = 2;
#endif
          } else if (js < nblk && (m & 0x18u) == 0x18u) {
            if constexpr (SPARSE) tc::fence_proxy_async_smem();    // K rows came through cp.async / plain stores
            tc::tc_fence_after();
            if (lane == 0) { FMLA_PTRACE_AT(gs, 2); FMLA_GTRACE_AT(gs, 0, 3); }
            if (tc::elect_one()) {
              s_block_pair(tmem + TMEM_S + sbs * 32, tmem + TMEM_Q, desc_q, tc::desc_advance(desc_k, kst * kKStageBytes), idesc_s);
              commit_both(S_FULL0 + sbs);
              commit_both(K_EMPTY0 + kst);
              FMLA_PTRACE_AT(gs, 3);
              FMLA_GTRACE_AT(gs, 0, 4);
              if (js == nblk - 1) commit_both(Q_EMPTY);
            }
            __syncwarp();
            ++js;
            did = true;
#ifdef FMLA_TRACE
            after_issue = 1;
#endif
          }
          if (did) {
            idle = 0;
          } else if (++idle > tc::kSpinLimit) {
            if (lane == 0) tc::report_status(status, 106);
            alive = false;
          }
#ifdef FMLA_PAIR_POLL_SLEEP
          else { __nanosleep(FMLA_PAIR_POLL_SLEEP); }
#endif
        }
        g += nblk;
        if (alive && tc::elect_one()) commit_both(O_FULL);
        __syncwarp();
        ++req;
      }
    }
  } else if (warp < 4) {
    // ================================ softmax / epilogue ================================
    const int r_row = tid & 63, th = tid >> 6;           // TMEM lane tid: row tid%64, token/column half tid/64
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t l_s_empty0 = lbar(S_EMPTY0), l_p_full0 = lbar(P_FULL0), l_o_empty = lbar(O_EMPTY);
    int g = 0, req = 0;
    bool aborted = false;        // uniform over the 128 softmax threads: only read right after a bar_sync
    for (int wi = 0; wi < tile.n_work; ++wi) {
      const Work r = get_work<WM>(P, tile, wi);
      const int nblk = r.blk_hi - r.blk_lo;
      float m_run = neg_inf();     // running maximum (base-2 scaled logits)
      float m_used = 0.f;          // the maximum O and l are currently scaled with
      float l_part = 0.f;          // this thread's share of the row sum
      for (int j = 0; j < nblk && !aborted; ++j, ++g) {
        const int st = g & 1;
        uint32_t sv[32];
        uint32_t vbits = 0xffffffffu;
        if (tc::mbar_wait(bar(S_FULL0 + st), (g >> 1) & 1, status, 108)) {
          if (tid == 0) { FMLA_PTRACE_AT(g, 6); FMLA_GTRACE_AT(g, rank, 0); }
          tc::tc_fence_after();
          tc::tmem_ld32(tmem + lane_addr + TMEM_S + st * 32, sv);
          tc::tmem_wait_ld();
          tc::tc_fence_before();
        } else {
          *sAbort = 1;
#pragma unroll
          for (int i = 0; i < 32; ++i) sv[i] = 0u;
        }
        __syncwarp();
        if (lane == 0) tc::mbar_arrive_cluster(l_s_empty0 + st * 8);
        if (tid == 0) { FMLA_PTRACE_AT(g, 7); FMLA_GTRACE_AT(g, rank, 1); }

        if constexpr (SPARSE) {
          vbits = sValid[(g % 6) * 2 + th];
        } else {
          const int tok0 = (r.blk_lo + j) * 64 + th * 32;
          if (tok0 + 32 > r.border) vbits = tok0 >= r.border ? 0u : (0xffffffffu >> (32 - (r.border - tok0)));
        }
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
        if (tid == 0) FMLA_PTRACE_AT(g, 8);
        mx = fmaxf(mx, xch[tid ^ 64]);
        const float m_new = fmaxf(m_run, mx);

        bool need = false;
        if (j == 0 || (m_run == neg_inf() && m_new != neg_inf())) {
          m_used = (m_new == neg_inf()) ? 0.f : m_new;      // O and l are exactly zero so far
        } else {
          need = (m_new - m_used) > kRescaleThreshold;
        }
        m_run = m_new;
        const bool any_need = __any_sync(0xffffffffu, need);
        // P has two buffers (block g uses buffer g & 1): writing it needs P V of block g-2 to be complete;
        // rescaling O needs every earlier P V to be complete, i.e. that of block g-1 (they complete in order)
        if (any_need) {
          if (j > 0 && !tc::mbar_wait(bar(P_EMPTY0 + ((g - 1) & 1)), ((g - 1) >> 1) & 1, status, 109)) *sAbort = 1;
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
        if (!tc::mbar_wait(bar(P_EMPTY0 + st), ((g >> 1) & 1) ^ 1, status, 109)) *sAbort = 1;
        if (tid == 0) FMLA_PTRACE_AT(g, 9);
        // P[row][th*32 .. +32) -> K-major 128B-swizzled A operand: 16-byte chunk (th*4 + q) ^ (row & 7)
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4)
          pst_shared_v4(sP + st * kChunkBytes + r_row * 128 + ((((th * 4 + q4) ^ (r_row & 7))) << 4),
                        make_uint4(pk[q4 * 4], pk[q4 * 4 + 1], pk[q4 * 4 + 2], pk[q4 * 4 + 3]));
        tc::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive_cluster(l_p_full0 + st * 8);
        if (tid == 0) { FMLA_PTRACE_AT(g, 11); FMLA_GTRACE_AT(g, rank, 2); }
      }

      // ---- epilogue of this work item ---------------------------------------------------
      float* xch = sMx + 256;
      if (tid == 0) FMLA_PTRACE_AT(g - 1, 14);
      bar_sync(1, 128);
      xch[tid] = l_part;
      bar_sync(1, 128);
      if (*sAbort) aborted = true;
      if (aborted) break;
      const float l = l_part + xch[tid ^ 64];
      const int head = tile.head0 + r_row;
      const float inv = (l == 0.f || nblk == 0) ? 0.f : 1.f / l;
      bool have_o = nblk > 0;
      if (have_o) {
        if (!tc::mbar_wait(bar(O_FULL), req & 1, status, 110)) { *sAbort = 1; have_o = false; }
        tc::tc_fence_after();
      }
      const int q_seq_per_hk = PREFILL ? 0 : p.s_q * p.hq_per_hk;
      const int row_in_group = PREFILL ? 0 : tile.sq * p.hq_per_hk + tile.hb * 64 + r_row;   // regrouped row index within the kv head
      __nv_bfloat16* o_final = PREFILL
          ? reinterpret_cast<__nv_bfloat16*>(P.sp.out) + ((int64_t)r.batch * P.sp.h_q + head) * 512
          : reinterpret_cast<__nv_bfloat16*>(p.out) + r.batch * p.o_stride_b + tile.sq * p.o_stride_s + head * p.o_stride_h;
      const int64_t part_row = PREFILL ? 0 : ((int64_t)r.split_slot * p.h_k + tile.kh) * q_seq_per_hk + row_in_group;
      float* o_part = PREFILL ? nullptr : p.o_accum + part_row * 512;
      // The read of chunk c + 1 is in flight while chunk c is scaled and stored (two register sets), and every store
      // is one full 32-byte sector per thread (each thread writes its own row, so the rows of a warp instruction are
      // 1 KB or 2 KB apart: with 16-byte stores the load/store unit handled twice as many half-filled sectors).
      constexpr int kSets = WM == kSparseDecode ? 1 : 2;      // the FP8 decode (480 threads, 128 registers) has no room for a second set
      uint32_t ov[kSets][32];
      if (have_o && kSets == 2) tc::tmem_ld32(tmem + lane_addr + TMEM_O, ov[0]);
#pragma unroll 2
      for (int c = 0; c < 8; ++c) {
        uint32_t* cur = ov[c % kSets];
        if (have_o) {
          if constexpr (kSets == 1) tc::tmem_ld32(tmem + lane_addr + TMEM_O + c * 32, ov[0]);
          tc::tmem_wait_ld();
          if (kSets == 2 && c + 1 < 8) tc::tmem_ld32(tmem + lane_addr + TMEM_O + (c + 1) * 32, ov[(c + 1) % kSets]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) cur[i] = 0u;
        }
        const int col = (c >> 2) * 256 + th * 128 + (c & 3) * 32;
        if (r.no_split) {
#pragma unroll
          for (int q8 = 0; q8 < 2; ++q8) {
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
              w[i] = pack_16x2<F16>(__uint_as_float(cur[q8 * 16 + 2 * i]) * inv, __uint_as_float(cur[q8 * 16 + 2 * i + 1]) * inv);
            st_global_32B(o_final + col + q8 * 16, w);
          }
        } else {
#pragma unroll
          for (int q8 = 0; q8 < 4; ++q8) {
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = __float_as_uint(__uint_as_float(cur[q8 * 8 + i]) * inv);
            st_global_32B(o_part + col + q8 * 8, w);
          }
        }
      }
      if (nblk > 0) {
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive_cluster(l_o_empty);
        ++req;
      }
      if (tid == 0) FMLA_PTRACE_AT(g - 1, 15);
      if constexpr (PREFILL) {
        if (th == 0) {      // base-2 quantities; a row without any valid index gives out 0, max_logits -inf, lse -inf
          const int64_t o = (int64_t)r.batch * P.sp.h_q + head;
          P.sp.max_logits[o] = inv == 0.f ? neg_inf() : m_run;
          P.sp.lse[o] = inv == 0.f ? neg_inf() : log2f(l) + m_used;
        }
      } else if (th == 0) {
        if (r.no_split) {
          p.softmax_lse[((int64_t)r.batch * p.h_q + head) * p.s_q + tile.sq] = inv == 0.f ? pos_inf() : (log2f(l) + m_used) * kLn2;
        } else {
          p.lse_accum[part_row] = inv == 0.f ? neg_inf() : log2f(l) + m_used;
          if (p.no_split_hint && tid == 0) tc::report_status(status, 41);     // a split request although the caller ruled it out
        }
      }
      // ---- merge of a split request by whoever delivers its last partial ----------------
      // Every CTA that has written a partial of (request, query token, this 64-head tile) counts itself in; the one
      // that completes the count reads all partials back (they were written during this kernel: coherent loads)
      // and writes the final rows, math of csrc/smxx/mla_combine.cu:71-107, 128-151.  The counter returns to zero.
      if (!PREFILL && !r.no_split && p.arrival_counters != nullptr) {
        __threadfence();
        bar_sync(1, 128);
        int* sMerge = reinterpret_cast<int*>(smem + MISC_OFF + 16);
        if (tid == 0) {
          const int lo = __ldg(p.num_splits + r.batch), nsp = __ldg(p.num_splits + r.batch + 1) - lo;
          const int n_hb = p.hq_per_hk >> 6;
          int* ctr = p.arrival_counters + (((int64_t)r.batch * p.s_q + tile.sq) * p.h_k + tile.kh) * n_hb + tile.hb;
          const bool last = atomicAdd(ctr, 1) == nsp - 1;
          if (last) *ctr = 0;
          sMerge[0] = last ? nsp : 0;
          sMerge[1] = lo;
        }
        bar_sync(1, 128);
        const int nsp = sMerge[0], lo = sMerge[1];
        if (nsp > 0) {
          __threadfence();
          const int64_t rows_per_slot = (int64_t)p.h_k * q_seq_per_hk;
          for (int rr = 0; rr < 16; ++rr) {
            const int row = warp * 16 + rr;                              // one warp per row, 16 rows per warp
            const int64_t prow = ((int64_t)lo * p.h_k + tile.kh) * q_seq_per_hk + tile.sq * p.hq_per_hk + tile.hb * 64 + row;
            const float* lse_p = p.lse_accum + prow;
            float mx = neg_inf();
            for (int i = lane; i < nsp; i += 32) mx = fmaxf(mx, __ldcv(lse_p + i * rows_per_slot));
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            if (mx == neg_inf()) mx = 0.f;
            float sum = 0.f;
            for (int i = lane; i < nsp; i += 32) sum += exp2f(__ldcv(lse_p + i * rows_per_slot) - mx);
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            const float glse = (sum == 0.f || sum != sum) ? pos_inf() : log2f(sum) + mx;
            const int hd = tile.head0 + row;
            if (lane == 0) p.softmax_lse[((int64_t)r.batch * p.h_q + hd) * p.s_q + tile.sq] = glse * kLn2;
            float4 acc[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int i = 0; i < nsp; ++i) {
              const float w = exp2f(__ldcv(lse_p + i * rows_per_slot) - glse);
              if (w == 0.f) continue;
              const float4* src = reinterpret_cast<const float4*>(p.o_accum + (prow + i * rows_per_slot) * 512);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float4 v = __ldcv(src + j * 32 + lane);
                acc[j].x += w * v.x; acc[j].y += w * v.y; acc[j].z += w * v.z; acc[j].w += w * v.w;
              }
            }
            __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + r.batch * p.o_stride_b + tile.sq * p.o_stride_s + hd * p.o_stride_h;
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<uint2*>(orow + (j * 32 + lane) * 4) =
                  make_uint2(pack_16x2<F16>(acc[j].x, acc[j].y), pack_16x2<F16>(acc[j].z, acc[j].w));
          }
        }
      }
    }
  }

  // neither CTA may leave (or give its tensor memory back) while its peer can still address it
  tc::tc_fence_before();
  __syncthreads();
  tc::cluster_sync_all();
  if (warp == 5) tc::tmem_dealloc_pair(tmem, 512);
#ifdef FMLA_TRACE
  if (tid == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_pair_span[(blockIdx.z * gridDim.x + blockIdx.x) * 2 + 1] = (long long)t;
  }
#endif
}

// ---- host side ----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn pair_encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess) f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// 16-bit tensor [d3][d2][d1][d0=576] with element strides s1,s2,s3 ; box {64, b1, b2, 1}
static bool pair_map_4d(CUtensorMap* m, const void* base, uint64_t d1, uint64_t d2, uint64_t d3, int64_t s1, int64_t s2, int64_t s3,
                        uint32_t b1, uint32_t b2) {
  EncodeTiledFn enc = pair_encode_fn();
  if (!enc) return false;
  cuuint64_t dims[4] = {576, d1, d2, d3};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(s1) * 2, static_cast<cuuint64_t>(s2) * 2, static_cast<cuuint64_t>(s3) * 2};
  cuuint32_t box[4] = {64, b1, b2, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool decode_sparse_pair_applies(const DecodeKernelParams& p) { return p.h_k == 1 && p.hq_per_hk == 128 && !p.is_f16; }

cudaError_t launch_decode_sparse_pair(const DecodeKernelParams& p, cudaStream_t stream) {
  TcParams P = {};
  P.d = p;
  CUtensorMap tq;
  // q [b][s_q][h_q][576] ; box = 64 heads x 64 columns
  if (!pair_map_4d(&tq, p.q, p.h_q, p.s_q, p.b, p.q_stride_h, p.q_stride_s, p.q_stride_b, 64, 1)) return cudaErrorInvalidValue;
  auto kern = mla_pair_kernel<false, kSparseDecode>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ptc::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  kern<<<dim3(2, p.s_q, p.num_sm_parts), ptc::kSparseDecodeThreads, ptc::SMEM_BYTES, stream>>>(P, tq, tq, tq);   // the K / V maps are not used in this mode
  return cudaGetLastError();
}

bool sparse_prefill_pair_applies(const SparsePrefillKernelParams& sp) { return sp.h_q == 128; }

cudaError_t launch_sparse_prefill_pair(const SparsePrefillKernelParams& sp, cudaStream_t stream) {
  TcParams P = {};
  P.sp = sp;
  CUtensorMap tq;
  // q [s_q][h_q][576] as (col, head, token, 1)
  if (!pair_map_4d(&tq, sp.q, sp.h_q, sp.s_q, 1, sp.q_stride_h, sp.q_stride_s, sp.q_stride_s * sp.s_q, 64, 1)) return cudaErrorInvalidValue;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 148;
  const int lanes = max(1, min(sp.s_q, sms / 2));
  auto kern = mla_pair_kernel<false, kSparsePrefill>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ptc::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  kern<<<dim3(2, lanes, 1), ptc::kPrefillThreads, ptc::SMEM_BYTES, stream>>>(P, tq, tq, tq);    // the K / V maps are not used in this mode
  return cudaGetLastError();
}

bool decode_dense_pair_applies(const DecodeKernelParams& p) { return p.hq_per_hk % 128 == 0; }

cudaError_t launch_decode_dense_pair(const DecodeKernelParams& p, cudaStream_t stream) {
  TcParams P = {};
  P.d = p;
  static const int prefetch = [] {
    const char* v = getenv("FMLA_PAIR_PREFETCH");
    return v ? atoi(v) : 0;
  }();
  P.d.l2_prefetch_dist = prefetch;
  CUtensorMap tq, tk, tv;
  // q [b][s_q][h_q][576] ; box = 64 heads x 64 columns
  if (!pair_map_4d(&tq, p.q, p.h_q, p.s_q, p.b, p.q_stride_h, p.q_stride_s, p.q_stride_b, 64, 1)) return cudaErrorInvalidValue;
  // cache [num_blocks][64][h_k][576] addressed as (col, head, row-in-page, page): boxes of 32 rows (K part) and 64 rows (V part)
  if (!pair_map_4d(&tk, p.kcache, p.h_k, 64, p.num_blocks, p.k_stride_head, p.k_stride_row, p.k_stride_block, 1, 32)) return cudaErrorInvalidValue;
  if (!pair_map_4d(&tv, p.kcache, p.h_k, 64, p.num_blocks, p.k_stride_head, p.k_stride_row, p.k_stride_block, 1, 64)) return cudaErrorInvalidValue;
  const int n_hb = p.hq_per_hk / 64;
  const dim3 grid(p.s_q * n_hb, p.h_k, p.num_sm_parts);
  static bool attr_set[2] = {false, false};      // idempotent, so a race between threads is harmless
  if (p.is_f16) {
    auto kern = mla_pair_kernel<true, kDense>;
    if (!attr_set[1]) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ptc::SMEM_BYTES);
      if (e != cudaSuccess) return e;
      attr_set[1] = true;
    }
    kern<<<grid, ptc::kThreads, ptc::SMEM_BYTES, stream>>>(P, tq, tk, tv);
  } else {
    auto kern = mla_pair_kernel<false, kDense>;
    if (!attr_set[0]) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ptc::SMEM_BYTES);
      if (e != cudaSuccess) return e;
      attr_set[0] = true;
    }
    kern<<<grid, ptc::kThreads, ptc::SMEM_BYTES, stream>>>(P, tq, tk, tv);
  }
  return cudaGetLastError();
}

#ifdef FMLA_TRACE
extern "C" int fmla_debug_read_pair_trace(long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_pair_trace, sizeof(long long) * n);
}
extern "C" int fmla_debug_read_pair_gt(long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_pair_gt, sizeof(long long) * n);
}
extern "C" int fmla_debug_read_pair_head(long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_pair_head, sizeof(long long) * n);
}
extern "C" int fmla_debug_read_pair_span(long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_pair_span, sizeof(long long) * n);
}
#endif

cudaError_t set_status_mirror_pair(int* mapped_host_word) { return tc::set_status_mirror(mapped_host_word); }

cudaError_t read_decode_pair_status(int* host_status, bool reset) {
  cudaError_t e = cudaMemcpyFromSymbol(host_status, g_decode_pair_status, sizeof(int));
  if (e != cudaSuccess) return e;
  if (reset && *host_status != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_decode_pair_status, &zero, sizeof(int));
  }
  return e;
}

}  // namespace fmla
