// Work decomposition shared by the MLA attention kernels (mla_tc.cu, mla_pair.cu): which tile of heads and
// which stretch of the split-KV schedule a CTA owns, and the requests / query tokens it walks.
#pragma once

#include "kernels.h"

namespace fmla {

enum TcMode { kDense = 0, kSparseDecode = 1, kSparsePrefill = 2 };

struct TcParams {
  DecodeKernelParams d;          // decode modes
  SparsePrefillKernelParams sp;  // prefill mode
};

// One unit of work of a CTA: a request (decode) or a query token (prefill) and the range of
// 64-token blocks of its key list that this CTA covers.
struct Work {
  int batch;                 // request index (decode) / query token (prefill)
  int blk_lo, blk_hi;
  int seqlen, border;        // dense: cached tokens, first masked token
  int split_slot;
  bool no_split;
  const int* idx;            // sparse: the index list of this (request, query token)
};

// Which tile and which stretch of the schedule a CTA owns.
struct Tile {
  int sq, hb, kh, head0, nvalid;
  int begin_idx, end_idx, begin_block, end_block, begin_split;
  int n_work;
};

template <int MODE>
__device__ __forceinline__ Tile make_tile(const TcParams& P) {
  Tile t;
  if constexpr (MODE == kSparsePrefill) {
    // persistent over query tokens: this CTA takes tokens blockIdx.y, blockIdx.y + gridDim.y, ... so that the
    // Q load and the output stores of one token overlap with the blocks of its neighbours
    t.hb = blockIdx.x; t.sq = blockIdx.y; t.kh = 0;
    t.head0 = t.hb * 64; t.nvalid = 64;
    t.begin_idx = t.end_idx = 0; t.begin_block = 0; t.end_block = P.sp.topk / 64; t.begin_split = 0;
    t.n_work = (P.sp.s_q - static_cast<int>(blockIdx.y) + static_cast<int>(gridDim.y) - 1) / static_cast<int>(gridDim.y);
  } else {
    const DecodeKernelParams& p = P.d;
    int part;
    if constexpr (MODE == kDense) {
      const int n_hb = (p.hq_per_hk + 63) >> 6;
      t.sq = blockIdx.x / n_hb; t.hb = blockIdx.x % n_hb; t.kh = blockIdx.y; part = blockIdx.z;
    } else {
      t.hb = blockIdx.x; t.sq = blockIdx.y; t.kh = 0; part = blockIdx.z;
    }
    t.head0 = t.kh * p.hq_per_hk + t.hb * 64;
    t.nvalid = min(64, p.hq_per_hk - t.hb * 64);
    const int4 md = __ldg(reinterpret_cast<const int4*>(p.tile_scheduler_metadata + part * 8));
    t.begin_idx = md.x; t.begin_block = md.y; t.end_idx = md.z; t.end_block = md.w;
    t.begin_split = __ldg(p.tile_scheduler_metadata + part * 8 + 4);
    t.n_work = t.begin_idx >= p.b ? 0 : t.end_idx - t.begin_idx + 1;
  }
  return t;
}

template <int MODE>
__device__ __forceinline__ Work get_work(const TcParams& P, const Tile& t, int i) {
  Work w;
  if constexpr (MODE == kSparsePrefill) {
    w.batch = t.sq + i * static_cast<int>(gridDim.y);          // the query token
    w.blk_lo = 0; w.blk_hi = P.sp.topk / 64;
    w.seqlen = P.sp.topk; w.border = P.sp.topk;
    w.split_slot = 0; w.no_split = true;
    w.idx = P.sp.indices + (int64_t)w.batch * P.sp.indices_stride_s;
  } else {
    const DecodeKernelParams& p = P.d;
    const int batch = t.begin_idx + i;
    w.batch = batch;
    int nblk_total, nblk_visible;
    if constexpr (MODE == kDense) {
      w.seqlen = __ldg(p.seqlens_k + batch);
      nblk_total = (w.seqlen + 63) >> 6;
      w.border = p.is_causal ? w.seqlen - (p.s_q - 1 - t.sq) : w.seqlen;
      nblk_visible = w.border > 0 ? (w.border + 63) >> 6 : 0;
      w.idx = nullptr;
    } else {
      w.seqlen = p.topk; w.border = p.topk;
      nblk_total = nblk_visible = p.topk >> 6;
      w.idx = p.indices + batch * p.indices_stride_b + t.sq * p.indices_stride_s;
    }
    w.blk_lo = batch == t.begin_idx ? t.begin_block : 0;
    w.blk_hi = min(min(batch == t.end_idx ? t.end_block : nblk_total, nblk_total), nblk_visible);
    if (w.blk_hi < w.blk_lo) w.blk_hi = w.blk_lo;
    const int lo = __ldg(p.num_splits + batch);
    w.no_split = !p.force_partial && __ldg(p.num_splits + batch + 1) - lo == 1;
    w.split_slot = lo + (batch == t.begin_idx ? t.begin_split : 0);
  }
  return w;
}

}  // namespace fmla
