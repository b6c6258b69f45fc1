// Split-KV tile scheduler: cuts the (request, 64-token block) work list of a
// decode batch into num_sm_parts contiguous, block-balanced partitions.
//
// Same algorithm and output contract as csrc/smxx/get_mla_metadata.cu:8-89
// (greedy walk with a fixed per-visit overhead of 5 blocks), restructured as a
// block-wide prefix sum followed by a serial walk over partitions on one
// thread; batch size is unbounded (request sizes are re-read from global memory
// instead of being staged in shared memory).  Words 5..7 of each row are
// written as zero.  An inconsistent walk cannot occur for valid inputs; it is
// not asserted on the device.
#include "kernels.h"

namespace fmla {

constexpr int kFixedOverheadBlocks = 5;   // csrc/pybind.cpp:308,323,341
constexpr int kBlockN = 64;

__global__ void __launch_bounds__(256) get_mla_metadata_kernel(const int* __restrict__ seqlens_k, int batch,
                                                              int num_sm_parts, int topk, int* __restrict__ md,
                                                              int* __restrict__ num_splits) {
  __shared__ int s_partial[256];
  int local = 0;
  for (int i = threadIdx.x; i < batch; i += blockDim.x) {
    const int len = topk == -1 ? seqlens_k[i] : topk;
    local += max(len - 1, 0) / kBlockN + 1 + kFixedOverheadBlocks;
  }
  s_partial[threadIdx.x] = local;
  __syncthreads();
  for (int off = 128; off >= 1; off >>= 1) {
    if (threadIdx.x < off) s_partial[threadIdx.x] += s_partial[threadIdx.x + off];
    __syncthreads();
  }
  if (threadIdx.x != 0) return;
  const int total = s_partial[0];
  const int payload = (total + num_sm_parts - 1) / num_sm_parts + kFixedOverheadBlocks;

  auto len_of = [&](int i) { return topk == -1 ? seqlens_k[i] : topk; };
  auto blocks_of = [&](int i) { return max(len_of(i) - 1, 0) / kBlockN + 1; };

  int now_idx = 0, now_block = 0, now_split = 0, cum = 0;
  num_splits[0] = 0;
  for (int i = 0; i < num_sm_parts; ++i) {
    int row[8] = {now_idx, now_block, 0, 0, now_split, 0, 0, 0};
    int remain = payload;
    while (now_idx < batch) {
      const int rem_blocks = blocks_of(now_idx) - now_block;
      if (remain >= rem_blocks + kFixedOverheadBlocks) {
        cum += now_split + 1;
        num_splits[now_idx + 1] = cum;
        remain -= rem_blocks + kFixedOverheadBlocks;
        ++now_idx;
        now_block = 0;
        now_split = 0;
      } else {
        if (remain - kFixedOverheadBlocks > 0) {
          now_block += remain - kFixedOverheadBlocks;
          ++now_split;
          remain = 0;
        }
        break;
      }
    }
    if (now_block > 0) {
      row[2] = now_idx;
      row[3] = now_block;
    } else {
      row[2] = now_idx - 1;
      row[3] = now_idx >= 1 ? (len_of(now_idx - 1) == 0 ? 0 : blocks_of(now_idx - 1)) : 0;
    }
    int4* dst = reinterpret_cast<int4*>(md + i * 8);
    dst[0] = make_int4(row[0], row[1], row[2], row[3]);
    dst[1] = make_int4(row[4], 0, 0, 0);
  }
}

cudaError_t launch_get_mla_metadata(const int* seqlens_k, int batch, int num_sm_parts, int topk, int* md,
                                    int* num_splits, cudaStream_t stream) {
  get_mla_metadata_kernel<<<1, 256, 0, stream>>>(seqlens_k, batch, num_sm_parts, topk, md, num_splits);
  return cudaGetLastError();
}

}  // namespace fmla
