// Split-KV tile scheduler: cuts the (request, 64-token block) work list of a decode batch into num_sm_parts
// contiguous partitions.
//
// Output contract of csrc/smxx/get_mla_metadata.cu:8-89 of the reference (rows [begin_idx, begin_block,
// end_idx inclusive, end_block exclusive, begin_n_split_idx, 0, 0, 0]; num_splits = exclusive prefix of the number
// of partitions that touch each request), computed differently: the reference walks the partitions one after
// the other on a single thread; here every cut is a closed-form position on the line of request costs, found
// by a binary search over the cost prefix sums, so all partitions are computed in parallel by one thread
// block (a few microseconds for any batch size).
//
//   cost of a request = its block count (a zero-length request counts one block) + a fixed overhead of 5,
//                       laid out on a line as [overhead | blocks]
//   cut k             = k * pitch on that line; pitch = ceil(total / parts) when there are more requests than
//                       parts (a partition then carries at most pitch + one overhead, the bound of the
//                       reference's greedy walk), ceil(total / parts) + overhead otherwise (the slack lets a
//                       batch of similar requests fall one request per partition instead of being cut everywhere)
//   a cut inside an overhead stretch moves to the start of that request
//   partition k       = everything between cuts k and k+1; equal cuts give an empty partition (begin_idx = batch)
// The integer statement of the same algorithm, against which the kernel is checked bit for bit, is
// oracle/scheduler.py:schedule_cut_ref.
#include "kernels.h"

namespace fmla {

constexpr int kFixedOverheadBlocks = 5;   // csrc/pybind.cpp:308,323,341
constexpr int kBlockN = 64;
constexpr int kSchedThreads = 1024;
constexpr int kMaxParts = 1023;           // one thread per cut

struct Cut { int req, off; };

// grid 1 x 1024.  num_splits ([batch + 1] ints) doubles as the scratch for the cost prefix sums: it is only
// overwritten with its final contents after every cut has been located.
__global__ void __launch_bounds__(kSchedThreads) get_mla_metadata_kernel(const int* __restrict__ seqlens_k, int batch,
                                                                         int num_sm_parts, int topk, int* __restrict__ md,
                                                                         int* __restrict__ num_splits) {
  __shared__ int s_scan[kSchedThreads];
  __shared__ int s_carry;
  __shared__ Cut s_cut[kMaxParts + 2];
  __shared__ unsigned char s_new[kMaxParts + 2];     // cut k differs from cut k-1
  const int tid = threadIdx.x;
  auto len_of = [&](int i) { return topk == -1 ? __ldg(seqlens_k + i) : topk; };
  auto real_blocks = [&](int i) { const int l = len_of(i); return l == 0 ? 0 : (l + kBlockN - 1) / kBlockN; };
  auto cost_of = [&](int i) { return max(real_blocks(i), 1) + kFixedOverheadBlocks; };

  // in-place exclusive scan of `n` values produced by value(i) into dst[0..n] (dst[n] = total), 1024 at a time
  auto exclusive_scan = [&](int n, auto value, int* dst) {
    if (tid == 0) s_carry = 0;
    __syncthreads();
    for (int base = 0; base < n; base += kSchedThreads) {
      const int i = base + tid;
      const int v = i < n ? value(i) : 0;
      s_scan[tid] = v;
      __syncthreads();
      for (int off = 1; off < kSchedThreads; off <<= 1) {
        const int add = tid >= off ? s_scan[tid - off] : 0;
        __syncthreads();
        s_scan[tid] += add;
        __syncthreads();
      }
      const int carry = s_carry;
      if (i < n) dst[i] = carry + s_scan[tid] - v;
      __syncthreads();
      if (tid == kSchedThreads - 1) s_carry = carry + s_scan[tid];
      __syncthreads();
    }
    if (tid == 0) dst[n] = s_carry;
    __syncthreads();
  };

  // 1. cost prefix sums -> num_splits (scratch use)
  exclusive_scan(batch, cost_of, num_splits);
  __threadfence_block();
  const int total = num_splits[batch];
  const int pitch = (total + num_sm_parts - 1) / num_sm_parts + (batch <= num_sm_parts ? kFixedOverheadBlocks : 0);

  // 2. cut k, k = 0 .. parts
  if (tid <= num_sm_parts) {
    Cut c;
    const long long x = static_cast<long long>(tid) * pitch;
    if (tid >= num_sm_parts || x >= total) {
      c.req = batch; c.off = 0;
    } else {
      int lo = 0, hi = batch;                 // last request r with prefix[r] <= x
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (num_splits[mid] <= x) lo = mid; else hi = mid;
      }
      const int off = static_cast<int>(x) - num_splits[lo] - kFixedOverheadBlocks;
      c.req = lo; c.off = off <= 0 ? 0 : off;
      if (c.off >= max(real_blocks(lo), 1)) { c.req = lo + 1; c.off = 0; }      // cannot happen for x < prefix[lo + 1]; kept as a guard
    }
    s_cut[tid] = c;
  }
  __syncthreads();
  if (tid <= num_sm_parts) s_new[tid] = tid == 0 || s_cut[tid].req != s_cut[tid - 1].req || s_cut[tid].off != s_cut[tid - 1].off;
  __syncthreads();

  // 3. every request is touched by one partition plus one per distinct cut strictly inside it
  for (int i = tid; i < batch; i += kSchedThreads) num_splits[i] = 1;
  __syncthreads();
  if (tid >= 1 && tid < num_sm_parts && s_new[tid] && s_cut[tid].off > 0) atomicAdd(num_splits + s_cut[tid].req, 1);
  __syncthreads();

  // 4. metadata rows
  if (tid < num_sm_parts) {
    const Cut a = s_cut[tid], e = s_cut[tid + 1];
    int row[5] = {batch, 0, batch - 1, 0, 0};
    if (a.req != e.req || a.off != e.off) {
      int split = 0;
      if (a.off > 0)
        for (int j = tid; j >= 1 && s_cut[j].req == a.req && s_cut[j].off > 0; --j) split += s_new[j];
      row[0] = a.req; row[1] = a.off; row[4] = split;
      if (e.off > 0) { row[2] = e.req; row[3] = e.off; }
      else { row[2] = e.req - 1; row[3] = real_blocks(e.req - 1); }
    }
    int4* dst = reinterpret_cast<int4*>(md + tid * 8);
    dst[0] = make_int4(row[0], row[1], row[2], row[3]);
    dst[1] = make_int4(row[4], 0, 0, 0);
  }
  __syncthreads();

  // 5. counts -> exclusive prefix, in place
  exclusive_scan(batch, [&](int i) { return num_splits[i]; }, num_splits);
}

cudaError_t launch_get_mla_metadata(const int* seqlens_k, int batch, int num_sm_parts, int topk, int* md,
                                    int* num_splits, cudaStream_t stream) {
  if (num_sm_parts > kMaxParts) return cudaErrorInvalidValue;
  get_mla_metadata_kernel<<<1, kSchedThreads, 0, stream>>>(seqlens_k, batch, num_sm_parts, topk, md, num_splits);
  return cudaGetLastError();
}

}  // namespace fmla
