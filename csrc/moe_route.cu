// Routing of a MoE layer on the device, in two launches instead of the dozen library kernels of softmax + topk +
// argsort + bincount + cumsum:
//   moe_topk_kernel   one warp per token: the k largest gate logits and their weights (softmax over all experts,
//                     renormalised over the k kept ones - which is the softmax over the k kept logits).
//   moe_sort_kernel   one CTA: a stable counting sort of the token copies by expert.  Writes the copy indices
//                     ordered by expert (`sorted_copy`) and the prefix of the per-expert counts (`expert_start`),
//                     the two tables the dispatch kernel of moe_a2a.cu reads.
// The reference has no routing code: its AllToAll programs (examples/mscclang/alltoall_allpairs.py) move fixed-size
// chunks; data-dependent counts are what the fused MoE path adds.
#include <cuda_runtime.h>

#include <cstdint>

#include "moe_a2a.h"

namespace msccl {
namespace sm100 {

namespace {

constexpr int kSortThreads = 1024;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kTopkMax = 8;

// logits [tokens, experts] fp32 -> experts [tokens, k] int32 (descending by logit, ties to the lower id), weights fp32
__global__ void moe_topk_kernel(const float* __restrict__ logits, int tokens, int experts, int k, int* __restrict__ out_e,
                                float* __restrict__ out_w) {
  const int lane = threadIdx.x % 32;
  const int token = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  if (token >= tokens) return;
  const float* row = logits + static_cast<size_t>(token) * experts;
  constexpr int kPerLane = kMoeMaxExperts / 32;
  float v[kPerLane];
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < experts ? row[e] : -INFINITY;
  }
  float top_v[kTopkMax];
  int top_e[kTopkMax];
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i)
      if (v[i] > best) { best = v[i]; best_e = i * 32 + lane; }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, off);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
      if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
    }
    top_v[j] = best;
    top_e[j] = best_e;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i)
      if (i * 32 + lane == best_e) v[i] = -INFINITY;
  }
  if (lane == 0) {
    float sum = 0.0f;
    for (int j = 0; j < k; ++j) sum += __expf(top_v[j] - top_v[0]);
    for (int j = 0; j < k; ++j) {
      out_e[static_cast<size_t>(token) * k + j] = top_e[j];
      out_w[static_cast<size_t>(token) * k + j] = __expf(top_v[j] - top_v[0]) / sum;
    }
  }
}

// Stable counting sort of `n` copies by expert id, one CTA.  Warp w owns the contiguous range [w * per, (w + 1) * per);
// inside a batch of 32 copies __match_any_sync ranks the copies of one expert by lane.
__global__ void __launch_bounds__(kSortThreads, 1)
moe_sort_kernel(const int* __restrict__ expert_of, int n, int experts, int* __restrict__ sorted_copy, int* __restrict__ expert_start) {
  __shared__ int warp_base[kSortWarps][kMoeMaxExperts];      // first counts, then where the warp's next copy of e goes
  __shared__ int start[kMoeMaxExperts + 1];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const unsigned int lt = (1u << lane) - 1u;
  for (int i = threadIdx.x; i < kSortWarps * kMoeMaxExperts; i += kSortThreads) (&warp_base[0][0])[i] = 0;
  __syncthreads();
  const int per = ((n + kSortWarps - 1) / kSortWarps + 31) / 32 * 32;
  const int lo = min(n, warp * per), hi = min(n, lo + per);
  for (int i0 = lo; i0 < hi; i0 += 32) {
    const int i = i0 + lane;
    const bool in = i < hi;
    int e = in ? expert_of[i] : -1;
    if (in && (e < 0 || e >= experts)) e = experts - 1;      // ids are checked on the host side of the caller
    const unsigned int same = __match_any_sync(0xffffffffu, e);
    if (in && (same & lt) == 0) warp_base[warp][e] += __popc(same);
    __syncwarp();
  }
  __syncthreads();
  // exclusive prefix over experts of the totals, then over warps inside each expert
  if (threadIdx.x < experts) {
    int total = 0;
    for (int w = 0; w < kSortWarps; ++w) total += warp_base[w][threadIdx.x];
    start[threadIdx.x + 1] = total;
  }
  if (threadIdx.x == 0) start[0] = 0;
  __syncthreads();
  if (threadIdx.x == 0)
    for (int e = 0; e < experts; ++e) start[e + 1] += start[e];
  __syncthreads();
  if (threadIdx.x < experts) {
    int run = start[threadIdx.x];
    for (int w = 0; w < kSortWarps; ++w) {
      const int c = warp_base[w][threadIdx.x];
      warp_base[w][threadIdx.x] = run;
      run += c;
    }
  }
  for (int e = threadIdx.x; e <= experts; e += kSortThreads) expert_start[e] = start[e];
  __syncthreads();
  for (int i0 = lo; i0 < hi; i0 += 32) {
    const int i = i0 + lane;
    const bool in = i < hi;
    int e = in ? expert_of[i] : -1;
    if (in && (e < 0 || e >= experts)) e = experts - 1;
    const unsigned int same = __match_any_sync(0xffffffffu, e);
    int pos = 0;
    if (in) pos = warp_base[warp][e] + __popc(same & lt);
    __syncwarp();
    if (in && (same & lt) == 0) warp_base[warp][e] += __popc(same);
    __syncwarp();
    if (in) sorted_copy[pos] = i;
  }
}

}  // namespace

cudaError_t launch_moe_topk(const float* logits, int tokens, int experts, int k, int* out_experts, float* out_weights,
                            cudaStream_t stream) {
  if (tokens < 1 || experts < 1 || experts > kMoeMaxExperts || k < 1 || k > kTopkMax || k > experts) return cudaErrorInvalidValue;
  const int warps = 8;
  moe_topk_kernel<<<(tokens + warps - 1) / warps, warps * 32, 0, stream>>>(logits, tokens, experts, k, out_experts, out_weights);
  return cudaGetLastError();
}

cudaError_t launch_moe_sort(const int* expert_of, int n, int experts, int* sorted_copy, int* expert_start, cudaStream_t stream) {
  if (n < 1 || experts < 1 || experts > kMoeMaxExperts) return cudaErrorInvalidValue;
  moe_sort_kernel<<<1, kSortThreads, 0, stream>>>(expert_of, n, experts, sorted_copy, expert_start);
  return cudaGetLastError();
}

}  // namespace sm100
}  // namespace msccl
