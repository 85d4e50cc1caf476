// Reduction side of the fused GEMM -> reduce-scatter kernels (bf16 and block-scaled fp8 operands, fused_tp.cu and
// fused_tp_fp8.cu): CTAs that do no GEMM wait for the per-(source, row block) counters peers bump after storing
// their partial tiles, and add up the n partial slabs of a row block as soon as it is complete.
#pragma once
#include "fused_tp.h"
#include "pipeline_sm100.cuh"

namespace msccl {
namespace sm100 {

constexpr int kReduceSlices = 8;       // a row block is reduced in this many independent pieces

// Sum of the n partial slabs over 16-byte vectors [first, first + count) of this rank's shard, in rank order, fp32
// accumulation, one rounding to bf16.  RU vectors per thread and pass; the loads of NR sources are all issued before
// the first add (the loop over sources is unrolled for that), so RU x NR loads are in flight per thread.  The number
// of ranks is a multiple of NR (NR = 1 serves any count).
template <int RU, int NR, typename Args>
__device__ __forceinline__ void reduce_vectors(const Args& g, const char* my_slabs, size_t slab_bytes, size_t first, size_t count) {
  char* out = static_cast<char*>(g.out);
  const size_t stride = blockDim.x;
#pragma unroll 1
  for (size_t i = threadIdx.x; i < count; i += stride * RU) {
    float acc[RU][8];
#pragma unroll
    for (int u = 0; u < RU; ++u)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[u][e] = 0.0f;
#pragma unroll 1
    for (int s0 = 0; s0 < g.nranks; s0 += NR) {
      uint4 in[NR][RU];
#pragma unroll
      for (int r = 0; r < NR; ++r)
#pragma unroll
        for (int u = 0; u < RU; ++u) {
          const size_t ii = i + u * stride;
          if (ii < count) in[r][u] = *reinterpret_cast<const uint4*>(my_slabs + (s0 + r) * slab_bytes + (first + ii) * 16);
        }
#pragma unroll
      for (int r = 0; r < NR; ++r) {
#pragma unroll
        for (int u = 0; u < RU; ++u) {
          const uint32_t w[4] = {in[r][u].x, in[r][u].y, in[r][u].z, in[r][u].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[u][2 * e] += __uint_as_float(w[e] << 16);
            acc[u][2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      const size_t ii = i + u * stride;
      if (ii < count)
        *reinterpret_cast<uint4*>(out + (first + ii) * 16) =
            make_uint4(pack_bf16(acc[u][0], acc[u][1]), pack_bf16(acc[u][2], acc[u][3]), pack_bf16(acc[u][4], acc[u][5]),
                       pack_bf16(acc[u][6], acc[u][7]));
    }
  }
}

// Reduction work of one launch: items (row block, slice) handed out through a counter in the rank's flag page, the
// row blocks in the order they become complete.  The dedicated reducer CTAs pull items from the start; the GEMM CTAs
// join once their tiles are done, so the tail of the reduction has the whole GPU.  `per_block` counts every source
// adds per (source, row block) and launch.
template <typename Args>
__device__ __forceinline__ void reduce_items(const Args& g, FusedPage* page, const char* my_slabs, size_t slab_bytes,
                                             int blocks_per_rank, unsigned long long per_block) {
  __shared__ int s_item;
  __shared__ int s_ok;
  const int total = blocks_per_rank * kReduceSlices;
  const size_t block_vectors = static_cast<size_t>(BM) * g.N * 2 / 16;
  const size_t slice_vectors = (block_vectors + kReduceSlices - 1) / kReduceSlices;
  while (true) {
    __syncthreads();
    if (threadIdx.x == 0) {
      s_item = static_cast<int>(atomicAdd(&page->rs_work, 1u));
      s_ok = 1;
    }
    __syncthreads();
    const int item = s_item;
    if (item >= total) break;
    const int b = g.reduce_order[item / kReduceSlices], slice = item % kReduceSlices;
    if (static_cast<int>(threadIdx.x) < g.nranks) {
      volatile int never = 0;
      if (!wait_flag_ge(&page->rs_count[threadIdx.x][b], page->rs_base[threadIdx.x][b] + per_block, &never)) {
        if (g.error_words != nullptr && atomicCAS(&g.error_words[0], 0, static_cast<int>(GEMM_TIMEOUT_FLAG)) == 0) {
          g.error_words[1] = blockIdx.x;
          g.error_words[2] = 3;
          g.error_words[3] = threadIdx.x * 64 + b;
        }
        s_ok = 0;
      }
    }
    __syncthreads();
    if (s_ok == 0) break;
    const size_t begin = min(block_vectors, slice_vectors * slice);
    const size_t count = min(block_vectors, begin + slice_vectors) - begin;
    const size_t first = static_cast<size_t>(b) * block_vectors + begin;
    // keep about 16 loads per thread in flight whatever the number of ranks
    if (g.nranks == 2) reduce_vectors<4, 2>(g, my_slabs, slab_bytes, first, count);
    else if (g.nranks == 4) reduce_vectors<4, 4>(g, my_slabs, slab_bytes, first, count);
    else if (g.nranks % 8 == 0) reduce_vectors<2, 8>(g, my_slabs, slab_bytes, first, count);
    else reduce_vectors<4, 1>(g, my_slabs, slab_bytes, first, count);
  }
}

// The last CTA of a launch to finish moves the counter bases on and advances the launch epoch.
template <typename Args>
__device__ __forceinline__ void finish_rs_launch(const Args& g, FusedPage* page, int blocks_per_rank, unsigned long long per_block,
                                                 unsigned long long epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&page->rs_done, 1u) == gridDim.x - 1u) {
      // every CTA of this rank is through: the reducers have seen all counters of this launch
      for (int s = 0; s < g.nranks; ++s)
        for (int b = 0; b < blocks_per_rank; ++b) page->rs_base[s][b] += per_block;
      page->rs_done = 0;
      page->rs_work = 0;
      page->rs_epoch = epoch;
    }
  }
}

}  // namespace sm100
}  // namespace msccl
