// Reduction side of the fused GEMM -> reduce-scatter kernels (bf16 and block-scaled fp8 operands, fused_tp.cu and
// fused_tp_fp8.cu): CTAs that do no GEMM wait for the per-(source, row block) counters peers bump after storing
// their partial tiles, and add up the n partial slabs of a row block as soon as it is complete.
#pragma once
#include "fused_tp.h"
#include "pipeline_sm100.cuh"

namespace msccl {
namespace sm100 {

// Sum of the n partial slabs of row block b (rows [b*BM, (b+1)*BM) of this rank's shard), in rank order,
// fp32 accumulation, one rounding to bf16.  `part` of `parts` CTAs.
template <typename Args>
__device__ __forceinline__ void reduce_row_block(const Args& g, const char* my_slabs, size_t slab_bytes, int b, int part, int parts) {
  constexpr int RU = 4;          // vectors per thread per pass; with 8 sources that is 32 loads in flight
  const size_t first = static_cast<size_t>(b) * BM * g.N * 2 / 16;
  const size_t count = static_cast<size_t>(BM) * g.N * 2 / 16;
  const size_t stride = static_cast<size_t>(parts) * blockDim.x;
  char* out = static_cast<char*>(g.out);
  for (size_t i = static_cast<size_t>(part) * blockDim.x + threadIdx.x; i < count; i += stride * RU) {
    uint4 in[RU][kFusedMaxRanks];
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      const size_t ii = i + u * stride;
#pragma unroll
      for (int s = 0; s < kFusedMaxRanks; ++s)
        if (s < g.nranks && ii < count) in[u][s] = *reinterpret_cast<const uint4*>(my_slabs + s * slab_bytes + (first + ii) * 16);
    }
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      const size_t ii = i + u * stride;
      if (ii >= count) break;
      float acc8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int s = 0; s < kFusedMaxRanks; ++s) {
        if (s < g.nranks) {
          const uint32_t w[4] = {in[u][s].x, in[u][s].y, in[u][s].z, in[u][s].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc8[2 * e] += __uint_as_float(w[e] << 16);
            acc8[2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
          }
        }
      }
      *reinterpret_cast<uint4*>(out + (first + ii) * 16) =
          make_uint4(pack_bf16(acc8[0], acc8[1]), pack_bf16(acc8[2], acc8[3]), pack_bf16(acc8[4], acc8[5]), pack_bf16(acc8[6], acc8[7]));
    }
  }
}

// Body of a reducer CTA: the rank's row blocks in the order they become complete.  `per_block` counts every source
// adds per (source, row block) and launch.
template <typename Args>
__device__ __forceinline__ void reducer_cta(const Args& g, FusedPage* page, const char* my_slabs, size_t slab_bytes,
                                            int blocks_per_rank, unsigned long long per_block, int part, int parts) {
  __shared__ int s_ok;
  for (int i = 0; i < blocks_per_rank; ++i) {
    const int b = g.reduce_order[i];
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
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
    reduce_row_block(g, my_slabs, slab_bytes, b, part, parts);
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
      page->rs_epoch = epoch;
    }
  }
}

}  // namespace sm100
}  // namespace msccl
