// The comm CTAs of the block-scaled fp8 all-gather -> GEMM kernels (fused_tp_fp8.cu, fused_tp_fp8_2cta.cu): the first
// g.comm_ctas CTAs of the grid push the local shard to every peer in 128-row blocks - the e4m3 values of a block,
// then its K/128 scale blocks of 512 bytes - and publish one flag per block.
#pragma once
#include <cuda_runtime.h>

#include "fused_tp.h"
#include "gemm_sm100.cuh"
#include "pipeline_sm100.cuh"
#include "prims.cuh"

namespace msccl {
namespace sm100 {

__device__ __forceinline__ void push_f8_blocks(const AgGemmF8Args& g, FusedPage* page, unsigned long long epoch, size_t parity_off) {
  const int blocks_per_rank = g.rows_per_rank / BM;
  const size_t value_bytes = static_cast<size_t>(BM) * g.K;                  // one block of values
  const size_t scale_bytes = static_cast<size_t>(g.K / 128) * 512;           // and its scales
  const size_t all_values = static_cast<size_t>(g.rows_per_rank) * g.nranks * g.K;
  const int C = g.comm_ctas;
  const int parts = C >= blocks_per_rank ? C / blocks_per_rank : 1;
  const int part = C >= blocks_per_rank ? static_cast<int>(blockIdx.x) / blocks_per_rank : 0;
  const int b_first = C >= blocks_per_rank ? static_cast<int>(blockIdx.x) % blocks_per_rank : static_cast<int>(blockIdx.x);
  const int b_step = C >= blocks_per_rank ? blocks_per_rank * parts : C;
  const size_t vecs = (value_bytes + scale_bytes) / 16;                    // values first, then the scale blocks
  const size_t value_vecs = value_bytes / 16;
  const size_t per_part = (vecs + parts - 1) / parts;
  const size_t v0 = min(vecs, per_part * part), v1 = min(vecs, v0 + per_part);
  for (int b = b_first; b < blocks_per_rank && part < parts; b += b_step) {
    const char* src_values = static_cast<const char*>(g.x_local) + b * value_bytes;
    const char* src_scales = static_cast<const char*>(g.sf_local) + b * scale_bytes;
    const size_t dst_values = parity_off + (static_cast<size_t>(g.rank) * blocks_per_rank + b) * value_bytes;
    const size_t dst_scales = parity_off + all_values + (static_cast<size_t>(g.rank) * blocks_per_rank + b) * scale_bytes;
    constexpr int U = 8;
    for (size_t base = v0 + threadIdx.x; base < v1; base += static_cast<size_t>(blockDim.x) * U) {
      uint4 d[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t v = base + static_cast<size_t>(u) * blockDim.x;
        if (v < v1) d[u] = *reinterpret_cast<const uint4*>(v < value_vecs ? src_values + v * 16 : src_scales + (v - value_vecs) * 16);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t v = base + static_cast<size_t>(u) * blockDim.x;
        if (v >= v1) continue;
        const size_t off = v < value_vecs ? dst_values + v * 16 : dst_scales + (v - value_vecs) * 16;
        if (g.mc_base != nullptr) {
          multimem_st16(g.mc_base + off, d[u]);
        } else {
          for (int q = 1; q < g.nranks; ++q) *reinterpret_cast<uint4*>(g.heap_bases[(g.rank + q) % g.nranks] + off) = d[u];
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      fence_acq_rel_sys();
      if (atomicAdd(&page->ag_block_count[b], 1u) == static_cast<unsigned int>(parts) - 1u) {
        page->ag_block_count[b] = 0;
        fence_acq_rel_sys();
        for (int q = 1; q < g.nranks; ++q)
          st_release_sys(&g.pages[(g.rank + q) % g.nranks]->ag_flag[g.rank][b], epoch);
      }
    }
  }
}

}  // namespace sm100
}  // namespace msccl
