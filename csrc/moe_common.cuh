// Pieces shared by the fused MoE kernels (moe_a2a.cu on single CTAs, moe_a2a_2cta.cu on CTA pairs): the enumeration
// of the grouped GEMM tiles and the per-launch tables that every CTA derives from the all-gathered expert counts.
#pragma once
#include <cuda_runtime.h>

#include "fused_tp.h"
#include "moe_a2a.h"
#include "pipeline_sm100.cuh"

namespace msccl {
namespace sm100 {

struct TileInfo { int expert, m0, tn, rows; };

// Grouped tile enumeration: experts in order, column tiles of an expert, then its row tiles fastest
// (m_tiles[e] = ceil(rows_e / 128)).  The CTAs that run side by side therefore share a handful of
// weight tiles and read the expert's rows - a few MB - from L2: the weights of one expert (235 MB of
// gate and up rows at hidden 4096, ffn 14336) do not fit into L2, and with the column tiles fastest
// every row tile streamed them from DRAM again.  Returns false when `tile` is past the end.
__device__ __forceinline__ bool decode_grouped(int tile, const int* rows_per_expert, int local_experts, int tiles_n,
                                               TileInfo& t) {
  int base = 0;
  for (int e = 0; e < local_experts; ++e) {
    const int mt = (rows_per_expert[e] + BM - 1) / BM;
    const int here = mt * tiles_n;
    if (tile < base + here) {
      const int in_e = tile - base;
      t.expert = e;
      t.m0 = (in_e % mt) * BM;
      t.tn = in_e / mt;
      t.rows = min(BM, rows_per_expert[e] - t.m0);
      return true;
    }
    base += here;
  }
  return false;
}

__device__ __forceinline__ int total_grouped_tiles(const int* rows_per_expert, int local_experts, int tiles_n) {
  int total = 0;
  for (int e = 0; e < local_experts; ++e) total += ((rows_per_expert[e] + BM - 1) / BM) * tiles_n;
  return total;
}

// The same enumeration for CTA pairs: a pair owns two consecutive row tiles of one expert (256 rows) and one
// column tile; CTA `r` of the pair gets row tile 2 * p + r, which is empty (rows == 0) behind an odd last tile.
__device__ __forceinline__ bool decode_grouped_pair(int tile, const int* rows_per_expert, int local_experts, int tiles_n, int r,
                                                    TileInfo& t) {
  int base = 0;
  for (int e = 0; e < local_experts; ++e) {
    const int pt = (rows_per_expert[e] + 2 * BM - 1) / (2 * BM);
    const int here = pt * tiles_n;
    if (tile < base + here) {
      const int in_e = tile - base;
      t.expert = e;
      t.m0 = (2 * (in_e % pt) + r) * BM;
      t.tn = in_e / pt;
      t.rows = max(0, min(BM, rows_per_expert[e] - t.m0));
      return true;
    }
    base += here;
  }
  return false;
}

__device__ __forceinline__ int total_grouped_pair_tiles(const int* rows_per_expert, int local_experts, int tiles_n) {
  int total = 0;
  for (int e = 0; e < local_experts; ++e) total += ((rows_per_expert[e] + 2 * BM - 1) / (2 * BM)) * tiles_n;
  return total;
}

struct MoeShared {
  int rows_per_expert[kMoeMaxLocalExperts];                    // rows of each local expert (all sources)
  int seg_start[kMoeMaxLocalExperts][kFusedMaxRanks + 1];      // per local expert: first row of each source's segment
  int my_offset[kMoeMaxExperts];                               // where my copies start inside every (global) expert
  int ok;
};

// Wait for the count rows of all sources (flag 0) and derive the segment tables.
__device__ __forceinline__ bool load_counts(const MoeArgs& g, FusedPage* page, unsigned long long epoch, int parity, MoeShared* sh,
                            volatile int* abort_flag) {
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int s = 0; s < g.nranks && ok; ++s)
      if (!wait_flag_ge(&page->moe_flag[s][0], epoch, abort_flag)) {
        gemm_fail(g.error_words, abort_flag, GEMM_TIMEOUT_FLAG, 4, s);
        ok = 0;
      }
    sh->ok = ok;
  }
  __syncthreads();
  if (sh->ok == 0) return false;
  const int* counts = reinterpret_cast<const int*>(g.heap_bases[g.rank] + g.moe_off + g.lay.counts_off +
                                                   static_cast<size_t>(parity) * g.lay.counts_parity);
  for (int e = threadIdx.x; e < g.num_experts; e += blockDim.x) {
    int before_me = 0, total = 0;
    for (int s = 0; s < g.nranks; ++s) {
      const int c = counts[s * g.num_experts + e];
      if (s < g.rank) before_me += c;
      total += c;
    }
    sh->my_offset[e] = before_me;
    const int first_local = g.rank * g.local_experts;
    if (e >= first_local && e < first_local + g.local_experts) {
      const int le = e - first_local;
      sh->rows_per_expert[le] = total;
      int run = 0;
      for (int s = 0; s < g.nranks; ++s) {
        sh->seg_start[le][s] = run;
        run += counts[s * g.num_experts + e];
      }
      sh->seg_start[le][g.nranks] = run;
      if (total > g.cap) gemm_fail(g.error_words, abort_flag, 5 /* expert over capacity */, 4, e);
    }
  }
  __syncthreads();
  return *abort_flag == 0;
}

// The comm CTAs of the dispatch kernel (the first g.comm_ctas CTAs of the grid): all-gather the per-expert counts,
// then scatter my token copies into the owners' dispatch buffers and publish one flag per destination.
__device__ __forceinline__ void moe_comm_role(const MoeArgs& g, FusedPage* page, unsigned long long epoch, int parity, MoeShared* sh,
                                          volatile int* abort_flag) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int copies = g.tokens * g.topk;
  const size_t row_bytes = static_cast<size_t>(g.hidden) * 2;
  if (blockIdx.x == 0) {
    // all-gather my per-expert counts: row `rank` of every rank's count matrix
    for (int q = 0; q < g.nranks; ++q) {
      int* dst = reinterpret_cast<int*>(g.heap_bases[(g.rank + q) % g.nranks] + g.moe_off + g.lay.counts_off +
                                        static_cast<size_t>(parity) * g.lay.counts_parity) + g.rank * g.num_experts;
      for (int e = threadIdx.x; e < g.num_experts; e += blockDim.x) dst[e] = g.expert_start[e + 1] - g.expert_start[e];
    }
    __syncthreads();
    if (threadIdx.x < g.nranks) {
      fence_acq_rel_sys();
      st_release_sys(&g.pages[threadIdx.x]->moe_flag[g.rank][0], epoch);
    }
  }
  if (!load_counts(g, page, epoch, parity, sh, abort_flag)) return;
  {
    // scatter rows: one warp per token copy, copies taken in expert order
    const int warps = g.comm_ctas * (kGemmThreads / 32);
    const int gw = blockIdx.x * (kGemmThreads / 32) + warp;
    for (int i = gw; i < copies; i += warps) {
      const int c = g.sorted_copy[i];
      // expert of position i: binary search in expert_start
      int lo = 0, hi = g.num_experts;
      while (hi - lo > 1) {
        const int mid = (lo + hi) / 2;
        if (g.expert_start[mid] <= i) lo = mid; else hi = mid;
      }
      const int e = lo, dst_rank = e / g.local_experts, le = e % g.local_experts;
      const int row = sh->my_offset[e] + (i - g.expert_start[e]);
      if (row >= g.cap) continue;                               // over capacity: already reported as an error
      char* base = g.heap_bases[dst_rank] + g.moe_off;
      char* dst = base + g.lay.dispatch_off + static_cast<size_t>(parity) * g.lay.dispatch_parity +
                  (static_cast<size_t>(le) * g.cap + row) * row_bytes;
      const char* src = static_cast<const char*>(g.x) + static_cast<size_t>(c / g.topk) * row_bytes;
      const int vecs = static_cast<int>(row_bytes / 16);
      for (int v0 = lane; v0 < vecs; v0 += 32 * 8) {
        uint4 d[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (v0 + u * 32 < vecs) d[u] = *reinterpret_cast<const uint4*>(src + (v0 + u * 32) * 16);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (v0 + u * 32 < vecs) *reinterpret_cast<uint4*>(dst + (v0 + u * 32) * 16) = d[u];
      }
      if (lane == 0) {
        int4* meta = reinterpret_cast<int4*>(base + g.lay.meta_off + static_cast<size_t>(parity) * g.lay.meta_parity) +
                     static_cast<size_t>(le) * g.cap + row;
        *meta = make_int4(g.rank, c, __float_as_int(g.copy_weight[c]), 0);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      fence_acq_rel_sys();
      if (atomicAdd(&page->ag_block_count[0], 1u) == static_cast<unsigned int>(g.comm_ctas) - 1u) {
        page->ag_block_count[0] = 0;
        fence_acq_rel_sys();
        for (int q = 0; q < g.nranks; ++q) st_release_sys(&g.pages[(g.rank + q) % g.nranks]->moe_flag[g.rank][1], epoch);
      }
    }
  }
}

// The tail of the combine kernel, run by every CTA: wait until every peer has stored its expert outputs for my tokens,
// sum the top-k slots of each token, and let the last CTA advance the launch epoch.  `cta` of `ctas` share the sum.
__device__ __forceinline__ void moe_sum_and_finish(const MoeArgs& g, FusedPage* page, unsigned long long epoch, int parity,
                                                   volatile int* abort_flag) {
  const int ctas = gridDim.x, cta = blockIdx.x;
  const size_t row_bytes = static_cast<size_t>(g.hidden) * 2;
  // ---------------------------------------------------------------- combine: y[t] = sum over k of combine[t*topk + k]
  const unsigned long long per_launch = 4ull * gridDim.x;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int s = 0; s < g.nranks && ok; ++s)
      if (!wait_flag_ge(&page->moe_count[s], page->moe_base[s] + per_launch, abort_flag)) {
        gemm_fail(g.error_words, abort_flag, GEMM_TIMEOUT_FLAG, 3, s);
        ok = 0;
      }
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok != 0) {
    const char* comb = g.heap_bases[g.rank] + g.moe_off + g.lay.combine_off + static_cast<size_t>(parity) * g.lay.combine_parity;
    const size_t vec_per_row = row_bytes / 16;
    const size_t total = static_cast<size_t>(g.tokens) * vec_per_row;
    for (size_t v = static_cast<size_t>(cta) * blockDim.x + threadIdx.x; v < total; v += static_cast<size_t>(ctas) * blockDim.x) {
      const size_t tkn = v / vec_per_row, col = v % vec_per_row;
      float a8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int k = 0; k < g.topk; ++k) {
        const uint4 d = *reinterpret_cast<const uint4*>(comb + ((tkn * g.topk + k) * vec_per_row + col) * 16);
        const uint32_t wv[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          a8[2 * e] += __uint_as_float(wv[e] << 16);
          a8[2 * e + 1] += __uint_as_float(wv[e] & 0xffff0000u);
        }
      }
      *reinterpret_cast<uint4*>(static_cast<char*>(g.y) + v * 16) =
          make_uint4(pack_bf16(a8[0], a8[1]), pack_bf16(a8[2], a8[3]), pack_bf16(a8[4], a8[5]), pack_bf16(a8[6], a8[7]));
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&page->moe_done, 1u) == gridDim.x - 1u) {
      for (int s = 0; s < g.nranks; ++s) page->moe_base[s] += per_launch;
      page->moe_done = 0;
      page->moe_pad = 0;
      page->moe_epoch = epoch;
    }
  }
}

}  // namespace sm100
}  // namespace msccl
