// The fused MoE kernels of moe_a2a.cu on CTA pairs (tcgen05 cta_group::2).  A cluster of two CTAs owns 256 rows of
// one expert (two consecutive 128-row tiles) times one 256-column tile: each CTA stages its own row tile of the
// dispatched tokens and its own half of the expert's weight tile, the leader issues the MMAs for both, and each CTA
// reads the accumulator of its own rows back (pair_pipeline.cuh).  Per output element the pair reads half as much of
// the weights from shared memory as two independent CTAs - the limit of the single-CTA pipeline.
//
// What the all-to-all adds stays per CTA: the producer of CTA r waits for the sources whose rows its own tile covers,
// the epilogue of CTA r sends its own rows home.  Behind an odd last tile of an expert the second CTA of the pair
// computes on rows that nobody stores (rows == 0).  Comm CTAs, count exchange, buffers and the final sum over the
// top-k slots are those of moe_a2a.cu (moe_common.cuh); operand loads carry no multicast.  Every wait is bounded.
#include <cuda.h>
#include <cuda_runtime.h>

#include "gemm_sm100.h"
#include "moe_a2a.h"
#include "moe_common.cuh"
#include "pair_pipeline.cuh"
#include "pipeline_sm100.cuh"

namespace msccl {
namespace sm100 {

namespace {

// ============================================================ dispatch + grouped GEMM1 (SwiGLU) on CTA pairs
__global__ void __launch_bounds__(kGemmThreads, 1)
moe_dispatch_gemm_2cta_kernel(const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_a1,
                              const __grid_constant__ CUtensorMap map_b, MoeArgs g) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ MoeShared sh;
  __shared__ int s_skip;
  const PairPipe p = carve_pair<kAgStages>(smem_raw);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  FusedPage* page = g.pages[g.rank];
  const unsigned long long epoch = page->moe_epoch + 1;
  const int parity = static_cast<int>(epoch & 1ull);
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int cluster = static_cast<int>(cluster_id_x()), clusters = static_cast<int>(num_clusters_x());
  const int comm_clusters = g.comm_ctas / 2;
  bool skip = false;

  if (cluster < comm_clusters) {
    // ---------------------------------------------------------------- comm CTAs (whole clusters, no tensor memory)
    skip = g.error_words != nullptr && *reinterpret_cast<volatile int*>(g.error_words) != 0;
    if (threadIdx.x == 0) *p.abort_flag = 0;
    __syncthreads();
    if (!skip) moe_comm_role(g, page, epoch, parity, &sh, p.abort_flag);
  } else {
    // ---------------------------------------------------------------- GEMM pairs
    if (threadIdx.x == 0) s_skip = (g.error_words != nullptr && *reinterpret_cast<volatile int*>(g.error_words) != 0) ? 1 : 0;
    init_pair<kAgStages>(p);
    if (threadIdx.x == 0) prefetch_tensormap(&map_b);
    if (warp == 1) tmem_alloc_pair(p.tmem_slot, kPTmemCols);
    tc_fence_before_sync();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *p.tmem_slot;
    skip = ld_shared_cluster_u32(map_to_cta(smem_u32(&s_skip), 0)) != 0;      // the leader's reading decides for the pair
    const bool have_counts = !skip && load_counts(g, page, epoch, parity, &sh, p.abort_flag);
    const int pairs = clusters - comm_clusters, pair = cluster - comm_clusters;
    const int n_out = 2 * g.ffn, tiles_n = n_out / PBN, k_blocks = g.hidden / BK;
    const int num_tiles = have_counts ? total_grouped_pair_tiles(sh.rows_per_expert, g.local_experts, tiles_n) : 0;
    const int my_tiles = num_tiles > pair ? (num_tiles - pair + pairs - 1) / pairs : 0;

    if (warp == 0) {
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        unsigned int landed = 0;                                  // bit s: all rows of source s have arrived
        for (int tile = pair; tile < num_tiles && ok; tile += pairs) {
          TileInfo t;
          decode_grouped_pair(tile, sh.rows_per_expert, g.local_experts, tiles_n, static_cast<int>(cta_rank), t);
          for (int s = 0; s < g.nranks && ok; ++s) {
            const bool covers = sh.seg_start[t.expert][s] < t.m0 + t.rows && sh.seg_start[t.expert][s + 1] > t.m0;
            if (covers && !(landed & (1u << s))) {
              if (!wait_flag_ge(&page->moe_flag[s][1], epoch, p.abort_flag)) {
                gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_FLAG, 0, s);
                ok = false;
              }
              landed |= 1u << s;
              fence_proxy_async();                                // peer stores (generic proxy) before my tensor loads
            }
          }
          const int a_row = t.expert * g.cap + t.m0;
          const int b_row = t.expert * n_out + t.tn * PBN + static_cast<int>(cta_rank) * (PBN / 2);
          for (int kb = 0; kb < k_blocks && ok; ++kb) {
            if (!mbar_wait(&p.empty_bar[stage], phase ^ 1, p.abort_flag)) {
              gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_EMPTY, 0, stage);
              ok = false;
              break;
            }
            uint8_t* a_dst = p.stage_base + static_cast<size_t>(stage) * kPStageBytes;
            if (leader) mbar_expect_tx(&p.full_bar[stage], 2 * kPStageBytes);
            const uint32_t leader_full = map_to_cta(smem_u32(&p.full_bar[stage]), 0);
            if (parity) tma_load_2d_pair(a_dst, &map_a1, leader_full, kb * BK, a_row);
            else tma_load_2d_pair(a_dst, &map_a0, leader_full, kb * BK, a_row);
            tma_load_2d_pair(a_dst + kPABytes, &map_b, leader_full, kb * BK, b_row);
            if (++stage == kAgStages) { stage = 0; phase ^= 1; }
          }
        }
        if (!ok) drain_pair<kAgStages>(p, leader);
      }
    } else if (warp == 1) {
      if (lane == 0 && leader) mma_role_pair<kAgStages>(p, tmem_base, my_tiles, k_blocks, g.error_words);
    } else {
      const int quarter = warp % 4;
      int acc = 0;
      uint32_t acc_phase = 0;
      __nv_bfloat16* h = static_cast<__nv_bfloat16*>(g.h);
      constexpr int H = PBN / 2;
      for (int tile = pair; tile < num_tiles; tile += pairs) {
        TileInfo t;
        decode_grouped_pair(tile, sh.rows_per_expert, g.local_experts, tiles_n, static_cast<int>(cta_rank), t);
        bool ok = mbar_wait(&p.acc_full[acc], acc_phase, p.abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_ACC, 2, acc);
          break;
        }
        tc_fence_after_sync();
        const int r_in_tile = quarter * 32 + lane;
        const size_t row = static_cast<size_t>(t.expert) * g.cap + t.m0 + r_in_tile;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * PBN);
        if (quarter * 32 < t.rows) {                              // warp-uniform: this quarter holds real rows
#pragma unroll 1
          for (int c = 0; c < H; c += 32) {
            uint32_t gt[32], up[32];
            tmem_ld32(taddr + c, gt);
            tmem_ld32(taddr + H + c, up);
            tc_wait_ld();
            if (r_in_tile < t.rows) {
              uint4* out = reinterpret_cast<uint4*>(h + row * g.ffn + t.tn * H + c);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const float gv = __uint_as_float(gt[8 * v + e]);
                  o[e] = gv / (1.0f + __expf(-gv)) * __uint_as_float(up[8 * v + e]);
                }
                out[v] = make_uint4(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]), pack_bf16(o[4], o[5]), pack_bf16(o[6], o[7]));
              }
            }
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&p.acc_empty[acc]), 0));   // the leader's barrier
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    tc_fence_before_sync();
    cluster_sync_all();                                          // nothing of the pair is in flight any more
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc_pair(tmem_base, kPTmemCols);
    }
  }
  if (skip) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&page->moe_done, 1u) == gridDim.x - 1u) {
      page->moe_done = 0;
      page->moe_pad = 1;                                         // the epoch advances after the second kernel
    }
  }
}

// ============================================================ grouped GEMM2 + combine on CTA pairs
__global__ void __launch_bounds__(kGemmThreads, 1)
moe_gemm_combine_2cta_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, MoeArgs g) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ MoeShared sh;
  __shared__ int s_skip;
  const PairPipe p = carve_pair<kRsStages>(smem_raw);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  FusedPage* page = g.pages[g.rank];
  const unsigned long long epoch = page->moe_epoch + 1;
  const int parity = static_cast<int>(epoch & 1ull);
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int pair = static_cast<int>(cluster_id_x()), pairs = static_cast<int>(num_clusters_x());
  if (threadIdx.x == 0) s_skip = (g.error_words != nullptr && *reinterpret_cast<volatile int*>(g.error_words) != 0) ? 1 : 0;
  init_pair<kRsStages>(p);
  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 1) tmem_alloc_pair(p.tmem_slot, kPTmemCols);
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *p.tmem_slot;
  const bool skip = ld_shared_cluster_u32(map_to_cta(smem_u32(&s_skip), 0)) != 0;
  const bool have_counts = !skip && load_counts(g, page, epoch, parity, &sh, p.abort_flag);   // flags are already set: no wait
  const int tiles_n = g.hidden / PBN, k_blocks = g.ffn / BK;
  const int num_tiles = have_counts ? total_grouped_pair_tiles(sh.rows_per_expert, g.local_experts, tiles_n) : 0;
  const int my_tiles = num_tiles > pair ? (num_tiles - pair + pairs - 1) / pairs : 0;
  const size_t row_bytes = static_cast<size_t>(g.hidden) * 2;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += pairs) {
        TileInfo t;
        decode_grouped_pair(tile, sh.rows_per_expert, g.local_experts, tiles_n, static_cast<int>(cta_rank), t);
        const int a_row = t.expert * g.cap + t.m0;
        const int b_row = t.expert * g.hidden + t.tn * PBN + static_cast<int>(cta_rank) * (PBN / 2);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&p.empty_bar[stage], phase ^ 1, p.abort_flag)) {
            gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_EMPTY, 0, stage);
            ok = false;
            break;
          }
          uint8_t* a_dst = p.stage_base + static_cast<size_t>(stage) * kPStageBytes;
          if (leader) mbar_expect_tx(&p.full_bar[stage], 2 * kPStageBytes);
          const uint32_t leader_full = map_to_cta(smem_u32(&p.full_bar[stage]), 0);
          tma_load_2d_pair(a_dst, &map_a, leader_full, kb * BK, a_row);
          tma_load_2d_pair(a_dst + kPABytes, &map_b, leader_full, kb * BK, b_row);
          if (++stage == kRsStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) drain_pair<kRsStages>(p, leader);
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) mma_role_pair<kRsStages>(p, tmem_base, my_tiles, k_blocks, g.error_words);
  } else {
    const int quarter = warp % 4;
    int acc = 0;
    uint32_t acc_phase = 0;
    const int4* meta_base = reinterpret_cast<const int4*>(g.heap_bases[g.rank] + g.moe_off + g.lay.meta_off +
                                                          static_cast<size_t>(parity) * g.lay.meta_parity);
    for (int tile = pair; tile < num_tiles; tile += pairs) {
      TileInfo t;
      decode_grouped_pair(tile, sh.rows_per_expert, g.local_experts, tiles_n, static_cast<int>(cta_rank), t);
      bool ok = mbar_wait(&p.acc_full[acc], acc_phase, p.abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_ACC, 2, acc);
        break;
      }
      tc_fence_after_sync();
      const int r_in_tile = quarter * 32 + lane;
      const bool valid = r_in_tile < t.rows;
      const bool any = quarter * 32 < t.rows;                     // warp-uniform: this quarter holds real rows
      int4 m = make_int4(0, 0, 0, 0);
      if (valid) m = meta_base[static_cast<size_t>(t.expert) * g.cap + t.m0 + r_in_tile];
      const float w = valid ? __int_as_float(m.z) : 0.0f;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * PBN);
      uint8_t* stage_warp = p.staging + (warp - 2) * kStagingPerWarp;
      if (any) stage_quarter_bf16(taddr, stage_warp, lane, w);   // row = lane: scaled by its own gate weight
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&p.acc_empty[acc]), 0));   // free once it sits in shared memory
      // every row goes home: combine[parity][copy][hidden] on the rank that owns the token, one row (512 contiguous
      // bytes) per store instruction; the row's address comes from the lane that holds its metadata
      char* my_dst = nullptr;
      if (valid)
        my_dst = g.heap_bases[m.x] + g.moe_off + g.lay.combine_off + static_cast<size_t>(parity) * g.lay.combine_parity +
                 static_cast<size_t>(m.y) * row_bytes + static_cast<size_t>(t.tn) * PBN * 2;
      const unsigned long long mine_u = reinterpret_cast<unsigned long long>(my_dst);
      if (any) {
#pragma unroll 1
        for (int r0 = 0; r0 < 32; r0 += 8) {
          uint4 d[8];
          unsigned long long ptr[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            ptr[u] = __shfl_sync(0xffffffffu, mine_u, r0 + u);
            d[u] = *reinterpret_cast<const uint4*>(stage_warp + (r0 + u) * kStagePitch + lane * 16);
          }
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (ptr[u] != 0) *reinterpret_cast<uint4*>(reinterpret_cast<char*>(ptr[u]) + lane * 16) = d[u];
        }
      }
      __syncwarp();
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    // this warp's rows are on their way: tell every rank (one count per epilogue warp and CTA)
    __syncwarp();
    if (!skip && lane < g.nranks) {
      fence_acq_rel_sys();
      red_add_release_sys(&g.pages[lane]->moe_count[g.rank], 1ull);
    }
  }
  tc_fence_before_sync();
  cluster_sync_all();                                            // nothing of the pair is in flight any more
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kPTmemCols);
  }
  if (skip) return;
  moe_sum_and_finish(g, page, epoch, parity, p.abort_flag);
}

}  // namespace

// Same contracts as launch_moe_dispatch_gemm / launch_moe_gemm_combine; additionally an even number of comm CTAs.
// `grid` is the number of CTAs wanted (0: as many pairs as the device holds at once); every rank must pass the same.
cudaError_t launch_moe_dispatch_gemm_2cta(const MoeArgs& g, int grid, cudaStream_t stream) {
  if (g.hidden % BK != 0 || (2 * g.ffn) % PBN != 0 || g.nranks > kFusedMaxRanks || g.local_experts > kMoeMaxLocalExperts ||
      g.num_experts > kMoeMaxExperts || g.comm_ctas < 2 || g.comm_ctas % 2 != 0)
    return cudaErrorInvalidValue;
  static int resident = 0;
  if (resident == 0) {
    cudaError_t err = pair_clusters(moe_dispatch_gemm_2cta_kernel, kAgSmemBytes, &resident);
    if (err != cudaSuccess) return err;
  }
  int clusters = resident;
  if (grid > 0 && grid / 2 < clusters) clusters = grid / 2;
  if (clusters <= g.comm_ctas / 2) return cudaErrorLaunchOutOfResources;
  const char* disp = g.heap_bases_host[g.rank] + g.moe_off + g.lay.dispatch_off;
  const uint64_t rows = static_cast<uint64_t>(g.local_experts) * g.cap;
  CUtensorMap a0 = make_bf16_kmajor_map(disp, rows, g.hidden, g.hidden, BM);
  CUtensorMap a1 = make_bf16_kmajor_map(disp + g.lay.dispatch_parity, rows, g.hidden, g.hidden, BM);
  CUtensorMap b = make_bf16_kmajor_map(g.w_gate_up, static_cast<uint64_t>(g.local_experts) * 2 * g.ffn, g.hidden, g.hidden, PBN / 2);
  return launch_pairs(moe_dispatch_gemm_2cta_kernel, kAgSmemBytes, clusters, stream, a0, a1, b, g);
}

cudaError_t launch_moe_gemm_combine_2cta(const MoeArgs& g, int grid, cudaStream_t stream) {
  if (g.hidden % PBN != 0 || g.ffn % BK != 0 || g.nranks > kFusedMaxRanks || g.local_experts > kMoeMaxLocalExperts)
    return cudaErrorInvalidValue;
  static int resident = 0;
  if (resident == 0) {
    cudaError_t err = pair_clusters(moe_gemm_combine_2cta_kernel, kRsSmemBytes, &resident);
    if (err != cudaSuccess) return err;
  }
  int clusters = resident;
  if (grid > 0 && grid / 2 < clusters) clusters = grid / 2;
  if (clusters < 1) return cudaErrorLaunchOutOfResources;
  CUtensorMap a = make_bf16_kmajor_map(g.h, static_cast<uint64_t>(g.local_experts) * g.cap, g.ffn, g.ffn, BM);
  CUtensorMap b = make_bf16_kmajor_map(g.w_down, static_cast<uint64_t>(g.local_experts) * g.hidden, g.ffn, g.ffn, PBN / 2);
  return launch_pairs(moe_gemm_combine_2cta_kernel, kRsSmemBytes, clusters, stream, a, b, g);
}

}  // namespace sm100
}  // namespace msccl
