// The fused tensor-parallel kernels of fused_tp.cu on CTA pairs (tcgen05 cta_group::2): a cluster of two CTAs
// owns one 256 x 256 output tile, each CTA stages its own 128 rows of A and its own 128 rows of the B tile (32 KB per
// stage), the leader issues the MMAs for both, and each CTA ends up with the accumulator of its own 128 rows in its
// own tensor memory (structure and barrier protocol of gemm_2cta_sm100.cu).  Per output element a pair reads half as
// much of B from shared memory as two independent 128 x 256 CTAs, which is what limits the single-CTA pipeline.
//
// What the collectives add is per CTA, so the pair changes little:
//   all-gather -> GEMM       the two row blocks of a pair tile are two consecutive entries of the order table; CTA r
//                            waits for the flag of entry 2t + r only and loads it from the LOCAL gathered buffer (no
//                            multicast, no peer memory); the comm CTAs are whole clusters that never touch TMEM.
//   GEMM -> reduce-scatter   CTA r stores the partial tile of entry 2t + r into its owner's slab and bumps the
//                            (source, row block) counter there; the last clusters of the grid only reduce, and the
//                            GEMM CTAs join them when their tiles are out (fused_reduce.cuh).
// Operand loads are per-CTA tensor loads completing on the leader's mbarrier (cp.async.bulk.tensor ... cta_group::2
// without multicast).  Every wait is bounded.
#include <cuda.h>
#include <cuda_runtime.h>

#include "fused_reduce.cuh"
#include "fused_tp.h"
#include "gemm_sm100.cuh"
#include "gemm_sm100.h"
#include "pair_pipeline.cuh"
#include "pipeline_sm100.cuh"
#include "prims.cuh"

namespace msccl {
namespace sm100 {

namespace {

// ============================================================ all-gather -> GEMM (+SwiGLU) on CTA pairs
template <int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
ag_gemm_2cta_kernel(const __grid_constant__ CUtensorMap map_local, const __grid_constant__ CUtensorMap map_gath0,
                    const __grid_constant__ CUtensorMap map_gath1, const __grid_constant__ CUtensorMap map_b, AgGemmArgs g) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_skip;
  const PairPipe p = carve_pair<kAgStages>(smem_raw);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  FusedPage* page = g.pages[g.rank];
  const unsigned long long epoch = page->ag_epoch + 1;
  const int parity = static_cast<int>(epoch & 1ull);
  const int blocks_per_rank = g.rows_per_rank / BM;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int cluster = static_cast<int>(cluster_id_x()), clusters = static_cast<int>(num_clusters_x());
  const int comm_clusters = g.comm_ctas / 2;
  bool skip = false;

  if (cluster < comm_clusters) {
    // ------------------------------------------------------------------ comm CTAs: push my shard (as in fused_tp.cu)
    skip = g.error_words != nullptr && *reinterpret_cast<volatile int*>(g.error_words) != 0;
    const size_t block_bytes = static_cast<size_t>(BM) * g.K * 2;
    const size_t vecs = block_bytes / 16;
    const int C = g.comm_ctas;
    const int parts = C >= blocks_per_rank ? C / blocks_per_rank : 1;
    const int part = C >= blocks_per_rank ? static_cast<int>(blockIdx.x) / blocks_per_rank : 0;
    const int b_first = C >= blocks_per_rank ? static_cast<int>(blockIdx.x) % blocks_per_rank : static_cast<int>(blockIdx.x);
    const int b_step = C >= blocks_per_rank ? blocks_per_rank * parts : C;
    const size_t per_part = (vecs + parts - 1) / parts;
    const size_t v0 = min(vecs, per_part * part), v1 = min(vecs, v0 + per_part);
    const size_t dst_off = g.gathered_off + static_cast<size_t>(parity) * g.gathered_bytes +
                           static_cast<size_t>(g.rank) * g.rows_per_rank * g.K * 2;
    for (int b = b_first; b < blocks_per_rank && part < parts && !skip; b += b_step) {
      const char* src = static_cast<const char*>(g.x_local) + b * block_bytes;
      constexpr int U = 16;       // 256 bytes per thread in flight: the copy is latency bound otherwise
      for (size_t base = v0 + threadIdx.x; base < v1; base += static_cast<size_t>(blockDim.x) * U) {
        uint4 d[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const size_t v = base + static_cast<size_t>(u) * blockDim.x;
          if (v < v1) d[u] = *reinterpret_cast<const uint4*>(src + v * 16);
        }
        if (g.mc_base != nullptr) {
          char* dst = g.mc_base + dst_off + b * block_bytes;
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const size_t v = base + static_cast<size_t>(u) * blockDim.x;
            if (v < v1) multimem_st16(dst + v * 16, d[u]);
          }
        } else {
          for (int q = 1; q < g.nranks; ++q) {
            char* dst = g.heap_bases[(g.rank + q) % g.nranks] + dst_off + b * block_bytes;
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const size_t v = base + static_cast<size_t>(u) * blockDim.x;
              if (v < v1) *reinterpret_cast<uint4*>(dst + v * 16) = d[u];
            }
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
  } else {
    // ------------------------------------------------------------------ GEMM pairs
    // An earlier launch gave up: skip the work.  The leader's reading decides for the pair.
    if (threadIdx.x == 0) s_skip = (g.error_words != nullptr && *reinterpret_cast<volatile int*>(g.error_words) != 0) ? 1 : 0;
    init_pair<kAgStages>(p);
    if (threadIdx.x == 0) {
      prefetch_tensormap(&map_local);
      prefetch_tensormap(&map_b);
    }
    if (warp == 1) tmem_alloc_pair(p.tmem_slot, kPTmemCols);
    tc_fence_before_sync();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *p.tmem_slot;
    skip = ld_shared_cluster_u32(map_to_cta(smem_u32(&s_skip), 0)) != 0;

    const int pairs = clusters - comm_clusters, pair = cluster - comm_clusters;
    const int tiles_n = g.N / PBN;
    const int num_tiles = (blocks_per_rank * g.nranks / 2) * tiles_n;
    const int k_blocks = g.K / BK;
    const int my_tiles = (num_tiles - pair + pairs - 1) / pairs;

    if (skip) {
      // nothing to do; fall through to the common exit
    } else if (warp == 0) {
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = pair; tile < num_tiles && ok; tile += pairs) {
          const int tn = tile % tiles_n, mb = 2 * (tile / tiles_n) + static_cast<int>(cta_rank);
          const int src = g.order[2 * mb], b = g.order[2 * mb + 1];
          const bool local = src == g.rank;
          if (!local) {
            if (!wait_flag_ge(&page->ag_flag[src][b], epoch, p.abort_flag)) {
              gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_FLAG, 0, src * 64 + b);
              ok = false;
              break;
            }
            fence_proxy_async();       // peer stores (generic proxy) before my TMA reads (async proxy)
          }
          const int a_row = local ? b * BM : src * g.rows_per_rank + b * BM;
          const int b_row = tn * PBN + static_cast<int>(cta_rank) * (PBN / 2);
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(&p.empty_bar[stage], phase ^ 1, p.abort_flag)) {
              gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_EMPTY, 0, stage);
              ok = false;
              break;
            }
            uint8_t* a_dst = p.stage_base + static_cast<size_t>(stage) * kPStageBytes;
            if (leader) mbar_expect_tx(&p.full_bar[stage], 2 * kPStageBytes);
            const uint32_t leader_full = map_to_cta(smem_u32(&p.full_bar[stage]), 0);
            if (local) tma_load_2d_pair(a_dst, &map_local, leader_full, kb * BK, a_row);
            else if (parity) tma_load_2d_pair(a_dst, &map_gath1, leader_full, kb * BK, a_row);
            else tma_load_2d_pair(a_dst, &map_gath0, leader_full, kb * BK, a_row);
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
      __nv_bfloat16* d = static_cast<__nv_bfloat16*>(g.d);
      for (int tile = pair; tile < num_tiles; tile += pairs) {
        const int tn = tile % tiles_n, mb = 2 * (tile / tiles_n) + static_cast<int>(cta_rank);
        const int src = g.order[2 * mb], b = g.order[2 * mb + 1];
        bool ok = mbar_wait(&p.acc_full[acc], acc_phase, p.abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_ACC, 2, acc);
          break;
        }
        tc_fence_after_sync();
        const size_t row = static_cast<size_t>(src) * g.rows_per_rank + b * BM + quarter * 32 + lane;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * PBN);
        if (EPI == 0) {
#pragma unroll 1
          for (int c = 0; c < PBN; c += 32) {
            uint32_t r[32];
            tmem_ld32(taddr + c, r);
            tc_wait_ld();
            uint4* out = reinterpret_cast<uint4*>(d + row * g.ldd + tn * PBN + c);
#pragma unroll
            for (int v = 0; v < 4; ++v)
              out[v] = make_uint4(pack_bf16(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1])),
                                  pack_bf16(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3])),
                                  pack_bf16(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5])),
                                  pack_bf16(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7])));
          }
        } else {
          constexpr int H = PBN / 2;
#pragma unroll 1
          for (int c = 0; c < H; c += 32) {
            uint32_t gt[32], up[32];
            tmem_ld32(taddr + c, gt);
            tmem_ld32(taddr + H + c, up);
            tc_wait_ld();
            uint4* out = reinterpret_cast<uint4*>(d + row * g.ldd + tn * H + c);
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
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&p.acc_empty[acc]), 0));   // the leader's barrier
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    tc_fence_before_sync();
    cluster_sync_all();                                // nothing of the pair is in flight any more
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc_pair(tmem_base, kPTmemCols);
    }
  }
  if (skip) return;
  // the last CTA to finish advances the launch epoch of this rank
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&page->ag_done, 1u) == gridDim.x - 1u) {
      page->ag_done = 0;
      page->ag_epoch = epoch;
    }
  }
}

// ============================================================ GEMM -> reduce-scatter on CTA pairs
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_rs_2cta_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmRsArgs g) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_skip;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  FusedPage* page = g.pages[g.rank];
  const unsigned long long epoch = page->rs_epoch + 1;
  const int parity = static_cast<int>(epoch & 1ull);
  const int blocks_per_rank = g.rows_per_rank / BM;
  const int tiles_n = g.N / PBN;
  const int k_blocks = g.K / BK;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int cluster = static_cast<int>(cluster_id_x()), clusters = static_cast<int>(num_clusters_x());
  const int pairs = clusters - g.reduce_ctas / 2;      // clusters that run the GEMM
  const size_t slab_bytes = static_cast<size_t>(g.rows_per_rank) * g.N * 2;
  const size_t parity_off = g.partial_off + static_cast<size_t>(parity) * g.nranks * slab_bytes;
  const unsigned long long per_block = 4ull * static_cast<unsigned long long>(tiles_n);   // counts per (source, row block) and launch
  bool skip = false;

  if (cluster >= pairs) {
    // ------------------------------------------------------------------ reducer clusters
    skip = g.error_words != nullptr && *reinterpret_cast<volatile int*>(g.error_words) != 0;
    if (!skip) reduce_items(g, page, g.heap_bases[g.rank] + parity_off, slab_bytes, blocks_per_rank, per_block);
  } else {
    const PairPipe p = carve_pair<kRsStages>(smem_raw);
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
    skip = ld_shared_cluster_u32(map_to_cta(smem_u32(&s_skip), 0)) != 0;
    const int num_tiles = (blocks_per_rank * g.nranks / 2) * tiles_n;
    const int my_tiles = (num_tiles - cluster + pairs - 1) / pairs;

    if (skip) {
      // nothing to do; fall through to the common exit
    } else if (warp == 0) {
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = cluster; tile < num_tiles && ok; tile += pairs) {
          const int tn = tile % tiles_n, rb = 2 * (tile / tiles_n) + static_cast<int>(cta_rank);
          const int owner = g.order[2 * rb], b = g.order[2 * rb + 1];
          const int a_row = owner * g.rows_per_rank + b * BM;
          const int b_row = tn * PBN + static_cast<int>(cta_rank) * (PBN / 2);
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
      int pend_owner = -1, pend_b = 0;                      // the tile whose stores were issued last
      for (int tile = cluster; tile < num_tiles; tile += pairs) {
        const int tn = tile % tiles_n, rb = 2 * (tile / tiles_n) + static_cast<int>(cta_rank);
        const int owner = g.order[2 * rb], b = g.order[2 * rb + 1];
        bool ok = mbar_wait(&p.acc_full[acc], acc_phase, p.abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_ACC, 2, acc);
          break;
        }
        tc_fence_after_sync();
        // destination: the owner's slab for source = me, local row inside the owner's shard
        char* slab = g.heap_bases[owner] + parity_off + static_cast<size_t>(g.rank) * slab_bytes;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * PBN);
        uint8_t* stage_warp = p.staging + (warp - 2) * kStagingPerWarp;
        stage_quarter_bf16(taddr, stage_warp, lane, 1.0f);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&p.acc_empty[acc]), 0));   // free as soon as it sits in shared memory
        // count the previous tile on its owner: its stores were issued a whole tile ago, so the release has nothing
        // left to wait for (a release right behind the stores, let alone a system-scope fence, cost 8-30 us a tile)
        if (pend_owner >= 0 && lane == 0) red_add_release_sys(&g.pages[pend_owner]->rs_count[g.rank][pend_b], 1ull);
        // one row (512 contiguous bytes) per store instruction, 8 rows in flight
        char* dst0 = slab + ((static_cast<size_t>(b) * BM + quarter * 32) * g.N + static_cast<size_t>(tn) * PBN) * 2 + lane * 16;
#pragma unroll 1
        for (int r0 = 0; r0 < 32; r0 += 8) {
          uint4 d[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) d[u] = *reinterpret_cast<const uint4*>(stage_warp + (r0 + u) * kStagePitch + lane * 16);
#pragma unroll
          for (int u = 0; u < 8; ++u) *reinterpret_cast<uint4*>(dst0 + static_cast<size_t>(r0 + u) * g.N * 2) = d[u];
        }
        __syncwarp();
        pend_owner = owner;                                  // published while the next tile is staged (or after the loop)
        pend_b = b;
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      // the last tile of this warp
      if (pend_owner >= 0 && lane == 0) red_add_release_sys(&g.pages[pend_owner]->rs_count[g.rank][pend_b], 1ull);
    }
    tc_fence_before_sync();
    cluster_sync_all();                                // nothing of the pair is in flight any more
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc_pair(tmem_base, kPTmemCols);
    }
    // the tiles of this CTA are out: help with the reduction
    if (!skip) reduce_items(g, page, g.heap_bases[g.rank] + parity_off, slab_bytes, blocks_per_rank, per_block);
  }
  if (skip) return;
  finish_rs_launch(g, page, blocks_per_rank, per_block, epoch);
}

}  // namespace

// Same contract as launch_ag_gemm; additionally N % 256 == 0, an even number of row blocks in total and an even
// number of comm CTAs.  `grid` is the number of CTAs wanted (0: as many pairs as the device holds at once).
cudaError_t launch_ag_gemm_2cta(const AgGemmArgs& g, int epilogue, int grid, cudaStream_t stream) {
  if (g.K % BK != 0 || g.N % PBN != 0 || g.rows_per_rank % BM != 0 || g.rows_per_rank / BM > kFusedMaxBlocks ||
      g.nranks > kFusedMaxRanks || g.comm_ctas < 2 || g.comm_ctas % 2 != 0 || g.order == nullptr ||
      (g.rows_per_rank / BM * g.nranks) % 2 != 0)
    return cudaErrorInvalidValue;
  static int resident[2] = {0, 0};
  const int e = epilogue != 0;
  if (resident[e] == 0) {
    cudaError_t err = e ? pair_clusters(ag_gemm_2cta_kernel<1>, kAgSmemBytes, &resident[e])
                        : pair_clusters(ag_gemm_2cta_kernel<0>, kAgSmemBytes, &resident[e]);
    if (err != cudaSuccess) return err;
  }
  int clusters = resident[e];
  if (grid > 0 && grid / 2 < clusters) clusters = grid / 2;
  if (clusters <= g.comm_ctas / 2) return cudaErrorLaunchOutOfResources;
  const uint64_t all_rows = static_cast<uint64_t>(g.rows_per_rank) * g.nranks;
  CUtensorMap map_local = make_bf16_kmajor_map(g.x_local, g.rows_per_rank, g.K, g.K, BM);
  const char* gath = g.heap_bases_host[g.rank] + g.gathered_off;
  CUtensorMap map_g0 = make_bf16_kmajor_map(gath, all_rows, g.K, g.K, BM);
  CUtensorMap map_g1 = make_bf16_kmajor_map(gath + g.gathered_bytes, all_rows, g.K, g.K, BM);
  CUtensorMap map_b = make_bf16_kmajor_map(g.b, g.N, g.K, g.ldb, PBN / 2);
  return e ? launch_pairs(ag_gemm_2cta_kernel<1>, kAgSmemBytes, clusters, stream, map_local, map_g0, map_g1, map_b, g)
           : launch_pairs(ag_gemm_2cta_kernel<0>, kAgSmemBytes, clusters, stream, map_local, map_g0, map_g1, map_b, g);
}

// Same contract as launch_gemm_rs; additionally N % 256 == 0, an even number of row blocks in total and an even
// number of reducer CTAs.
cudaError_t launch_gemm_rs_2cta(const GemmRsArgs& g, int grid, cudaStream_t stream) {
  if (g.K % BK != 0 || g.N % PBN != 0 || g.rows_per_rank % BM != 0 || g.rows_per_rank / BM > kFusedMaxBlocks ||
      g.nranks > kFusedMaxRanks || g.reduce_ctas < 2 || g.reduce_ctas % 2 != 0 || g.order == nullptr ||
      g.reduce_order == nullptr || (g.rows_per_rank / BM * g.nranks) % 2 != 0)
    return cudaErrorInvalidValue;
  static int resident = 0;
  if (resident == 0) {
    cudaError_t err = pair_clusters(gemm_rs_2cta_kernel, kRsSmemBytes, &resident);
    if (err != cudaSuccess) return err;
  }
  int clusters = resident;
  if (grid > 0 && grid / 2 < clusters) clusters = grid / 2;
  if (clusters <= g.reduce_ctas / 2) return cudaErrorLaunchOutOfResources;
  CUtensorMap map_a = make_bf16_kmajor_map(g.a, static_cast<uint64_t>(g.rows_per_rank) * g.nranks, g.K, g.lda, BM);
  CUtensorMap map_b = make_bf16_kmajor_map(g.b, g.N, g.K, g.ldb, PBN / 2);
  return launch_pairs(gemm_rs_2cta_kernel, kRsSmemBytes, clusters, stream, map_a, map_b, g);
}

}  // namespace sm100
}  // namespace msccl
