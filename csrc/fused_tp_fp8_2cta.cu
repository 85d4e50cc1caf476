// The block-scaled fp8 tensor-parallel kernels of fused_tp_fp8.cu on CTA pairs (tcgen05 cta_group::2, 256 x 256
// tiles): the MX pipeline of the plain pair GEMM (mxfp8_pair.cuh) with the collectives of fused_tp_2cta.cu around it.
//
//   all-gather -> GEMM       the two row blocks of a pair tile are two consecutive entries of the order table; CTA r
//       waits for the flag of entry 2t + r and fetches its 128 rows of e4m3 values and their scale block from the
//       LOCAL gathered buffer (values and scales are both tensor loads that complete on the leader's mbarrier; no
//       multicast, no peer memory), its half of the weight tile and the scales of all 256 weight rows.
//   GEMM -> reduce-scatter   CTA r packs its partial tile to bf16 in shared memory, stores it into the owner's slab
//       and bumps the (source, row block) counter there; reducer clusters and the work items are those of the bf16
//       kernel (fused_reduce.cuh).
// One 256-column accumulator (two plus the scale columns do not fit into tensor memory): the epilogue releases it as
// soon as the tile sits in shared memory.  Every wait is bounded.
#include <cuda.h>
#include <cuda_runtime.h>

#include "fused_fp8_push.cuh"
#include "fused_reduce.cuh"
#include "fused_tp.h"
#include "gemm_sm100.cuh"
#include "gemm_sm100.h"
#include "mxfp8_pair.cuh"
#include "pair_pipeline.cuh"
#include "pipeline_sm100.cuh"
#include "prims.cuh"

namespace msccl {
namespace sm100 {

namespace {

struct QPipe {
  uint8_t* stage_base;
  uint8_t* epi;                                        // staged epilogue: 4 warps x 32 rows x 128 bf16
  uint64_t *full_bar, *empty_bar, *acc_full, *acc_empty;
  uint32_t* tmem_slot;
  volatile int* abort_flag;
};

__device__ __forceinline__ QPipe carve_q(uint8_t* smem_raw) {
  QPipe p;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  p.stage_base = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(kQStages) * kQStageBytes);
  p.full_bar = bars;                                   // leader only: loads of both CTAs complete here
  p.empty_bar = bars + kQStages;                       // per CTA: commit from the leader
  p.acc_full = bars + 2 * kQStages;                    // per CTA: commit from the leader
  p.acc_empty = bars + 2 * kQStages + 1;               // leader only: 8 epilogue warps of the pair
  p.tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kQStages + 2);
  p.abort_flag = reinterpret_cast<volatile int*>(p.tmem_slot + 1);
  p.epi = smem + static_cast<size_t>(kQStages) * kQStageBytes + 256;
  return p;
}

__device__ __forceinline__ void init_q(const QPipe& p) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < kQStages; ++s) {
      mbar_init(&p.full_bar[s], 1);
      mbar_init(&p.empty_bar[s], 1);
    }
    mbar_init(p.acc_full, 1);
    mbar_init(p.acc_empty, 8);
    *p.abort_flag = 0;
    mbar_fence_init();
  }
}

__device__ __forceinline__ void drain_q(const QPipe& p, bool leader) {
  if (leader) {
    for (int s = 0; s < kQStages; ++s)
      for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&p.full_bar[s], 0) && !mbar_try_wait(&p.full_bar[s], 1); ++i) {}
  } else {
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {}
  }
}

// One stage of a pair tile: this CTA's rows of A and of B, the scales of its A rows and of all 256 B rows.
__device__ __forceinline__ void load_stage_q(const QPipe& p, int stage, bool leader, const CUtensorMap* map_a, int a_row,
                                             const CUtensorMap* map_sfa, int sfa_block, const CUtensorMap* map_b, int b_row,
                                             const CUtensorMap* map_sfb, int sfb_block0, int sfb_block1, int kb) {
  uint8_t* a_dst = p.stage_base + static_cast<size_t>(stage) * kQStageBytes;
  uint8_t* b_dst = a_dst + kQABytes;
  uint8_t* sf_dst = b_dst + kQBBytes;
  if (leader) mbar_expect_tx(&p.full_bar[stage], 2 * kQLoadBytes);
  const uint32_t leader_full = map_to_cta(smem_u32(&p.full_bar[stage]), 0);
  tma_load_2d_pair8(a_dst, map_a, leader_full, kb * QBK, a_row);
  tma_load_2d_pair8(b_dst, map_b, leader_full, kb * QBK, b_row);
  tma_load_2d_pair8(sf_dst, map_sfa, leader_full, 0, sfa_block + kb);
  tma_load_2d_pair8(sf_dst + kQSfBytes, map_sfb, leader_full, 0, sfb_block0 + kb);
  tma_load_2d_pair8(sf_dst + 2 * kQSfBytes, map_sfb, leader_full, 0, sfb_block1 + kb);
}

// 32 staged rows of kQStageCols bf16 -> `dst0` (row pitch `pitch_bytes`), 16 lanes per row, 8 stores in flight.
__device__ __forceinline__ void store_staged_rows(const uint8_t* epi, char* dst0, size_t pitch_bytes, int lane, int rows_valid) {
  constexpr int kLanesPerRow = kQStageCols * 2 / 16, kRowsPerStore = 32 / kLanesPerRow;
  const int sub_row = lane / kLanesPerRow, sub_col = (lane % kLanesPerRow) * 16;
#pragma unroll 1
  for (int r0 = 0; r0 < 32; r0 += 8 * kRowsPerStore) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = *reinterpret_cast<const uint4*>(epi + (r0 + u * kRowsPerStore + sub_row) * kQEpiPitch + sub_col);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int rr = r0 + u * kRowsPerStore + sub_row;
      if (rr < rows_valid) *reinterpret_cast<uint4*>(dst0 + static_cast<size_t>(rr) * pitch_bytes + sub_col) = v[u];
    }
  }
}

// 32 accumulator columns of this lane's row -> bf16 in the staging row.
__device__ __forceinline__ void pack_chunk(const uint32_t (&r)[32], uint8_t* epi, int lane, int col) {
  uint4* dst = reinterpret_cast<uint4*>(epi + lane * kQEpiPitch + col * 2);
#pragma unroll
  for (int v = 0; v < 4; ++v)
    dst[v] = make_uint4(pack_bf16(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1])),
                        pack_bf16(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3])),
                        pack_bf16(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5])),
                        pack_bf16(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7])));
}

// kQStageCols accumulator columns starting at `taddr` -> bf16 staging rows; the tensor-memory load of the next 32
// columns is in flight while these are packed.
__device__ __forceinline__ void stage_plain_cols(uint32_t taddr, uint8_t* epi, int lane) {
  uint32_t r[2][32];
  tmem_ld32(taddr, r[0]);
#pragma unroll
  for (int c = 0; c < kQStageCols; c += 32) {
    const int cur = (c / 32) & 1;
    tc_wait_ld();
    if (c + 32 < kQStageCols) tmem_ld32(taddr + c + 32, r[cur ^ 1]);
    pack_chunk(r[cur], epi, lane, c);
  }
}

// SwiGLU of a whole tile: gate columns [0, 128) and up columns [128, 256) of the accumulator -> 128 bf16 columns.
__device__ __forceinline__ void stage_swiglu_cols(uint32_t taddr, uint8_t* epi, int lane) {
  constexpr int H = QBN / 2;
  uint32_t gt[2][32], up[2][32];
  tmem_ld32(taddr, gt[0]);
  tmem_ld32(taddr + H, up[0]);
#pragma unroll
  for (int c = 0; c < H; c += 32) {
    const int cur = (c / 32) & 1;
    tc_wait_ld();
    if (c + 32 < H) {
      tmem_ld32(taddr + c + 32, gt[cur ^ 1]);
      tmem_ld32(taddr + H + c + 32, up[cur ^ 1]);
    }
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      const float gv = __uint_as_float(gt[cur][e]);
      gt[cur][e] = __float_as_uint(gv / (1.0f + __expf(-gv)) * __uint_as_float(up[cur][e]));
    }
    pack_chunk(gt[cur], epi, lane, c);
  }
}

// ============================================================ all-gather -> GEMM (+SwiGLU), MX fp8, CTA pairs
struct AgF8Maps {
  CUtensorMap local, gath0, gath1, b;              // values
  CUtensorMap sf_local, sf_gath0, sf_gath1, sfb;   // scale blocks of 512 bytes
};

template <int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
ag_gemm_mxfp8_2cta_kernel(const __grid_constant__ AgF8Maps maps, AgGemmF8Args g) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_skip;
  const QPipe p = carve_q(smem_raw);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  FusedPage* page = g.pages[g.rank];
  const unsigned long long epoch = page->ag_epoch + 1;
  const int parity = static_cast<int>(epoch & 1ull);
  const int blocks_per_rank = g.rows_per_rank / BM;
  const int k_blocks = g.K / QBK;
  const size_t parity_off = g.gathered_off + static_cast<size_t>(parity) * g.gathered_bytes;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int cluster = static_cast<int>(cluster_id_x()), clusters = static_cast<int>(num_clusters_x());
  const int comm_clusters = g.comm_ctas / 2;
  bool skip = false;

  if (cluster < comm_clusters) {
    // ------------------------------------------------------------------ comm CTAs (whole clusters, no tensor memory)
    skip = g.error_words != nullptr && *reinterpret_cast<volatile int*>(g.error_words) != 0;
    if (!skip) push_f8_blocks(g, page, epoch, parity_off);
  } else {
    // ------------------------------------------------------------------ GEMM pairs
    if (threadIdx.x == 0) s_skip = (g.error_words != nullptr && *reinterpret_cast<volatile int*>(g.error_words) != 0) ? 1 : 0;
    init_q(p);
    if (threadIdx.x == 0) {
      prefetch_tensormap(&maps.local);
      prefetch_tensormap(&maps.b);
      prefetch_tensormap(&maps.sf_local);
      prefetch_tensormap(&maps.sfb);
    }
    if (warp == 1) tmem_alloc_pair(p.tmem_slot, kQTmemCols);
    tc_fence_before_sync();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *p.tmem_slot;
    skip = ld_shared_cluster_u32(map_to_cta(smem_u32(&s_skip), 0)) != 0;       // the leader's reading decides for the pair

    const int pairs = clusters - comm_clusters, pair = cluster - comm_clusters;
    const int tiles_n = g.N / QBN;
    const int num_tiles = (blocks_per_rank * g.nranks / 2) * tiles_n;
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
            fence_proxy_async();       // peer stores (generic proxy) before my tensor loads (async proxy)
          }
          const CUtensorMap* map_a = local ? &maps.local : (parity ? &maps.gath1 : &maps.gath0);
          const CUtensorMap* map_sfa = local ? &maps.sf_local : (parity ? &maps.sf_gath1 : &maps.sf_gath0);
          const int a_row = local ? b * BM : src * g.rows_per_rank + b * BM;
          const int sfa_block = (local ? b : src * blocks_per_rank + b) * k_blocks;
          const int b_row = tn * QBN + static_cast<int>(cta_rank) * (QBN / 2);
          const int sfb_block0 = tn * 2 * k_blocks, sfb_block1 = sfb_block0 + k_blocks;
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(&p.empty_bar[stage], phase ^ 1, p.abort_flag)) {
              gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_EMPTY, 0, stage);
              ok = false;
              break;
            }
            load_stage_q(p, stage, leader, map_a, a_row, map_sfa, sfa_block, &maps.b, b_row, &maps.sfb, sfb_block0, sfb_block1, kb);
            if (++stage == kQStages) { stage = 0; phase ^= 1; }
          }
        }
        if (!ok) drain_q(p, leader);
      }
    } else if (warp == 1) {
      if (lane == 0 && leader)
        mma_role_mx_pair<kQStages>(p.stage_base, p.full_bar, p.empty_bar, p.acc_full, p.acc_empty, tmem_base, my_tiles, k_blocks,
                                   p.abort_flag, g.error_words);
    } else {
      const int quarter = warp % 4;
      uint32_t acc_phase = 0;
      __nv_bfloat16* d = static_cast<__nv_bfloat16*>(g.d);
      uint8_t* epi = p.epi + (warp - 2) * kQEpiPerWarp;
      for (int tile = pair; tile < num_tiles; tile += pairs) {
        const int tn = tile % tiles_n, mb = 2 * (tile / tiles_n) + static_cast<int>(cta_rank);
        const int src = g.order[2 * mb], b = g.order[2 * mb + 1];
        bool ok = mbar_wait(p.acc_full, acc_phase, p.abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_ACC, 2, 0);
          break;
        }
        tc_fence_after_sync();
        const size_t row0 = static_cast<size_t>(src) * g.rows_per_rank + b * BM + quarter * 32;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        if (EPI == 0) {
#pragma unroll 1
          for (int c0 = 0; c0 < QBN; c0 += kQStageCols) {
            stage_plain_cols(taddr + c0, epi, lane);
            if (c0 + kQStageCols == QBN) {
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(p.acc_empty), 0));   // the accumulator is read
            } else {
              __syncwarp();
            }
            store_staged_rows(epi, reinterpret_cast<char*>(d + row0 * g.ldd + tn * QBN + c0), static_cast<size_t>(g.ldd) * 2, lane, 32);
            __syncwarp();
          }
        } else {
          constexpr int H = QBN / 2;       // the tile holds 128 gate columns followed by the 128 up columns of the same features
          stage_swiglu_cols(taddr, epi, lane);
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(p.acc_empty), 0));       // the accumulator is read
          store_staged_rows(epi, reinterpret_cast<char*>(d + row0 * g.ldd + tn * H), static_cast<size_t>(g.ldd) * 2, lane, 32);
          __syncwarp();
        }
        acc_phase ^= 1;
      }
    }
    tc_fence_before_sync();
    cluster_sync_all();                                // nothing of the pair is in flight any more
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc_pair(tmem_base, kQTmemCols);
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

// ============================================================ GEMM -> reduce-scatter, MX fp8 operands, CTA pairs
struct RsF8Maps {
  CUtensorMap a, b, sfa, sfb;
};

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_rs_mxfp8_2cta_kernel(const __grid_constant__ RsF8Maps maps, GemmRsF8Args g) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_skip;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  FusedPage* page = g.pages[g.rank];
  const unsigned long long epoch = page->rs_epoch + 1;
  const int parity = static_cast<int>(epoch & 1ull);
  const int blocks_per_rank = g.rows_per_rank / BM;
  const int tiles_n = g.N / QBN;
  const int k_blocks = g.K / QBK;
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
    const QPipe p = carve_q(smem_raw);
    if (threadIdx.x == 0) s_skip = (g.error_words != nullptr && *reinterpret_cast<volatile int*>(g.error_words) != 0) ? 1 : 0;
    init_q(p);
    if (threadIdx.x == 0) {
      prefetch_tensormap(&maps.a);
      prefetch_tensormap(&maps.b);
      prefetch_tensormap(&maps.sfa);
      prefetch_tensormap(&maps.sfb);
    }
    if (warp == 1) tmem_alloc_pair(p.tmem_slot, kQTmemCols);
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
          const int row_block = owner * blocks_per_rank + b;
          const int b_row = tn * QBN + static_cast<int>(cta_rank) * (QBN / 2);
          const int sfb_block0 = tn * 2 * k_blocks, sfb_block1 = sfb_block0 + k_blocks;
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(&p.empty_bar[stage], phase ^ 1, p.abort_flag)) {
              gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_EMPTY, 0, stage);
              ok = false;
              break;
            }
            load_stage_q(p, stage, leader, &maps.a, row_block * BM, &maps.sfa, row_block * k_blocks, &maps.b, b_row, &maps.sfb,
                         sfb_block0, sfb_block1, kb);
            if (++stage == kQStages) { stage = 0; phase ^= 1; }
          }
        }
        if (!ok) drain_q(p, leader);
      }
    } else if (warp == 1) {
      if (lane == 0 && leader)
        mma_role_mx_pair<kQStages>(p.stage_base, p.full_bar, p.empty_bar, p.acc_full, p.acc_empty, tmem_base, my_tiles, k_blocks,
                                   p.abort_flag, g.error_words);
    } else {
      const int quarter = warp % 4;
      uint32_t acc_phase = 0;
      uint8_t* epi = p.epi + (warp - 2) * kQEpiPerWarp;
      int pend_owner = -1, pend_b = 0;                      // the tile whose stores were issued last
      for (int tile = cluster; tile < num_tiles; tile += pairs) {
        const int tn = tile % tiles_n, rb = 2 * (tile / tiles_n) + static_cast<int>(cta_rank);
        const int owner = g.order[2 * rb], b = g.order[2 * rb + 1];
        bool ok = mbar_wait(p.acc_full, acc_phase, p.abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_ACC, 2, 0);
          break;
        }
        tc_fence_after_sync();
        // count the previous tile on its owner: its stores were issued a whole tile ago, so the release has nothing
        // left to wait for (a release right behind the stores, let alone a system-scope fence, cost 8-30 us a tile)
        if (pend_owner >= 0 && lane == 0) red_add_release_sys(&g.pages[pend_owner]->rs_count[g.rank][pend_b], 1ull);
        // destination: the owner's slab for source = me, local row inside the owner's shard
        char* slab = g.heap_bases[owner] + parity_off + static_cast<size_t>(g.rank) * slab_bytes;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
        for (int c0 = 0; c0 < QBN; c0 += kQStageCols) {
          stage_plain_cols(taddr + c0, epi, lane);
          if (c0 + kQStageCols == QBN) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(p.acc_empty), 0));     // the accumulator is read
          } else {
            __syncwarp();
          }
          char* dst0 = slab + ((static_cast<size_t>(b) * BM + quarter * 32) * g.N + static_cast<size_t>(tn) * QBN + c0) * 2;
          store_staged_rows(epi, dst0, static_cast<size_t>(g.N) * 2, lane, 32);
          __syncwarp();
        }
        pend_owner = owner;                                  // published while the next tile is staged (or after the loop)
        pend_b = b;
        acc_phase ^= 1;
      }
      // the last tile of this warp
      if (pend_owner >= 0 && lane == 0) red_add_release_sys(&g.pages[pend_owner]->rs_count[g.rank][pend_b], 1ull);
    }
    tc_fence_before_sync();
    cluster_sync_all();                                // nothing of the pair is in flight any more
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc_pair(tmem_base, kQTmemCols);
    }
    // the tiles of this CTA are out: help with the reduction
    if (!skip) reduce_items(g, page, g.heap_bases[g.rank] + parity_off, slab_bytes, blocks_per_rank, per_block);
  }
  if (skip) return;
  finish_rs_launch(g, page, blocks_per_rank, per_block, epoch);
}

}  // namespace

// Same contract as launch_ag_gemm_mxfp8; additionally N % 256 == 0, an even number of row blocks in total and an
// even number of comm CTAs; with the SwiGLU epilogue the weight rows are interleaved per 256 (128 gate, 128 up).
cudaError_t launch_ag_gemm_mxfp8_2cta(const AgGemmF8Args& g, int epilogue, int grid, cudaStream_t stream) {
  if (g.K % QBK != 0 || g.N % QBN != 0 || g.rows_per_rank % BM != 0 || g.rows_per_rank / BM > kFusedMaxBlocks ||
      g.nranks > kFusedMaxRanks || g.comm_ctas < 2 || g.comm_ctas % 2 != 0 || g.order == nullptr ||
      (g.rows_per_rank / BM * g.nranks) % 2 != 0)
    return cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(g.sf_local) % 16 != 0 || reinterpret_cast<uintptr_t>(g.sfb) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(g.x_local) % 16 != 0 || g.gathered_off % 1024 != 0 || g.gathered_bytes % 1024 != 0)
    return cudaErrorInvalidValue;
  static int resident[2] = {0, 0};
  const int e = epilogue != 0;
  if (resident[e] == 0) {
    cudaError_t err = e ? pair_clusters(ag_gemm_mxfp8_2cta_kernel<1>, kQSmemBytes, &resident[e])
                        : pair_clusters(ag_gemm_mxfp8_2cta_kernel<0>, kQSmemBytes, &resident[e]);
    if (err != cudaSuccess) return err;
  }
  int clusters = resident[e];
  if (grid > 0 && grid / 2 < clusters) clusters = grid / 2;
  if (clusters <= g.comm_ctas / 2) return cudaErrorLaunchOutOfResources;
  const uint64_t all_rows = static_cast<uint64_t>(g.rows_per_rank) * g.nranks;
  const uint64_t k_blocks = static_cast<uint64_t>(g.K / QBK);
  const char* gath = g.heap_bases_host[g.rank] + g.gathered_off;
  const size_t all_values = static_cast<size_t>(all_rows) * g.K;
  AgF8Maps maps;
  maps.local = make_u8_kmajor_map(g.x_local, g.rows_per_rank, g.K, g.K, BM);
  maps.gath0 = make_u8_kmajor_map(gath, all_rows, g.K, g.K, BM);
  maps.gath1 = make_u8_kmajor_map(gath + g.gathered_bytes, all_rows, g.K, g.K, BM);
  maps.b = make_u8_kmajor_map(g.b, g.N, g.K, g.ldb, QBN / 2);
  maps.sf_local = make_block512_map(g.sf_local, static_cast<uint64_t>(g.rows_per_rank / BM) * k_blocks);
  maps.sf_gath0 = make_block512_map(gath + all_values, all_rows / BM * k_blocks);
  maps.sf_gath1 = make_block512_map(gath + g.gathered_bytes + all_values, all_rows / BM * k_blocks);
  maps.sfb = make_block512_map(g.sfb, static_cast<uint64_t>(g.N / 128) * k_blocks);
  return e ? launch_pairs(ag_gemm_mxfp8_2cta_kernel<1>, kQSmemBytes, clusters, stream, maps, g)
           : launch_pairs(ag_gemm_mxfp8_2cta_kernel<0>, kQSmemBytes, clusters, stream, maps, g);
}

// Same contract as launch_gemm_rs_mxfp8; additionally N % 256 == 0, an even number of row blocks in total and an
// even number of reducer CTAs.
cudaError_t launch_gemm_rs_mxfp8_2cta(const GemmRsF8Args& g, int grid, cudaStream_t stream) {
  if (g.K % QBK != 0 || g.N % QBN != 0 || g.rows_per_rank % BM != 0 || g.rows_per_rank / BM > kFusedMaxBlocks ||
      g.nranks > kFusedMaxRanks || g.reduce_ctas < 2 || g.reduce_ctas % 2 != 0 || g.order == nullptr ||
      g.reduce_order == nullptr || (g.rows_per_rank / BM * g.nranks) % 2 != 0)
    return cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(g.sfa) % 16 != 0 || reinterpret_cast<uintptr_t>(g.sfb) % 16 != 0) return cudaErrorInvalidValue;
  static int resident = 0;
  if (resident == 0) {
    cudaError_t err = pair_clusters(gemm_rs_mxfp8_2cta_kernel, kQSmemBytes, &resident);
    if (err != cudaSuccess) return err;
  }
  int clusters = resident;
  if (grid > 0 && grid / 2 < clusters) clusters = grid / 2;
  if (clusters <= g.reduce_ctas / 2) return cudaErrorLaunchOutOfResources;
  const uint64_t all_rows = static_cast<uint64_t>(g.rows_per_rank) * g.nranks;
  const uint64_t k_blocks = static_cast<uint64_t>(g.K / QBK);
  RsF8Maps maps;
  maps.a = make_u8_kmajor_map(g.a, all_rows, g.K, g.lda, BM);
  maps.b = make_u8_kmajor_map(g.b, g.N, g.K, g.ldb, QBN / 2);
  maps.sfa = make_block512_map(g.sfa, all_rows / BM * k_blocks);
  maps.sfb = make_block512_map(g.sfb, static_cast<uint64_t>(g.N / 128) * k_blocks);
  return launch_pairs(gemm_rs_mxfp8_2cta_kernel, kQSmemBytes, clusters, stream, maps, g);
}

}  // namespace sm100
}  // namespace msccl
