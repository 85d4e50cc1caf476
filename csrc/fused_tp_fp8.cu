// Fused tensor-parallel kernels with block-scaled fp8 operands (OCP MX: e4m3 values, one UE8M0 scale per 32 K
// elements of a row) for sm_100a.  Same structure as the bf16 kernels of fused_tp.cu - comm CTAs push the local
// shard to every peer in 128-row blocks with one flag per block while the other CTAs run the persistent GEMM;
// partial tiles go straight into the owner's slab with per-(source, block) counters and a few CTAs only reduce -
// on the single-CTA MX pipeline of gemm_mxfp8_sm100.cu:
//
//   all-gather -> GEMM   what travels per block is 128 x K value bytes plus K/128 scale blocks of 512 bytes, half
//       of what the bf16 kernel moves; the producer fetches the values with TMA and the scale blocks with untiled
//       bulk copies, both from the LOCAL gathered buffer (never from peer memory, never with multicast); the MMA
//       issuer copies the scales into tensor memory and issues tcgen05.mma.kind::mxf8f6f4.block_scale.
//   GEMM -> reduce-scatter   the partial sums leave as bf16, so slabs, counters and the reducer CTAs are those of
//       the bf16 kernel (fused_reduce.cuh).
//
// Row blocks are walked in the order tables lowered from the schedule programs (msccl.ops.schedules).  Every wait
// is bounded.
#include <cuda.h>
#include <cuda_runtime.h>

#include "fused_reduce.cuh"
#include "fused_tp.h"
#include "gemm_sm100.cuh"
#include "gemm_sm100.h"
#include "fused_fp8_push.cuh"
#include "mxfp8_sm100.cuh"
#include "pipeline_sm100.cuh"
#include "prims.cuh"

namespace msccl {
namespace sm100 {

namespace {

constexpr int kRsF8Stages = 5;                                   // one stage less than the plain kernel: room for staging
constexpr int kF8StagePitch = FBN * 2 + 16;                      // bytes per staged row of 128 bf16 (+16: bank spread)
constexpr int kF8StagingPerWarp = 32 * kF8StagePitch;
constexpr size_t kRsF8SmemBytes = 1024 + static_cast<size_t>(kRsF8Stages) * kF8StageBytes + 256 + 4 * kF8StagingPerWarp;

struct F8Pipe {
  uint8_t* stage_base;
  uint8_t* staging;
  uint64_t *full_bar, *empty_bar, *acc_full, *acc_empty;
  uint32_t* tmem_slot;
  volatile int* abort_flag;
};

template <int STAGES>
__device__ __forceinline__ F8Pipe carve_f8(uint8_t* smem_raw) {
  F8Pipe p;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  p.stage_base = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(STAGES) * kF8StageBytes);
  p.full_bar = bars;
  p.empty_bar = bars + STAGES;
  p.acc_full = bars + 2 * STAGES;
  p.acc_empty = bars + 2 * STAGES + 2;
  p.tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  p.abort_flag = reinterpret_cast<volatile int*>(p.tmem_slot + 1);
  p.staging = smem + static_cast<size_t>(STAGES) * kF8StageBytes + 256;
  return p;
}

template <int STAGES>
__device__ __forceinline__ void init_f8(const F8Pipe& p) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&p.full_bar[s], 1);
      mbar_init(&p.empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&p.acc_full[a], 1);
      mbar_init(&p.acc_empty[a], 4);
    }
    *p.abort_flag = 0;
    mbar_fence_init();
  }
}

template <int STAGES>
__device__ __forceinline__ void drain_f8(const F8Pipe& p) {
  for (int s = 0; s < STAGES; ++s)
    for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&p.full_bar[s], 0) && !mbar_try_wait(&p.full_bar[s], 1); ++i) {}
}

// MMA issuer of the MX pipeline: `my_tiles` tiles of `k_blocks` stages each.
template <int STAGES>
__device__ __forceinline__ void mma_role_f8(const F8Pipe& p, uint32_t tmem_base, int my_tiles, int k_blocks, int* error_words) {
  int stage = 0, acc = 0;
  uint32_t phase = 0, acc_phase = 0, sf_set = 0;
  for (int t = 0; t < my_tiles; ++t) {
    if (!mbar_wait(&p.acc_empty[acc], acc_phase ^ 1, p.abort_flag)) {
      gemm_fail(error_words, p.abort_flag, GEMM_TIMEOUT_ACC, 1, acc);
      return;
    }
    tc_fence_after_sync();
    const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * FBN);
    for (int kb = 0; kb < k_blocks; ++kb) {
      if (!mbar_wait(&p.full_bar[stage], phase, p.abort_flag)) {
        gemm_fail(error_words, p.abort_flag, GEMM_TIMEOUT_FULL, 1, stage);
        return;
      }
      tc_fence_after_sync();
      const uint32_t a_addr = smem_u32(p.stage_base + static_cast<size_t>(stage) * kF8StageBytes);
      const uint32_t sf_addr = a_addr + kF8ABytes + kF8BBytes;
      const uint64_t adesc = smem_desc_sw128(a_addr);
      const uint64_t bdesc = smem_desc_sw128(a_addr + kF8ABytes);
      // scales of this K block -> tensor memory (4 columns for A's 128 rows, 4 for B's)
      const uint32_t sfa_t = tmem_base + kSfTmemBase + sf_set * 8;
      const uint32_t sfb_t = sfa_t + 4;
      tmem_cp_scales(sfa_t, smem_desc_scales(sf_addr));
      tmem_cp_scales(sfb_t, smem_desc_scales(sf_addr + kSfBytes));
#pragma unroll
      for (uint32_t k = 0; k < FBK / 32; ++k)
        umma_mxf8(tmem_d, adesc + static_cast<uint64_t>(k * 2), bdesc + static_cast<uint64_t>(k * 2), idesc_mxf8(BM, FBN, k), sfa_t,
                  sfb_t, (kb | static_cast<int>(k)) != 0);
      tc_commit(&p.empty_bar[stage]);
      sf_set ^= 1;
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
    tc_commit(&p.acc_full[acc]);
    if (++acc == 2) { acc = 0; acc_phase ^= 1; }
  }
}

// ============================================================ all-gather -> GEMM (+SwiGLU), MX fp8
template <int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
ag_gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap map_local, const __grid_constant__ CUtensorMap map_gath0,
                     const __grid_constant__ CUtensorMap map_gath1, const __grid_constant__ CUtensorMap map_b, AgGemmF8Args g) {
  extern __shared__ uint8_t smem_raw[];
  const F8Pipe p = carve_f8<kF8Stages>(smem_raw);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  FusedPage* page = g.pages[g.rank];
  if (g.error_words != nullptr && *reinterpret_cast<volatile int*>(g.error_words) != 0) return;   // an earlier launch gave up
  const unsigned long long epoch = page->ag_epoch + 1;
  const int parity = static_cast<int>(epoch & 1ull);
  const int blocks_per_rank = g.rows_per_rank / BM;
  const int k_blocks = g.K / FBK;
  const size_t scale_bytes = static_cast<size_t>(k_blocks) * kSfBytes;       // and its scales
  const size_t all_values = static_cast<size_t>(g.rows_per_rank) * g.nranks * g.K;
  const size_t parity_off = g.gathered_off + static_cast<size_t>(parity) * g.gathered_bytes;

  if (static_cast<int>(blockIdx.x) < g.comm_ctas) {
    // ------------------------------------------------------------------ comm CTAs: push my shard, block by block
    push_f8_blocks(g, page, epoch, parity_off);
  } else {
    // ------------------------------------------------------------------ GEMM CTAs
    init_f8<kF8Stages>(p);
    if (threadIdx.x == 0) {
      prefetch_tensormap(&map_local);
      prefetch_tensormap(&map_b);
    }
    if (warp == 1) tmem_alloc(p.tmem_slot, kF8TmemCols);
    tc_fence_before_sync();
    asm volatile("bar.sync 1, %0;" ::"r"(kGemmThreads) : "memory");
    tc_fence_after_sync();
    const uint32_t tmem_base = *p.tmem_slot;

    const int gemm_ctas = gridDim.x - g.comm_ctas;
    const int cta = blockIdx.x - g.comm_ctas;
    const int tiles_n = g.N / FBN;
    const int num_tiles = blocks_per_rank * g.nranks * tiles_n;
    const int my_tiles = (num_tiles - cta + gemm_ctas - 1) / gemm_ctas;
    const char* gathered = g.heap_bases[g.rank] + parity_off;

    if (warp == 0) {
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = cta; tile < num_tiles && ok; tile += gemm_ctas) {
          const int tn = tile % tiles_n, mb = tile / tiles_n;
          const int src = g.order[2 * mb], b = g.order[2 * mb + 1];
          const bool local = src == g.rank;
          if (!local) {
            if (!wait_flag_ge(&page->ag_flag[src][b], epoch, p.abort_flag)) {
              gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_FLAG, 0, src * 64 + b);
              ok = false;
              break;
            }
            fence_proxy_async();       // peer stores (generic proxy) before my TMA / bulk reads (async proxy)
          }
          const int a_row = local ? b * BM : src * g.rows_per_rank + b * BM;
          const char* sfa_tile = local ? static_cast<const char*>(g.sf_local) + b * scale_bytes
                                       : gathered + all_values + (static_cast<size_t>(src) * blocks_per_rank + b) * scale_bytes;
          const char* sfb_tile = static_cast<const char*>(g.sfb) + static_cast<size_t>(tn) * scale_bytes;
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(&p.empty_bar[stage], phase ^ 1, p.abort_flag)) {
              gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_EMPTY, 0, stage);
              ok = false;
              break;
            }
            uint8_t* a_dst = p.stage_base + static_cast<size_t>(stage) * kF8StageBytes;
            uint8_t* b_dst = a_dst + kF8ABytes;
            uint8_t* sf_dst = b_dst + kF8BBytes;
            mbar_expect_tx(&p.full_bar[stage], kF8StageBytes);
            if (local) tma_load_2d(a_dst, &map_local, &p.full_bar[stage], kb * FBK, a_row);
            else if (parity) tma_load_2d(a_dst, &map_gath1, &p.full_bar[stage], kb * FBK, a_row);
            else tma_load_2d(a_dst, &map_gath0, &p.full_bar[stage], kb * FBK, a_row);
            tma_load_2d(b_dst, &map_b, &p.full_bar[stage], kb * FBK, tn * FBN);
            bulk_load(sf_dst, sfa_tile + static_cast<size_t>(kb) * kSfBytes, kSfBytes, &p.full_bar[stage]);
            bulk_load(sf_dst + kSfBytes, sfb_tile + static_cast<size_t>(kb) * kSfBytes, kSfBytes, &p.full_bar[stage]);
            if (++stage == kF8Stages) { stage = 0; phase ^= 1; }
          }
        }
        if (!ok) drain_f8<kF8Stages>(p);
      }
    } else if (warp == 1) {
      if (lane == 0) mma_role_f8<kF8Stages>(p, tmem_base, my_tiles, k_blocks, g.error_words);
    } else {
      const int quarter = warp % 4;
      int acc = 0;
      uint32_t acc_phase = 0;
      __nv_bfloat16* d = static_cast<__nv_bfloat16*>(g.d);
      for (int tile = cta; tile < num_tiles; tile += gemm_ctas) {
        const int tn = tile % tiles_n, mb = tile / tiles_n;
        const int src = g.order[2 * mb], b = g.order[2 * mb + 1];
        bool ok = mbar_wait(&p.acc_full[acc], acc_phase, p.abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_ACC, 2, acc);
          break;
        }
        tc_fence_after_sync();
        const size_t row = static_cast<size_t>(src) * g.rows_per_rank + b * BM + quarter * 32 + lane;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * FBN);
        if (EPI == 0) {
#pragma unroll 1
          for (int c = 0; c < FBN; c += 32) {
            uint32_t r[32];
            tmem_ld32(taddr + c, r);
            tc_wait_ld();
            uint4* out = reinterpret_cast<uint4*>(d + row * g.ldd + tn * FBN + c);
#pragma unroll
            for (int v = 0; v < 4; ++v)
              out[v] = make_uint4(pack_bf16(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1])),
                                  pack_bf16(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3])),
                                  pack_bf16(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5])),
                                  pack_bf16(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7])));
          }
        } else {
          constexpr int H = FBN / 2;       // the tile holds 64 gate columns followed by the 64 up columns of the same features
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
        if (lane == 0) mbar_arrive(&p.acc_empty[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    tc_fence_before_sync();
    asm volatile("bar.sync 1, %0;" ::"r"(kGemmThreads) : "memory");
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc(tmem_base, kF8TmemCols);
    }
  }
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

// ============================================================ GEMM -> reduce-scatter, MX fp8 operands
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_rs_mxfp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmRsF8Args g) {
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  FusedPage* page = g.pages[g.rank];
  if (g.error_words != nullptr && *reinterpret_cast<volatile int*>(g.error_words) != 0) return;   // an earlier launch gave up
  const unsigned long long epoch = page->rs_epoch + 1;
  const int parity = static_cast<int>(epoch & 1ull);
  const int blocks_per_rank = g.rows_per_rank / BM;
  const int tiles_n = g.N / FBN;
  const int num_tiles = blocks_per_rank * g.nranks * tiles_n;
  const int k_blocks = g.K / FBK;
  const int ctas = static_cast<int>(gridDim.x) - g.reduce_ctas;       // CTAs that run the GEMM
  const int cta = blockIdx.x;
  const size_t slab_bytes = static_cast<size_t>(g.rows_per_rank) * g.N * 2;
  const size_t parity_off = g.partial_off + static_cast<size_t>(parity) * g.nranks * slab_bytes;
  const unsigned long long per_block = 4ull * static_cast<unsigned long long>(tiles_n);   // counts per (source, row block) and launch

  if (cta >= ctas) {
    reduce_items(g, page, g.heap_bases[g.rank] + parity_off, slab_bytes, blocks_per_rank, per_block);
  } else {
    const F8Pipe p = carve_f8<kRsF8Stages>(smem_raw);
    const int my_tiles = (num_tiles - cta + ctas - 1) / ctas;
    const size_t scale_bytes = static_cast<size_t>(k_blocks) * kSfBytes;
    init_f8<kRsF8Stages>(p);
    if (threadIdx.x == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
    }
    if (warp == 1) tmem_alloc(p.tmem_slot, kF8TmemCols);
    tc_fence_before_sync();
    asm volatile("bar.sync 1, %0;" ::"r"(kGemmThreads) : "memory");
    tc_fence_after_sync();
    const uint32_t tmem_base = *p.tmem_slot;

    if (warp == 0) {
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = cta; tile < num_tiles && ok; tile += ctas) {
          const int tn = tile % tiles_n, rb = tile / tiles_n;
          const int owner = g.order[2 * rb], b = g.order[2 * rb + 1];
          const int row_block = owner * blocks_per_rank + b;
          const char* sfa_tile = static_cast<const char*>(g.sfa) + static_cast<size_t>(row_block) * scale_bytes;
          const char* sfb_tile = static_cast<const char*>(g.sfb) + static_cast<size_t>(tn) * scale_bytes;
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(&p.empty_bar[stage], phase ^ 1, p.abort_flag)) {
              gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_EMPTY, 0, stage);
              ok = false;
              break;
            }
            uint8_t* a_dst = p.stage_base + static_cast<size_t>(stage) * kF8StageBytes;
            uint8_t* b_dst = a_dst + kF8ABytes;
            uint8_t* sf_dst = b_dst + kF8BBytes;
            mbar_expect_tx(&p.full_bar[stage], kF8StageBytes);
            tma_load_2d(a_dst, &map_a, &p.full_bar[stage], kb * FBK, row_block * BM);
            tma_load_2d(b_dst, &map_b, &p.full_bar[stage], kb * FBK, tn * FBN);
            bulk_load(sf_dst, sfa_tile + static_cast<size_t>(kb) * kSfBytes, kSfBytes, &p.full_bar[stage]);
            bulk_load(sf_dst + kSfBytes, sfb_tile + static_cast<size_t>(kb) * kSfBytes, kSfBytes, &p.full_bar[stage]);
            if (++stage == kRsF8Stages) { stage = 0; phase ^= 1; }
          }
        }
        if (!ok) drain_f8<kRsF8Stages>(p);
      }
    } else if (warp == 1) {
      if (lane == 0) mma_role_f8<kRsF8Stages>(p, tmem_base, my_tiles, k_blocks, g.error_words);
    } else {
      const int quarter = warp % 4;
      int acc = 0;
      uint32_t acc_phase = 0;
      int pend_owner = -1, pend_b = 0;                      // the tile whose stores were issued last
      for (int tile = cta; tile < num_tiles; tile += ctas) {
        const int tn = tile % tiles_n, rb = tile / tiles_n;
        const int owner = g.order[2 * rb], b = g.order[2 * rb + 1];
        bool ok = mbar_wait(&p.acc_full[acc], acc_phase, p.abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_ACC, 2, acc);
          break;
        }
        tc_fence_after_sync();
        char* slab = g.heap_bases[owner] + parity_off + static_cast<size_t>(g.rank) * slab_bytes;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * FBN);
        uint8_t* stage_warp = p.staging + (warp - 2) * kF8StagingPerWarp;
        // this lane's row of the quarter -> shared memory as bf16
#pragma unroll 1
        for (int c = 0; c < FBN; c += 32) {
          uint32_t r[32];
          tmem_ld32(taddr + c, r);
          tc_wait_ld();
          uint4* dst = reinterpret_cast<uint4*>(stage_warp + lane * kF8StagePitch + c * 2);
#pragma unroll
          for (int v = 0; v < 4; ++v)
            dst[v] = make_uint4(pack_bf16(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1])),
                                pack_bf16(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3])),
                                pack_bf16(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5])),
                                pack_bf16(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7])));
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p.acc_empty[acc]);      // the accumulator is free as soon as it sits in shared memory
        // count the previous tile on its owner: its stores were issued a whole tile ago, so the release has nothing
        // left to wait for (a release right behind the stores, let alone a system-scope fence, cost 8-30 us a tile)
        if (pend_owner >= 0 && lane == 0) red_add_release_sys(&g.pages[pend_owner]->rs_count[g.rank][pend_b], 1ull);
        // two rows (256 contiguous bytes each) per store instruction, 16 rows in flight
        const int half = lane / 16, piece = lane % 16;
        char* dst0 = slab + ((static_cast<size_t>(b) * BM + quarter * 32 + half) * g.N + static_cast<size_t>(tn) * FBN) * 2 + piece * 16;
#pragma unroll 1
        for (int r0 = 0; r0 < 32; r0 += 16) {
          uint4 d[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            d[u] = *reinterpret_cast<const uint4*>(stage_warp + (r0 + 2 * u + half) * kF8StagePitch + piece * 16);
#pragma unroll
          for (int u = 0; u < 8; ++u) *reinterpret_cast<uint4*>(dst0 + static_cast<size_t>(r0 + 2 * u) * g.N * 2) = d[u];
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
    asm volatile("bar.sync 1, %0;" ::"r"(kGemmThreads) : "memory");
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc(tmem_base, kF8TmemCols);
    }
    // the tiles of this CTA are out: help with the reduction
    reduce_items(g, page, g.heap_bases[g.rank] + parity_off, slab_bytes, blocks_per_rank, per_block);
  }
  finish_rs_launch(g, page, blocks_per_rank, per_block, epoch);
}

}  // namespace

cudaError_t launch_ag_gemm_mxfp8(const AgGemmF8Args& g, int epilogue, int grid, cudaStream_t stream) {
  if (g.K % FBK != 0 || g.N % FBN != 0 || g.rows_per_rank % BM != 0 || g.rows_per_rank / BM > kFusedMaxBlocks ||
      g.nranks > kFusedMaxRanks || g.comm_ctas < 1 || grid <= g.comm_ctas || g.order == nullptr)
    return cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(g.sf_local) % 16 != 0 || reinterpret_cast<uintptr_t>(g.sfb) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(g.x_local) % 16 != 0 || g.gathered_off % 1024 != 0 || g.gathered_bytes % 1024 != 0)
    return cudaErrorInvalidValue;
  const uint64_t all_rows = static_cast<uint64_t>(g.rows_per_rank) * g.nranks;
  CUtensorMap map_local = make_u8_kmajor_map(g.x_local, g.rows_per_rank, g.K, g.K, BM);
  const char* gath = g.heap_bases_host[g.rank] + g.gathered_off;
  CUtensorMap map_g0 = make_u8_kmajor_map(gath, all_rows, g.K, g.K, BM);
  CUtensorMap map_g1 = make_u8_kmajor_map(gath + g.gathered_bytes, all_rows, g.K, g.K, BM);
  CUtensorMap map_b = make_u8_kmajor_map(g.b, g.N, g.K, g.ldb, FBN);
  auto launch = [&](auto kernel) {
    static bool configured[2] = {false, false};          // the attribute is sticky: set it once per kernel
    cudaError_t e = cudaSuccess;
    if (!configured[epilogue != 0]) {
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kF8SmemBytes));
      configured[epilogue != 0] = e == cudaSuccess;
    }
    if (e != cudaSuccess) return e;
    kernel<<<grid, kGemmThreads, kF8SmemBytes, stream>>>(map_local, map_g0, map_g1, map_b, g);
    return cudaGetLastError();
  };
  return epilogue == 0 ? launch(ag_gemm_mxfp8_kernel<0>) : launch(ag_gemm_mxfp8_kernel<1>);
}

cudaError_t launch_gemm_rs_mxfp8(const GemmRsF8Args& g, int grid, cudaStream_t stream) {
  if (g.K % FBK != 0 || g.N % FBN != 0 || g.rows_per_rank % BM != 0 || g.rows_per_rank / BM > kFusedMaxBlocks ||
      g.nranks > kFusedMaxRanks || g.reduce_ctas < 1 || grid <= g.reduce_ctas || g.order == nullptr ||
      g.reduce_order == nullptr)
    return cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(g.sfa) % 16 != 0 || reinterpret_cast<uintptr_t>(g.sfb) % 16 != 0) return cudaErrorInvalidValue;
  CUtensorMap map_a = make_u8_kmajor_map(g.a, static_cast<uint64_t>(g.rows_per_rank) * g.nranks, g.K, g.lda, BM);
  CUtensorMap map_b = make_u8_kmajor_map(g.b, g.N, g.K, g.ldb, FBN);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_rs_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kRsF8SmemBytes));
    if (e != cudaSuccess) return e;
    configured = true;
  }
  gemm_rs_mxfp8_kernel<<<grid, kGemmThreads, kRsF8SmemBytes, stream>>>(map_a, map_b, g);
  return cudaGetLastError();
}

}  // namespace sm100
}  // namespace msccl
