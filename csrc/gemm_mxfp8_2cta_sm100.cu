// Block-scaled fp8 GEMM on CTA pairs (tcgen05 cta_group::2): the large-tile version of
// gemm_mxfp8_sm100.cu.  Same data contract: A [M,K] and B [N,K] e4m3 K-major, one UE8M0 scale per
// 32 K elements of a row, scales pre-arranged in 512-byte blocks per (128 rows, 128 K), bf16 result.
//
// Why a second kernel: fp8 halves the time of every MMA but not the bytes it needs.  A 128 x 128 tile
// asks its SM for 129 bytes of operands per clock from L2, about twice what an SM can take in, and the
// tensor pipe idles (measured 37 % active).  A pair that shares a 256 x 256 tile needs 67 bytes per
// clock and SM:
//   CTA r of the pair stages rows [128 r, 128 r + 128) of A and of B, the scales of its own A rows
//   (512 bytes) and the scales of all 256 B rows (1 KB; each CTA multiplies its 128 rows with all of B)
//   per 128-byte K block, all as tensor loads that complete on the leader's mbarrier; the leader issues tcgen05.cp.cta_group::2 (scales to tensor memory in both
//   CTAs) and tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale (M 256, N 256, K 32).
// Tensor memory: one 256-column accumulator plus 12 scale columns per pipeline stage.  Two accumulator
// stages of 256 columns would fill all 512 columns, so the epilogue of a tile cannot run beside the
// next tile's MMAs as a whole; what is kept off the critical path is its second half: the epilogue warps
// pack the accumulator to bf16 in shared memory, release it, and only then store to global memory.
// Barriers and failure handling as in gemm_2cta_sm100.cu.
#include <cuda.h>
#include <cuda_runtime.h>

#include "gemm_sm100.cuh"
#include "gemm_sm100.h"
#include "mxfp8_pair.cuh"
#include "umma_2cta.cuh"

namespace msccl {
namespace sm100 {

namespace {

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_mxfp8_2cta_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                       __nv_bfloat16* __restrict__ d, int M, int N, int K, int ldd, int* error_words) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* stage_base = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(kQStages) * kQStageBytes);
  uint64_t* full_bar = bars;                         // leader only: loads of both CTAs complete here
  uint64_t* empty_bar = bars + kQStages;             // per CTA: commit from the leader
  uint64_t* acc_full = bars + 2 * kQStages;          // per CTA: commit from the leader
  uint64_t* acc_empty = bars + 2 * kQStages + 1;     // leader only: 8 epilogue warps of the pair
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kQStages + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* epi_base = smem + static_cast<size_t>(kQStages) * kQStageBytes + 256;

  __shared__ int s_skip;                             // the leader's reading decides for the pair
  if (threadIdx.x == 0) s_skip = (error_words != nullptr && *reinterpret_cast<volatile int*>(error_words) != 0) ? 1 : 0;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int tiles_m = (M + QBM - 1) / QBM, tiles_n = N / QBN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = K / QBK;
  const int first_tile = static_cast<int>(cluster_id_x()), tile_step = static_cast<int>(num_clusters_x());

  if (threadIdx.x == 0) {
    for (int s = 0; s < kQStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 8);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    prefetch_tensormap(&map_sfa);
    prefetch_tensormap(&map_sfb);
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, kQTmemCols);
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool skip = ld_shared_cluster_u32(map_to_cta(smem_u32(&s_skip), 0)) != 0;

  if (skip) {
    // an earlier launch gave up: nothing to do
  } else if (warp == 0) {
    // ---------------------------------------------------------------- producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const int sfa_tiles_per_pair = 2;              // 128-row scale blocks per 256-row tile
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, kQGroupM, tm, tn);
        const int a_row = tm * QBM + static_cast<int>(cta_rank) * BM;
        const int b_row = tn * QBN + static_cast<int>(cta_rank) * (QBN / 2);
        // scale blocks are indexed [128-row block][K block]
        const int sfa_block = (tm * sfa_tiles_per_pair + static_cast<int>(cta_rank)) * k_blocks;
        const int sfb_block0 = tn * 2 * k_blocks, sfb_block1 = sfb_block0 + k_blocks;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_EMPTY, 0, stage);
            ok = false;
            break;
          }
          uint8_t* a_dst = stage_base + static_cast<size_t>(stage) * kQStageBytes;
          uint8_t* b_dst = a_dst + kQABytes;
          uint8_t* sf_dst = b_dst + kQBBytes;          // [SFA own rows | SFB rows 0-127 | SFB rows 128-255]
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * kQLoadBytes);
          const uint32_t leader_full = map_to_cta(smem_u32(&full_bar[stage]), 0);
          tma_load_2d_pair8(a_dst, &map_a, leader_full, kb * QBK, a_row);
          tma_load_2d_pair8(b_dst, &map_b, leader_full, kb * QBK, b_row);
          tma_load_2d_pair8(sf_dst, &map_sfa, leader_full, 0, sfa_block + kb);
          tma_load_2d_pair8(sf_dst + kQSfBytes, &map_sfb, leader_full, 0, sfb_block0 + kb);
          tma_load_2d_pair8(sf_dst + 2 * kQSfBytes, &map_sfb, leader_full, 0, sfb_block1 + kb);
          if (++stage == kQStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // let issued loads land before shared memory is released (see gemm_2cta_sm100.cu)
        if (leader) {
          for (int s = 0; s < kQStages; ++s)
            for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&full_bar[s], 0) && !mbar_try_wait(&full_bar[s], 1); ++i) {}
        } else {
          unsigned long long t0, t1;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
          do { asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1)); } while (t1 - t0 < 200000ull);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader only)
    if (lane == 0 && leader) {
      int stage = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
        if (!mbar_wait(acc_empty, acc_phase ^ 1, abort_flag)) {
          gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_ACC, 1, 0);
          break;
        }
        tc_fence_after_sync();
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_FULL, 1, stage);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(stage_base + static_cast<size_t>(stage) * kQStageBytes);
          const uint32_t sf_addr = a_addr + kQABytes + kQBBytes;
          const uint64_t adesc = smem_desc_sw128(a_addr);
          const uint64_t bdesc = smem_desc_sw128(a_addr + kQABytes);
          // this stage's scale columns: 4 for A's 128 rows per CTA, 8 for B's 256 rows
          const uint32_t sfa_t = tmem_base + kQSfTmemBase + static_cast<uint32_t>(stage) * 12;
          const uint32_t sfb_t = sfa_t + 4;
          tmem_cp_scales_pair(sfa_t, smem_desc_scales_pair(sf_addr));
          tmem_cp_scales_pair(sfb_t, smem_desc_scales_pair(sf_addr + kQSfBytes));
          tmem_cp_scales_pair(sfb_t + 4, smem_desc_scales_pair(sf_addr + 2 * kQSfBytes));
#pragma unroll
          for (uint32_t k = 0; k < QBK / 32; ++k)
            umma_mxf8_pair(tmem_base, adesc + static_cast<uint64_t>(k * 2), bdesc + static_cast<uint64_t>(k * 2), idesc_mxf8_pair(k),
                           sfa_t, sfb_t, (kb | static_cast<int>(k)) != 0);
          tc_commit_pair(&empty_bar[stage], 3);
          if (++stage == kQStages) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit_pair(acc_full, 3);
        acc_phase ^= 1;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5, both CTAs)
    const int quarter = warp % 4;
    uint32_t acc_phase = 0;
    for (int tile = first_tile; tile < num_tiles; tile += tile_step) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, kQGroupM, tm, tn);
      bool ok = mbar_wait(acc_full, acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_ACC, 2, 0);
        break;
      }
      tc_fence_after_sync();
      const int row0 = tm * QBM + static_cast<int>(cta_rank) * BM + quarter * 32;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      uint8_t* epi = epi_base + (warp - 2) * kQEpiPerWarp;
      constexpr int kLanesPerRow = kQStageCols * 2 / 16, kRowsPerStore = 32 / kLanesPerRow;
#pragma unroll 1
      for (int c0 = 0; c0 < QBN; c0 += kQStageCols) {
        // tensor memory -> registers -> shared memory; the load of the next 32 columns is in flight while these are packed
        uint32_t r[2][32];
        tmem_ld32(taddr + c0, r[0]);
#pragma unroll
        for (int c = 0; c < kQStageCols; c += 32) {
          const int cur = (c / 32) & 1;
          tc_wait_ld();
          if (c + 32 < kQStageCols) tmem_ld32(taddr + c0 + c + 32, r[cur ^ 1]);
          uint4* dst = reinterpret_cast<uint4*>(epi + lane * kQEpiPitch + c * 2);
#pragma unroll
          for (int v = 0; v < 4; ++v)
            dst[v] = make_uint4(pack_bf16(__uint_as_float(r[cur][8 * v + 0]), __uint_as_float(r[cur][8 * v + 1])),
                                pack_bf16(__uint_as_float(r[cur][8 * v + 2]), __uint_as_float(r[cur][8 * v + 3])),
                                pack_bf16(__uint_as_float(r[cur][8 * v + 4]), __uint_as_float(r[cur][8 * v + 5])),
                                pack_bf16(__uint_as_float(r[cur][8 * v + 6]), __uint_as_float(r[cur][8 * v + 7])));
        }
        if (c0 + kQStageCols == QBN) {
          // the accumulator has been read completely: the MMAs of the next tile may overwrite it
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(acc_empty), 0));
        } else {
          __syncwarp();
        }
        // shared memory -> global: kRowsPerStore rows of kQStageCols bf16 per instruction, eight instructions in flight
        const int sub_row = lane / kLanesPerRow, sub_col = (lane % kLanesPerRow) * 16;
        __nv_bfloat16* out0 = d + static_cast<size_t>(row0) * ldd + tn * QBN + c0;
#pragma unroll 1
        for (int r0 = 0; r0 < 32; r0 += 8 * kRowsPerStore) {
          uint4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            v[u] = *reinterpret_cast<const uint4*>(epi + (r0 + u * kRowsPerStore + sub_row) * kQEpiPitch + sub_col);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int rr = r0 + u * kRowsPerStore + sub_row;
            if (row0 + rr < M)
              *reinterpret_cast<uint4*>(reinterpret_cast<char*>(out0 + static_cast<size_t>(rr) * ldd) + sub_col) = v[u];
          }
        }
        __syncwarp();                                  // the staging rows are read: the next pass may overwrite them
      }
      acc_phase ^= 1;
    }
  }

  tc_fence_before_sync();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kQTmemCols);
  }
}

int max_pairs_mxfp8() {
  static int cached[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
  if (cudaFuncSetAttribute(gemm_mxfp8_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kQSmemBytes)) !=
      cudaSuccess)
    return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * sm_count(), 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = kQSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, gemm_mxfp8_2cta_kernel, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (dev >= 0 && dev < 64) cached[dev] = clusters;
  return clusters;
}

}  // namespace

// Same contract as gemm_mxfp8; N % 256 == 0, K % 128 == 0.  The packed A scales must cover a multiple
// of 256 rows (pack_mx_scales pads to 128; the caller passes ceil(M / 256) * 2 row blocks).
cudaError_t gemm_mxfp8_2cta(const void* a, const void* sfa, const void* b, const void* sfb, void* d, int M, int N, int K, int lda,
                            int ldb, int ldd, int* error_words, int max_pairs, cudaStream_t stream) {
  if (K % QBK != 0 || N % QBN != 0 || M <= 0) return cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(sfa) % 16 != 0 || reinterpret_cast<uintptr_t>(sfb) % 16 != 0) return cudaErrorInvalidValue;
  int pairs = max_pairs_mxfp8();
  if (pairs <= 0) return cudaErrorLaunchOutOfResources;
  if (max_pairs > 0 && max_pairs < pairs) pairs = max_pairs;
  const int tiles = ((M + QBM - 1) / QBM) * (N / QBN);
  if (tiles < pairs) pairs = tiles;
  CUtensorMap map_a = make_u8_kmajor_map(a, M, K, lda, BM);
  CUtensorMap map_b = make_u8_kmajor_map(b, N, K, ldb, QBN / 2);
  CUtensorMap map_sfa = make_block512_map(sfa, static_cast<uint64_t>((M + QBM - 1) / QBM) * 2 * (K / QBK));
  CUtensorMap map_sfb = make_block512_map(sfb, static_cast<uint64_t>(N / 128) * (K / QBK));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = kQSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gemm_mxfp8_2cta_kernel, map_a, map_b, map_sfa, map_sfb, static_cast<__nv_bfloat16*>(d), M, N, K,
                            ldd, error_words);
}

}  // namespace sm100
}  // namespace msccl
