// Two-CTA persistent tcgen05 GEMM for sm_100a: D[M,N] = A[M,K] * B[N,K]^T, bf16 in, fp32 accumulate
// in tensor memory, bf16 out, optional SwiGLU epilogue (same contract as gemm_sm100.cu).
//
// A cluster of two CTAs owns one 256 x 256 output tile per step:
//   CTA r of the pair loads rows [128 r, 128 r + 128) of the tile's A block and rows
//   [128 r, 128 r + 128) of its B block into its own shared memory (32 KB per stage instead of the
//   48 KB a single CTA needs for 128 x 256, so six stages fit), the leader's MMA thread issues
//   tcgen05.mma.cta_group::2 (M 256, N 256, K 16) which reads both CTAs' shared memory, and each CTA
//   ends up with the 128 x 256 accumulator of its own rows in its own tensor memory.
// Per output element the pair reads half as much of B from shared memory as two independent
// 128 x 256 CTAs would; that traffic is what limits the single-CTA kernel.
//
// Synchronisation (all mbarriers sit at the same shared-memory offsets in both CTAs):
//   full[s]      leader only.  Both producers' loads complete on it; the leader's producer posts the
//                expected byte count of the pair.
//   empty[s]     one per CTA; the leader's tcgen05.commit arrives on both when the MMAs that read
//                stage s are done.
//   acc_full[a]  one per CTA; arrives (commit) when a tile's accumulator is complete.
//   acc_empty[a] leader only; the eight epilogue warps of the pair arrive on it.
// Every wait is bounded (gemm_sm100.cuh); a CTA that gives up raises the error word, and its
// partner runs into its own limit.  Both CTAs meet at a cluster barrier before tensor memory is
// freed, so no arrival can target a CTA that has already exited.
#include <cuda.h>
#include <cuda_runtime.h>

#include "gemm_sm100.cuh"
#include "gemm_sm100.h"
#include "umma_2cta.cuh"

namespace msccl {
namespace sm100 {

namespace {

constexpr int PBM = 256;                      // tile rows of the pair
constexpr int PBN = 256;                      // tile columns of the pair
constexpr int kPStages = 6;
constexpr int kPGroupM = 8;                   // 8 pair rows = 2048 rows of A per L2-resident group
constexpr int kPABytes = BM * BK * 2;         // this CTA's 128 rows of A: 16 KB
constexpr int kPBBytes = (PBN / 2) * BK * 2;  // this CTA's 128 rows of B: 16 KB
constexpr int kPStageBytes = kPABytes + kPBBytes;
constexpr int kPTmemCols = 2 * PBN;           // two accumulator stages
constexpr size_t kPSmemBytes = 1024 + static_cast<size_t>(kPStages) * kPStageBytes + 256;

// Tensor load of one CTA of a pair: data lands in this CTA's shared memory, the bytes are counted on
// the mbarrier at `bar_cluster_addr`, which may belong to the partner.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}

template <int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      __nv_bfloat16* __restrict__ d, int M, int N, int K, int ldd, int* error_words) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* stage_base = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(kPStages) * kPStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kPStages;
  uint64_t* acc_full = bars + 2 * kPStages;
  uint64_t* acc_empty = bars + 2 * kPStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kPStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // An earlier launch gave up: skip the work.  The leader's reading decides for the pair, so that
  // both CTAs take the same path even if the word changes between their two loads.
  __shared__ int s_skip;
  if (threadIdx.x == 0) s_skip = (error_words != nullptr && *reinterpret_cast<volatile int*>(error_words) != 0) ? 1 : 0;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int tiles_m = (M + PBM - 1) / PBM, tiles_n = N / PBN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = K / BK;
  const int first_tile = static_cast<int>(cluster_id_x()), tile_step = static_cast<int>(num_clusters_x());

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 8);                   // four epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, kPTmemCols);
  tc_fence_before_sync();
  cluster_sync_all();                                // barriers of both CTAs are initialised, tensor memory is allocated
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool skip = ld_shared_cluster_u32(map_to_cta(smem_u32(&s_skip), 0)) != 0;

  if (skip) {
    // nothing to do; fall through to the common exit
  } else if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, kPGroupM, tm, tn);
        const int a_row = tm * PBM + static_cast<int>(cta_rank) * BM;
        const int b_row = tn * PBN + static_cast<int>(cta_rank) * (PBN / 2);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_EMPTY, 0, stage);
            ok = false;
            break;
          }
          uint8_t* a_dst = stage_base + static_cast<size_t>(stage) * kPStageBytes;
          uint8_t* b_dst = a_dst + kPABytes;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * kPStageBytes);
          const uint32_t leader_full = map_to_cta(smem_u32(&full_bar[stage]), 0);
          tma_load_2d_pair(a_dst, &map_a, leader_full, kb * BK, a_row);
          tma_load_2d_pair(b_dst, &map_b, leader_full, kb * BK, b_row);
          if (++stage == kPStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Let the loads that were issued land before shared memory is released.  The leader can watch
        // the barriers they complete on; the partner cannot, and allows them 200 us (a load takes a
        // few microseconds, and a producer only fails after its own wait of seconds or on abort).
        if (leader) {
          for (int s = 0; s < kPStages; ++s)
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
      constexpr uint32_t idesc = idesc_bf16_f32(PBM, PBN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) {
          gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_ACC, 1, acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * PBN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_FULL, 1, stage);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(stage_base + static_cast<size_t>(stage) * kPStageBytes);
          const uint64_t adesc = smem_desc_sw128(a_addr);
          const uint64_t bdesc = smem_desc_sw128(a_addr + kPABytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16_pair(tmem_d, adesc + static_cast<uint64_t>(k * 2), bdesc + static_cast<uint64_t>(k * 2), idesc, (kb | k) != 0);
          tc_commit_pair(&empty_bar[stage], 3);      // stage free in both CTAs
          if (++stage == kPStages) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit_pair(&acc_full[acc], 3);   // accumulator complete in both CTAs
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5, both CTAs)
    const int quarter = warp % 4;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = first_tile; tile < num_tiles; tile += tile_step) {
      int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, kPGroupM, tm, tn);
      bool ok = mbar_wait(&acc_full[acc], acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_ACC, 2, acc);
        break;
      }
      tc_fence_after_sync();
      const int row = tm * PBM + static_cast<int>(cta_rank) * BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * PBN);
      if (EPI == 0) {
#pragma unroll 1
        for (int c = 0; c < PBN; c += 32) {
          uint32_t r[32];
          tmem_ld32(taddr + c, r);
          tc_wait_ld();
          if (row < M) {
            uint4* out = reinterpret_cast<uint4*>(d + static_cast<size_t>(row) * ldd + tn * PBN + c);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              out[v] = make_uint4(pack_bf16(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1])),
                                  pack_bf16(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3])),
                                  pack_bf16(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5])),
                                  pack_bf16(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7])));
            }
          }
        }
      } else {
        constexpr int H = PBN / 2;
#pragma unroll 1
        for (int c = 0; c < H; c += 32) {
          uint32_t g[32], u[32];
          tmem_ld32(taddr + c, g);
          tmem_ld32(taddr + H + c, u);
          tc_wait_ld();
          if (row < M) {
            uint4* out = reinterpret_cast<uint4*>(d + static_cast<size_t>(row) * ldd + tn * H + c);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float o[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float gv = __uint_as_float(g[8 * v + e]);
                o[e] = gv / (1.0f + __expf(-gv)) * __uint_as_float(u[8 * v + e]);
              }
              out[v] = make_uint4(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]), pack_bf16(o[4], o[5]), pack_bf16(o[6], o[7]));
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));   // the leader's barrier
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

}  // namespace

// How many CTA pairs can be resident at once (pairs need two SMs of the same cluster-capable group).
int max_cta_pairs(int epilogue) {
  static int cached[64][2] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const int e = epilogue ? 1 : 0;
  if (dev >= 0 && dev < 64 && cached[dev][e] > 0) return cached[dev][e];
  auto kernel = epilogue ? gemm_bf16_2cta_kernel<1> : gemm_bf16_2cta_kernel<0>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kPSmemBytes)) != cudaSuccess) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * sm_count(), 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = kPSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (dev >= 0 && dev < 64) cached[dev][e] = clusters;
  return clusters;
}

// Same contract as gemm_bf16 with bn = 256; N % 256 == 0, K % 64 == 0.
cudaError_t gemm_bf16_2cta(const void* a, const void* b, void* d, int M, int N, int K, int lda, int ldb, int ldd, int epilogue,
                           int* error_words, int max_pairs, cudaStream_t stream) {
  if (K % BK != 0 || N % PBN != 0 || M <= 0) return cudaErrorInvalidValue;
  int pairs = max_cta_pairs(epilogue);
  if (pairs <= 0) return cudaErrorLaunchOutOfResources;
  if (max_pairs > 0 && max_pairs < pairs) pairs = max_pairs;
  const int tiles = ((M + PBM - 1) / PBM) * (N / PBN);
  if (tiles < pairs) pairs = tiles;
  CUtensorMap map_a = make_bf16_kmajor_map(a, M, K, lda, BM);
  CUtensorMap map_b = make_bf16_kmajor_map(b, N, K, ldb, PBN / 2);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = kPSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  auto* out = static_cast<__nv_bfloat16*>(d);
  if (epilogue == 0) return cudaLaunchKernelEx(&cfg, gemm_bf16_2cta_kernel<0>, map_a, map_b, out, M, N, K, ldd, error_words);
  return cudaLaunchKernelEx(&cfg, gemm_bf16_2cta_kernel<1>, map_a, map_b, out, M, N, K, ldd, error_words);
}

}  // namespace sm100
}  // namespace msccl
