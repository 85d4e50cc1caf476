// Block-scaled fp8 GEMM for sm_100a: D[M,N] = (A * 2^(sfa-127))[M,K] * (B * 2^(sfb-127))[N,K]^T.
// A and B are e4m3, K-major; one UE8M0 scale byte covers 32 consecutive K elements of one row
// (the OCP "MX" format).  The scaling is done by the tensor core itself:
// tcgen05.mma.kind::mxf8f6f4.block_scale reads the scale bytes from tensor memory, where
// tcgen05.cp puts them from shared memory.  fp32 accumulation in tensor memory, bf16 result.
//
// Same warp roles as the bf16 kernel (gemm_sm100.cuh): TMA producer, MMA issuer, 4 epilogue warps,
// persistent CTAs.  Differences:
//   * a pipeline stage holds 128 bytes of K (128 elements, four K=32 MMAs) of A (128 rows) and
//     B (128 rows) plus their 2 x 512 bytes of scales, fetched with two untiled bulk copies;
//   * tile 128 x 128: two accumulator stages take 256 of the 512 TMEM columns, the scale buffers
//     (two sets, alternating per K block) sit behind them;
//   * scales arrive pre-arranged in global memory as one 512-byte block per (128 rows, 128 K):
//     byte (r % 32) * 16 + (r / 32) * 4 + j holds the scale of row r for K elements [32 j, 32 j + 32).
//     That is the order tcgen05.cp.32x128b.warpx4 needs: lane r % 32 of every TMEM lane quarter
//     receives the 16 bytes of rows r % 32 + {0, 32, 64, 96}, one 32-bit column per row, and the
//     instruction descriptor's scale id picks byte j of the column.
// Every wait is bounded as in the bf16 kernel.
#include <cuda.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "gemm_sm100.cuh"
#include "gemm_sm100.h"
#include "mxfp8_sm100.cuh"

namespace msccl {
namespace sm100 {

namespace {

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb, __nv_bfloat16* __restrict__ d, int M, int N,
                  int K, int ldd, int* error_words) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* stage_base = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(kF8Stages) * kF8StageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kF8Stages;
  uint64_t* acc_full = bars + 2 * kF8Stages;
  uint64_t* acc_empty = bars + 2 * kF8Stages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kF8Stages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (error_words != nullptr && *reinterpret_cast<volatile int*>(error_words) != 0) return;   // an earlier launch gave up
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = N / FBN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = K / FBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kF8Stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 1) tmem_alloc(tmem_slot, kF8TmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, kF8GroupM, tm, tn);
        const uint8_t* sfa_tile = sfa + static_cast<size_t>(tm) * k_blocks * kSfBytes;
        const uint8_t* sfb_tile = sfb + static_cast<size_t>(tn) * k_blocks * kSfBytes;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_EMPTY, 0, stage);
            ok = false;
            break;
          }
          uint8_t* a_dst = stage_base + static_cast<size_t>(stage) * kF8StageBytes;
          uint8_t* b_dst = a_dst + kF8ABytes;
          uint8_t* sfa_dst = b_dst + kF8BBytes;
          mbar_expect_tx(&full_bar[stage], kF8StageBytes);
          tma_load_2d(a_dst, &map_a, &full_bar[stage], kb * FBK, tm * BM);
          tma_load_2d(b_dst, &map_b, &full_bar[stage], kb * FBK, tn * FBN);
          bulk_load(sfa_dst, sfa_tile + static_cast<size_t>(kb) * kSfBytes, kSfBytes, &full_bar[stage]);
          bulk_load(sfa_dst + kSfBytes, sfb_tile + static_cast<size_t>(kb) * kSfBytes, kSfBytes, &full_bar[stage]);
          if (++stage == kF8Stages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        for (int s = 0; s < kF8Stages; ++s)
          for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&full_bar[s], 0) && !mbar_try_wait(&full_bar[s], 1); ++i) {}
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      uint32_t sf_set = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) {
          gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_ACC, 1, acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * FBN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_FULL, 1, stage);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(stage_base + static_cast<size_t>(stage) * kF8StageBytes);
          const uint32_t sf_addr = a_addr + kF8ABytes + kF8BBytes;
          const uint64_t adesc = smem_desc_sw128(a_addr);
          const uint64_t bdesc = smem_desc_sw128(a_addr + kF8ABytes);
          // scales of this K block -> tensor memory (4 columns for A's 128 rows, 4 for B's)
          const uint32_t sfa_t = tmem_base + kSfTmemBase + sf_set * 8;
          const uint32_t sfb_t = sfa_t + 4;
          tmem_cp_scales(sfa_t, smem_desc_scales(sf_addr));
          tmem_cp_scales(sfb_t, smem_desc_scales(sf_addr + kSfBytes));
#pragma unroll
          for (uint32_t k = 0; k < FBK / 32; ++k) {
            // K advances by 32 elements = 32 bytes inside the 128-byte swizzle row
            umma_mxf8(tmem_d, adesc + static_cast<uint64_t>(k * 2), bdesc + static_cast<uint64_t>(k * 2), idesc_mxf8(BM, FBN, k),
                      sfa_t, sfb_t, (kb | static_cast<int>(k)) != 0);
          }
          tc_commit(&empty_bar[stage]);
          sf_set ^= 1;
          if (++stage == kF8Stages) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int quarter = warp % 4;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, kF8GroupM, tm, tn);
      bool ok = mbar_wait(&acc_full[acc], acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_ACC, 2, acc);
        break;
      }
      tc_fence_after_sync();
      const int row = tm * BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * FBN);
#pragma unroll 1
      for (int c = 0; c < FBN; c += 32) {
        uint32_t r[32];
        tmem_ld32(taddr + c, r);
        tc_wait_ld();
        if (row < M) {
          uint4* out = reinterpret_cast<uint4*>(d + static_cast<size_t>(row) * ldd + tn * FBN + c);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            out[v] = make_uint4(pack_bf16(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1])),
                                pack_bf16(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3])),
                                pack_bf16(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5])),
                                pack_bf16(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7])));
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kF8TmemCols);
  }
}

}  // namespace

// D[M,N] (bf16) = block-scaled A[M,K] * B[N,K]^T (e4m3).  K % 128 == 0, N % 128 == 0.
// sfa: ceil(M/128) * (K/128) blocks of 512 bytes, sfb: (N/128) * (K/128) blocks (layout at the top).
cudaError_t gemm_mxfp8(const void* a, const void* sfa, const void* b, const void* sfb, void* d, int M, int N, int K, int lda,
                       int ldb, int ldd, int* error_words, int max_ctas, cudaStream_t stream) {
  if (K % FBK != 0 || N % FBN != 0 || M <= 0) return cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(sfa) % 16 != 0 || reinterpret_cast<uintptr_t>(sfb) % 16 != 0) return cudaErrorInvalidValue;
  CUtensorMap map_a = make_u8_kmajor_map(a, M, K, lda, BM);
  CUtensorMap map_b = make_u8_kmajor_map(b, N, K, ldb, FBN);
  const int tiles = ((M + BM - 1) / BM) * (N / FBN);
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = tiles;
  static bool configured[64] = {};                 // the attribute is per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kF8SmemBytes));
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  gemm_mxfp8_kernel<<<grid, kGemmThreads, kF8SmemBytes, stream>>>(map_a, map_b, static_cast<const uint8_t*>(sfa),
                                                                 static_cast<const uint8_t*>(sfb),
                                                                 static_cast<__nv_bfloat16*>(d), M, N, K, ldd, error_words);
  return cudaGetLastError();
}

}  // namespace sm100
}  // namespace msccl
