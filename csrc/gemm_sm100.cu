// Persistent tcgen05 GEMM for sm_100a: D[M,N] = A[M,K] * B[N,K]^T (bf16 in, fp32 accumulate in
// tensor memory, bf16 out), optionally with a fused SwiGLU epilogue.  See gemm_sm100.cuh for the
// warp roles.  The same main loop is reused by the fused all-gather->GEMM and
// GEMM->reduce-scatter kernels (fused_tp.cu) and by the grouped expert GEMM (moe_a2a.cu).
#include <cuda.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "gemm_sm100.cuh"
#include "gemm_sm100.h"

namespace msccl {
namespace sm100 {

namespace {

constexpr int kGroupM = 16;          // 16 tile rows = 2048 rows of A per L2-resident group

template <int BN> struct GemmSmem {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kAccStages = 2;
  static constexpr int kTmemCols = kAccStages * BN;          // 512 for BN=256, 256 for BN=128
  static constexpr size_t kBytes = 1024 /*alignment slack*/ + static_cast<size_t>(kStages) * kStageBytes + 256;
};

// EPI 0: D = acc (bf16).  EPI 1: SwiGLU - columns [0,BN/2) of a tile are "gate", [BN/2,BN) are
// "up" for the same BN/2 output features; D[M, N/2] = silu(gate) * up.
template <int BN, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 __nv_bfloat16* __restrict__ d, int M, int N, int K, int ldd, int* error_words) {
  using S = GemmSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* stage_base = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(S::kStages) * S::kStageBytes);
  uint64_t* full_bar = bars;                         // [kStages]   TMA -> MMA
  uint64_t* empty_bar = bars + S::kStages;           // [kStages]   MMA -> TMA
  uint64_t* acc_full = bars + 2 * S::kStages;        // [2]         MMA -> epilogue
  uint64_t* acc_empty = bars + 2 * S::kStages + 2;   // [2]         epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S::kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (error_words != nullptr && *reinterpret_cast<volatile int*>(error_words) != 0) return;   // an earlier launch gave up
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = N / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);                   // one arrival per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 1) tmem_alloc(tmem_slot, S::kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued_unconsumed = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, kGroupM, tm, tn);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_EMPTY, 0, stage);
            ok = false;
            break;
          }
          uint8_t* a_dst = stage_base + static_cast<size_t>(stage) * S::kStageBytes;
          uint8_t* b_dst = a_dst + S::kABytes;
          mbar_expect_tx(&full_bar[stage], S::kStageBytes);
          tma_load_2d(a_dst, &map_a, &full_bar[stage], kb * BK, tm * BM);
          tma_load_2d(b_dst, &map_b, &full_bar[stage], kb * BK, tn * BN);
          ++issued_unconsumed;
          if (++stage == S::kStages) { stage = 0; phase ^= 1; }
        }
      }
      (void)issued_unconsumed;
      if (!ok) {
        // let every load that was issued land before shared memory is released
        for (int s = 0; s < S::kStages; ++s)
          for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&full_bar[s], 0) && !mbar_try_wait(&full_bar[s], 1); ++i) {}
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16_f32(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) {
          gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_ACC, 1, acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_FULL, 1, stage);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(stage_base + static_cast<size_t>(stage) * S::kStageBytes);
          const uint64_t adesc = smem_desc_sw128(a_addr);
          const uint64_t bdesc = smem_desc_sw128(a_addr + S::kABytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing K by 16 elements = 32 bytes inside the 128-byte swizzle row
            umma_bf16(tmem_d, adesc + static_cast<uint64_t>(k * 2), bdesc + static_cast<uint64_t>(k * 2), idesc,
                      (kb | k) != 0);
          }
          tc_commit(&empty_bar[stage]);              // stage reusable once these MMAs have read it
          if (++stage == S::kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&acc_full[acc]);           // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int quarter = warp % 4;                    // TMEM lanes [32*quarter, 32*quarter+32)
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, kGroupM, tm, tn);
      bool ok = mbar_wait(&acc_full[acc], acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_ACC, 2, acc);
        break;
      }
      tc_fence_after_sync();
      const int row = tm * BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
      if (EPI == 0) {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld32(taddr + c, r);
          tc_wait_ld();
          if (row < M) {
            uint4* out = reinterpret_cast<uint4*>(d + static_cast<size_t>(row) * ldd + tn * BN + c);
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
        constexpr int H = BN / 2;
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
      if (lane == 0) mbar_arrive(&acc_empty[acc]);   // accumulator stage free for the MMA warp
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, S::kTmemCols);
  }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || p == nullptr)
      throw std::runtime_error("cuTensorMapEncodeTiled is not available");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

}  // namespace

// Tensor map for a row-major [rows, cols] bf16 matrix (cols contiguous), box = [box_rows, 64 cols],
// 128-byte swizzle.  `ld` is the row pitch in elements.
CUtensorMap make_bf16_kmajor_map(const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || (ld * 2) % 16 != 0)
    throw std::runtime_error("TMA needs a 16-byte aligned base address and row pitch");
  CUtensorMap map;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), box_rows};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = encode_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r)));
  return map;
}

// Tensor map for a row-major [rows, cols] matrix of 8-bit elements (cols contiguous), box = [box_rows, 128 cols],
// 128-byte swizzle.  `ld` is the row pitch in bytes.
CUtensorMap make_u8_kmajor_map(const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || ld % 16 != 0)
    throw std::runtime_error("TMA needs a 16-byte aligned base address and row pitch");
  CUtensorMap map;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = encode_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r)));
  return map;
}

// Tensor map over an array of 512-byte blocks (the packed scale factors): block i is row i of a
// [blocks, 128] matrix of 32-bit words, box = one row, no swizzle.
CUtensorMap make_block512_map(const void* base, uint64_t blocks) {
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) throw std::runtime_error("TMA needs a 16-byte aligned base address");
  CUtensorMap map;
  cuuint64_t dims[2] = {128, blocks};
  cuuint64_t strides[1] = {512};
  cuuint32_t box[2] = {128, 1};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = encode_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r)));
  return map;
}

int sm_count() {
  static int count = 0;
  if (count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
  }
  return count;
}

// D[M, N or N/2] = epilogue(A[M,K] * B[N,K]^T).  K % 64 == 0, N % 256 == 0 (128 with bn=128).
cudaError_t gemm_bf16(const void* a, const void* b, void* d, int M, int N, int K, int lda, int ldb, int ldd, int epilogue,
                      int bn, int* error_words, int max_ctas, cudaStream_t stream) {
  if (K % BK != 0 || N % bn != 0 || (bn != 128 && bn != 256) || M <= 0) return cudaErrorInvalidValue;
  CUtensorMap map_a = make_bf16_kmajor_map(a, M, K, lda, BM);
  CUtensorMap map_b = make_bf16_kmajor_map(b, N, K, ldb, bn);
  const int tiles = ((M + BM - 1) / BM) * (N / bn);
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = tiles;
  auto* out = static_cast<__nv_bfloat16*>(d);
#define MSCCL_LAUNCH_GEMM(BN_, EPI_)                                                                                      \
  do {                                                                                                                    \
    auto kernel = gemm_bf16_kernel<BN_, EPI_>;                                                                            \
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,                            \
                                         static_cast<int>(GemmSmem<BN_>::kBytes));                                        \
    if (e != cudaSuccess) return e;                                                                                       \
    kernel<<<grid, kGemmThreads, GemmSmem<BN_>::kBytes, stream>>>(map_a, map_b, out, M, N, K, ldd, error_words);          \
  } while (0)
  if (bn == 256 && epilogue == 0) MSCCL_LAUNCH_GEMM(256, 0);
  else if (bn == 256) MSCCL_LAUNCH_GEMM(256, 1);
  else if (epilogue == 0) MSCCL_LAUNCH_GEMM(128, 0);
  else MSCCL_LAUNCH_GEMM(128, 1);
#undef MSCCL_LAUNCH_GEMM
  return cudaGetLastError();
}

}  // namespace sm100
}  // namespace msccl
