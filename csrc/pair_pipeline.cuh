// The tile pipeline of a CTA pair (tcgen05 cta_group::2), shared by the fused kernels that run on pairs
// (fused_tp_2cta.cu, moe_a2a_2cta.cu): a cluster of two CTAs owns one 256 x 256 output tile; each CTA stages its own
// 128 rows of A and its own 128 rows of the B tile (32 KB per stage) with tensor loads that complete on the leader's
// mbarrier (no multicast), the leader issues the MMAs for both, and each CTA ends up with the accumulator of its own
// 128 rows in its own tensor memory.  Two accumulator stages of 256 columns.  Every wait is bounded.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "gemm_sm100.cuh"
#include "gemm_sm100.h"
#include "pipeline_sm100.cuh"
#include "prims.cuh"
#include "umma_2cta.cuh"

namespace msccl {
namespace sm100 {

constexpr int PBN = 256;                      // tile columns of the pair
constexpr int kPABytes = BM * BK * 2;         // this CTA's 128 rows of A: 16 KB
constexpr int kPBBytes = (PBN / 2) * BK * 2;  // this CTA's 128 rows of B: 16 KB
constexpr int kPStageBytes = kPABytes + kPBBytes;
constexpr int kPTmemCols = 2 * PBN;           // two accumulator stages
constexpr int kAgStages = 6;
constexpr int kRsStages = 4;                  // room for the staged epilogue
constexpr size_t kAgSmemBytes = 1024 + static_cast<size_t>(kAgStages) * kPStageBytes + 256;
constexpr size_t kRsSmemBytes = 1024 + static_cast<size_t>(kRsStages) * kPStageBytes + 256 + 4 * kStagingPerWarp;

__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}

struct PairPipe {
  uint8_t* stage_base;
  uint8_t* staging;
  uint64_t *full_bar, *empty_bar, *acc_full, *acc_empty;
  uint32_t* tmem_slot;
  volatile int* abort_flag;
};

template <int STAGES>
__device__ __forceinline__ PairPipe carve_pair(uint8_t* smem_raw) {
  PairPipe p;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  p.stage_base = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(STAGES) * kPStageBytes);
  p.full_bar = bars;
  p.empty_bar = bars + STAGES;
  p.acc_full = bars + 2 * STAGES;
  p.acc_empty = bars + 2 * STAGES + 2;
  p.tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  p.abort_flag = reinterpret_cast<volatile int*>(p.tmem_slot + 1);
  p.staging = smem + static_cast<size_t>(STAGES) * kPStageBytes + 256;
  return p;
}

template <int STAGES>
__device__ __forceinline__ void init_pair(const PairPipe& p) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&p.full_bar[s], 1);
      mbar_init(&p.empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&p.acc_full[a], 1);
      mbar_init(&p.acc_empty[a], 8);                 // four epilogue warps in each CTA of the pair
    }
    *p.abort_flag = 0;
    mbar_fence_init();
  }
}

// A producer that gave up lets the loads it issued land before shared memory is released: the leader can watch the
// barriers they complete on; the partner cannot and allows them 200 us.
template <int STAGES>
__device__ __forceinline__ void drain_pair(const PairPipe& p, bool leader) {
  if (leader) {
    for (int s = 0; s < STAGES; ++s)
      for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&p.full_bar[s], 0) && !mbar_try_wait(&p.full_bar[s], 1); ++i) {}
  } else {
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {}
  }
}

// MMA issuer of a pair (leader only): `my_tiles` tiles of `k_blocks` stages each.
template <int STAGES>
__device__ __forceinline__ void mma_role_pair(const PairPipe& p, uint32_t tmem_base, int my_tiles, int k_blocks, int* error_words) {
  constexpr uint32_t idesc = idesc_bf16_f32(2 * BM, PBN);
  int stage = 0, acc = 0;
  uint32_t phase = 0, acc_phase = 0;
  for (int t = 0; t < my_tiles; ++t) {
    if (!mbar_wait(&p.acc_empty[acc], acc_phase ^ 1, p.abort_flag)) {
      gemm_fail(error_words, p.abort_flag, GEMM_TIMEOUT_ACC, 1, acc);
      return;
    }
    tc_fence_after_sync();
    const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * PBN);
    for (int kb = 0; kb < k_blocks; ++kb) {
      if (!mbar_wait(&p.full_bar[stage], phase, p.abort_flag)) {
        gemm_fail(error_words, p.abort_flag, GEMM_TIMEOUT_FULL, 1, stage);
        return;
      }
      tc_fence_after_sync();
      const uint32_t a_addr = smem_u32(p.stage_base + static_cast<size_t>(stage) * kPStageBytes);
      const uint64_t adesc = smem_desc_sw128(a_addr);
      const uint64_t bdesc = smem_desc_sw128(a_addr + kPABytes);
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; ++k)
        umma_bf16_pair(tmem_d, adesc + static_cast<uint64_t>(k * 2), bdesc + static_cast<uint64_t>(k * 2), idesc, (kb | k) != 0);
      tc_commit_pair(&p.empty_bar[stage], 3);        // stage free in both CTAs
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
    tc_commit_pair(&p.acc_full[acc], 3);             // accumulator complete in both CTAs
    if (++acc == 2) { acc = 0; acc_phase ^= 1; }
  }
}

// Host side: how many clusters of two CTAs the device holds at once, and the cluster launch.
template <typename Kernel>
cudaError_t pair_clusters(Kernel kernel, size_t smem, int* clusters) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * sm_count(), 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaOccupancyMaxActiveClusters(clusters, kernel, &cfg);
}

template <typename Kernel, typename... Args>
cudaError_t launch_pairs(Kernel kernel, size_t smem, int clusters, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}


}  // namespace sm100
}  // namespace msccl
