// Pieces of the block-scaled fp8 pipeline on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles, K blocks of 128 bytes)
// shared by the plain GEMM (gemm_mxfp8_2cta_sm100.cu) and the fused tensor-parallel kernels (fused_tp_fp8_2cta.cu):
// tile geometry, the per-CTA tensor load that completes on the leader's mbarrier, the scale copy into the tensor
// memory of both CTAs, the tcgen05.mma.kind::mxf8f6f4.block_scale issue, and the MMA issuer loop.
//
// Per stage a CTA holds [A: its 128 rows | B: its 128 rows of the tile | scales of its A rows (512 B) | scales of B
// rows 0-127 | scales of B rows 128-255]; tensor memory holds one 256-column accumulator and 12 scale columns per
// stage.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "gemm_sm100.cuh"
#include "gemm_sm100.h"
#include "umma_2cta.cuh"

namespace msccl {
namespace sm100 {

constexpr int QBM = 256, QBN = 256, QBK = 128;
constexpr int kQStages = 5;                        // pipeline stages; the shared memory of a sixth holds the staged epilogue
constexpr int kQGroupM = 8;
constexpr int kQABytes = BM * QBK;                 // 16 KB: this CTA's 128 rows of A
constexpr int kQBBytes = (QBN / 2) * QBK;          // 16 KB: this CTA's 128 rows of B
constexpr int kQSfBytes = 512;                     // scales of 128 rows x 128 K
constexpr int kQLoadBytes = kQABytes + kQBBytes + 3 * kQSfBytes;   // bytes one CTA loads per stage
constexpr int kQStageBytes = 34 * 1024;            // stage pitch: operand tiles stay 1024-byte aligned
constexpr int kQTmemCols = 512;                    // [0,256) accumulator, then 12 scale columns per stage
constexpr int kQSfTmemBase = QBN;
// Staged epilogue: an epilogue warp packs its 32 rows x kQStageCols columns to bf16 in shared memory (one row per
// lane), then stores whole row segments with consecutive lanes on consecutive 16 bytes.  After the last pass into
// shared memory the accumulator is free for the next tile while the stores are still being issued.
constexpr int kQStageCols = 128;
constexpr int kQEpiPitch = kQStageCols * 2 + 16;   // bytes per staged row (16 of padding spread the banks)
constexpr int kQEpiPerWarp = 32 * kQEpiPitch;
constexpr size_t kQSmemBytes = 1024 + static_cast<size_t>(kQStages) * kQStageBytes + 256 + 4 * kQEpiPerWarp;
static_assert(kQLoadBytes <= kQStageBytes, "stage pitch too small");
static_assert(kQSmemBytes <= 227 * 1024, "shared memory of one CTA");

__device__ __forceinline__ void tma_load_2d_pair8(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ uint64_t smem_desc_scales_pair(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>(128 >> 4) << 32;     // stride between the four 8-row groups of a 32 x 16-byte block
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}
// Scales shared memory -> tensor memory in both CTAs of the pair (each from its own shared memory).
__device__ __forceinline__ void tmem_cp_scales_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ uint32_t idesc_mxf8_pair(uint32_t sf) {
  return (sf << 4) | (1u << 23) | (static_cast<uint32_t>(QBN >> 3) << 17) | (static_cast<uint32_t>(QBM >> 4) << 24) | (sf << 29);
}
__device__ __forceinline__ void umma_mxf8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa_taddr,
                                               uint32_t sfb_taddr, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate)), "r"(sfa_taddr), "r"(sfb_taddr)
      : "memory");
}

// MMA issuer of a pair (one thread of the leader): `my_tiles` tiles of `k_blocks` stages.  full_bar / acc_empty are the
// leader's barriers, empty_bar / acc_full exist in both CTAs and are committed to with the pair mask.
template <int STAGES>
__device__ __forceinline__ void mma_role_mx_pair(uint8_t* stage_base, uint64_t* full_bar, uint64_t* empty_bar, uint64_t* acc_full,
                                                 uint64_t* acc_empty, uint32_t tmem_base, int my_tiles, int k_blocks,
                                                 volatile int* abort_flag, int* error_words) {
  int stage = 0;
  uint32_t phase = 0, acc_phase = 0;
  for (int t = 0; t < my_tiles; ++t) {
    if (!mbar_wait(acc_empty, acc_phase ^ 1, abort_flag)) {
      gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_ACC, 1, 0);
      return;
    }
    tc_fence_after_sync();
    for (int kb = 0; kb < k_blocks; ++kb) {
      if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
        gemm_fail(error_words, abort_flag, GEMM_TIMEOUT_FULL, 1, stage);
        return;
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
        umma_mxf8_pair(tmem_base, adesc + static_cast<uint64_t>(k * 2), bdesc + static_cast<uint64_t>(k * 2), idesc_mxf8_pair(k), sfa_t,
                       sfb_t, (kb | static_cast<int>(k)) != 0);
      tc_commit_pair(&empty_bar[stage], 3);
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
    tc_commit_pair(acc_full, 3);
    acc_phase ^= 1;
  }
}

}  // namespace sm100
}  // namespace msccl
