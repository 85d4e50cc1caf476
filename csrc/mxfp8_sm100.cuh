// Pieces of the single-CTA block-scaled fp8 (OCP MX: e4m3 values, one UE8M0 scale per 32 K elements of a row)
// pipeline shared by the plain GEMM (gemm_mxfp8_sm100.cu) and the fused tensor-parallel kernels
// (fused_tp_fp8.cu): tile geometry, the untiled bulk copy for scale blocks, the scale copy into tensor memory
// and the tcgen05.mma.kind::mxf8f6f4.block_scale issue.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "gemm_sm100.cuh"

namespace msccl {
namespace sm100 {

constexpr int FBN = 128;                       // tile columns
constexpr int FBK = 128;                       // K elements (= bytes) per stage
constexpr int kF8Stages = 6;
constexpr int kF8GroupM = 16;                  // tile rows per L2-resident group
constexpr int kF8ABytes = BM * FBK;            // 16 KB
constexpr int kF8BBytes = FBN * FBK;           // 16 KB
constexpr int kSfBytes = 512;                  // scales of 128 rows x 128 K
constexpr int kF8StageBytes = kF8ABytes + kF8BBytes + 2 * kSfBytes;   // multiple of 1024
constexpr int kF8TmemCols = 512;               // [0,256) accumulators, [256,272) scale buffers
constexpr int kSfTmemBase = 2 * FBN;
constexpr size_t kF8SmemBytes = 1024 + static_cast<size_t>(kF8Stages) * kF8StageBytes + 256;
static_assert(kF8StageBytes % 1024 == 0, "operand tiles must stay 1024-byte aligned for SWIZZLE_128B");

// Untiled bulk copy global -> shared, completion counted on an mbarrier.  Both addresses and the
// size are multiples of 16 bytes.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Shared-memory descriptor of a scale block: 32 rows of 16 bytes, no swizzle; the four 8-row core
// matrices are 128 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_scales(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>(128 >> 4) << 32;     // stride byte offset between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;            // descriptor version for sm_100
  return d;
}
__device__ __forceinline__ void tmem_cp_scales(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// Instruction descriptor for e4m3 x e4m3 with UE8M0 scales, both operands K-major; `sf` selects
// which byte of the scale columns applies to this K=32 step.
__device__ __forceinline__ uint32_t idesc_mxf8(int m, int n, uint32_t sf) {
  return (sf << 4) | (1u << 23) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24) | (sf << 29);
}
__device__ __forceinline__ void umma_mxf8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa_taddr,
                                          uint32_t sfb_taddr, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate)), "r"(sfa_taddr), "r"(sfb_taddr)
      : "memory");
}

}  // namespace sm100
}  // namespace msccl
