// Blackwell (sm_100a) GEMM building blocks: mbarrier, TMA (non-multicast), tcgen05.mma with TMEM
// accumulators, tcgen05.ld epilogue.  D[M,N] = A[M,K] * B[N,K]^T, A and B K-major bf16, fp32
// accumulation in tensor memory.
//
// Kernel shape used by all GEMM-shaped kernels of this package:
//   persistent CTAs (one per SM), 192 threads:
//     warp 0      TMA producer   - one thread issues cp.async.bulk.tensor loads into a ring of
//                                  SWIZZLE_128B shared-memory stages, completion on mbarriers
//     warp 1      MMA issuer     - one thread issues tcgen05.mma (128 x BN x 16 per instruction),
//                                  tcgen05.commit releases stages and publishes accumulators
//     warps 2..5  epilogue       - tcgen05.ld the accumulator (one TMEM lane quarter per warp),
//                                  convert, store; double-buffered against the next tile's MMAs
// Every mbarrier wait is bounded; on expiry the kernel raises an error word in global memory,
// drains its outstanding TMA loads, frees its tensor memory and returns.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace msccl {
namespace sm100 {

constexpr int BM = 128;           // tile rows  (= TMEM lanes, one tcgen05.mma M)
constexpr int BK = 64;            // 64 bf16 = 128 bytes = one swizzle atom row
constexpr int UMMA_K = 16;        // K per tcgen05.mma for 16-bit inputs
constexpr int kGemmThreads = 192;
constexpr unsigned long long kMbarTimeoutNs = 10ull * 1000 * 1000 * 1000;   // longest wait on one mbarrier

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return done != 0;
}
// Bounded wait; false = gave up (or another role already failed).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long now;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
  const unsigned long long deadline = now + kMbarTimeoutNs;
  for (uint32_t i = 0;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u) {
      if (*abort_flag != 0) return false;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (now > deadline) return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

// ---- tensor memory -----------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {        // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, 128-byte rows, SWIZZLE_128B; 8-row groups are
// 1024 bytes apart (stride byte offset); the leading byte offset is unused for this layout.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>(1) << 16;            // leading byte offset (16 B), ignored
  d |= static_cast<uint64_t>(1024 >> 4) << 32;    // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;            // descriptor version for sm_100
  d |= static_cast<uint64_t>(2) << 61;            // SWIZZLE_128B
  return d;
}
// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, M x N tile.
__host__ __device__ constexpr uint32_t idesc_bf16_f32(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
      : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Tile order of the persistent kernels.  Tiles that run at the same time have consecutive indices;
// walking `group_m` tile rows per tile column before moving to the next column keeps the A rows of a
// group (group_m x tile_rows x K) and the B columns in flight resident in L2.  Plain column-major
// order re-reads all of A from HBM once per tile column as soon as A outgrows L2.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  const int per_group = group_m * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * group_m;
  const int rows = min(group_m, tiles_m - first_m);
  const int in_group = tile - g * per_group;
  tm = first_m + in_group % rows;
  tn = in_group / rows;
}

// Error word layout in global memory: [0] code (0 ok), [1] block, [2] role, [3] detail.
enum GemmError : int { GEMM_OK = 0, GEMM_TIMEOUT_FULL = 1, GEMM_TIMEOUT_EMPTY = 2, GEMM_TIMEOUT_ACC = 3, GEMM_TIMEOUT_FLAG = 4 };

__device__ __forceinline__ void gemm_fail(int* error_words, volatile int* abort_flag, int code, int role, int detail) {
  *abort_flag = 1;
  if (error_words != nullptr && atomicCAS(&error_words[0], 0, code) == 0) {
    error_words[1] = blockIdx.x;
    error_words[2] = role;
    error_words[3] = detail;
  }
}

}  // namespace sm100
}  // namespace msccl
