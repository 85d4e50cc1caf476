// Pieces shared by the fused compute+collective kernels (fused_tp.cu, moe_a2a.cu): the 128x256
// tile pipeline (shared-memory carve-up, mbarrier set, MMA issuer role) and bounded waits on flags
// that peers write over NVLink.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "gemm_sm100.cuh"
#include "prims.cuh"

namespace msccl {
namespace sm100 {

constexpr int BN = 256;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;
constexpr int kBBytes = BN * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 2 * BN;
constexpr size_t kSmemBytes = 1024 + static_cast<size_t>(kStages) * kStageBytes + 256;
constexpr unsigned long long kFlagTimeoutNs = 5ull * 1000 * 1000 * 1000;   // per wait on a peer

__device__ __forceinline__ bool wait_flag_ge(const unsigned long long* flag, unsigned long long want, volatile int* abort_flag) {
  const unsigned long long deadline = global_timer_ns() + kFlagTimeoutNs;
  for (unsigned int i = 0;; ++i) {
    if (ld_acquire_sys(flag) >= want) return true;
    if ((i & 255u) == 255u && (*abort_flag != 0 || global_timer_ns() > deadline)) return false;
  }
}

__device__ __forceinline__ void multimem_st16(void* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void red_add_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

constexpr int kStagePitch = BN * 2 + 16;                 // bytes per staged row: 512 + 16 of padding (bank spread)
constexpr int kStagingPerWarp = 32 * kStagePitch;        // one epilogue warp stages 32 rows x 256 bf16
constexpr size_t kSmemBytesStaged = 1024 + 3 * static_cast<size_t>(kStageBytes) + 256 + 4 * kStagingPerWarp;

struct Pipe {
  uint8_t* staging;                                      // only valid for the 3-stage + staging layout
  uint8_t* stage_base;
  uint64_t *full_bar, *empty_bar, *acc_full, *acc_empty;
  uint32_t* tmem_slot;
  volatile int* abort_flag;
};

template <int STAGES = kStages>
__device__ __forceinline__ Pipe carve_smem(uint8_t* smem_raw) {
  Pipe p;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  p.stage_base = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(STAGES) * kStageBytes);
  p.full_bar = bars;
  p.empty_bar = bars + STAGES;
  p.acc_full = bars + 2 * STAGES;
  p.acc_empty = bars + 2 * STAGES + 2;
  p.tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  p.staging = smem + static_cast<size_t>(STAGES) * kStageBytes + 256;
  p.abort_flag = reinterpret_cast<volatile int*>(p.tmem_slot + 1);
  return p;
}

template <int STAGES = kStages>
__device__ __forceinline__ void init_pipe(const Pipe& p) {
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

// MMA issuer shared by both kernels: consumes `my_tiles` tiles of k_blocks stages each.
template <int STAGES = kStages>
__device__ __forceinline__ void mma_role(const Pipe& p, uint32_t tmem_base, int my_tiles, int k_blocks, int* error_words) {
  constexpr uint32_t idesc = idesc_bf16_f32(BM, BN);
  int stage = 0, acc = 0;
  uint32_t phase = 0, acc_phase = 0;
  for (int t = 0; t < my_tiles; ++t) {
    if (!mbar_wait(&p.acc_empty[acc], acc_phase ^ 1, p.abort_flag)) {
      gemm_fail(error_words, p.abort_flag, GEMM_TIMEOUT_ACC, 1, acc);
      return;
    }
    tc_fence_after_sync();
    const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
    for (int kb = 0; kb < k_blocks; ++kb) {
      if (!mbar_wait(&p.full_bar[stage], phase, p.abort_flag)) {
        gemm_fail(error_words, p.abort_flag, GEMM_TIMEOUT_FULL, 1, stage);
        return;
      }
      tc_fence_after_sync();
      const uint32_t a_addr = smem_u32(p.stage_base + static_cast<size_t>(stage) * kStageBytes);
      const uint64_t adesc = smem_desc_sw128(a_addr);
      const uint64_t bdesc = smem_desc_sw128(a_addr + kABytes);
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; ++k)
        umma_bf16(tmem_d, adesc + static_cast<uint64_t>(k * 2), bdesc + static_cast<uint64_t>(k * 2), idesc, (kb | k) != 0);
      tc_commit(&p.empty_bar[stage]);
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
    tc_commit(&p.acc_full[acc]);
    if (++acc == 2) { acc = 0; acc_phase ^= 1; }
  }
}

template <int STAGES = kStages>
__device__ __forceinline__ void drain_loads(const Pipe& p) {
  for (int s = 0; s < STAGES; ++s)
    for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&p.full_bar[s], 0) && !mbar_try_wait(&p.full_bar[s], 1); ++i) {}
}


// ---- staged epilogue -----------------------------------------------------------------------
// An epilogue warp holds 32 rows x 256 fp32 columns of the accumulator, one row per lane.  Storing
// from registers gives every lane its own row: fine for local HBM, wasteful over NVLink where only
// full contiguous lines travel efficiently.  Staging the bf16 tile in shared memory lets the warp
// write one row per instruction, 32 lanes x 16 bytes = 512 contiguous bytes.
__device__ __forceinline__ void stage_quarter_bf16(uint32_t taddr, uint8_t* stage_warp, int lane, float scale) {
#pragma unroll 1
  for (int c = 0; c < BN; c += 32) {
    uint32_t r[32];
    tmem_ld32(taddr + c, r);
    tc_wait_ld();
    uint4* dst = reinterpret_cast<uint4*>(stage_warp + lane * kStagePitch + c * 2);
#pragma unroll
    for (int v = 0; v < 4; ++v)
      dst[v] = make_uint4(pack_bf16(scale * __uint_as_float(r[8 * v + 0]), scale * __uint_as_float(r[8 * v + 1])),
                          pack_bf16(scale * __uint_as_float(r[8 * v + 2]), scale * __uint_as_float(r[8 * v + 3])),
                          pack_bf16(scale * __uint_as_float(r[8 * v + 4]), scale * __uint_as_float(r[8 * v + 5])),
                          pack_bf16(scale * __uint_as_float(r[8 * v + 6]), scale * __uint_as_float(r[8 * v + 7])));
  }
  __syncwarp();
}

}  // namespace sm100
}  // namespace msccl
