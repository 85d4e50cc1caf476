// Fused MoE expert-parallel kernels for sm_100a (top-k routing, experts sharded over GPUs).
//
//   dispatch + GEMM1   comm CTAs all-gather the per-expert copy counts (a few hundred bytes), derive
//                      where each of their token copies lands on the owning GPU (rows of one expert
//                      are contiguous, ordered by source rank), and scatter the token rows straight
//                      into the owners' dispatch buffers over NVLink, then publish one flag per
//                      source.  GEMM CTAs run the grouped gate/up GEMM with fused SwiGLU over the
//                      experts of this GPU; a tile waits only for the sources whose rows it covers.
//   GEMM2 + combine    grouped down projection; the epilogue multiplies each row by its gate weight
//                      and stores it directly into the combine buffer of the GPU that owns the
//                      token (the all-to-all back), then all CTAs sum the top-k slots of the local
//                      tokens once every peer has reported completion.
//
// This is the MSCCLang AllToAll pattern (reference examples/mscclang/alltoall_allpairs.py:14-17)
// generalised to data-dependent counts and fused with the expert GEMMs.  Buffers written by peers
// are double buffered by launch parity; every wait is bounded.
#include <cuda.h>
#include <cuda_runtime.h>

#include "gemm_sm100.h"
#include "moe_a2a.h"
#include "moe_common.cuh"
#include "pipeline_sm100.cuh"

namespace msccl {
namespace sm100 {

namespace {

// ============================================================ dispatch + grouped GEMM1 (SwiGLU)
__global__ void __launch_bounds__(kGemmThreads, 1)
moe_dispatch_gemm_kernel(const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_a1,
                         const __grid_constant__ CUtensorMap map_b, MoeArgs g) {
  extern __shared__ uint8_t smem_raw[];
  const Pipe p = carve_smem(smem_raw);
  __shared__ MoeShared sh;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  FusedPage* page = g.pages[g.rank];
  if (g.error_words != nullptr && *reinterpret_cast<volatile int*>(g.error_words) != 0) return;
  const unsigned long long epoch = page->moe_epoch + 1;
  const int parity = static_cast<int>(epoch & 1ull);
  if (threadIdx.x == 0) *p.abort_flag = 0;
  __syncthreads();

  if (static_cast<int>(blockIdx.x) < g.comm_ctas) {
    // ---------------------------------------------------------------- comm CTAs
    moe_comm_role(g, page, epoch, parity, &sh, p.abort_flag);
  } else {
    // ---------------------------------------------------------------- GEMM CTAs
    init_pipe(p);
    if (threadIdx.x == 0) prefetch_tensormap(&map_b);
    if (warp == 1) tmem_alloc(p.tmem_slot, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *p.tmem_slot;
    const bool have_counts = load_counts(g, page, epoch, parity, &sh, p.abort_flag);
    const int gemm_ctas = gridDim.x - g.comm_ctas, cta = blockIdx.x - g.comm_ctas;
    const int n_out = 2 * g.ffn, tiles_n = n_out / BN, k_blocks = g.hidden / BK;
    const int num_tiles = have_counts ? total_grouped_tiles(sh.rows_per_expert, g.local_experts, tiles_n) : 0;
    const int my_tiles = num_tiles > cta ? (num_tiles - cta + gemm_ctas - 1) / gemm_ctas : 0;

    if (warp == 0) {
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        unsigned int landed = 0;                                  // bit s: all rows of source s have arrived
        for (int tile = cta; tile < num_tiles && ok; tile += gemm_ctas) {
          TileInfo t;
          decode_grouped(tile, sh.rows_per_expert, g.local_experts, tiles_n, t);
          for (int s = 0; s < g.nranks && ok; ++s) {
            const bool covers = sh.seg_start[t.expert][s] < t.m0 + t.rows && sh.seg_start[t.expert][s + 1] > t.m0;
            if (covers && !(landed & (1u << s))) {
              if (!wait_flag_ge(&page->moe_flag[s][1], epoch, p.abort_flag)) {
                gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_FLAG, 0, s);
                ok = false;
              }
              landed |= 1u << s;
              fence_proxy_async();
            }
          }
          const int a_row = t.expert * g.cap + t.m0;
          const int b_row = t.expert * n_out + t.tn * BN;
          for (int kb = 0; kb < k_blocks && ok; ++kb) {
            if (!mbar_wait(&p.empty_bar[stage], phase ^ 1, p.abort_flag)) {
              gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_EMPTY, 0, stage);
              ok = false;
              break;
            }
            uint8_t* a_dst = p.stage_base + static_cast<size_t>(stage) * kStageBytes;
            mbar_expect_tx(&p.full_bar[stage], kStageBytes);
            if (parity) tma_load_2d(a_dst, &map_a1, &p.full_bar[stage], kb * BK, a_row);
            else tma_load_2d(a_dst, &map_a0, &p.full_bar[stage], kb * BK, a_row);
            tma_load_2d(a_dst + kABytes, &map_b, &p.full_bar[stage], kb * BK, b_row);
            if (++stage == kStages) { stage = 0; phase ^= 1; }
          }
        }
        if (!ok) drain_loads(p);
      }
    } else if (warp == 1) {
      if (lane == 0) mma_role(p, tmem_base, my_tiles, k_blocks, g.error_words);
    } else {
      const int quarter = warp % 4;
      int acc = 0;
      uint32_t acc_phase = 0;
      __nv_bfloat16* h = static_cast<__nv_bfloat16*>(g.h);
      constexpr int H = BN / 2;
      for (int tile = cta; tile < num_tiles; tile += gemm_ctas) {
        TileInfo t;
        decode_grouped(tile, sh.rows_per_expert, g.local_experts, tiles_n, t);
        bool ok = mbar_wait(&p.acc_full[acc], acc_phase, p.abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_ACC, 2, acc);
          break;
        }
        tc_fence_after_sync();
        const int r_in_tile = quarter * 32 + lane;
        const size_t row = static_cast<size_t>(t.expert) * g.cap + t.m0 + r_in_tile;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
#pragma unroll 1
        for (int c = 0; c < H; c += 32) {
          uint32_t gt[32], up[32];
          tmem_ld32(taddr + c, gt);
          tmem_ld32(taddr + H + c, up);
          tc_wait_ld();
          if (r_in_tile < t.rows) {
            uint4* out = reinterpret_cast<uint4*>(h + row * g.ffn + t.tn * H + c);
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
    __syncthreads();
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc(tmem_base, kTmemCols);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&page->moe_done, 1u) == gridDim.x - 1u) {
      page->moe_done = 0;
      // the epoch advances after the second kernel; remember that the first half ran
      page->moe_pad = 1;
    }
  }
}

// ============================================================ grouped GEMM2 + combine
__global__ void __launch_bounds__(kGemmThreads, 1)
moe_gemm_combine_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, MoeArgs g) {
  extern __shared__ uint8_t smem_raw[];
  const Pipe p = carve_smem<3>(smem_raw);
  __shared__ MoeShared sh;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  FusedPage* page = g.pages[g.rank];
  if (g.error_words != nullptr && *reinterpret_cast<volatile int*>(g.error_words) != 0) return;
  const unsigned long long epoch = page->moe_epoch + 1;
  const int parity = static_cast<int>(epoch & 1ull);
  init_pipe<3>(p);
  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 1) tmem_alloc(p.tmem_slot, kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *p.tmem_slot;
  const bool have_counts = load_counts(g, page, epoch, parity, &sh, p.abort_flag);   // flags are already set: no wait
  const int ctas = gridDim.x, cta = blockIdx.x;
  const int tiles_n = g.hidden / BN, k_blocks = g.ffn / BK;
  const int num_tiles = have_counts ? total_grouped_tiles(sh.rows_per_expert, g.local_experts, tiles_n) : 0;
  const int my_tiles = num_tiles > cta ? (num_tiles - cta + ctas - 1) / ctas : 0;
  const size_t row_bytes = static_cast<size_t>(g.hidden) * 2;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += ctas) {
        TileInfo t;
        decode_grouped(tile, sh.rows_per_expert, g.local_experts, tiles_n, t);
        const int a_row = t.expert * g.cap + t.m0;
        const int b_row = t.expert * g.hidden + t.tn * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&p.empty_bar[stage], phase ^ 1, p.abort_flag)) {
            gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_EMPTY, 0, stage);
            ok = false;
            break;
          }
          uint8_t* a_dst = p.stage_base + static_cast<size_t>(stage) * kStageBytes;
          mbar_expect_tx(&p.full_bar[stage], kStageBytes);
          tma_load_2d(a_dst, &map_a, &p.full_bar[stage], kb * BK, a_row);
          tma_load_2d(a_dst + kABytes, &map_b, &p.full_bar[stage], kb * BK, b_row);
          if (++stage == 3) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) drain_loads<3>(p);
    }
  } else if (warp == 1) {
    if (lane == 0) mma_role<3>(p, tmem_base, my_tiles, k_blocks, g.error_words);
  } else {
    const int quarter = warp % 4;
    int acc = 0;
    uint32_t acc_phase = 0;
    const int4* meta_base = reinterpret_cast<const int4*>(g.heap_bases[g.rank] + g.moe_off + g.lay.meta_off +
                                                          static_cast<size_t>(parity) * g.lay.meta_parity);
    for (int tile = cta; tile < num_tiles; tile += ctas) {
      TileInfo t;
      decode_grouped(tile, sh.rows_per_expert, g.local_experts, tiles_n, t);
      bool ok = mbar_wait(&p.acc_full[acc], acc_phase, p.abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_ACC, 2, acc);
        break;
      }
      tc_fence_after_sync();
      const int r_in_tile = quarter * 32 + lane;
      const bool valid = r_in_tile < t.rows;
      int4 m = make_int4(0, 0, 0, 0);
      if (valid) m = meta_base[static_cast<size_t>(t.expert) * g.cap + t.m0 + r_in_tile];
      const float w = valid ? __int_as_float(m.z) : 0.0f;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
      uint8_t* stage_warp = p.staging + (warp - 2) * kStagingPerWarp;
      stage_quarter_bf16(taddr, stage_warp, lane, w);            // row = lane: scaled by its own gate weight
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p.acc_empty[acc]);
      // every row goes home: combine[parity][copy][hidden] on the rank that owns the token.  The warp
      // writes one row per instruction (512 contiguous bytes); the row's address comes from the lane
      // that holds its metadata.
      char* my_dst = nullptr;
      if (valid)
        my_dst = g.heap_bases[m.x] + g.moe_off + g.lay.combine_off + static_cast<size_t>(parity) * g.lay.combine_parity +
                 static_cast<size_t>(m.y) * row_bytes + static_cast<size_t>(t.tn) * BN * 2;
      const unsigned long long mine_u = reinterpret_cast<unsigned long long>(my_dst);
#pragma unroll 1
      for (int r0 = 0; r0 < 32; r0 += 8) {
        uint4 d[8];
        unsigned long long ptr[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          ptr[u] = __shfl_sync(0xffffffffu, mine_u, r0 + u);
          d[u] = *reinterpret_cast<const uint4*>(stage_warp + (r0 + u) * kStagePitch + lane * 16);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (ptr[u] != 0) *reinterpret_cast<uint4*>(reinterpret_cast<char*>(ptr[u]) + lane * 16) = d[u];
      }
      __syncwarp();
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    // this warp's rows are on their way: tell every rank (one count per epilogue warp and CTA)
    __syncwarp();
    if (lane < g.nranks) {
      fence_acq_rel_sys();
      red_add_release_sys(&g.pages[lane]->moe_count[g.rank], 1ull);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }

  moe_sum_and_finish(g, page, epoch, parity, p.abort_flag);
}

}  // namespace

cudaError_t launch_moe_dispatch_gemm(const MoeArgs& g, int grid, cudaStream_t stream) {
  if (g.hidden % BN != 0 || (2 * g.ffn) % BN != 0 || g.hidden % BK != 0 || g.nranks > kFusedMaxRanks ||
      g.local_experts > kMoeMaxLocalExperts || g.num_experts > kMoeMaxExperts || g.comm_ctas < 1 || grid <= g.comm_ctas)
    return cudaErrorInvalidValue;
  const char* disp = g.heap_bases_host[g.rank] + g.moe_off + g.lay.dispatch_off;
  const uint64_t rows = static_cast<uint64_t>(g.local_experts) * g.cap;
  CUtensorMap a0 = make_bf16_kmajor_map(disp, rows, g.hidden, g.hidden, BM);
  CUtensorMap a1 = make_bf16_kmajor_map(disp + g.lay.dispatch_parity, rows, g.hidden, g.hidden, BM);
  CUtensorMap b = make_bf16_kmajor_map(g.w_gate_up, static_cast<uint64_t>(g.local_experts) * 2 * g.ffn, g.hidden, g.hidden, BN);
  cudaError_t e = cudaFuncSetAttribute(moe_dispatch_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kSmemBytes));
  if (e != cudaSuccess) return e;
  moe_dispatch_gemm_kernel<<<grid, kGemmThreads, kSmemBytes, stream>>>(a0, a1, b, g);
  return cudaGetLastError();
}

cudaError_t launch_moe_gemm_combine(const MoeArgs& g, int grid, cudaStream_t stream) {
  if (g.hidden % BN != 0 || g.ffn % BK != 0 || g.nranks > kFusedMaxRanks || g.local_experts > kMoeMaxLocalExperts || grid < 1)
    return cudaErrorInvalidValue;
  CUtensorMap a = make_bf16_kmajor_map(g.h, static_cast<uint64_t>(g.local_experts) * g.cap, g.ffn, g.ffn, BM);
  CUtensorMap b = make_bf16_kmajor_map(g.w_down, static_cast<uint64_t>(g.local_experts) * g.hidden, g.ffn, g.ffn, BN);
  cudaError_t e = cudaFuncSetAttribute(moe_gemm_combine_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kSmemBytesStaged));
  if (e != cudaSuccess) return e;
  moe_gemm_combine_kernel<<<grid, kGemmThreads, kSmemBytesStaged, stream>>>(a, b, g);
  return cudaGetLastError();
}

}  // namespace sm100
}  // namespace msccl
