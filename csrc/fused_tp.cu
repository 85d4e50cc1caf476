// Fused tensor-parallel kernels for sm_100a: the collective and the tcgen05 GEMM run in ONE
// kernel and overlap tile by tile.
//
//   all-gather -> GEMM   D[n*Ml, N] = epilogue(gather(X)[n*Ml, K] * B[N, K]^T)
//       A few "comm" CTAs push this rank's token shard X[Ml, K] into the gathered buffer of every
//       rank (multimem.st through NVSwitch when a multicast window exists, else peer stores) in
//       128-row blocks and publish one flag per block.  The other CTAs are the persistent GEMM:
//       their TMA producer waits for the flag of the block a tile needs, then loads it from the
//       LOCAL gathered buffer (never from peer memory, never with multicast).  Tiles are ordered
//       block-major so that consumption follows arrival; tiles of the local shard need no flag.
//
//   GEMM -> reduce-scatter   Y_owner[Ml, N] = sum over ranks of (H_r[n*Ml, K] * B_r[N, K]^T)[owner rows]
//       The epilogue converts each accumulator tile to bf16 and stores it straight into the owner
//       rank's partial buffer over NVLink, then bumps the counter of its (source, row block) on the
//       owner.  The row blocks are produced in the order of a table lowered from the schedule program
//       (msccl.ops.schedules): block-major, so that block b of every owner is complete long before the
//       GEMM ends.  A few CTAs at the end of the grid do no GEMM: they wait for the counters of one row
//       block after the other and sum its n partials in fp32, in rank order, while the GEMM CTAs are
//       still producing the later blocks.
//
// Buffers that peers write are double buffered by launch parity, so no barrier is needed between
// consecutive calls (a rank can be at most one call ahead of a peer: it needs the peer's data of
// call k+1 before it can finish it).  Every wait is bounded.
#include <cuda.h>
#include <cuda_runtime.h>

#include "gemm_sm100.cuh"
#include "gemm_sm100.h"
#include "fused_reduce.cuh"
#include "fused_tp.h"
#include "pipeline_sm100.cuh"
#include "prims.cuh"

namespace msccl {
namespace sm100 {

namespace {

static_assert(sizeof(FusedPage) <= 64 * 1024, "the fused-kernel flag page must fit its 64 KiB slot of the heap");

// Tile -> (column tile, row block).  Row blocks are numbered in arrival order (block-major over
// sources).  Default: column tile fastest (CTAs running together share a row block of A).
// tuning bit 0: groups of 8 row blocks with the row block fastest inside a group, which makes CTAs
// running together share column tiles of B instead.
__device__ __forceinline__ void ag_decode(int tile, int tiles_n, int row_blocks, int tuning, int& tn, int& mb) {
  if ((tuning & 1) == 0) {
    tn = tile % tiles_n;
    mb = tile / tiles_n;
  } else {
    constexpr int G = 8;
    const int per_group = G * tiles_n;
    const int group = tile / per_group, in_group = tile % per_group;
    const int rows_here = min(G, row_blocks - group * G);
    mb = group * G + in_group % rows_here;
    tn = in_group / rows_here;
  }
}

// ============================================================ all-gather -> GEMM (+SwiGLU)
template <int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap map_local, const __grid_constant__ CUtensorMap map_gath0,
               const __grid_constant__ CUtensorMap map_gath1, const __grid_constant__ CUtensorMap map_b, AgGemmArgs g) {
  extern __shared__ uint8_t smem_raw[];
  const Pipe p = carve_smem(smem_raw);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  FusedPage* page = g.pages[g.rank];
  if (g.error_words != nullptr && *reinterpret_cast<volatile int*>(g.error_words) != 0) return;   // an earlier launch gave up
  const unsigned long long epoch = page->ag_epoch + 1;
  const int parity = static_cast<int>(epoch & 1ull);
  const int blocks_per_rank = g.rows_per_rank / BM;

  if (static_cast<int>(blockIdx.x) < g.comm_ctas) {
    // ------------------------------------------------------------------ comm CTAs: push my shard
    // Blocks are pushed in parallel, not one after the other: publishing a block costs a
    // system-scope fence (an NVLink round trip), and doing that eight times in a row would delay
    // the last block by tens of microseconds.  With at least as many comm CTAs as blocks, block b
    // is handled by the CTAs c with c % blocks == b; otherwise CTA c walks blocks c, c + C, ...
    const size_t block_bytes = static_cast<size_t>(BM) * g.K * 2;
    const size_t vecs = block_bytes / 16;
    const int C = g.comm_ctas;
    const int parts = C >= blocks_per_rank ? C / blocks_per_rank : 1;
    const int part = C >= blocks_per_rank ? static_cast<int>(blockIdx.x) / blocks_per_rank : 0;
    const int b_first = C >= blocks_per_rank ? static_cast<int>(blockIdx.x) % blocks_per_rank : static_cast<int>(blockIdx.x);
    const int b_step = C >= blocks_per_rank ? blocks_per_rank : C;
    const size_t per_part = (vecs + parts - 1) / parts;
    const size_t v0 = min(vecs, per_part * part), v1 = min(vecs, v0 + per_part);
    const size_t dst_off = g.gathered_off + static_cast<size_t>(parity) * g.gathered_bytes +
                           static_cast<size_t>(g.rank) * g.rows_per_rank * g.K * 2;
    for (int b = b_first; b < blocks_per_rank && part < parts; b += (C >= blocks_per_rank ? blocks_per_rank * parts : b_step)) {
      const char* src = static_cast<const char*>(g.x_local) + b * block_bytes;
      constexpr int U = 16;       // 256 bytes per thread in flight: the copy is latency bound otherwise
      for (size_t base = v0 + threadIdx.x; base < v1; base += static_cast<size_t>(blockDim.x) * U) {
        uint4 d[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const size_t v = base + static_cast<size_t>(u) * blockDim.x;
          if (v < v1) d[u] = *reinterpret_cast<const uint4*>(src + v * 16);
        }
        if (g.mc_base != nullptr) {
          char* dst = g.mc_base + dst_off + b * block_bytes;
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const size_t v = base + static_cast<size_t>(u) * blockDim.x;
            if (v < v1) multimem_st16(dst + v * 16, d[u]);
          }
        } else {
          for (int q = 1; q < g.nranks; ++q) {
            char* dst = g.heap_bases[(g.rank + q) % g.nranks] + dst_off + b * block_bytes;
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const size_t v = base + static_cast<size_t>(u) * blockDim.x;
              if (v < v1) *reinterpret_cast<uint4*>(dst + v * 16) = d[u];
            }
          }
        }
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        fence_acq_rel_sys();
        if (atomicAdd(&page->ag_block_count[b], 1u) == static_cast<unsigned int>(parts) - 1u) {
          page->ag_block_count[b] = 0;
          fence_acq_rel_sys();
          for (int q = 1; q < g.nranks; ++q)
            st_release_sys(&g.pages[(g.rank + q) % g.nranks]->ag_flag[g.rank][b], epoch);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ GEMM CTAs
    init_pipe(p);
    if (threadIdx.x == 0) {
      prefetch_tensormap(&map_local);
      prefetch_tensormap(&map_b);
    }
    if (warp == 1) tmem_alloc(p.tmem_slot, kTmemCols);
    tc_fence_before_sync();
    asm volatile("bar.sync 1, %0;" ::"r"(kGemmThreads) : "memory");
    tc_fence_after_sync();
    const uint32_t tmem_base = *p.tmem_slot;

    const int gemm_ctas = gridDim.x - g.comm_ctas;
    const int cta = blockIdx.x - g.comm_ctas;
    const int tiles_n = g.N / BN;
    const int num_tiles = blocks_per_rank * g.nranks * tiles_n;
    const int k_blocks = g.K / BK;
    const int my_tiles = (num_tiles - cta + gemm_ctas - 1) / gemm_ctas;

    if (warp == 0) {
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = cta; tile < num_tiles && ok; tile += gemm_ctas) {
          int tn, mb;
          ag_decode(tile, tiles_n, blocks_per_rank * g.nranks, g.tuning, tn, mb);
          const int src = g.order[2 * mb], b = g.order[2 * mb + 1];
          const bool local = src == g.rank;
          if (!local) {
            if (!wait_flag_ge(&page->ag_flag[src][b], epoch, p.abort_flag)) {
              gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_FLAG, 0, src * 64 + b);
              ok = false;
              break;
            }
            fence_proxy_async();       // peer stores (generic proxy) before my TMA reads (async proxy)
          }
          const int a_row = local ? b * BM : src * g.rows_per_rank + b * BM;
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(&p.empty_bar[stage], phase ^ 1, p.abort_flag)) {
              gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_EMPTY, 0, stage);
              ok = false;
              break;
            }
            uint8_t* a_dst = p.stage_base + static_cast<size_t>(stage) * kStageBytes;
            mbar_expect_tx(&p.full_bar[stage], kStageBytes);
            if (local) tma_load_2d(a_dst, &map_local, &p.full_bar[stage], kb * BK, a_row);
            else if (parity) tma_load_2d(a_dst, &map_gath1, &p.full_bar[stage], kb * BK, a_row);
            else tma_load_2d(a_dst, &map_gath0, &p.full_bar[stage], kb * BK, a_row);
            tma_load_2d(a_dst + kABytes, &map_b, &p.full_bar[stage], kb * BK, tn * BN);
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
      __nv_bfloat16* d = static_cast<__nv_bfloat16*>(g.d);
      for (int tile = cta; tile < num_tiles; tile += gemm_ctas) {
        int tn, mb;
        ag_decode(tile, tiles_n, blocks_per_rank * g.nranks, g.tuning, tn, mb);
        const int src = g.order[2 * mb], b = g.order[2 * mb + 1];
        bool ok = mbar_wait(&p.acc_full[acc], acc_phase, p.abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_ACC, 2, acc);
          break;
        }
        tc_fence_after_sync();
        const size_t row = static_cast<size_t>(src) * g.rows_per_rank + b * BM + quarter * 32 + lane;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
        if (EPI == 0) {
#pragma unroll 1
          for (int c = 0; c < BN; c += 32) {
            uint32_t r[32];
            tmem_ld32(taddr + c, r);
            tc_wait_ld();
            uint4* out = reinterpret_cast<uint4*>(d + row * g.ldd + tn * BN + c);
#pragma unroll
            for (int v = 0; v < 4; ++v)
              out[v] = make_uint4(pack_bf16(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1])),
                                  pack_bf16(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3])),
                                  pack_bf16(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5])),
                                  pack_bf16(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7])));
          }
        } else {
          constexpr int H = BN / 2;
#pragma unroll 1
          for (int c = 0; c < H; c += 32) {
            uint32_t gt[32], up[32];
            tmem_ld32(taddr + c, gt);
            tmem_ld32(taddr + H + c, up);
            tc_wait_ld();
            uint4* out = reinterpret_cast<uint4*>(d + row * g.ldd + tn * H + c);
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
    asm volatile("bar.sync 1, %0;" ::"r"(kGemmThreads) : "memory");
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc(tmem_base, kTmemCols);
    }
  }
  // the last CTA to finish advances the launch epoch of this rank
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&page->ag_done, 1u) == gridDim.x - 1u) {
      page->ag_done = 0;
      page->ag_epoch = epoch;
    }
  }
}

// ============================================================ GEMM -> reduce-scatter
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmRsArgs g) {
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  FusedPage* page = g.pages[g.rank];
  if (g.error_words != nullptr && *reinterpret_cast<volatile int*>(g.error_words) != 0) return;   // an earlier launch gave up
  const unsigned long long epoch = page->rs_epoch + 1;
  const int parity = static_cast<int>(epoch & 1ull);
  const int blocks_per_rank = g.rows_per_rank / BM;
  const int tiles_n = g.N / BN;
  const int num_tiles = blocks_per_rank * g.nranks * tiles_n;
  const int k_blocks = g.K / BK;
  const int ctas = static_cast<int>(gridDim.x) - g.reduce_ctas;       // CTAs that run the GEMM
  const int cta = blockIdx.x;
  // partial buffer on every rank: [parity][source rank][rows_per_rank][N] bf16
  const size_t slab_bytes = static_cast<size_t>(g.rows_per_rank) * g.N * 2;
  const size_t parity_off = g.partial_off + static_cast<size_t>(parity) * g.nranks * slab_bytes;
  // Every source adds one count per (epilogue warp, tile) it stored: 4 * tiles_n per (source, row block) and
  // launch.  The counters are never reset; rs_base remembers where the previous launch left them.
  const unsigned long long per_block = 4ull * static_cast<unsigned long long>(tiles_n);

  if (cta >= ctas) {
    // ------------------------------------------------------------------ reducer CTAs
    reduce_items(g, page, g.heap_bases[g.rank] + parity_off, slab_bytes, blocks_per_rank, per_block);
  } else {
    // ------------------------------------------------------------------ GEMM CTAs
    const Pipe p = carve_smem<3>(smem_raw);
    const int my_tiles = (num_tiles - cta + ctas - 1) / ctas;
    init_pipe<3>(p);
    if (threadIdx.x == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
    }
    if (warp == 1) tmem_alloc(p.tmem_slot, kTmemCols);
    tc_fence_before_sync();
    asm volatile("bar.sync 1, %0;" ::"r"(kGemmThreads) : "memory");
    tc_fence_after_sync();
    const uint32_t tmem_base = *p.tmem_slot;

    // tile -> (owner, row block of the owner's shard, column tile): row blocks in the order of the table
    auto decode = [&](int tile, int& owner, int& b, int& tn) {
      tn = tile % tiles_n;
      const int rb = tile / tiles_n;
      owner = g.order[2 * rb];
      b = g.order[2 * rb + 1];
    };

    if (warp == 0) {
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = cta; tile < num_tiles && ok; tile += ctas) {
          int owner, b, tn;
          decode(tile, owner, b, tn);
          const int a_row = owner * g.rows_per_rank + b * BM;
          for (int kb = 0; kb < k_blocks; ++kb) {
            if (!mbar_wait(&p.empty_bar[stage], phase ^ 1, p.abort_flag)) {
              gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_EMPTY, 0, stage);
              ok = false;
              break;
            }
            uint8_t* a_dst = p.stage_base + static_cast<size_t>(stage) * kStageBytes;
            mbar_expect_tx(&p.full_bar[stage], kStageBytes);
            tma_load_2d(a_dst, &map_a, &p.full_bar[stage], kb * BK, a_row);
            tma_load_2d(a_dst + kABytes, &map_b, &p.full_bar[stage], kb * BK, tn * BN);
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
      int pend_owner = -1, pend_b = 0;                      // the tile whose stores were issued last
      for (int tile = cta; tile < num_tiles; tile += ctas) {
        int owner, b, tn;
        decode(tile, owner, b, tn);
        bool ok = mbar_wait(&p.acc_full[acc], acc_phase, p.abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_ACC, 2, acc);
          break;
        }
        tc_fence_after_sync();
        // destination: the owner's slab for source = me, local row inside the owner's shard
        char* slab = g.heap_bases[owner] + parity_off + static_cast<size_t>(g.rank) * slab_bytes;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
        uint8_t* stage_warp = p.staging + (warp - 2) * kStagingPerWarp;
        stage_quarter_bf16(taddr, stage_warp, lane, 1.0f);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p.acc_empty[acc]);      // accumulator is free as soon as it sits in shared memory
        // count the previous tile on its owner: its stores were issued a whole tile ago, so the release has nothing
        // left to wait for (a release right behind the stores, let alone a system-scope fence, cost 8-30 us a tile)
        if (pend_owner >= 0 && lane == 0) red_add_release_sys(&g.pages[pend_owner]->rs_count[g.rank][pend_b], 1ull);
        // one row (512 contiguous bytes) per store instruction, 8 rows in flight
        char* dst0 = slab + ((static_cast<size_t>(b) * BM + quarter * 32) * g.N + static_cast<size_t>(tn) * BN) * 2 + lane * 16;
#pragma unroll 1
        for (int r0 = 0; r0 < 32; r0 += 8) {
          uint4 d[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) d[u] = *reinterpret_cast<const uint4*>(stage_warp + (r0 + u) * kStagePitch + lane * 16);
#pragma unroll
          for (int u = 0; u < 8; ++u) *reinterpret_cast<uint4*>(dst0 + static_cast<size_t>(r0 + u) * g.N * 2) = d[u];
        }
        __syncwarp();
        pend_owner = owner;                                  // published while the next tile is staged (or after the loop)
        pend_b = b;
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      // the last tile of this warp
      if (pend_owner >= 0 && lane == 0) red_add_release_sys(&g.pages[pend_owner]->rs_count[g.rank][pend_b], 1ull);
    }
    tc_fence_before_sync();
    asm volatile("bar.sync 1, %0;" ::"r"(kGemmThreads) : "memory");
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc(tmem_base, kTmemCols);
    }
    // the tiles of this CTA are out: help with the reduction
    reduce_items(g, page, g.heap_bases[g.rank] + parity_off, slab_bytes, blocks_per_rank, per_block);
  }

  finish_rs_launch(g, page, blocks_per_rank, per_block, epoch);
}

}  // namespace

cudaError_t launch_ag_gemm(const AgGemmArgs& g, int epilogue, int grid, cudaStream_t stream) {
  if (g.K % BK != 0 || g.N % BN != 0 || g.rows_per_rank % BM != 0 || g.rows_per_rank / BM > kFusedMaxBlocks ||
      g.nranks > kFusedMaxRanks || g.comm_ctas < 1 || grid <= g.comm_ctas || g.order == nullptr)
    return cudaErrorInvalidValue;
  const uint64_t all_rows = static_cast<uint64_t>(g.rows_per_rank) * g.nranks;
  CUtensorMap map_local = make_bf16_kmajor_map(g.x_local, g.rows_per_rank, g.K, g.K, BM);
  const char* gath = g.heap_bases_host[g.rank] + g.gathered_off;
  CUtensorMap map_g0 = make_bf16_kmajor_map(gath, all_rows, g.K, g.K, BM);
  CUtensorMap map_g1 = make_bf16_kmajor_map(gath + g.gathered_bytes, all_rows, g.K, g.K, BM);
  CUtensorMap map_b = make_bf16_kmajor_map(g.b, g.N, g.K, g.ldb, BN);
  auto launch = [&](auto kernel) {
    static bool configured[2] = {false, false};          // the attribute is sticky: set it once per kernel
    cudaError_t e = cudaSuccess;
    if (!configured[epilogue != 0]) {
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes));
      configured[epilogue != 0] = e == cudaSuccess;
    }
    if (e != cudaSuccess) return e;
    kernel<<<grid, kGemmThreads, kSmemBytes, stream>>>(map_local, map_g0, map_g1, map_b, g);
    return cudaGetLastError();
  };
  return epilogue == 0 ? launch(ag_gemm_kernel<0>) : launch(ag_gemm_kernel<1>);
}

cudaError_t launch_gemm_rs(const GemmRsArgs& g, int grid, cudaStream_t stream) {
  if (g.K % BK != 0 || g.N % BN != 0 || g.rows_per_rank % BM != 0 || g.rows_per_rank / BM > kFusedMaxBlocks ||
      g.nranks > kFusedMaxRanks || g.reduce_ctas < 1 || grid <= g.reduce_ctas || g.order == nullptr ||
      g.reduce_order == nullptr)
    return cudaErrorInvalidValue;
  CUtensorMap map_a = make_bf16_kmajor_map(g.a, static_cast<uint64_t>(g.rows_per_rank) * g.nranks, g.K, g.lda, BM);
  CUtensorMap map_b = make_bf16_kmajor_map(g.b, g.N, g.K, g.ldb, BN);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_rs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kSmemBytesStaged));
    if (e != cudaSuccess) return e;
    configured = true;
  }
  gemm_rs_kernel<<<grid, kGemmThreads, kSmemBytesStaged, stream>>>(map_a, map_b, g);
  return cudaGetLastError();
}

}  // namespace sm100
}  // namespace msccl
