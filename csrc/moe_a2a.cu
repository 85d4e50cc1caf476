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
#include "pipeline_sm100.cuh"

namespace msccl {
namespace sm100 {

namespace {

struct TileInfo { int expert, m0, tn, rows; };

// Grouped tile enumeration: experts in order, column tiles of an expert, then its row tiles fastest
// (m_tiles[e] = ceil(rows_e / 128)).  The CTAs that run side by side therefore share a handful of
// weight tiles and read the expert's rows - a few MB - from L2: the weights of one expert (235 MB of
// gate and up rows at hidden 4096, ffn 14336) do not fit into L2, and with the column tiles fastest
// every row tile streamed them from DRAM again.  Returns false when `tile` is past the end.
__device__ __forceinline__ bool decode_grouped(int tile, const int* rows_per_expert, int local_experts, int tiles_n,
                                               TileInfo& t) {
  int base = 0;
  for (int e = 0; e < local_experts; ++e) {
    const int mt = (rows_per_expert[e] + BM - 1) / BM;
    const int here = mt * tiles_n;
    if (tile < base + here) {
      const int in_e = tile - base;
      t.expert = e;
      t.m0 = (in_e % mt) * BM;
      t.tn = in_e / mt;
      t.rows = min(BM, rows_per_expert[e] - t.m0);
      return true;
    }
    base += here;
  }
  return false;
}

__device__ __forceinline__ int total_grouped_tiles(const int* rows_per_expert, int local_experts, int tiles_n) {
  int total = 0;
  for (int e = 0; e < local_experts; ++e) total += ((rows_per_expert[e] + BM - 1) / BM) * tiles_n;
  return total;
}

struct MoeShared {
  int rows_per_expert[kMoeMaxLocalExperts];                    // rows of each local expert (all sources)
  int seg_start[kMoeMaxLocalExperts][kFusedMaxRanks + 1];      // per local expert: first row of each source's segment
  int my_offset[kMoeMaxExperts];                               // where my copies start inside every (global) expert
  int ok;
};

// Wait for the count rows of all sources (flag 0) and derive the segment tables.
__device__ bool load_counts(const MoeArgs& g, FusedPage* page, unsigned long long epoch, int parity, MoeShared* sh,
                            volatile int* abort_flag) {
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int s = 0; s < g.nranks && ok; ++s)
      if (!wait_flag_ge(&page->moe_flag[s][0], epoch, abort_flag)) {
        gemm_fail(g.error_words, abort_flag, GEMM_TIMEOUT_FLAG, 4, s);
        ok = 0;
      }
    sh->ok = ok;
  }
  __syncthreads();
  if (sh->ok == 0) return false;
  const int* counts = reinterpret_cast<const int*>(g.heap_bases[g.rank] + g.moe_off + g.lay.counts_off +
                                                   static_cast<size_t>(parity) * g.lay.counts_parity);
  for (int e = threadIdx.x; e < g.num_experts; e += blockDim.x) {
    int before_me = 0, total = 0;
    for (int s = 0; s < g.nranks; ++s) {
      const int c = counts[s * g.num_experts + e];
      if (s < g.rank) before_me += c;
      total += c;
    }
    sh->my_offset[e] = before_me;
    const int first_local = g.rank * g.local_experts;
    if (e >= first_local && e < first_local + g.local_experts) {
      const int le = e - first_local;
      sh->rows_per_expert[le] = total;
      int run = 0;
      for (int s = 0; s < g.nranks; ++s) {
        sh->seg_start[le][s] = run;
        run += counts[s * g.num_experts + e];
      }
      sh->seg_start[le][g.nranks] = run;
      if (total > g.cap) gemm_fail(g.error_words, abort_flag, 5 /* expert over capacity */, 4, e);
    }
  }
  __syncthreads();
  return *abort_flag == 0;
}

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
  const int copies = g.tokens * g.topk;
  const size_t row_bytes = static_cast<size_t>(g.hidden) * 2;

  if (static_cast<int>(blockIdx.x) < g.comm_ctas) {
    // ---------------------------------------------------------------- comm CTAs
    if (blockIdx.x == 0) {
      // all-gather my per-expert counts: row `rank` of every rank's count matrix
      for (int q = 0; q < g.nranks; ++q) {
        int* dst = reinterpret_cast<int*>(g.heap_bases[(g.rank + q) % g.nranks] + g.moe_off + g.lay.counts_off +
                                          static_cast<size_t>(parity) * g.lay.counts_parity) + g.rank * g.num_experts;
        for (int e = threadIdx.x; e < g.num_experts; e += blockDim.x) dst[e] = g.expert_start[e + 1] - g.expert_start[e];
      }
      __syncthreads();
      if (threadIdx.x < g.nranks) {
        __threadfence_system();
        st_release_sys(&g.pages[threadIdx.x]->moe_flag[g.rank][0], epoch);
      }
    }
    if (!load_counts(g, page, epoch, parity, &sh, p.abort_flag)) goto finish;
    {
      // scatter rows: one warp per token copy, copies taken in expert order
      const int warps = g.comm_ctas * (kGemmThreads / 32);
      const int gw = blockIdx.x * (kGemmThreads / 32) + warp;
      for (int i = gw; i < copies; i += warps) {
        const int c = g.sorted_copy[i];
        // expert of position i: binary search in expert_start
        int lo = 0, hi = g.num_experts;
        while (hi - lo > 1) {
          const int mid = (lo + hi) / 2;
          if (g.expert_start[mid] <= i) lo = mid; else hi = mid;
        }
        const int e = lo, dst_rank = e / g.local_experts, le = e % g.local_experts;
        const int row = sh.my_offset[e] + (i - g.expert_start[e]);
        if (row >= g.cap) continue;                               // over capacity: already reported as an error
        char* base = g.heap_bases[dst_rank] + g.moe_off;
        char* dst = base + g.lay.dispatch_off + static_cast<size_t>(parity) * g.lay.dispatch_parity +
                    (static_cast<size_t>(le) * g.cap + row) * row_bytes;
        const char* src = static_cast<const char*>(g.x) + static_cast<size_t>(c / g.topk) * row_bytes;
        const int vecs = static_cast<int>(row_bytes / 16);
        for (int v0 = lane; v0 < vecs; v0 += 32 * 8) {
          uint4 d[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (v0 + u * 32 < vecs) d[u] = *reinterpret_cast<const uint4*>(src + (v0 + u * 32) * 16);
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (v0 + u * 32 < vecs) *reinterpret_cast<uint4*>(dst + (v0 + u * 32) * 16) = d[u];
        }
        if (lane == 0) {
          int4* meta = reinterpret_cast<int4*>(base + g.lay.meta_off + static_cast<size_t>(parity) * g.lay.meta_parity) +
                       static_cast<size_t>(le) * g.cap + row;
          *meta = make_int4(g.rank, c, __float_as_int(g.copy_weight[c]), 0);
        }
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence_system();
        if (atomicAdd(&page->ag_block_count[0], 1u) == static_cast<unsigned int>(g.comm_ctas) - 1u) {
          page->ag_block_count[0] = 0;
          __threadfence_system();
          for (int q = 0; q < g.nranks; ++q) st_release_sys(&g.pages[(g.rank + q) % g.nranks]->moe_flag[g.rank][1], epoch);
        }
      }
    }
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
finish:
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
      __threadfence_system();
      red_add_release_sys(&g.pages[lane]->moe_count[g.rank], 1ull);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }

  // ---------------------------------------------------------------- combine: y[t] = sum over k of combine[t*topk + k]
  const unsigned long long per_launch = 4ull * gridDim.x;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int s = 0; s < g.nranks && ok; ++s)
      if (!wait_flag_ge(&page->moe_count[s], page->moe_base[s] + per_launch, p.abort_flag)) {
        gemm_fail(g.error_words, p.abort_flag, GEMM_TIMEOUT_FLAG, 3, s);
        ok = 0;
      }
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok != 0) {
    const char* comb = g.heap_bases[g.rank] + g.moe_off + g.lay.combine_off + static_cast<size_t>(parity) * g.lay.combine_parity;
    const size_t vec_per_row = row_bytes / 16;
    const size_t total = static_cast<size_t>(g.tokens) * vec_per_row;
    for (size_t v = static_cast<size_t>(cta) * blockDim.x + threadIdx.x; v < total; v += static_cast<size_t>(ctas) * blockDim.x) {
      const size_t tkn = v / vec_per_row, col = v % vec_per_row;
      float a8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int k = 0; k < g.topk; ++k) {
        const uint4 d = *reinterpret_cast<const uint4*>(comb + ((tkn * g.topk + k) * vec_per_row + col) * 16);
        const uint32_t wv[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          a8[2 * e] += __uint_as_float(wv[e] << 16);
          a8[2 * e + 1] += __uint_as_float(wv[e] & 0xffff0000u);
        }
      }
      *reinterpret_cast<uint4*>(static_cast<char*>(g.y) + v * 16) =
          make_uint4(pack_bf16(a8[0], a8[1]), pack_bf16(a8[2], a8[3]), pack_bf16(a8[4], a8[5]), pack_bf16(a8[6], a8[7]));
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&page->moe_done, 1u) == gridDim.x - 1u) {
      for (int s = 0; s < g.nranks; ++s) page->moe_base[s] += per_launch;
      page->moe_done = 0;
      page->moe_pad = 0;
      page->moe_epoch = epoch;
    }
  }
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
