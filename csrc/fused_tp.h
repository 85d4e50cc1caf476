// Host API and shared structures of the fused tensor-parallel kernels (see fused_tp.cu).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace msccl {
namespace sm100 {

constexpr int kFusedMaxRanks = 8;
constexpr int kFusedMaxBlocks = 64;     // 128-row blocks per rank shard

// One per rank inside its symmetric heap; peers write the flag / counter arrays.
struct alignas(128) FusedPage {
  unsigned long long ag_flag[kFusedMaxRanks][kFusedMaxBlocks];    // [source][block] = launch epoch when the block has landed
  unsigned long long rs_count[kFusedMaxRanks][kFusedMaxBlocks];   // [source][block] += 1 per tile quarter stored
  unsigned long long rs_base[kFusedMaxRanks][kFusedMaxBlocks];    // local: rs_count at the end of the previous launch
  unsigned long long ag_epoch, rs_epoch;                           // local: launches completed
  unsigned int ag_block_count[kFusedMaxBlocks];                    // local: comm CTAs done with a block
  unsigned int ag_done, rs_done;                                   // local: CTAs of the running launch that finished
  unsigned int rs_work, rs_pad;                                    // local: reduction items of the running launch handed out
  // MoE dispatch / combine
  unsigned long long moe_flag[kFusedMaxRanks][4];
  unsigned long long moe_count[kFusedMaxRanks];                    // [source] += 1 per combine row group stored
  unsigned long long moe_base[kFusedMaxRanks];                     // local: moe_count at the end of the previous launch
  unsigned long long moe_epoch;
  unsigned int moe_done, moe_pad;
};

struct AgGemmArgs {
  const void* x_local;            // [rows_per_rank, K] bf16, contiguous
  const void* b;                  // [N, K] bf16
  void* d;                        // [nranks*rows_per_rank, N or N/2] bf16
  int rows_per_rank, N, K, ldb, ldd;
  int rank, nranks, comm_ctas;
  int tuning;                     // bit 0: order tiles row-block-fastest inside a (block, source) wave group
  const int* order;               // device array of nranks * blocks (source rank, block) pairs: the row blocks in the order
                                  // the GEMM tiles consume them, as lowered from the schedule program
  char* const* heap_bases;        // device array: every rank's heap as mapped here
  char* heap_bases_host[kFusedMaxRanks];
  FusedPage* pages[kFusedMaxRanks];
  char* mc_base;                  // multicast window of the heaps (null: peer stores)
  size_t gathered_off;            // offset of the gathered buffer [2][nranks*rows_per_rank, K] in every heap
  size_t gathered_bytes;          // bytes of one parity
  int* error_words;
};

struct GemmRsArgs {
  const void* a;                  // [nranks*rows_per_rank, K] bf16
  const void* b;                  // [N, K] bf16
  void* out;                      // [rows_per_rank, N] bf16: this rank's reduced rows
  int rows_per_rank, N, K, lda, ldb;
  int rank, nranks;
  char* const* heap_bases;
  FusedPage* pages[kFusedMaxRanks];
  size_t partial_off;             // offset of the partial buffer [2][nranks][rows_per_rank, N] in every heap
  int* error_words;
  const int* order;               // device array of nranks * blocks (owner rank, block) pairs: the row blocks in the order
                                  // the GEMM tiles produce them, as lowered from the schedule program
  const int* reduce_order;        // device array of blocks: this rank's row blocks in the order they become complete
  int reduce_ctas;                // CTAs (the last ones of the grid) that only reduce
};

// Block-scaled fp8 (OCP MX) variants: operands are e4m3 bytes plus UE8M0 scale blocks of 512 bytes per
// (128 rows, 128 K) in the arrangement tcgen05.cp wants (msccl.ops.gemm.pack_mx_scales).  Tiles are 128 x 128.
struct AgGemmF8Args {
  const void* x_local;            // [rows_per_rank, K] e4m3, contiguous
  const void* sf_local;           // [rows_per_rank/128][K/128][512] scales of x_local
  const void* b;                  // [N, K] e4m3
  const void* sfb;                // [N/128][K/128][512]
  void* d;                        // [nranks*rows_per_rank, N or N/2] bf16
  int rows_per_rank, N, K, ldb, ldd;
  int rank, nranks, comm_ctas;
  const int* order;               // as in AgGemmArgs
  char* const* heap_bases;
  char* heap_bases_host[kFusedMaxRanks];
  FusedPage* pages[kFusedMaxRanks];
  char* mc_base;
  size_t gathered_off;            // per parity: [nranks*rows_per_rank, K] values, then [nranks*rows_per_rank/128][K/128][512] scales
  size_t gathered_bytes;          // bytes of one parity (values + scales, rounded up to 1024)
  int* error_words;
};

struct GemmRsF8Args {
  const void* a;                  // [nranks*rows_per_rank, K] e4m3
  const void* sfa;                // [nranks*rows_per_rank/128][K/128][512]
  const void* b;                  // [N, K] e4m3
  const void* sfb;                // [N/128][K/128][512]
  void* out;                      // [rows_per_rank, N] bf16: this rank's reduced rows
  int rows_per_rank, N, K, lda, ldb;
  int rank, nranks;
  char* const* heap_bases;
  FusedPage* pages[kFusedMaxRanks];
  size_t partial_off;             // the bf16 partial buffer [2][nranks][rows_per_rank, N], as in GemmRsArgs
  int* error_words;
  const int* order;
  const int* reduce_order;
  int reduce_ctas;
};

cudaError_t launch_ag_gemm(const AgGemmArgs& args, int epilogue, int grid, cudaStream_t stream);
// the block-scaled fp8 kernels on CTA pairs (256 x 256 tiles; fused_tp_fp8_2cta.cu).  With the SwiGLU epilogue the
// weight rows are interleaved per 256 (128 gate rows, 128 up rows) instead of per 128.
cudaError_t launch_ag_gemm_mxfp8_2cta(const AgGemmF8Args& args, int epilogue, int grid, cudaStream_t stream);
cudaError_t launch_gemm_rs_mxfp8_2cta(const GemmRsF8Args& args, int grid, cudaStream_t stream);
// the same two kernels on CTA pairs (cta_group::2, 256 x 256 tiles; fused_tp_2cta.cu)
cudaError_t launch_ag_gemm_2cta(const AgGemmArgs& args, int epilogue, int grid, cudaStream_t stream);
cudaError_t launch_gemm_rs_2cta(const GemmRsArgs& args, int grid, cudaStream_t stream);
cudaError_t launch_ag_gemm_mxfp8(const AgGemmF8Args& args, int epilogue, int grid, cudaStream_t stream);
cudaError_t launch_gemm_rs_mxfp8(const GemmRsF8Args& args, int grid, cudaStream_t stream);
cudaError_t launch_gemm_rs(const GemmRsArgs& args, int grid, cudaStream_t stream);

}  // namespace sm100
}  // namespace msccl
