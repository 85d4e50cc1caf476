// Host API of the fused MoE kernels (see moe_a2a.cu).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "fused_tp.h"

namespace msccl {
namespace sm100 {

constexpr int kMoeMaxLocalExperts = 16;
constexpr int kMoeMaxExperts = 128;

// Layout of the MoE area inside every rank's symmetric heap (offsets relative to moe_off).
// Peers write everything except `hidden`.
//   counts   [2 parities][nranks sources][num_experts] int32
//   meta     [2][local_experts][cap] int4  (source rank, copy index = token*topk+k, weight bits, 0)
//   dispatch [2][local_experts][cap][hidden] bf16     rows routed to my experts
//   combine  [2][tokens*topk][hidden] bf16            expert outputs for my tokens, already weighted
struct MoeLayout {
  size_t counts_off, meta_off, dispatch_off, combine_off;
  size_t counts_parity, meta_parity, dispatch_parity, combine_parity;   // bytes of one parity
};

struct MoeArgs {
  int rank, nranks, tokens, topk, hidden, ffn, num_experts, local_experts, cap;
  int comm_ctas;
  char* const* heap_bases;                // device array
  char* heap_bases_host[kFusedMaxRanks];
  FusedPage* pages[kFusedMaxRanks];
  size_t moe_off;
  MoeLayout lay;
  // dispatch + first GEMM
  const void* x;                          // [tokens, hidden] bf16
  const int* sorted_copy;                 // [tokens*topk] copy indices ordered by expert
  const int* expert_start;                // [num_experts+1] prefix of my per-expert copy counts
  const float* copy_weight;               // [tokens*topk] gate weight of every copy
  const void* w_gate_up;                  // [local_experts*2*ffn, hidden] bf16, gate/up interleaved per 256 rows
  void* h;                                // [local_experts*cap, ffn] bf16 (local)
  // second GEMM + combine
  const void* w_down;                     // [local_experts*hidden, ffn] bf16
  void* y;                                // [tokens, hidden] bf16
  int* error_words;
};

cudaError_t launch_moe_dispatch_gemm(const MoeArgs& args, int grid, cudaStream_t stream);
cudaError_t launch_moe_gemm_combine(const MoeArgs& args, int grid, cudaStream_t stream);

}  // namespace sm100
}  // namespace msccl
