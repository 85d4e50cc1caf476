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
// The same two kernels on CTA pairs (moe_a2a_2cta.cu): comm_ctas must be even; grid 0 = all resident pairs.
cudaError_t launch_moe_dispatch_gemm_2cta(const MoeArgs& args, int grid, cudaStream_t stream);
cudaError_t launch_moe_gemm_combine_2cta(const MoeArgs& args, int grid, cudaStream_t stream);

// Routing on the device (moe_route.cu).  launch_moe_topk: logits [tokens, experts] fp32 -> the k largest experts of
// every token (int32, descending) and their renormalised softmax weights.  launch_moe_sort: stable counting sort of
// the n = tokens * k copies by expert -> sorted_copy [n] and expert_start [experts + 1].
cudaError_t launch_moe_topk(const float* logits, int tokens, int experts, int k, int* out_experts, float* out_weights,
                            cudaStream_t stream);
cudaError_t launch_moe_sort(const int* expert_of, int n, int experts, int* sorted_copy, int* expert_start, cudaStream_t stream);

}  // namespace sm100
}  // namespace msccl
