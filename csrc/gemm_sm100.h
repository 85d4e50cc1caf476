// Host API of the tcgen05 GEMM (see gemm_sm100.cu).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace msccl {
namespace sm100 {

CUtensorMap make_bf16_kmajor_map(const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);
CUtensorMap make_u8_kmajor_map(const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);
CUtensorMap make_block512_map(const void* base, uint64_t blocks);
int sm_count();
// bf16 [rows, K] -> e4m3 values + packed UE8M0 scale blocks (quantize_mx.cu)
cudaError_t quantize_mxfp8(const void* x, void* q, void* sf, int rows, int K, long long ldx, cudaStream_t stream);
// epilogue: 0 = plain bf16 store, 1 = SwiGLU over (gate | up) column halves of each tile.
cudaError_t gemm_bf16(const void* a, const void* b, void* d, int M, int N, int K, int lda, int ldb, int ldd, int epilogue,
                      int bn, int* error_words, int max_ctas, cudaStream_t stream);

// Two-CTA (cta_group::2) variant with 256 x 256 tiles per CTA pair, see gemm_2cta_sm100.cu.  N % 256 == 0.
cudaError_t gemm_bf16_2cta(const void* a, const void* b, void* d, int M, int N, int K, int lda, int ldb, int ldd, int epilogue,
                           int* error_words, int max_pairs, cudaStream_t stream);
int max_cta_pairs(int epilogue);
// Block-scaled fp8 (e4m3 with one UE8M0 scale per 32 K elements), see gemm_mxfp8_sm100.cu.
cudaError_t gemm_mxfp8(const void* a, const void* sfa, const void* b, const void* sfb, void* d, int M, int N, int K, int lda,
                       int ldb, int ldd, int* error_words, int max_ctas, cudaStream_t stream);
// The same on CTA pairs with 256 x 256 tiles (gemm_mxfp8_2cta_sm100.cu).  N % 256 == 0; sfa must hold an even
// number of 128-row blocks (2 * ceil(M / 256)).
cudaError_t gemm_mxfp8_2cta(const void* a, const void* sfa, const void* b, const void* sfb, void* d, int M, int N, int K, int lda,
                            int ldb, int ldd, int* error_words, int max_pairs, cudaStream_t stream);

}  // namespace sm100
}  // namespace msccl
