// Quantisation of bf16 activations to the block-scaled fp8 format of the MX GEMM kernels, in one pass: e4m3 values
// plus one UE8M0 scale per 32 consecutive K elements of a row, the scales written straight into the 512-byte blocks
// per (128 rows, 128 K) that tcgen05.cp consumes (byte (r % 32) * 16 + (r / 32) * 4 + j of a block = scale of row r
// for K elements [32 j, 32 j + 32)).  One thread owns one group of 32 elements: 64 bytes in, 32 bytes + 1 byte out.
// The scale is the smallest power of two that brings the group's largest magnitude inside the e4m3 range (448).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace msccl {
namespace sm100 {

namespace {

__global__ void __launch_bounds__(256) quantize_mx_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                                          uint8_t* __restrict__ sf, int rows, int K, long long ldx) {
  const int groups_per_row = K / 32;
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= static_cast<long long>(rows) * groups_per_row) return;
  const int row = static_cast<int>(t / groups_per_row), grp = static_cast<int>(t % groups_per_row);
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(row) * ldx + grp * 32);
  uint4 raw[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) raw[i] = src[i];
  float v[32];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      v[8 * i + 2 * e] = __uint_as_float(w[e] << 16);
      v[8 * i + 2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
    }
  }
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = fmaxf(amax, 1.0e-36f);
  // smallest e with amax / 2^e <= 448
  const float ratio = amax / 448.0f;
  int e = ilogbf(ratio);
  if (ldexpf(1.0f, e) < ratio) ++e;
  e = max(-127, min(127, e));
  const float inv = ldexpf(1.0f, -e);
  uint32_t packed[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i] * inv, v[4 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i + 2] * inv, v[4 * i + 3] * inv), __NV_SATFINITE, __NV_E4M3);
    packed[i] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
  }
  uint4* dst = reinterpret_cast<uint4*>(q + static_cast<long long>(row) * K + grp * 32);
  dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
  const int k_blocks = K / 128;
  const int tile = row / 128, r = row % 128, kb = grp / 4, j = grp % 4;
  sf[(static_cast<long long>(tile) * k_blocks + kb) * 512 + (r % 32) * 16 + (r / 32) * 4 + j] = static_cast<uint8_t>(e + 127);
}

}  // namespace

// x: [rows, K] bf16 with row pitch ldx (elements); q: [rows, K] e4m3 contiguous; sf: ceil(rows / 128) * (K / 128)
// blocks of 512 bytes (rows beyond `rows` inside the last block are not written).  K % 128 == 0, 16-byte aligned rows.
cudaError_t quantize_mxfp8(const void* x, void* q, void* sf, int rows, int K, long long ldx, cudaStream_t stream) {
  if (rows <= 0 || K <= 0 || K % 128 != 0 || ldx % 8 != 0 || reinterpret_cast<uintptr_t>(x) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(q) % 16 != 0)
    return cudaErrorInvalidValue;
  const long long threads = static_cast<long long>(rows) * (K / 32);
  const int grid = static_cast<int>((threads + 255) / 256);
  quantize_mx_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q),
                                              static_cast<uint8_t*>(sf), rows, K, ldx);
  return cudaGetLastError();
}

}  // namespace sm100
}  // namespace msccl
