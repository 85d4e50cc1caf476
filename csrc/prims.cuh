// Device primitives shared by the executor kernels: scoped loads/stores, bounded waits, and
// 16-byte vector arithmetic for fp32 / bf16 / fp16 sums (low-precision sums are formed in fp32
// and rounded once per addition, matching the CPU reference interpreter bit for bit).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "msccl_device.h"

namespace msccl {

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// Release / acquire fence at system scope.  __threadfence_system() is the sequentially consistent fence (fence.sc.sys),
// which costs several microseconds behind stores to a peer; the flag protocols here only need the ordering of a
// release (the data before the flag) or an acquire (the flag before the data), which is what this fence gives.
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_gpu(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_gpu(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_volatile_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_v4(uint4* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---- 16-byte vector sums ---------------------------------------------------------------
template <typename T> struct Vec16;

template <> struct Vec16<float> {
  static __device__ __forceinline__ uint4 add(uint4 a, uint4 b) {
    uint4 r;
    r.x = __float_as_uint(__uint_as_float(a.x) + __uint_as_float(b.x));
    r.y = __float_as_uint(__uint_as_float(a.y) + __uint_as_float(b.y));
    r.z = __float_as_uint(__uint_as_float(a.z) + __uint_as_float(b.z));
    r.w = __float_as_uint(__uint_as_float(a.w) + __uint_as_float(b.w));
    return r;
  }
};

__device__ __forceinline__ unsigned int add_bf16x2(unsigned int a, unsigned int b) {
  // bf16 -> fp32 is a 16-bit shift; the sum is rounded to nearest-even once
  float lo = __uint_as_float(a << 16) + __uint_as_float(b << 16);
  float hi = __uint_as_float(a & 0xffff0000u) + __uint_as_float(b & 0xffff0000u);
  __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned int*>(&r);
}
template <> struct Vec16<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 add(uint4 a, uint4 b) {
    return make_uint4(add_bf16x2(a.x, b.x), add_bf16x2(a.y, b.y), add_bf16x2(a.z, b.z), add_bf16x2(a.w, b.w));
  }
};

__device__ __forceinline__ unsigned int add_f16x2(unsigned int a, unsigned int b) {
  float2 fa = __half22float2(*reinterpret_cast<__half2*>(&a));
  float2 fb = __half22float2(*reinterpret_cast<__half2*>(&b));
  __half2 r = __floats2half2_rn(fa.x + fb.x, fa.y + fb.y);
  return *reinterpret_cast<unsigned int*>(&r);
}
template <> struct Vec16<__half> {
  static __device__ __forceinline__ uint4 add(uint4 a, uint4 b) {
    return make_uint4(add_f16x2(a.x, b.x), add_f16x2(a.y, b.y), add_f16x2(a.z, b.z), add_f16x2(a.w, b.w));
  }
};


// ---- element-wide accesses -----------------------------------------------------------------
// Buffers whose chunks are not multiples of 16 bytes are moved one element per access: Wide<T, sizeof(T)>.
// Wide<T, 16> is the 16-byte vector path.
template <typename T, int W> struct Wide;

template <typename T> struct Wide<T, 16> {
  using V = uint4;
  static __device__ __forceinline__ V add(V a, V b) { return Vec16<T>::add(a, b); }
};
template <> struct Wide<float, 4> {
  using V = unsigned int;
  static __device__ __forceinline__ V add(V a, V b) { return __float_as_uint(__uint_as_float(a) + __uint_as_float(b)); }
};
template <> struct Wide<__nv_bfloat16, 2> {
  using V = unsigned short;
  static __device__ __forceinline__ V add(V a, V b) {
    const float s = __uint_as_float(static_cast<unsigned int>(a) << 16) + __uint_as_float(static_cast<unsigned int>(b) << 16);
    return __bfloat16_as_ushort(__float2bfloat16_rn(s));
  }
};
template <> struct Wide<__half, 2> {
  using V = unsigned short;
  static __device__ __forceinline__ V add(V a, V b) {
    return __half_as_ushort(__float2half_rn(__half2float(__ushort_as_half(a)) + __half2float(__ushort_as_half(b))));
  }
};

__device__ __forceinline__ uint2 ld_volatile_v2(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_v2(uint2* p, uint2 v) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

}  // namespace msccl
