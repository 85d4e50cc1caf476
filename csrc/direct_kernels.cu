// Direct (non-interpreted) all-reduce kernels over symmetric memory for one NVSwitch box.
//
//   one-shot LL  : every rank pushes its message (all-reduce, all-gather) or one block per peer
//                  (reduce-scatter, all-to-all) into a private staging slot on the peer as 16-byte
//                  {data, flag, data, flag} packets; the receiver sums the n slots in rank order or
//                  copies them out.  One NVLink traversal, no barrier, no fence: the latency floor
//                  for small messages.  Input and output may be ordinary device memory.
//   two-shot     : in place on a symmetric buffer.  Rank r owns 1/n of the message: it reduces
//                  that slice across all ranks and publishes the result to all ranks.
//                  NVLS mode does both inside the switch (multimem.ld_reduce + multimem.st on the
//                  multicast window); P2P mode uses plain peer loads and stores, summing in rank
//                  order so that all ranks produce identical bits.
//
//   reduce-scatter: the first half of two-shot; rank r writes the sum of everyone's slice r to an
//                  ordinary local buffer instead of publishing it.
//   push         : all-gather and all-to-all.  Every rank stores its block(s) straight into the
//                  destination buffers of its peers (peer stores, or one multimem.st through the
//                  switch for all-gather), between two barriers: no staging copy on either side.
//
// All waits are bounded; on expiry the kernel writes a status code to the rank's sync page and
// returns.  These are the hand-tuned counterparts of the allreduce_one_shot / allreduce_two_shot
// MSCCLang programs (msccl/programs/allreduce.py), selected by the plan dispatcher by size.
#include <tuple>

#include "msccl_device.h"
#include "prims.cuh"

namespace msccl {

namespace {

constexpr int kDirectThreads = 512;

__device__ __forceinline__ void fail_direct(SyncPage* sync, unsigned int code, int rank, unsigned int aux0, unsigned int aux1) {
  if (atomicCAS(&sync->status[0], 0u, code) == 0u) {
    sync->status[1] = rank;
    sync->status[2] = blockIdx.x;
    sync->status[3] = 0;
    sync->status[4] = 0;
    sync->status[5] = aux0;
    sync->status[6] = aux1;
  }
  __threadfence();
  atomicExch(&sync->abort_flag, 1u);
}

// Barrier across ranks for CTA lane blockIdx.x.  Returns false if it timed out.
__device__ bool rank_barrier(SyncPage* const* syncs, int rank, int nranks, unsigned long long deadline, int* s_fail) {
  SyncPage* me = syncs[rank];
  const int lane = blockIdx.x;
  __syncthreads();
  if (threadIdx.x < nranks) {
    const unsigned long long e = me->cta_epoch[lane] + 1;
    fence_acq_rel_sys();
    st_release_sys(&syncs[threadIdx.x]->cta_barrier[lane][rank], e);
    unsigned int spins = 0;
    while (ld_acquire_sys(&me->cta_barrier[lane][threadIdx.x]) < e) {
      if ((++spins & 127u) == 0 && (global_timer_ns() > deadline || ld_volatile_u32(&me->abort_flag) != 0)) {
        *reinterpret_cast<volatile int*>(s_fail) = 1;
        fail_direct(me, STATUS_TIMEOUT_BARRIER, rank, threadIdx.x, lane);
        break;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) me->cta_epoch[lane] = me->cta_epoch[lane] + 1;
  __syncthreads();
  return *reinterpret_cast<volatile int*>(s_fail) == 0;
}

// ---- multimem wrappers ---------------------------------------------------------------------
template <typename T> struct Multimem;

template <> struct Multimem<float> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ void st(void* p, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
                 ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};
template <> struct Multimem<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ void st(void* p, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1,%2,%3,%4};"
                 ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};
template <> struct Multimem<__half> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ void st(void* p, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1,%2,%3,%4};"
                 ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};

// ---- two-shot, in place on a symmetric buffer ---------------------------------------------
// heap_bases[r] + offset = rank r's buffer as mapped here (P2P mode); mc = the same offset inside
// the multicast window (NVLS mode).
// PIPE (NVLS only): the in-switch loads of the next sweep are issued before the stores of the current one, so
// that reduction and broadcast traffic overlap inside every thread instead of alternating.
template <typename T, bool NVLS, bool PIPE>
__global__ void __launch_bounds__(kDirectThreads, 1)
twoshot_allreduce_kernel(char* const* heap_bases, char* mc, long long offset, long long bytes, int rank, int nranks,
                         SyncPage* const* syncs, unsigned long long timeout_ns, char* rs_out) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  const unsigned long long deadline = global_timer_ns() + timeout_ns;
  if (!rank_barrier(syncs, rank, nranks, deadline, &s_fail)) return;   // every rank's input is in place

  // slice of this rank, then of this CTA, in 16-byte vectors
  const long long vectors = bytes / 16;
  const long long per_rank = (vectors + nranks - 1) / nranks;
  const long long r_begin = min(vectors, per_rank * rank), r_end = min(vectors, r_begin + per_rank);
  const long long per_cta = (r_end - r_begin + gridDim.x - 1) / gridDim.x;
  const long long begin = min(r_end, r_begin + per_cta * blockIdx.x), end = min(r_end, begin + per_cta);

  if (NVLS && PIPE) {
    constexpr int U = 8;
    const long long stride = static_cast<long long>(blockDim.x) * U;
    uint4 cur[U], nxt[U];
    long long v = begin + threadIdx.x;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = v + static_cast<long long>(u) * blockDim.x;
      if (i < end) cur[u] = Multimem<T>::ld_reduce(mc + i * 16);
    }
    for (; v < end; v += stride) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = v + stride + static_cast<long long>(u) * blockDim.x;
        if (i < end) nxt[u] = Multimem<T>::ld_reduce(mc + i * 16);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = v + static_cast<long long>(u) * blockDim.x;
        if (i < end) {
          if (rs_out != nullptr) *reinterpret_cast<uint4*>(rs_out + (i - r_begin) * 16) = cur[u];
          else Multimem<T>::st(mc + i * 16, cur[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) cur[u] = nxt[u];
    }
  } else if (NVLS) {
    constexpr int U = 8;
    for (long long v = begin + threadIdx.x; v < end; v += static_cast<long long>(blockDim.x) * U) {
      uint4 acc[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        long long i = v + static_cast<long long>(u) * blockDim.x;
        if (i < end) acc[u] = Multimem<T>::ld_reduce(mc + i * 16);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        long long i = v + static_cast<long long>(u) * blockDim.x;
        if (i < end) {
          if (rs_out != nullptr) *reinterpret_cast<uint4*>(rs_out + (i - r_begin) * 16) = acc[u];
          else Multimem<T>::st(mc + i * 16, acc[u]);
        }
      }
    }
  } else {
    // peer loads: all n loads of two vectors are issued before the first add, sums in rank order
    constexpr int PU = 2;
    for (long long v = begin + threadIdx.x; v < end; v += static_cast<long long>(blockDim.x) * PU) {
      constexpr int R8 = 8;       // ranks loaded together; a box has at most 8 GPUs, more are summed in a tail loop
      uint4 part[PU][R8];
#pragma unroll
      for (int u = 0; u < PU; ++u) {
        const long long i = v + static_cast<long long>(u) * blockDim.x;
#pragma unroll
        for (int r = 0; r < R8; ++r)
          if (r < nranks && i < end) part[u][r] = *reinterpret_cast<const uint4*>(heap_bases[r] + offset + i * 16);
      }
#pragma unroll
      for (int u = 0; u < PU; ++u) {
        const long long i = v + static_cast<long long>(u) * blockDim.x;
        if (i >= end) break;
        uint4 acc = part[u][0];
#pragma unroll
        for (int r = 1; r < R8; ++r)
          if (r < nranks) acc = Vec16<T>::add(acc, part[u][r]);
        for (int r = R8; r < nranks; ++r)
          acc = Vec16<T>::add(acc, *reinterpret_cast<const uint4*>(heap_bases[r] + offset + i * 16));
        if (rs_out != nullptr) {
          *reinterpret_cast<uint4*>(rs_out + (i - r_begin) * 16) = acc;
        } else {
          for (int r = 0; r < nranks; ++r) *reinterpret_cast<uint4*>(heap_bases[(rank + r) % nranks] + offset + i * 16) = acc;
        }
      }
    }
  }
  rank_barrier(syncs, rank, nranks, deadline, &s_fail);               // every slice has been published (or read)
}

// ---- push: all-gather and all-to-all --------------------------------------------------------
// Block `rank` of the destination buffer of peer p (at `dst_offset` of its heap) receives
//   SAME_SRC (all-gather): the one source block;   otherwise (all-to-all): source block p.
// NVLS (all-gather only): one multimem.st per vector reaches every rank through the switch.
template <bool SAME_SRC, bool NVLS>
__global__ void __launch_bounds__(kDirectThreads, 1)
push_kernel(const char* src, char* const* heap_bases, char* mc, long long dst_offset, long long block_bytes, int rank,
            int nranks, SyncPage* const* syncs, unsigned long long timeout_ns) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  const unsigned long long deadline = global_timer_ns() + timeout_ns;
  if (!rank_barrier(syncs, rank, nranks, deadline, &s_fail)) return;   // every destination may be overwritten

  constexpr int U = 8;
  const long long vectors = block_bytes / 16;
  const long long per_cta = (vectors + gridDim.x - 1) / gridDim.x;
  const long long begin = min(vectors, per_cta * blockIdx.x), end = min(vectors, begin + per_cta);
  const long long nthreads = blockDim.x;
  const long long mine = dst_offset + block_bytes * rank;               // where my block lands in every destination
  for (long long v = begin + threadIdx.x; v < end; v += nthreads * U) {
    uint4 val[U];
    if (SAME_SRC) {
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (v + u * nthreads < end) val[u] = *reinterpret_cast<const uint4*>(src + (v + u * nthreads) * 16);
      if (NVLS) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (v + u * nthreads < end) Multimem<float>::st(mc + mine + (v + u * nthreads) * 16, val[u]);
      } else {
        for (int k = 1; k <= nranks; ++k) {
          char* dst = heap_bases[(rank + k) % nranks] + mine;
          if (dst == src) continue;                                     // in place: my block is already there
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (v + u * nthreads < end) *reinterpret_cast<uint4*>(dst + (v + u * nthreads) * 16) = val[u];
        }
      }
    } else {
      for (int k = 1; k <= nranks; ++k) {
        const int p = (rank + k) % nranks;
        const char* from = src + block_bytes * p;
        char* dst = heap_bases[p] + mine;
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (v + u * nthreads < end) val[u] = *reinterpret_cast<const uint4*>(from + (v + u * nthreads) * 16);
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (v + u * nthreads < end) *reinterpret_cast<uint4*>(dst + (v + u * nthreads) * 16) = val[u];
      }
    }
  }
  rank_barrier(syncs, rank, nranks, deadline, &s_fail);                 // every block has landed
}

// ---- one-shot LL ---------------------------------------------------------------------------
// staging[r] = rank r's staging area as mapped here: [2 parities][nranks senders][slot_bytes],
// slot_bytes >= 2 * block bytes (a packet carries 8 bytes of payload per 16).
// One kernel shape serves four collectives on blocks of `bytes`:
//   PER_PEER false: my one block goes to every rank          (all-reduce, all-gather)
//   PER_PEER true : block p of my input goes to rank p        (reduce-scatter, all-to-all)
//   SUM true      : out[v]       = sum over senders, in rank order   (all-reduce, reduce-scatter)
//   SUM false     : out[s][v]    = what sender s sent                (all-gather, all-to-all)
// No barrier and no fence: the flag travels inside every 16-byte packet.  Input and output may be
// ordinary device memory.
template <typename T, bool PER_PEER, bool SUM>
__global__ void __launch_bounds__(kDirectThreads, 1)
oneshot_ll_kernel(const void* in, void* out, char* const* staging, long long bytes, long long slot_bytes, int rank, int nranks,
                  SyncPage* sync, unsigned long long timeout_ns) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const unsigned long long deadline = global_timer_ns() + timeout_ns;
  const unsigned long long epoch = sync->ll_epoch + 1;       // same value on every rank (all launch in lockstep)
  const unsigned int flag = static_cast<unsigned int>(epoch);
  const long long parity_off = static_cast<long long>(epoch & 1) * nranks * slot_bytes;
  const long long vectors = bytes / 16;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;

  // push: vector v of the block for rank p goes to slot [parity][rank] of p (including myself)
  for (long long v = tid; v < vectors; v += nthreads) {
    if (PER_PEER) {
      for (int r = 0; r < nranks; ++r) {
        const int p = (rank + r) % nranks;
        const uint4 d = *reinterpret_cast<const uint4*>(static_cast<const char*>(in) + (static_cast<long long>(p) * vectors + v) * 16);
        uint4* pk = reinterpret_cast<uint4*>(staging[p] + parity_off + rank * slot_bytes) + 2 * v;
        st_volatile_v4(pk, make_uint4(d.x, flag, d.y, flag));
        st_volatile_v4(pk + 1, make_uint4(d.z, flag, d.w, flag));
      }
    } else {
      const uint4 d = *reinterpret_cast<const uint4*>(static_cast<const char*>(in) + v * 16);
      const uint4 p0 = make_uint4(d.x, flag, d.y, flag), p1 = make_uint4(d.z, flag, d.w, flag);
      for (int r = 0; r < nranks; ++r) {
        uint4* pk = reinterpret_cast<uint4*>(staging[(rank + r) % nranks] + parity_off + rank * slot_bytes) + 2 * v;
        st_volatile_v4(pk, p0);
        st_volatile_v4(pk + 1, p1);
      }
    }
  }
  // pull from the n slots of my own staging area.  All slots of a vector are polled together (the
  // loads overlap); only slots whose flags have not arrived yet are read again.
  const char* mine = staging[rank] + parity_off;
  for (long long v = tid; v < vectors; v += nthreads) {
    constexpr int R8 = 8;
    uint4 a[R8], b[R8];
    unsigned int pending = (nranks >= 32) ? 0xffffffffu : ((1u << nranks) - 1u);
    unsigned int spins = 0;
    while (pending != 0 && nranks <= R8) {
#pragma unroll
      for (int r = 0; r < R8; ++r) {
        if (pending & (1u << r)) {
          const uint4* pk = reinterpret_cast<const uint4*>(mine + r * slot_bytes) + 2 * v;
          a[r] = ld_volatile_v4(pk);
          b[r] = ld_volatile_v4(pk + 1);
        }
      }
#pragma unroll
      for (int r = 0; r < R8; ++r)
        if ((pending & (1u << r)) && a[r].y == flag && a[r].w == flag && b[r].y == flag && b[r].w == flag) pending &= ~(1u << r);
      if (pending != 0 && (++spins & 255u) == 0 && (s_fail != 0 || global_timer_ns() > deadline)) {
        if (atomicExch(&s_fail, 1) == 0) fail_direct(sync, STATUS_TIMEOUT_DATA, rank, __ffs(pending) - 1, 0);
        break;
      }
    }
    uint4 acc = make_uint4(0, 0, 0, 0);
    if (nranks <= R8) {
#pragma unroll
      for (int r = 0; r < R8; ++r) {
        if (r < nranks) {
          const uint4 d = make_uint4(a[r].x, a[r].z, b[r].x, b[r].z);
          if (SUM) acc = (r == 0) ? d : Vec16<T>::add(acc, d);
          else *reinterpret_cast<uint4*>(static_cast<char*>(out) + (static_cast<long long>(r) * vectors + v) * 16) = d;
        }
      }
    } else {
      for (int r = 0; r < nranks; ++r) {       // more than 8 ranks: one slot at a time
        const uint4* pk = reinterpret_cast<const uint4*>(mine + r * slot_bytes) + 2 * v;
        uint4 pa, pb;
        unsigned int sp = 0;
        while (true) {
          pa = ld_volatile_v4(pk);
          pb = ld_volatile_v4(pk + 1);
          if (pa.y == flag && pa.w == flag && pb.y == flag && pb.w == flag) break;
          if ((++sp & 255u) == 0 && (s_fail != 0 || global_timer_ns() > deadline)) {
            if (atomicExch(&s_fail, 1) == 0) fail_direct(sync, STATUS_TIMEOUT_DATA, rank, r, 0);
            break;
          }
        }
        const uint4 d = make_uint4(pa.x, pa.z, pb.x, pb.z);
        if (SUM) acc = (r == 0) ? d : Vec16<T>::add(acc, d);
        else *reinterpret_cast<uint4*>(static_cast<char*>(out) + (static_cast<long long>(r) * vectors + v) * 16) = d;
      }
    }
    if (SUM) *reinterpret_cast<uint4*>(static_cast<char*>(out) + v * 16) = acc;
  }
  // the last CTA to finish advances the epoch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&sync->ll_done, 1u) == gridDim.x - 1u) {
      sync->ll_done = 0;
      sync->ll_epoch = epoch;
    }
  }
}

// The CTAs of these kernels wait on the same-numbered CTA of every other rank (rank_barrier) or on packets any
// CTA of a peer may write, so all CTAs of a launch must be resident together - also when the GPU is shared with a
// GEMM on another stream.  A cooperative launch guarantees that (and fails instead of deadlocking when the grid
// cannot fit).
template <typename... Params, typename... Args>
cudaError_t launch_coresident(void (*kernel)(Params...), int ctas, cudaStream_t stream, Args... args) {
  std::tuple<Params...> values{static_cast<Params>(args)...};
  void* ptrs[sizeof...(Params)];
  std::apply([&](auto&... v) { int i = 0; ((ptrs[i++] = static_cast<void*>(&v)), ...); }, values);
  return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), dim3(ctas), dim3(kDirectThreads), ptrs, 0, stream);
}

template <typename T>
cudaError_t twoshot_typed(char* const* heap_bases, char* mc_base, long long offset, long long bytes, int rank, int nranks,
                          SyncPage* const* syncs, unsigned long long timeout_ns, int ctas, cudaStream_t stream, char* rs_out,
                          bool pipelined) {
  if (mc_base != nullptr && pipelined) {
    return launch_coresident(twoshot_allreduce_kernel<T, true, true>, ctas, stream, heap_bases, mc_base + offset, offset, bytes,
                             rank, nranks, syncs, timeout_ns, rs_out);
  }
  if (mc_base != nullptr) {
    return launch_coresident(twoshot_allreduce_kernel<T, true, false>, ctas, stream, heap_bases, mc_base + offset, offset, bytes,
                             rank, nranks, syncs, timeout_ns, rs_out);
  }
  return launch_coresident(twoshot_allreduce_kernel<T, false, false>, ctas, stream, heap_bases, static_cast<char*>(nullptr), offset,
                           bytes, rank, nranks, syncs, timeout_ns, rs_out);
}

// mode: 0 all-reduce, 1 all-gather, 2 reduce-scatter, 3 all-to-all
template <typename T>
cudaError_t oneshot_typed(const void* in, void* out, char* const* staging, long long bytes, long long slot_bytes, int rank,
                          int nranks, SyncPage* sync, unsigned long long timeout_ns, int ctas, int mode, cudaStream_t stream) {
  switch (mode) {
    case 0: return launch_coresident(oneshot_ll_kernel<T, false, true>, ctas, stream, in, out, staging, bytes, slot_bytes, rank, nranks, sync, timeout_ns);
    case 1: return launch_coresident(oneshot_ll_kernel<T, false, false>, ctas, stream, in, out, staging, bytes, slot_bytes, rank, nranks, sync, timeout_ns);
    case 2: return launch_coresident(oneshot_ll_kernel<T, true, true>, ctas, stream, in, out, staging, bytes, slot_bytes, rank, nranks, sync, timeout_ns);
    case 3: return launch_coresident(oneshot_ll_kernel<T, true, false>, ctas, stream, in, out, staging, bytes, slot_bytes, rank, nranks, sync, timeout_ns);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

cudaError_t launch_twoshot_allreduce(char* const* heap_bases, char* mc_base, long long offset, long long bytes, int dtype,
                                     int rank, int nranks, SyncPage* const* syncs, unsigned long long timeout_ns, int ctas,
                                     cudaStream_t stream, void* rs_out, bool pipelined) {
  if (bytes % 16 != 0 || offset % 16 != 0 || ctas < 1 || ctas > kMaxDirectCtas || nranks > kMaxRanks) return cudaErrorInvalidValue;
  // reduce-scatter: every rank's slice must be the same whole number of vectors
  if (rs_out != nullptr && (bytes % (16ll * nranks) != 0 || reinterpret_cast<uintptr_t>(rs_out) % 16 != 0)) return cudaErrorInvalidValue;
  char* out = static_cast<char*>(rs_out);
  switch (dtype) {
    case DT_F32: return twoshot_typed<float>(heap_bases, mc_base, offset, bytes, rank, nranks, syncs, timeout_ns, ctas, stream, out, pipelined);
    case DT_BF16: return twoshot_typed<__nv_bfloat16>(heap_bases, mc_base, offset, bytes, rank, nranks, syncs, timeout_ns, ctas, stream, out, pipelined);
    case DT_F16: return twoshot_typed<__half>(heap_bases, mc_base, offset, bytes, rank, nranks, syncs, timeout_ns, ctas, stream, out, pipelined);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_push(const void* src, bool same_src, char* const* heap_bases, char* mc_base, long long dst_offset,
                        long long block_bytes, int rank, int nranks, SyncPage* const* syncs, unsigned long long timeout_ns,
                        int ctas, cudaStream_t stream) {
  if (block_bytes % 16 != 0 || dst_offset % 16 != 0 || reinterpret_cast<uintptr_t>(src) % 16 != 0 || ctas < 1 ||
      ctas > kMaxDirectCtas || nranks > kMaxRanks)
    return cudaErrorInvalidValue;
  const char* s = static_cast<const char*>(src);
  char* const no_window = nullptr;
  if (!same_src) return launch_coresident(push_kernel<false, false>, ctas, stream, s, heap_bases, no_window, dst_offset, block_bytes, rank, nranks, syncs, timeout_ns);
  if (mc_base != nullptr) return launch_coresident(push_kernel<true, true>, ctas, stream, s, heap_bases, mc_base, dst_offset, block_bytes, rank, nranks, syncs, timeout_ns);
  return launch_coresident(push_kernel<true, false>, ctas, stream, s, heap_bases, no_window, dst_offset, block_bytes, rank, nranks, syncs, timeout_ns);
}

// One-shot LL collectives on blocks of `bytes` (mode: 0 all-reduce, 1 all-gather, 2 reduce-scatter, 3 all-to-all).
cudaError_t launch_oneshot(const void* in, void* out, char* const* staging, long long bytes, long long slot_bytes, int dtype,
                           int rank, int nranks, SyncPage* sync, unsigned long long timeout_ns, int ctas, int mode,
                           cudaStream_t stream) {
  if (bytes % 16 != 0 || 2 * bytes > slot_bytes || ctas < 1 || nranks > kMaxRanks) return cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(in) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0) return cudaErrorInvalidValue;
  switch (dtype) {
    case DT_F32: return oneshot_typed<float>(in, out, staging, bytes, slot_bytes, rank, nranks, sync, timeout_ns, ctas, mode, stream);
    case DT_BF16: return oneshot_typed<__nv_bfloat16>(in, out, staging, bytes, slot_bytes, rank, nranks, sync, timeout_ns, ctas, mode, stream);
    case DT_F16: return oneshot_typed<__half>(in, out, staging, bytes, slot_bytes, rank, nranks, sync, timeout_ns, ctas, mode, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace msccl
