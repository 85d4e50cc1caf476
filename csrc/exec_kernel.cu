// MSCCL-IR interpreter kernel for sm_100a: one CTA per <tb>, steps executed in order, data moved
// with peer stores over NVLink.
//
// Protocols
//   Simple : the sender writes a tile, fences, then publishes the tile count with a release store; the
//            receiver acquires the count before reading.  The tile goes into a FIFO slot of the receiving
//            GPU, or - when the matching receive is `r` / `rcs` and the receiver's buffer is mapped here -
//            straight into the receiver's destination slot (no second copy on the receiving side).
//   LL     : every 8 bytes of data travel with a 32-bit flag (the tile sequence number of this launch), so no
//            separate fence/flag round trip is needed; half of the bytes moved are payload.
//   LL128  : 128-byte lines of 120 bytes of data and one 64-bit flag, stored four lines at a time by one
//            warp-wide instruction; a line becomes visible as a whole, so the flag in its last 8 bytes
//            vouches for the other 120.
// FIFO traffic is flow controlled by a credit counter the receiver writes back into the sender's memory;
// stores into a receiver's buffer wait for the receiver to open the slot (a counter as well).  Every wait is
// bounded: when the deadline passes the CTA records what it was waiting for in the rank's status words,
// raises the rank's abort flag and returns.
//
// Thread 0 of a CTA does the waiting: it polls the flags its step needs and hands its verdict to the other
// warps; after the data movement one barrier separates it from the signals thread 0 sends - one system-scope
// fence per step, the flags themselves relaxed stores behind it.
//
// Large buffers are processed in iterations: iteration k handles elements [k*tile, (k+1)*tile) of every
// chunk, so one program serves any message size.  Chunks that are not multiples of 16 bytes run on
// element-wide accesses (template parameter W).
//
// Every step's slots are checked against the buffer sizes the host declared before anything is touched; a
// step outside them stops the rank with STATUS_BOUNDS.
#include <cstdio>
#include <type_traits>

#include "msccl_device.h"
#include "prims.cuh"

namespace msccl {

namespace {

constexpr int kUnroll = 8;        // accesses per thread in flight (copies are latency bound)
constexpr int kSmemSteps = 192;   // steps of a threadblock kept in shared memory
constexpr unsigned int kFullWarp = 0xffffffffu;

__device__ __forceinline__ unsigned long long pack_progress(unsigned long long epoch, int iter, int step_plus_1) {
  // 32 bits of launch epoch | 20 bits of iteration | 12 bits of step+1 (the host rejects plans beyond these)
  return (epoch << 32) | (static_cast<unsigned long long>(iter & 0xfffff) << 12) |
         static_cast<unsigned long long>(step_plus_1 & 0xfff);
}

struct Waiter {
  SyncPage* sync;
  unsigned long long deadline;

  // Spin until *flag >= want.  Returns false on timeout or when the rank was aborted.
  __device__ bool until_ge(const unsigned long long* flag, unsigned long long want, bool system_scope) const {
    unsigned int spins = 0;
    while (true) {
      unsigned long long v = system_scope ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
      if (v >= want) return true;
      if ((++spins & 127u) == 0) {
        if (ld_volatile_u32(&sync->abort_flag) != 0) return false;
        if (global_timer_ns() > deadline) return false;
      }
    }
  }
  // The same for a counter that keeps other information above kTailModeShift; the whole word is returned.
  __device__ bool until_count_ge(const unsigned long long* flag, unsigned long long want, unsigned long long* word) const {
    unsigned int spins = 0;
    while (true) {
      const unsigned long long v = ld_acquire_sys(flag);
      if ((v & kTailCountMask) >= want) { *word = v; return true; }
      if ((++spins & 127u) == 0) {
        if (ld_volatile_u32(&sync->abort_flag) != 0) return false;
        if (global_timer_ns() > deadline) return false;
      }
    }
  }
  __device__ bool expired() const {
    return ld_volatile_u32(&sync->abort_flag) != 0 || global_timer_ns() > deadline;
  }
};

__device__ void record_failure(SyncPage* sync, unsigned int code, int rank, int tb, int step, int iter,
                               unsigned int aux0, unsigned int aux1) {
  unsigned int already = ld_volatile_u32(&sync->abort_flag);
  if (already != 0 && code != STATUS_ABORTED && code != STATUS_BOUNDS) code = STATUS_ABORTED;
  if (atomicCAS(&sync->status[0], 0u, code) == 0u) {
    sync->status[1] = rank;
    sync->status[2] = tb;
    sync->status[3] = step;
    sync->status[4] = iter;
    sync->status[5] = aux0;
    sync->status[6] = aux1;
  }
  __threadfence();
  atomicExch(&sync->abort_flag, 1u);
}

template <int W> struct Access;
template <> struct Access<16> {
  static __device__ __forceinline__ uint4 ld(const char* p) { return *reinterpret_cast<const uint4*>(p); }
  static __device__ __forceinline__ void st(char* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }
};
template <> struct Access<4> {
  static __device__ __forceinline__ unsigned int ld(const char* p) { return *reinterpret_cast<const unsigned int*>(p); }
  static __device__ __forceinline__ void st(char* p, unsigned int v) { *reinterpret_cast<unsigned int*>(p) = v; }
};
template <> struct Access<2> {
  static __device__ __forceinline__ unsigned short ld(const char* p) { return *reinterpret_cast<const unsigned short*>(p); }
  static __device__ __forceinline__ void st(char* p, unsigned short v) { *reinterpret_cast<unsigned short*>(p) = v; }
};

// ---- plain memory (local buffers, Simple FIFO slots, a peer's buffer) ------------------------
//   value = in0[v];  if (add1) value = value + add1[v];  if (out0) out0[v] = value;  if (out1) out1[v] = value
template <typename T, int W>
__device__ __noinline__ void move_plain(const char* in0, const char* add1, char* out0, char* out1, long long n) {
  using VT = typename Wide<T, W>::V;
  const long long nthreads = blockDim.x;
  const long long stride = nthreads * kUnroll;
  for (long long base = threadIdx.x; base < n; base += stride) {
    if (base + (kUnroll - 1) * nthreads < n) {
      // full group: all loads are issued before the first use, with no per-access predicate
      VT val[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) val[u] = Access<W>::ld(in0 + (base + u * nthreads) * W);
      if (add1 != nullptr) {
        VT other[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) other[u] = Access<W>::ld(add1 + (base + u * nthreads) * W);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) val[u] = Wide<T, W>::add(val[u], other[u]);
      }
      if (out0 != nullptr) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) Access<W>::st(out0 + (base + u * nthreads) * W, val[u]);
      }
      if (out1 != nullptr) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) Access<W>::st(out1 + (base + u * nthreads) * W, val[u]);
      }
    } else {
      for (long long v = base; v < n; v += nthreads) {
        VT r = Access<W>::ld(in0 + v * W);
        if (add1 != nullptr) r = Wide<T, W>::add(r, Access<W>::ld(add1 + v * W));
        if (out0 != nullptr) Access<W>::st(out0 + v * W, r);
        if (out1 != nullptr) Access<W>::st(out1 + v * W, r);
      }
    }
  }
}

// dst[v] = ((dst[v] + src_0[v]) + src_1[v]) + ... : k local reduces into one slot as one pass over it.  Every
// partial sum is rounded to T, exactly as k separate passes would.
template <typename T, int W>
__device__ __noinline__ void move_batch(char* dst, const char* const* srcs, int nsrc, long long n) {
  using VT = typename Wide<T, W>::V;
  const long long nthreads = blockDim.x;
  constexpr int U = 4;
  for (long long base = threadIdx.x; base < n; base += nthreads * U) {
    VT val[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (base + u * nthreads < n) val[u] = Access<W>::ld(dst + (base + u * nthreads) * W);
    for (int k = 0; k < nsrc; ++k) {
      const char* s = srcs[k];
      VT other[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (base + u * nthreads < n) other[u] = Access<W>::ld(s + (base + u * nthreads) * W);
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (base + u * nthreads < n) val[u] = Wide<T, W>::add(val[u], other[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (base + u * nthreads < n) Access<W>::st(dst + (base + u * nthreads) * W, val[u]);
  }
}

// ---- LL packets -----------------------------------------------------------------------------
// W = 16: two 16-byte packets {data, flag, data, flag} per vector.  W = 4 / 2: one 8-byte packet {data, flag}.
template <int W> struct LLPacket;

template <> struct LLPacket<16> {
  static constexpr int kBytes = 32;
  static __device__ __forceinline__ uint4 load(const char* slot, long long v, unsigned int flag, const Waiter& w, int* fail) {
    const uint4* pk = reinterpret_cast<const uint4*>(slot) + 2 * v;
    uint4 a, b;
    unsigned int spins = 0;
    while (true) {
      a = ld_volatile_v4(pk);
      b = ld_volatile_v4(pk + 1);
      if (a.y == flag && a.w == flag && b.y == flag && b.w == flag) break;
      if ((++spins & 255u) == 0) {
        if (*reinterpret_cast<volatile int*>(fail) != 0 || w.expired()) {
          *reinterpret_cast<volatile int*>(fail) = 1;
          break;
        }
      }
    }
    return make_uint4(a.x, a.z, b.x, b.z);
  }
  static __device__ __forceinline__ void store(char* slot, long long v, uint4 d, unsigned int flag) {
    uint4* pk = reinterpret_cast<uint4*>(slot) + 2 * v;
    st_volatile_v4(pk, make_uint4(d.x, flag, d.y, flag));
    st_volatile_v4(pk + 1, make_uint4(d.z, flag, d.w, flag));
  }
};

template <int W> struct LLPacketNarrow {
  static constexpr int kBytes = 8;
  using VT = typename std::conditional<W == 4, unsigned int, unsigned short>::type;
  static __device__ __forceinline__ VT load(const char* slot, long long v, unsigned int flag, const Waiter& w, int* fail) {
    const uint2* pk = reinterpret_cast<const uint2*>(slot) + v;
    uint2 a;
    unsigned int spins = 0;
    while (true) {
      a = ld_volatile_v2(pk);
      if (a.y == flag) break;
      if ((++spins & 255u) == 0) {
        if (*reinterpret_cast<volatile int*>(fail) != 0 || w.expired()) {
          *reinterpret_cast<volatile int*>(fail) = 1;
          break;
        }
      }
    }
    return static_cast<VT>(a.x);
  }
  static __device__ __forceinline__ void store(char* slot, long long v, VT d, unsigned int flag) {
    st_volatile_v2(reinterpret_cast<uint2*>(slot) + v, make_uint2(static_cast<unsigned int>(d), flag));
  }
};
template <> struct LLPacket<4> : LLPacketNarrow<4> {};
template <> struct LLPacket<2> : LLPacketNarrow<2> {};

//   value = FIFO_IN ? fifo_in[v] : in0[v];  if (add1) value = value + add1[v];
//   if (out0) out0[v] = value;              if (FIFO_OUT) fifo_out[v] = value
template <typename T, int W, bool FIFO_IN, bool FIFO_OUT>
__device__ __noinline__ void move_ll(const char* in0, const char* add1, char* out0, const char* fifo_in, char* fifo_out,
                                      long long fifo_base_v, long long n, unsigned int flag_in, unsigned int flag_out,
                                      const Waiter& w, int* fail) {
  using VT = typename Wide<T, W>::V;
  const long long nthreads = blockDim.x;
  const long long stride = nthreads * kUnroll;
  for (long long base = threadIdx.x; base < n; base += stride) {
    if (base + (kUnroll - 1) * nthreads < n) {
      VT val[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long long v = base + u * nthreads;
        if (FIFO_IN) val[u] = LLPacket<W>::load(fifo_in, fifo_base_v + v, flag_in, w, fail);
        else val[u] = Access<W>::ld(in0 + v * W);
      }
      if (add1 != nullptr) {
        VT other[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) other[u] = Access<W>::ld(add1 + (base + u * nthreads) * W);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) val[u] = Wide<T, W>::add(val[u], other[u]);
      }
      if (out0 != nullptr) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) Access<W>::st(out0 + (base + u * nthreads) * W, val[u]);
      }
      if (FIFO_OUT) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) LLPacket<W>::store(fifo_out, fifo_base_v + base + u * nthreads, val[u], flag_out);
      }
    } else {
      for (long long v = base; v < n; v += nthreads) {
        VT r = FIFO_IN ? LLPacket<W>::load(fifo_in, fifo_base_v + v, flag_in, w, fail) : Access<W>::ld(in0 + v * W);
        if (add1 != nullptr) r = Wide<T, W>::add(r, Access<W>::ld(add1 + v * W));
        if (out0 != nullptr) Access<W>::st(out0 + v * W, r);
        if (FIFO_OUT) LLPacket<W>::store(fifo_out, fifo_base_v + v, r, flag_out);
      }
    }
  }
}

// ---- LL128 lines ----------------------------------------------------------------------------
// The payload is counted in 8-byte units; line L carries units [15 L, 15 L + 15).  Lane k of the eight lanes
// that own a line holds units 15 L + 2k and 15 L + 2k + 1; lane 7 holds unit 15 L + 14 and the flag.  The 32
// lanes of a warp store 4 consecutive lines with one 16-byte-per-lane instruction.
__device__ __forceinline__ uint4 ld_units(const char* base, long long u0, long long n8, int k) {
  uint4 r = make_uint4(0, 0, 0, 0);
  if (u0 < n8) {
    const uint2 a = *reinterpret_cast<const uint2*>(base + u0 * 8);
    r.x = a.x; r.y = a.y;
  }
  if (k < 7 && u0 + 1 < n8) {
    const uint2 b = *reinterpret_cast<const uint2*>(base + (u0 + 1) * 8);
    r.z = b.x; r.w = b.y;
  }
  return r;
}
__device__ __forceinline__ void st_units(char* base, long long u0, long long n8, int k, uint4 v) {
  if (u0 < n8) *reinterpret_cast<uint2*>(base + u0 * 8) = make_uint2(v.x, v.y);
  if (k < 7 && u0 + 1 < n8) *reinterpret_cast<uint2*>(base + (u0 + 1) * 8) = make_uint2(v.z, v.w);
}

template <typename T, bool FIFO_IN, bool FIFO_OUT>
__device__ __noinline__ void move_ll128(const char* in0, const char* add1, char* out0, const char* fifo_in, char* fifo_out,
                                         long long line_base, long long n8, unsigned long long flag_in,
                                         unsigned long long flag_out, const Waiter& w, int* fail) {
  const int k = threadIdx.x & 7;
  const long long g = threadIdx.x >> 3, groups = blockDim.x >> 3;
  const long long lines = (n8 + 14) / 15;
  const long long rounds = (lines + groups - 1) / groups;      // the same for every thread of the CTA
  const unsigned int in_lo = static_cast<unsigned int>(flag_in), in_hi = static_cast<unsigned int>(flag_in >> 32);
  constexpr int U = 4;
  for (long long r0 = 0; r0 < rounds; r0 += U) {
    uint4 val[U];
    bool act[U];
#pragma unroll
    for (int u = 0; u < U; ++u) act[u] = (r0 + u < rounds) && ((r0 + u) * groups + g < lines);
    if (FIFO_IN) {
      unsigned int pending = 0;                                   // warp-uniform: rounds still to be seen complete
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (r0 + u < rounds) pending |= 1u << u;
      unsigned int spins = 0;
      while (pending != 0) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (((pending >> u) & 1u) && act[u])
            val[u] = ld_volatile_v4(reinterpret_cast<const uint4*>(fifo_in + (line_base + (r0 + u) * groups + g) * 128 + k * 16));
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if ((pending >> u) & 1u) {
            const bool ok = !act[u] || k != 7 || (val[u].z == in_lo && val[u].w == in_hi);
            if (__all_sync(kFullWarp, ok)) pending &= ~(1u << u);
          }
        }
        if (pending != 0 && (++spins & 63u) == 0) {
          const bool give_up = (threadIdx.x & 31) == 0 && (*reinterpret_cast<volatile int*>(fail) != 0 || w.expired());
          if (__any_sync(kFullWarp, give_up)) {
            *reinterpret_cast<volatile int*>(fail) = 1;
            break;
          }
        }
      }
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (act[u]) val[u] = ld_units(in0, ((r0 + u) * groups + g) * 15 + 2 * k, n8, k);
    }
    if (add1 != nullptr) {
      uint4 other[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (act[u]) other[u] = ld_units(add1, ((r0 + u) * groups + g) * 15 + 2 * k, n8, k);
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (act[u]) val[u] = Vec16<T>::add(val[u], other[u]);
    }
    if (out0 != nullptr) {
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (act[u]) st_units(out0, ((r0 + u) * groups + g) * 15 + 2 * k, n8, k, val[u]);
    }
    if (FIFO_OUT) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (act[u]) {
          uint4 v = val[u];
          if (k == 7) {
            v.z = static_cast<unsigned int>(flag_out);
            v.w = static_cast<unsigned int>(flag_out >> 32);
          }
          st_volatile_v4(reinterpret_cast<uint4*>(fifo_out + (line_base + (r0 + u) * groups + g) * 128 + k * 16), v);
        }
      }
    }
  }
}

__device__ __forceinline__ bool is_send(int t) { return t == ST_SEND || t == ST_RCS || t == ST_RRS || t == ST_RRCS; }
__device__ __forceinline__ bool is_recv(int t) {
  return t == ST_RECV || t == ST_RCS || t == ST_RRS || t == ST_RRC || t == ST_RRCS;
}

template <typename T, int PROTO, int W>
__global__ void __launch_bounds__(kExecThreads, 1) exec_kernel(ExecArgs a) {
  __shared__ int s_fail;
  __shared__ unsigned long long s_decision;        // (pass << 3) | failed | data in place | store in place: thread 0's verdict
  __shared__ __align__(16) DevStep s_steps[kSmemSteps];      // filled with 16-byte copies
  const DevTb& tb = a.tbs[a.first_tb + blockIdx.x];
  const RankCtx& me = a.ranks[tb.rank];
  SyncPage* const sync = me.sync;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int my_rank = tb.rank, my_tb = tb.tb_in_rank, nsteps = tb.nsteps, step_begin = tb.step_begin;
  const int send_conn = tb.send_conn, recv_conn = tb.recv_conn;
  const int send_peer_id = tb.send_peer, recv_peer_id = tb.recv_peer, chan = tb.chan;
  const bool from_args = a.bufs_from_args != 0;
  char* bufs[3];
  long long elems[3];
#pragma unroll
  for (int b = 0; b < 3; ++b) {
    bufs[b] = static_cast<char*>(from_args ? a.local_buf[b] : me.buf[b]);
    elems[b] = from_args ? a.local_elems[b] : me.buf_elems[b];
  }

  // the steps of this threadblock: shared memory when they fit
  const DevStep* sp = a.steps + step_begin;
  if (nsteps <= kSmemSteps) {
    const uint4* g = reinterpret_cast<const uint4*>(sp);
    uint4* s = reinterpret_cast<uint4*>(s_steps);
    for (int i = tid; i < nsteps * 2; i += blockDim.x) s[i] = g[i];
    sp = s_steps;
  }

  // launch epoch: read by every CTA of this rank, advanced by the last one to finish
  const unsigned long long epoch = a.epoch_base + sync->exec_epoch + 1;
  Waiter w;
  w.sync = sync;
  w.deadline = global_timer_ns() + a.timeout_ns;
  if (tid == 0) { s_fail = 0; s_decision = 0; }

  const bool has_send = send_peer_id >= 0;
  const bool has_recv = recv_peer_id >= 0;
  const int remote_idx = chan * kMaxRanks + my_rank;       // this rank's slot in a peer's flag arrays
  // addresses on the peers (NVLink-mapped in multi-process mode)
  char* const send_fifo = has_send ? a.ranks[send_peer_id].fifo + tb.send_fifo_off : nullptr;
  unsigned long long* const send_tail = has_send ? &a.ranks[send_peer_id].sync->recv_tail[remote_idx] : nullptr;
  unsigned long long* const recv_credit = has_recv ? &a.ranks[recv_peer_id].sync->send_head[remote_idx] : nullptr;
  unsigned long long* const recv_open = has_recv ? &a.ranks[recv_peer_id].sync->recv_posted[remote_idx] : nullptr;
  const char* const recv_fifo = has_recv ? me.fifo + tb.recv_fifo_off : nullptr;
  unsigned long long sseq = has_send ? sync->send_seq[send_conn] : 0ull;
  unsigned long long rseq = has_recv ? sync->recv_seq[recv_conn] : 0ull;
  const unsigned long long sseq0 = sseq, rseq0 = rseq;
  // LL flags are unique per (launch, tile): FIFO memory is reused by other programs with other
  // layouts, so a flag must never equal anything an earlier launch may have left behind.
  const unsigned int flag_epoch = static_cast<unsigned int>(epoch & 0xfffffull) << 12;
  const unsigned long long flag_epoch128 = epoch << 24;

  // Opening receive slots.  A sender may store a tile straight into this rank's buffer once the slot is open:
  // nothing on this GPU touches it any more before the receive.  The host worked out after which step that
  // holds (DevStep::opens_*); slots that nothing touches at all before their receive are opened for every
  // iteration right here - being inside this kernel already means that everything queued before it on this
  // GPU's stream has finished with them.  Only thread 0 opens slots; `opened` is its running count.
  const bool opening = PROTO == PROTO_SIMPLE && has_recv && tb.nrecv > 0 && (tb.recv_bufmask & a.direct_mask) != 0;
  const bool eager = opening && tb.opens_at_start == tb.nrecv;
  unsigned long long opened = rseq0;
  if (eager && tid == 0) {
    opened = rseq0 + static_cast<unsigned long long>(tb.nrecv) * a.iterations;
    st_release_sys(recv_open, opened);
  }
  unsigned int mode_bits = 0;                      // thread 0: how the last kFifoSlots tiles were sent
  unsigned long long pass = 0;                     // steps executed so far by this CTA (tags the verdicts of thread 0)
  __syncthreads();

  const long long C = a.chunk_elems;
  const bool trace_on = a.trace != nullptr;
  unsigned long long* const trace = trace_on ? a.trace + static_cast<long long>(a.first_tb + blockIdx.x) * a.trace_steps * 6 : nullptr;
  bool failed = false;

  for (int it = 0; it < a.iterations && !failed; ++it) {
    const long long tile_off = static_cast<long long>(it) * a.tile_elems;
    const long long n = min(a.tile_elems, C - tile_off);          // elements of each chunk this iteration
    const long long V = n * static_cast<long long>(sizeof(T)) / W;   // accesses per chunk this iteration
    const long long lines = (2 * V + 14) / 15;                       // LL128: lines per chunk this iteration

    if (opening && !eager && tid == 0 && tb.opens_at_start > 0) {
      opened += tb.opens_at_start;
      st_release_sys(recv_open, opened);
    }
    int s = 0;
    while (s < nsteps && !failed) {
      const DevStep st = sp[s];
      const int nb = st.batch > 1 ? st.batch : 1;                   // steps executed by this pass
      const int last = s + nb - 1;
      const bool sends = is_send(st.type), recvs = is_recv(st.type);
      // may this tile be stored into / found in the destination slot itself?  Decided per tile below.
      const bool can_direct_send = PROTO == PROTO_SIMPLE && sends && (st.flags & SF_DIRECT_SEND) && ((a.direct_mask >> st.rbuf) & 1);
      const bool can_direct_recv = PROTO == PROTO_SIMPLE && recvs && (st.flags & SF_DIRECT_RECV) && ((a.direct_mask >> st.dstbuf) & 1);
      unsigned long long t0 = 0, t1 = 0;
      if (trace_on && tid == 0) t0 = global_timer_ns();

      // ---- bounds (every thread computes the same verdict) ----
      bool in_bounds = true;
      long long worst = 0;
      if (st.type != ST_NOP) {
        const bool reads_src = st.type == ST_SEND || st.type == ST_CPY || st.type == ST_RE;
        const bool uses_dst = st.type != ST_SEND;
        if (reads_src && (static_cast<long long>(st.srcoff) + st.cnt) * C > elems[st.srcbuf]) { in_bounds = false; worst = st.srcoff; }
        if (uses_dst && (static_cast<long long>(st.dstoff) + st.cnt) * C > elems[st.dstbuf]) { in_bounds = false; worst = st.dstoff; }
        if (can_direct_send) {
          const long long peer_elems = from_args ? a.local_elems[st.rbuf] : a.ranks[send_peer_id].buf_elems[st.rbuf];
          if ((static_cast<long long>(st.roff) + st.cnt) * C > peer_elems) { in_bounds = false; worst = st.roff; }
        }
        const long long fifo_bytes = PROTO == PROTO_SIMPLE ? st.cnt * V * W
                                     : (PROTO == PROTO_LL ? st.cnt * V * LLPacket<W>::kBytes : st.cnt * lines * 128);
        if ((sends || recvs) && fifo_bytes > a.slot_bytes) { in_bounds = false; worst = -1; }
      }
      for (int k = 1; k < nb && in_bounds; ++k) {
        const DevStep sk = sp[s + k];
        if (sk.type == ST_RE && (static_cast<long long>(sk.srcoff) + sk.cnt) * C > elems[sk.srcbuf]) { in_bounds = false; worst = sk.srcoff; }
      }

      // ---- waits ----
      // Thread 0 polls the flags in global memory (one poller per CTA: sixteen would only fight over the same lines in
      // L2) and leaves its verdict - go or failed, and which way the tile travels - in shared memory with a running
      // number, so it is never mistaken for the previous step's.  The other warps pick it up at a CTA barrier
      // (wait_mode 1, the default: parked warps cost nothing) or by polling shared memory (wait_mode 0: no barrier
      // before the movement, but measured slower - the pollers take issue slots from thread 0).
      unsigned int code = 0, aux0 = 0, aux1 = 0;
      bool direct_send = false, direct_recv = false;
      ++pass;
      if (tid == 0) {
        if (!in_bounds) {
          code = STATUS_BOUNDS; aux0 = st.type; aux1 = static_cast<unsigned int>(worst);
        }
        for (int k = 0; k < nb && code == 0; ++k) {
          const DevStep sk = (k == 0) ? st : sp[s + k];
          if (sk.depid >= 0 && !w.until_ge(&sync->progress[sk.depid], pack_progress(epoch, it, sk.deps + 1), false)) {
            code = STATUS_TIMEOUT_DEP; aux0 = sk.depid; aux1 = sk.deps;
          }
        }
        if (code == 0 && sends &&
            !w.until_ge(&sync->send_head[send_conn], sseq + 1 > kFifoSlots ? sseq + 1 - kFifoSlots : 0, true)) {
          code = STATUS_TIMEOUT_CREDIT; aux0 = send_peer_id; aux1 = chan;
        }
        // store this tile straight into the receiver's slot?  Only if the receiver has opened it by now.
        if (code == 0 && can_direct_send) direct_send = ld_acquire_sys(&sync->recv_posted[send_conn]) >= sseq + 1;
        if (code == 0 && recvs && PROTO == PROTO_SIMPLE) {
          // a receive that opens its own slot does so here: the barrier that ended the previous step and this step's
          // dependency wait are behind us
          if (opening && !eager && st.opens_before > 0) {
            opened += st.opens_before;
            st_release_sys(recv_open, opened);
          }
          unsigned long long word = 0;
          if (!w.until_count_ge(&sync->recv_tail[recv_conn], rseq + 1, &word)) {
            code = STATUS_TIMEOUT_DATA; aux0 = recv_peer_id; aux1 = chan;
          }
          direct_recv = can_direct_recv && ((word >> (kTailModeShift + static_cast<int>(rseq % kFifoSlots))) & 1ull) != 0;
        }
        if (code != 0) {
          record_failure(sync, code, my_rank, my_tb, s, it, aux0, aux1);
          *reinterpret_cast<volatile int*>(&s_fail) = 1;
        }
        *reinterpret_cast<volatile unsigned long long*>(&s_decision) =
            (pass << 3) | (code != 0 ? 4ull : 0ull) | (direct_recv ? 2ull : 0ull) | (direct_send ? 1ull : 0ull);
      }
      if (a.wait_mode == 1) __syncthreads();
      if (tid != 0 && lane == 0) {
        unsigned int spins = 0;
        unsigned long long d;
        while (((d = *reinterpret_cast<volatile unsigned long long*>(&s_decision)) >> 3) != pass) {
          __nanosleep(64);         // a busy loop here takes issue slots from thread 0's polling and from the signals
          if ((++spins & 4095u) == 0 && w.expired()) { d = 4ull; break; }
        }
        code = (d & 4ull) ? static_cast<unsigned int>(STATUS_ABORTED) : 0u;
        direct_recv = (d & 2ull) != 0;
        direct_send = (d & 1ull) != 0;
      }
      code = __shfl_sync(kFullWarp, code, 0);
      direct_send = __shfl_sync(kFullWarp, direct_send ? 1 : 0, 0) != 0;
      direct_recv = __shfl_sync(kFullWarp, direct_recv ? 1 : 0, 0) != 0;
      if (trace_on && tid == 0) t1 = global_timer_ns();

      // ---- data movement ----
      if (code == 0 && st.type != ST_NOP) {
        const char* fifo_in = (recvs && !direct_recv) ? recv_fifo + (rseq % kFifoSlots) * a.slot_bytes : nullptr;
        char* fifo_out = (sends && !direct_send) ? send_fifo + (sseq % kFifoSlots) * a.slot_bytes : nullptr;
        char* const sbase = bufs[st.srcbuf];
        char* const dbase = bufs[st.dstbuf];
        char* const rbase = direct_send ? (from_args ? a.peer_heap[send_peer_id] + a.sym_off[st.rbuf]
                                                     : static_cast<char*>(a.ranks[send_peer_id].buf[st.rbuf]))
                                        : nullptr;
        const unsigned int tile_in = static_cast<unsigned int>((rseq - rseq0) % 4095ull) + 1u;
        const unsigned int tile_out = static_cast<unsigned int>((sseq - sseq0) % 4095ull) + 1u;
        const unsigned int flag_in = flag_epoch | tile_in, flag_out = flag_epoch | tile_out;
        const unsigned long long flag_in128 = flag_epoch128 | (rseq - rseq0 + 1), flag_out128 = flag_epoch128 | (sseq - sseq0 + 1);
        for (int j = 0; j < st.cnt; ++j) {
          const long long src_e = (static_cast<long long>(st.srcoff) + j) * C + tile_off;
          const long long dst_e = (static_cast<long long>(st.dstoff) + j) * C + tile_off;
          const char* lsrc = sbase + src_e * sizeof(T);
          char* ldst = dbase + dst_e * sizeof(T);
          if (st.type == ST_CPY) {
            move_plain<T, W>(lsrc, nullptr, ldst, nullptr, V);
            continue;
          }
          if (st.type == ST_RE) {
            if (nb == 1) {
              move_plain<T, W>(ldst, lsrc, ldst, nullptr, V);
            } else {
              const char* srcs[kMaxBatch];
              int nsrc = 0;
              for (int k = 0; k < nb; ++k) {
                const DevStep sk = sp[s + k];
                if (sk.type == ST_RE && nsrc < kMaxBatch)
                  srcs[nsrc++] = bufs[sk.srcbuf] + ((static_cast<long long>(sk.srcoff) + j) * C + tile_off) * sizeof(T);
              }
              move_batch<T, W>(ldst, srcs, nsrc, V);
            }
            continue;
          }
          if constexpr (PROTO == PROTO_SIMPLE) {
            // FIFO slots and a peer's buffer are plain memory here
            const char* fin = fifo_in != nullptr ? fifo_in + static_cast<long long>(j) * V * W : nullptr;
            char* out1 = nullptr;
            if (sends) out1 = direct_send ? rbase + ((static_cast<long long>(st.roff) + j) * C + tile_off) * sizeof(T)
                                          : fifo_out + static_cast<long long>(j) * V * W;
            switch (st.type) {
              case ST_SEND: move_plain<T, W>(lsrc, nullptr, nullptr, out1, V); break;
              case ST_RECV: if (!direct_recv) move_plain<T, W>(fin, nullptr, ldst, nullptr, V); break;
              case ST_RCS:
                if (direct_recv) move_plain<T, W>(ldst, nullptr, nullptr, out1, V);
                else move_plain<T, W>(fin, nullptr, ldst, out1, V);
                break;
              case ST_RRC: move_plain<T, W>(fin, ldst, ldst, nullptr, V); break;
              case ST_RRS: move_plain<T, W>(fin, ldst, nullptr, out1, V); break;
              case ST_RRCS: move_plain<T, W>(fin, ldst, ldst, out1, V); break;
              default: break;
            }
          } else if constexpr (PROTO == PROTO_LL) {
            const long long fv = static_cast<long long>(j) * V;
            switch (st.type) {
              case ST_SEND: move_ll<T, W, false, true>(lsrc, nullptr, nullptr, nullptr, fifo_out, fv, V, 0, flag_out, w, &s_fail); break;
              case ST_RECV: move_ll<T, W, true, false>(nullptr, nullptr, ldst, fifo_in, nullptr, fv, V, flag_in, 0, w, &s_fail); break;
              case ST_RCS: move_ll<T, W, true, true>(nullptr, nullptr, ldst, fifo_in, fifo_out, fv, V, flag_in, flag_out, w, &s_fail); break;
              case ST_RRC: move_ll<T, W, true, false>(nullptr, ldst, ldst, fifo_in, nullptr, fv, V, flag_in, 0, w, &s_fail); break;
              case ST_RRS: move_ll<T, W, true, true>(nullptr, ldst, nullptr, fifo_in, fifo_out, fv, V, flag_in, flag_out, w, &s_fail); break;
              case ST_RRCS: move_ll<T, W, true, true>(nullptr, ldst, ldst, fifo_in, fifo_out, fv, V, flag_in, flag_out, w, &s_fail); break;
              default: break;
            }
          } else if constexpr (W == 16) {      // LL128 (only built for 16-byte chunks)
            const long long lb = static_cast<long long>(j) * lines;
            const long long n8 = 2 * V;
            switch (st.type) {
              case ST_SEND: move_ll128<T, false, true>(lsrc, nullptr, nullptr, nullptr, fifo_out, lb, n8, 0, flag_out128, w, &s_fail); break;
              case ST_RECV: move_ll128<T, true, false>(nullptr, nullptr, ldst, fifo_in, nullptr, lb, n8, flag_in128, 0, w, &s_fail); break;
              case ST_RCS: move_ll128<T, true, true>(nullptr, nullptr, ldst, fifo_in, fifo_out, lb, n8, flag_in128, flag_out128, w, &s_fail); break;
              case ST_RRC: move_ll128<T, true, false>(nullptr, ldst, ldst, fifo_in, nullptr, lb, n8, flag_in128, 0, w, &s_fail); break;
              case ST_RRS: move_ll128<T, true, true>(nullptr, ldst, nullptr, fifo_in, fifo_out, lb, n8, flag_in128, flag_out128, w, &s_fail); break;
              case ST_RRCS: move_ll128<T, true, true>(nullptr, ldst, ldst, fifo_in, fifo_out, lb, n8, flag_in128, flag_out128, w, &s_fail); break;
              default: break;
            }
          }
        }
      }
      __syncthreads();
      unsigned long long t_moved = 0;
      if (trace_on && tid == 0) t_moved = global_timer_ns();
      if (*reinterpret_cast<volatile int*>(&s_fail) != 0) {
        // a wait or a flag-in-data poll ran out of time (the first failure recorded wins)
        if (tid == 0) record_failure(sync, STATUS_TIMEOUT_DATA, my_rank, my_tb, s, it, recv_peer_id, chan);
        failed = true;
        break;
      }

      // ---- signals (one thread; the other warps go on to the next step's waits) ----
      if (tid == 0) {
        // One fence covers everything this step publishes (a system-scope fence costs a microsecond or more, so the flags
        // themselves are relaxed stores behind it): the tile written by all warps before the barrier comes before
        // its count; this rank's own accesses to a slot come before the slot is opened; the step's stores come
        // before the progress word other threadblocks wait on.  The credit alone needs no fence: every warp has used
        // what it read from the FIFO slot before it came to the barrier.
        unsigned int more = 0;
        bool any_dep = st.hasdep != 0;
        if (opening && !eager) more = st.opens_after;
        for (int k = 1; k < nb; ++k) {
          if (opening && !eager) more += sp[s + k].opens_after;
          any_dep = any_dep || sp[s + k].hasdep != 0;
        }
        const bool publishes_tile = sends && PROTO == PROTO_SIMPLE;
        if (publishes_tile || more > 0) fence_acq_rel_sys();
        else if (any_dep) __threadfence();
        if (publishes_tile) {
          const unsigned int bit = 1u << static_cast<int>(sseq % kFifoSlots);
          mode_bits = direct_send ? (mode_bits | bit) : (mode_bits & ~bit);
          st_relaxed_sys(send_tail, (static_cast<unsigned long long>(mode_bits) << kTailModeShift) | (sseq + 1));
        }
        if (more > 0) {
          opened += more;
          st_relaxed_sys(recv_open, opened);
        }
        if (recvs) st_relaxed_sys(recv_credit, rseq + 1);
        if (any_dep) st_relaxed_gpu(&sync->progress[my_tb], pack_progress(epoch, it, last + 1));
        if (trace_on && s < a.trace_steps) {
          const unsigned long long t2 = global_timer_ns();
          unsigned long long* rec = trace + static_cast<long long>(s) * 6;
          if (it == 0) rec[0] = t0;
          rec[1] = t2;
          rec[2] += t1 - t0;
          rec[3] += t_moved - t1;
          rec[4] += t2 - t_moved;
        }
      }
      if (sends) ++sseq;
      if (recvs) ++rseq;
      s += nb;
    }
  }

  // Drain: the FIFO layout belongs to this plan, so do not leave before the peer has consumed
  // everything (the next launch may use another layout).
  if (tid == 0) {
    if (!failed && has_send && !w.until_ge(&sync->send_head[send_conn], sseq, true)) {
      record_failure(sync, STATUS_TIMEOUT_DRAIN, my_rank, my_tb, nsteps, a.iterations, send_peer_id, chan);
    }
    if (has_send) sync->send_seq[send_conn] = sseq;
    if (has_recv) sync->recv_seq[recv_conn] = rseq;
    // the last threadblock of this rank to finish advances the launch epoch
    __threadfence();
    if (atomicAdd(&sync->exec_done, 1u) == static_cast<unsigned int>(tb.tbs_in_rank) - 1u) {
      sync->exec_done = 0;
      sync->exec_epoch = sync->exec_epoch + 1;
    }
  }
}

template <typename T, int PROTO, int W>
const void* kernel_ptr() { return reinterpret_cast<const void*>(&exec_kernel<T, PROTO, W>); }

// proto x width -> kernel; LL128 exists for 16-byte chunks only (the host runs such programs as LL otherwise)
template <typename T>
const void* pick_kernel(int proto, int width) {
  constexpr int E = static_cast<int>(sizeof(T));
  if (width == 16) {
    if (proto == PROTO_SIMPLE) return kernel_ptr<T, PROTO_SIMPLE, 16>();
    if (proto == PROTO_LL) return kernel_ptr<T, PROTO_LL, 16>();
    if (proto == PROTO_LL128) return kernel_ptr<T, PROTO_LL128, 16>();
  } else if (width == E) {
    if (proto == PROTO_SIMPLE) return kernel_ptr<T, PROTO_SIMPLE, E>();
    if (proto == PROTO_LL) return kernel_ptr<T, PROTO_LL, E>();
  }
  return nullptr;
}

const void* pick_kernel(int dtype, int proto, int width) {
  switch (dtype) {
    case DT_F32: return pick_kernel<float>(proto, width);
    case DT_BF16: return pick_kernel<__nv_bfloat16>(proto, width);
    case DT_F16: return pick_kernel<__half>(proto, width);
    default: return nullptr;
  }
}

}  // namespace

// Launch `grid` CTAs executing tbs[first_tb .. first_tb+grid).  `width` is the access size in bytes (16, or
// the element size for chunks that are not multiples of 16 bytes).  `cooperative` guarantees that all CTAs
// are co-resident, which the step dependencies between CTAs require.
cudaError_t launch_exec(const ExecArgs& args, int dtype, int proto, int width, int grid, cudaStream_t stream, bool cooperative) {
  const void* fn = pick_kernel(dtype, proto, width);
  if (fn == nullptr) return cudaErrorInvalidValue;
  ExecArgs copy = args;
  void* params[] = {&copy};
  if (cooperative) return cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kExecThreads), params, 0, stream);
  return cudaLaunchKernel(fn, dim3(grid), dim3(kExecThreads), params, 0, stream);
}

// Largest grid of exec_kernel CTAs that can be co-resident on the current device.
int max_coresident_ctas(int dtype, int proto, int width) {
  int per_sm = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceProp prop;
  cudaGetDeviceProperties(&prop, dev);
  const void* fn = pick_kernel(dtype, proto, width);
  if (fn == nullptr) return 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kExecThreads, 0);
  return per_sm * prop.multiProcessorCount;
}

}  // namespace msccl
