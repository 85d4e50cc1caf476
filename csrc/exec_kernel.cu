// MSCCL-IR interpreter kernel for sm_100a: one CTA per <tb>, steps executed in order, data moved
// with 16-byte peer stores over NVLink into per-connection FIFOs of the receiving GPU.
//
// Protocols
//   Simple : sender writes a tile into a FIFO slot, fences, then publishes the tile count with a
//            release store; the receiver acquires the count before reading.
//   LL     : every 16-byte packet carries 8 bytes of data and two copies of a 32-bit flag (the
//            tile sequence number), so no separate fence/flag round trip is needed.
//   LL128  : executed with the LL packet format.
// Both directions are flow controlled by a credit counter the receiver writes back into the
// sender's memory.  Every wait is bounded: when the deadline passes the CTA records what it was
// waiting for in the rank's status words, raises the rank's abort flag and returns.
//
// Large buffers are processed in iterations: iteration k handles elements
// [k*tile, (k+1)*tile) of every chunk, so one program serves any message size.
#include <cstdio>

#include "msccl_device.h"
#include "prims.cuh"

namespace msccl {

namespace {

constexpr int kUnroll = 8;     // 16-byte vectors per thread in flight (copies are latency bound)

__device__ __forceinline__ unsigned long long pack_progress(unsigned long long epoch, int iter, int step_plus_1) {
  // 32 bits of launch epoch | 20 bits of iteration | 12 bits of step+1
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
};

__device__ void record_failure(SyncPage* sync, unsigned int code, int rank, int tb, int step, int iter,
                               unsigned int aux0, unsigned int aux1) {
  unsigned int already = ld_volatile_u32(&sync->abort_flag);
  if (already != 0 && code != STATUS_ABORTED) code = STATUS_ABORTED;
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

// ---- FIFO accessors -----------------------------------------------------------------------
// A "vector" is 16 bytes of payload.  Simple stores it as is; LL spreads it over two packets.
template <int PROTO> struct Fifo;

template <> struct Fifo<PROTO_SIMPLE> {
  static __device__ __forceinline__ uint4 load(const char* slot, long long v, unsigned int, const Waiter&, int* fail) {
    return *reinterpret_cast<const uint4*>(slot + v * 16);
  }
  static __device__ __forceinline__ void store(char* slot, long long v, uint4 d, unsigned int) {
    *reinterpret_cast<uint4*>(slot + v * 16) = d;
  }
};

template <> struct Fifo<PROTO_LL> {
  static __device__ __forceinline__ uint4 load(const char* slot, long long v, unsigned int flag, const Waiter& w,
                                               int* fail) {
    const uint4* pk = reinterpret_cast<const uint4*>(slot) + 2 * v;
    uint4 a, b;
    unsigned int spins = 0;
    while (true) {
      a = ld_volatile_v4(pk);
      b = ld_volatile_v4(pk + 1);
      if (a.y == flag && a.w == flag && b.y == flag && b.w == flag) break;
      if ((++spins & 255u) == 0) {
        if (*reinterpret_cast<volatile int*>(fail) != 0 || ld_volatile_u32(&w.sync->abort_flag) != 0 ||
            global_timer_ns() > w.deadline) {
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

// Move `vectors` 16-byte vectors for one chunk of a step.
//   value = FIFO_IN ? fifo_in[v] : in0[v];  if (in1) value = in1[v] + value;
//   if (out_local) out_local[v] = value;    if (FIFO_OUT) fifo_out[v] = value;
template <typename T, int PROTO, bool FIFO_IN, bool FIFO_OUT>
__device__ __noinline__ void move_vectors(const char* in0, const char* in1, char* out_local, const char* fifo_in,
                                             char* fifo_out, long long fifo_base_v, long long vectors,
                                             unsigned int flag_in, unsigned int flag_out, const Waiter& w, int* fail) {
  const long long nthreads = blockDim.x;
  const long long stride = nthreads * kUnroll;
  const bool reduce = in1 != nullptr;
  for (long long base = threadIdx.x; base < vectors; base += stride) {
    if (base + (kUnroll - 1) * nthreads < vectors) {
      // full group: all loads are issued before the first use, with no per-vector predicate
      uint4 val[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long long v = base + u * nthreads;
        if (FIFO_IN) {
          val[u] = Fifo<PROTO>::load(fifo_in, fifo_base_v + v, flag_in, w, fail);
        } else {
          val[u] = *reinterpret_cast<const uint4*>(in0 + v * 16);
        }
      }
      if (reduce) {
        uint4 other[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) other[u] = *reinterpret_cast<const uint4*>(in1 + (base + u * nthreads) * 16);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) val[u] = Vec16<T>::add(other[u], val[u]);
      }
      if (out_local != nullptr) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) *reinterpret_cast<uint4*>(out_local + (base + u * nthreads) * 16) = val[u];
      }
      if (FIFO_OUT) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) Fifo<PROTO>::store(fifo_out, fifo_base_v + base + u * nthreads, val[u], flag_out);
      }
    } else {
      for (long long v = base; v < vectors; v += nthreads) {
        uint4 r = FIFO_IN ? Fifo<PROTO>::load(fifo_in, fifo_base_v + v, flag_in, w, fail)
                          : *reinterpret_cast<const uint4*>(in0 + v * 16);
        if (reduce) r = Vec16<T>::add(*reinterpret_cast<const uint4*>(in1 + v * 16), r);
        if (out_local != nullptr) *reinterpret_cast<uint4*>(out_local + v * 16) = r;
        if (FIFO_OUT) Fifo<PROTO>::store(fifo_out, fifo_base_v + v, r, flag_out);
      }
    }
  }
}

template <typename T, int PROTO>
__global__ void __launch_bounds__(kExecThreads, 1) exec_kernel(ExecArgs a) {
  __shared__ int s_fail;
  const DevTb& tb = a.tbs[a.first_tb + blockIdx.x];
  const RankCtx& me = a.ranks[tb.rank];
  SyncPage* const sync = me.sync;
  const int tid = threadIdx.x;
  const int my_rank = tb.rank, my_tb = tb.tb_in_rank, nsteps = tb.nsteps, step_begin = tb.step_begin;
  const int send_conn = tb.send_conn, recv_conn = tb.recv_conn;
  const int send_peer_id = tb.send_peer, recv_peer_id = tb.recv_peer, chan = tb.chan;
  char* const buf0 = static_cast<char*>(a.bufs_from_args ? a.local_buf[0] : me.buf[0]);
  char* const buf1 = static_cast<char*>(a.bufs_from_args ? a.local_buf[1] : me.buf[1]);
  char* const buf2 = static_cast<char*>(a.bufs_from_args ? a.local_buf[2] : me.buf[2]);

  // launch epoch: read by every CTA of this rank, advanced by the last one to finish
  const unsigned long long epoch = sync->exec_epoch + 1;
  Waiter w;
  w.sync = sync;
  w.deadline = global_timer_ns() + a.timeout_ns;
  if (tid == 0) s_fail = 0;

  const bool has_send = send_peer_id >= 0;
  const bool has_recv = recv_peer_id >= 0;
  const int remote_idx = chan * kMaxRanks + my_rank;       // this rank's slot in a peer's flag arrays
  // addresses on the peers (NVLink-mapped in multi-process mode)
  char* const send_fifo = has_send ? a.ranks[send_peer_id].fifo + tb.send_fifo_off : nullptr;
  unsigned long long* const send_tail = has_send ? &a.ranks[send_peer_id].sync->recv_tail[remote_idx] : nullptr;
  unsigned long long* const recv_credit = has_recv ? &a.ranks[recv_peer_id].sync->send_head[remote_idx] : nullptr;
  const char* const recv_fifo = has_recv ? me.fifo + tb.recv_fifo_off : nullptr;
  unsigned long long sseq = has_send ? sync->send_seq[send_conn] : 0ull;
  unsigned long long rseq = has_recv ? sync->recv_seq[recv_conn] : 0ull;
  const unsigned long long sseq0 = sseq, rseq0 = rseq;
  // LL flags are unique per (launch, tile): FIFO memory is reused by other programs with other
  // layouts, so a flag must never equal anything an earlier launch may have left behind.
  const unsigned int flag_epoch = static_cast<unsigned int>(epoch & 0xfffffull) << 12;
  __syncthreads();

  const long long C = a.chunk_elems;
  bool failed = false;

  for (int it = 0; it < a.iterations && !failed; ++it) {
    const long long tile_off = static_cast<long long>(it) * a.tile_elems;
    const long long n = min(a.tile_elems, C - tile_off);          // elements of each chunk this iteration
    const long long V = n * static_cast<long long>(sizeof(T)) / 16;  // vectors per chunk this iteration

    for (int s = 0; s < nsteps && !failed; ++s) {
      const DevStep st = a.steps[step_begin + s];
      const bool sends = st.type == ST_SEND || st.type == ST_RCS || st.type == ST_RRS || st.type == ST_RRCS;
      const bool recvs = st.type == ST_RECV || st.type == ST_RCS || st.type == ST_RRS || st.type == ST_RRC ||
                         st.type == ST_RRCS;

      // ---- waits (one thread) ----
      if (tid == 0) {
        unsigned int code = 0, aux0 = 0, aux1 = 0;
        if (st.depid >= 0 &&
            !w.until_ge(&sync->progress[st.depid], pack_progress(epoch, it, st.deps + 1), false)) {
          code = STATUS_TIMEOUT_DEP; aux0 = st.depid; aux1 = st.deps;
        }
        if (code == 0 && sends && !w.until_ge(&sync->send_head[send_conn], sseq + 1 > kFifoSlots ? sseq + 1 - kFifoSlots : 0, true)) {
          code = STATUS_TIMEOUT_CREDIT; aux0 = send_peer_id; aux1 = chan;
        }
        if (code == 0 && recvs && PROTO == PROTO_SIMPLE &&
            !w.until_ge(&sync->recv_tail[recv_conn], rseq + 1, true)) {
          code = STATUS_TIMEOUT_DATA; aux0 = recv_peer_id; aux1 = chan;
        }
        if (code != 0) {
          record_failure(sync, code, my_rank, my_tb, s, it, aux0, aux1);
          s_fail = 1;
        }
      }
      __syncthreads();
      if (s_fail != 0) { failed = true; break; }

      // ---- data movement ----
      if (st.type != ST_NOP) {
        const char* fifo_in = recvs ? recv_fifo + (rseq % kFifoSlots) * a.slot_bytes : nullptr;
        char* fifo_out = sends ? send_fifo + (sseq % kFifoSlots) * a.slot_bytes : nullptr;
        char* const sbase = st.srcbuf == 0 ? buf0 : (st.srcbuf == 1 ? buf1 : buf2);
        char* const dbase = st.dstbuf == 0 ? buf0 : (st.dstbuf == 1 ? buf1 : buf2);
        const unsigned int flag_in = flag_epoch | (static_cast<unsigned int>((rseq - rseq0) % 4095ull) + 1u);
        const unsigned int flag_out = flag_epoch | (static_cast<unsigned int>((sseq - sseq0) % 4095ull) + 1u);
        for (int j = 0; j < st.cnt; ++j) {
          const long long src_e = (static_cast<long long>(st.srcoff) + j) * C + tile_off;
          const long long dst_e = (static_cast<long long>(st.dstoff) + j) * C + tile_off;
          const char* lsrc = sbase + src_e * sizeof(T);
          char* ldst = dbase + dst_e * sizeof(T);
          const long long fv = static_cast<long long>(j) * V;
          switch (st.type) {
            case ST_SEND:
              move_vectors<T, PROTO, false, true>(lsrc, nullptr, nullptr, nullptr, fifo_out, fv, V, 0, flag_out, w, &s_fail);
              break;
            case ST_RECV:
              move_vectors<T, PROTO, true, false>(nullptr, nullptr, ldst, fifo_in, nullptr, fv, V, flag_in, 0, w, &s_fail);
              break;
            case ST_RCS:
              move_vectors<T, PROTO, true, true>(nullptr, nullptr, ldst, fifo_in, fifo_out, fv, V, flag_in, flag_out, w, &s_fail);
              break;
            case ST_RRC:
              move_vectors<T, PROTO, true, false>(nullptr, ldst, ldst, fifo_in, nullptr, fv, V, flag_in, 0, w, &s_fail);
              break;
            case ST_RRS:
              move_vectors<T, PROTO, true, true>(nullptr, ldst, nullptr, fifo_in, fifo_out, fv, V, flag_in, flag_out, w, &s_fail);
              break;
            case ST_RRCS:
              move_vectors<T, PROTO, true, true>(nullptr, ldst, ldst, fifo_in, fifo_out, fv, V, flag_in, flag_out, w, &s_fail);
              break;
            case ST_CPY:
              move_vectors<T, PROTO, false, false>(lsrc, nullptr, ldst, nullptr, nullptr, 0, V, 0, 0, w, &s_fail);
              break;
            case ST_RE:
              move_vectors<T, PROTO, false, false>(lsrc, ldst, ldst, nullptr, nullptr, 0, V, 0, 0, w, &s_fail);
              break;
            default:
              break;
          }
        }
      }
      __syncthreads();
      if (s_fail != 0) {          // an LL poll ran out of time
        if (tid == 0) record_failure(sync, STATUS_TIMEOUT_DATA, my_rank, my_tb, s, it, recv_peer_id, chan);
        failed = true;
        break;
      }

      // ---- signals (one thread) ----
      if (tid == 0) {
        if (sends && PROTO == PROTO_SIMPLE) {
          __threadfence_system();
          st_release_sys(send_tail, sseq + 1);
        }
        if (recvs) st_release_sys(recv_credit, rseq + 1);
        if (st.hasdep) {
          __threadfence();
          st_release_gpu(&sync->progress[my_tb], pack_progress(epoch, it, s + 1));
        }
      }
      if (sends) ++sseq;
      if (recvs) ++rseq;
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
      sync->exec_epoch = epoch;
    }
  }
}

template <typename T>
cudaError_t launch_typed(const ExecArgs& args, int proto, int grid, cudaStream_t stream, bool cooperative) {
  ExecArgs copy = args;
  void* params[] = {&copy};
  const void* fn = (proto == PROTO_SIMPLE) ? reinterpret_cast<const void*>(&exec_kernel<T, PROTO_SIMPLE>)
                                            : reinterpret_cast<const void*>(&exec_kernel<T, PROTO_LL>);
  if (cooperative) return cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kExecThreads), params, 0, stream);
  return cudaLaunchKernel(fn, dim3(grid), dim3(kExecThreads), params, 0, stream);
}

}  // namespace

// Launch `grid` CTAs executing tbs[first_tb .. first_tb+grid).  `cooperative` guarantees that
// all CTAs are co-resident, which the step dependencies between CTAs require.
cudaError_t launch_exec(const ExecArgs& args, int dtype, int proto, int grid, cudaStream_t stream, bool cooperative) {
  switch (dtype) {
    case DT_F32: return launch_typed<float>(args, proto, grid, stream, cooperative);
    case DT_BF16: return launch_typed<__nv_bfloat16>(args, proto, grid, stream, cooperative);
    case DT_F16: return launch_typed<__half>(args, proto, grid, stream, cooperative);
    default: return cudaErrorInvalidValue;
  }
}

// Largest grid of exec_kernel CTAs that can be co-resident on the current device.
int max_coresident_ctas(int dtype, int proto) {
  int per_sm = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceProp prop;
  cudaGetDeviceProperties(&prop, dev);
  const void* fn = reinterpret_cast<const void*>(&exec_kernel<float, PROTO_SIMPLE>);
  if (dtype == DT_BF16) fn = (proto == PROTO_SIMPLE) ? reinterpret_cast<const void*>(&exec_kernel<__nv_bfloat16, PROTO_SIMPLE>)
                                                      : reinterpret_cast<const void*>(&exec_kernel<__nv_bfloat16, PROTO_LL>);
  else if (dtype == DT_F16) fn = (proto == PROTO_SIMPLE) ? reinterpret_cast<const void*>(&exec_kernel<__half, PROTO_SIMPLE>)
                                                          : reinterpret_cast<const void*>(&exec_kernel<__half, PROTO_LL>);
  else if (proto != PROTO_SIMPLE) fn = reinterpret_cast<const void*>(&exec_kernel<float, PROTO_LL>);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kExecThreads, 0);
  return per_sm * prop.multiProcessorCount;
}

}  // namespace msccl
