// Allocation-free variant of the interpreter launch: see no_alloc.h for the contract.
#include "no_alloc.h"

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "msccl_device.h"

namespace msccl {
cudaError_t launch_exec(const ExecArgs& args, int dtype, int proto, int width, int grid, cudaStream_t stream, bool cooperative);
int max_coresident_ctas(int dtype, int proto, int width);
}  // namespace msccl

namespace {

using namespace msccl;

// Layout of the fixed array (offsets in bytes).
constexpr size_t kSyncStride = 128 * 1024;                      // one SyncPage per rank, padded
constexpr size_t kOffSync = 0;
constexpr size_t kOffRankCtx = kOffSync + MSCCL_NOALLOC_MAX_RANKS * kSyncStride;
constexpr size_t kOffTbs = kOffRankCtx + 4096;
constexpr size_t kOffSteps = kOffTbs + 12288;                   // 148 * 64 = 9472
constexpr size_t kOffFifo = kOffSteps + 131072;                 // 4096 * 32
constexpr size_t kOffScratch = kOffFifo + static_cast<size_t>(MSCCL_NOALLOC_MAX_RANKS) * MSCCL_NOALLOC_FIFO_PER_RANK;
constexpr size_t kEnd = kOffScratch + static_cast<size_t>(MSCCL_NOALLOC_MAX_RANKS) * MSCCL_NOALLOC_SCRATCH_PER_RANK;
static_assert(sizeof(SyncPage) <= kSyncStride, "sync page does not fit its slot");
static_assert(sizeof(RankCtx) * MSCCL_NOALLOC_MAX_RANKS <= 4096, "rank contexts do not fit their slot");
static_assert(sizeof(DevTb) * MSCCL_NOALLOC_MAX_TBS <= 12288, "threadblock table does not fit its slot");
static_assert(sizeof(DevStep) * MSCCL_NOALLOC_MAX_STEPS <= 131072, "step table does not fit its slot");
static_assert(kEnd <= MSCCL_NOALLOC_BYTES, "fixed scratch array is too small for its layout");
static_assert(kOffFifo % 256 == 0 && kOffScratch % 256 == 0, "areas must stay 256-byte aligned");

constexpr int kMaxStepsPerTb = 4094;            // the progress word keeps 12 bits of step + 1
constexpr long long kMaxIterations = 1 << 20;   // ... and 20 bits of iteration

// The scratch itself.  In host code this name is a handle for cudaGetSymbolAddress, not an address
// a kernel can use.
static __device__ __align__(256) unsigned char g_noalloc_scratch[MSCCL_NOALLOC_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
unsigned char* g_device_base[kMaxDevices] = {};
unsigned long long g_calls[kMaxDevices] = {};       // launches made on each device: the flag epoch of the next one
thread_local char g_last_error[256] = "";

int fail_cuda(cudaError_t e, const char* what) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
  return MSCCL_NOALLOC_CUDA_ERROR;
}

int reject(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

// Device address of the array on the current device; looked up once per device.
int scratch_base(unsigned char** out, int* device) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "device index %d outside the supported range", dev);
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_device_base[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress");
    g_device_base[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_device_base[dev];
  if (device != nullptr) *device = dev;
  return MSCCL_NOALLOC_OK;
}

bool is_send_type(int t) { return t == ST_SEND || t == ST_RCS || t == ST_RRS || t == ST_RRCS; }
bool is_recv_type(int t) { return t == ST_RECV || t == ST_RCS || t == ST_RRS || t == ST_RRC || t == ST_RRCS; }

// Every index the kernel will form from the tables, checked on the host.  used[r][b]: chunks of buffer b rank r's
// program addresses.
int validate_tables(const DevTb* tbs, int num_tbs, const DevStep* steps, int num_steps, int nranks, long long slot_bytes,
                    int max_cnt, long long used[][3]) {
  int tbs_of_rank[MSCCL_NOALLOC_MAX_RANKS] = {};
  for (int i = 0; i < num_tbs; ++i) {
    const DevTb& t = tbs[i];
    if (t.rank < 0 || t.rank >= nranks || t.send_peer < -1 || t.send_peer >= nranks || t.recv_peer < -1 || t.recv_peer >= nranks)
      return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d names a rank outside 0..%d", i, nranks - 1);
    ++tbs_of_rank[t.rank];
  }
  for (int i = 0; i < num_tbs; ++i) {
    const DevTb& t = tbs[i];
    if (t.tbs_in_rank != tbs_of_rank[t.rank] || t.tbs_in_rank > kMaxTbsPerRank)
      return reject(t.tbs_in_rank > kMaxTbsPerRank ? MSCCL_NOALLOC_TOO_LARGE : MSCCL_NOALLOC_BAD_ARGUMENT,
                    "threadblock %d: rank %d runs %d threadblocks (table says %d, limit %d)", i, t.rank, tbs_of_rank[t.rank],
                    t.tbs_in_rank, kMaxTbsPerRank);
    if (t.tb_in_rank < 0 || t.tb_in_rank >= t.tbs_in_rank)
      return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d: index %d outside its rank's %d threadblocks", i, t.tb_in_rank, t.tbs_in_rank);
    if (t.nsteps < 0 || t.nsteps > kMaxStepsPerTb || t.step_begin < 0 || static_cast<long long>(t.step_begin) + t.nsteps > num_steps)
      return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d: steps [%d, %d) outside the %d steps passed (at most %d per threadblock)",
                    i, t.step_begin, t.step_begin + t.nsteps, num_steps, kMaxStepsPerTb);
    if (t.chan < 0 || t.chan >= kMaxChannels)
      return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d: channel %d outside 0..%d", i, t.chan, kMaxChannels - 1);
    if ((t.send_peer >= 0 && t.send_conn != t.chan * kMaxRanks + t.send_peer) || (t.send_peer < 0 && t.send_conn != -1) ||
        (t.recv_peer >= 0 && t.recv_conn != t.chan * kMaxRanks + t.recv_peer) || (t.recv_peer < 0 && t.recv_conn != -1))
      return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d: connection ids do not match its channel and peers", i);
    const long long span = static_cast<long long>(kFifoSlots) * slot_bytes;
    if ((t.recv_peer >= 0 && (t.recv_fifo_off < 0 || t.recv_fifo_off % 128 != 0)) ||
        (t.send_peer >= 0 && (t.send_fifo_off < 0 || t.send_fifo_off % 128 != 0)))
      return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d: FIFO offsets must be non-negative multiples of 128", i);
    if ((t.recv_peer >= 0 && t.recv_fifo_off + span > MSCCL_NOALLOC_FIFO_PER_RANK) ||
        (t.send_peer >= 0 && t.send_fifo_off + span > MSCCL_NOALLOC_FIFO_PER_RANK))
      return reject(MSCCL_NOALLOC_TOO_LARGE, "FIFO slots of %lld bytes do not fit the fixed %d-byte FIFO area", slot_bytes,
                    MSCCL_NOALLOC_FIFO_PER_RANK);
    if (t.opens_at_start < 0 || t.nrecv < 0 || t.nrecv > t.nsteps || (t.recv_bufmask & ~7) != 0)
      return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d: bad receive summary", i);
    int recv_steps = 0;
    long long opens = t.opens_at_start;
    for (int s = 0; s < t.nsteps; ++s) {
      const DevStep& st = steps[t.step_begin + s];
      if (st.type > ST_RE || st.srcbuf > BUF_SCRATCH || st.dstbuf > BUF_SCRATCH || st.rbuf > BUF_SCRATCH)
        return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d step %d: unknown step type or buffer", i, s);
      if (st.cnt < 0 || st.cnt > max_cnt || st.srcoff < 0 || st.dstoff < 0 || st.roff < 0)
        return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d step %d: count %d (max_cnt %d) or a negative offset", i, s, st.cnt, max_cnt);
      if (st.depid < -1 || st.depid >= t.tbs_in_rank || st.deps < -1 || st.deps >= kMaxStepsPerTb || (st.depid >= 0 && st.deps < 0))
        return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d step %d: dependency (%d, %d) outside its rank's threadblocks", i, s,
                      st.depid, st.deps);
      if ((is_send_type(st.type) && t.send_peer < 0) || (is_recv_type(st.type) && t.recv_peer < 0))
        return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d step %d: sends or receives without a peer", i, s);
      if ((st.flags & ~(SF_DIRECT_SEND | SF_DIRECT_RECV)) != 0 || ((st.flags & SF_DIRECT_SEND) && !is_send_type(st.type)) ||
          ((st.flags & SF_DIRECT_RECV) && st.type != ST_RECV && st.type != ST_RCS))
        return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d step %d: direct flags do not fit the step type", i, s);
      if (is_recv_type(st.type)) ++recv_steps;
      if (st.opens_before > 0 && !is_recv_type(st.type))
        return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d step %d: only a receive can open its own slot", i, s);
      opens += static_cast<long long>(st.opens_after) + st.opens_before;
      if (st.batch > 1) {
        int sources = 0;
        if (st.type != ST_RE || s + st.batch > t.nsteps)
          return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d step %d: batch of %d steps runs past the threadblock", i, s, st.batch);
        for (int k = 0; k < st.batch; ++k) {
          const DevStep& sk = steps[t.step_begin + s + k];
          if (sk.type == ST_RE) {
            ++sources;
            if (sk.dstbuf != st.dstbuf || sk.dstoff != st.dstoff || sk.cnt != st.cnt)
              return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d step %d: batched reduces must share one destination", i, s + k);
          } else if (sk.type != ST_NOP) {
            return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d step %d: only re and nop steps can be batched", i, s + k);
          }
        }
        if (sources > kMaxBatch)
          return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d step %d: %d reduces in one batch (limit %d)", i, s, sources, kMaxBatch);
      }
      if (st.type == ST_NOP) continue;
      long long* mine = used[t.rank];
      if (st.type == ST_SEND || st.type == ST_CPY || st.type == ST_RE)
        if (static_cast<long long>(st.srcoff) + st.cnt > mine[st.srcbuf]) mine[st.srcbuf] = static_cast<long long>(st.srcoff) + st.cnt;
      if (st.type != ST_SEND)
        if (static_cast<long long>(st.dstoff) + st.cnt > mine[st.dstbuf]) mine[st.dstbuf] = static_cast<long long>(st.dstoff) + st.cnt;
      if (st.flags & SF_DIRECT_SEND) {
        long long* theirs = used[t.send_peer];
        if (static_cast<long long>(st.roff) + st.cnt > theirs[st.rbuf]) theirs[st.rbuf] = static_cast<long long>(st.roff) + st.cnt;
      }
    }
    // every receive is opened exactly once per iteration (or none is: a plan compiled without direct stores)
    if (t.nrecv != (t.recv_peer >= 0 ? recv_steps : 0) || (opens != 0 && opens != recv_steps))
      return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "threadblock %d: %d receive steps, summary says %d with %lld openings", i, recv_steps,
                    t.nrecv, opens);
  }
  return MSCCL_NOALLOC_OK;
}

}  // namespace

extern "C" {

__attribute__((visibility("default"))) const char* msccl_noalloc_last_error(void) { return g_last_error; }

__attribute__((visibility("default"))) int msccl_exec_noalloc(
    const void* host_tbs, int num_tbs, const void* host_steps, int num_steps, int nranks, const void* const* inputs,
    void* const* outputs, const int* scratch_chunks, long long chunk_elems, long long slot_bytes, int max_cnt, int dtype,
    int proto, cudaStream_t stream) {
  g_last_error[0] = '\0';
  if (host_tbs == nullptr || host_steps == nullptr || inputs == nullptr || outputs == nullptr || scratch_chunks == nullptr ||
      chunk_elems <= 0 || slot_bytes <= 0 || max_cnt <= 0 || dtype < 0 || dtype > 2 || proto < 0 || proto > 2)
    return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "null pointer or value out of range");
  const long long elem = (dtype == DT_F32) ? 4 : 2;
  if (slot_bytes % 1024 != 0) return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "the FIFO slot size must be a multiple of 1024 bytes");
  if (nranks < 1 || nranks > MSCCL_NOALLOC_MAX_RANKS || num_tbs < 1 || num_tbs > MSCCL_NOALLOC_MAX_TBS ||
      num_steps < 0 || num_steps > MSCCL_NOALLOC_MAX_STEPS)
    return reject(MSCCL_NOALLOC_TOO_LARGE, "program too large: %d ranks (max %d), %d threadblocks (max %d), %d steps (max %d)",
                  nranks, MSCCL_NOALLOC_MAX_RANKS, num_tbs, MSCCL_NOALLOC_MAX_TBS, num_steps, MSCCL_NOALLOC_MAX_STEPS);
  const DevTb* tbs = static_cast<const DevTb*>(host_tbs);
  const DevStep* steps = static_cast<const DevStep*>(host_steps);
  long long used[MSCCL_NOALLOC_MAX_RANKS][3] = {};
  int rc = validate_tables(tbs, num_tbs, steps, num_steps, nranks, slot_bytes, max_cnt, used);
  if (rc != MSCCL_NOALLOC_OK) return rc;

  // Access width: 16-byte vectors when every chunk and buffer allows it, single elements otherwise.
  int width = (chunk_elems * elem) % 16 == 0 ? 16 : static_cast<int>(elem);
  for (int r = 0; r < nranks; ++r) {
    if (scratch_chunks[r] < 0 || used[r][BUF_SCRATCH] > scratch_chunks[r])
      return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "rank %d: steps address %lld chunks of scratch, %d declared", r, used[r][BUF_SCRATCH],
                    scratch_chunks[r]);
    if (static_cast<long long>(scratch_chunks[r]) * chunk_elems * elem > MSCCL_NOALLOC_SCRATCH_PER_RANK)
      return reject(MSCCL_NOALLOC_TOO_LARGE, "rank %d needs %lld bytes of scratch, the fixed area has %d per rank", r,
                    static_cast<long long>(scratch_chunks[r]) * chunk_elems * elem, MSCCL_NOALLOC_SCRATCH_PER_RANK);
    if (inputs[r] == nullptr || (outputs[r] == nullptr && used[r][BUF_OUTPUT] > 0))
      return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "rank %d: a buffer its program uses is missing", r);
    const uintptr_t in = reinterpret_cast<uintptr_t>(inputs[r]), out = reinterpret_cast<uintptr_t>(outputs[r]);
    if (in % elem != 0 || out % elem != 0) return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "rank %d: a buffer is not aligned to its element size", r);
    if (in % 16 != 0 || out % 16 != 0) width = static_cast<int>(elem);
  }
  if (proto == PROTO_LL128 && width != 16)
    return reject(MSCCL_NOALLOC_BAD_ARGUMENT, "LL128 programs need chunks and buffers that are multiples of 16 bytes");

  // Tile size: the largest step (max_cnt chunks) must fit one FIFO slot.
  long long tile;
  if (proto == PROTO_LL128) {
    const long long lines = slot_bytes / 128 / max_cnt;            // 15 units of 8 bytes per line, 2 units per vector
    tile = (lines * 15 / 2) * (16 / elem);
  } else {
    const long long fifo_bytes_per_access = proto == PROTO_SIMPLE ? width : (width == 16 ? 32 : 8);
    tile = slot_bytes / (static_cast<long long>(max_cnt) * fifo_bytes_per_access) * (width / elem);
  }
  if (tile <= 0) return reject(MSCCL_NOALLOC_TOO_LARGE, "FIFO slot too small for steps of %d chunks", max_cnt);
  if (tile > chunk_elems) tile = chunk_elems;
  const long long iterations = (chunk_elems + tile - 1) / tile;
  if (iterations >= kMaxIterations)
    return reject(MSCCL_NOALLOC_TOO_LARGE, "%lld iterations through the fixed FIFO area (limit %lld)", iterations, kMaxIterations);
  if (num_tbs > max_coresident_ctas(dtype, proto, width))
    return reject(MSCCL_NOALLOC_TOO_LARGE, "%d threadblocks cannot be co-resident on this device", num_tbs);

  unsigned char* base = nullptr;
  int dev = 0;
  rc = scratch_base(&base, &dev);
  if (rc != MSCCL_NOALLOC_OK) return rc;
  unsigned long long epoch_base;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    epoch_base = g_calls[dev]++;
  }

  // Per-rank contexts, built on the host stack and copied into the array (no allocation).
  RankCtx ctx[MSCCL_NOALLOC_MAX_RANKS];
  memset(ctx, 0, sizeof(ctx));
  for (int r = 0; r < nranks; ++r) {
    ctx[r].sync = reinterpret_cast<SyncPage*>(base + kOffSync + r * kSyncStride);
    ctx[r].fifo = reinterpret_cast<char*>(base + kOffFifo + static_cast<size_t>(r) * MSCCL_NOALLOC_FIFO_PER_RANK);
    ctx[r].buf[BUF_INPUT] = const_cast<void*>(inputs[r]);
    ctx[r].buf[BUF_OUTPUT] = outputs[r];
    ctx[r].buf[BUF_SCRATCH] = base + kOffScratch + static_cast<size_t>(r) * MSCCL_NOALLOC_SCRATCH_PER_RANK;
    // the caller vouches for its buffers holding every chunk the program addresses: those are the bounds
    ctx[r].buf_elems[BUF_INPUT] = used[r][BUF_INPUT] * chunk_elems;
    ctx[r].buf_elems[BUF_OUTPUT] = used[r][BUF_OUTPUT] * chunk_elems;
    ctx[r].buf_elems[BUF_SCRATCH] = static_cast<long long>(scratch_chunks[r]) * chunk_elems;
  }
  cudaError_t e;
  // Flags and counters start from zero on every call: the array still holds the previous call's.  The FIFO
  // area is not cleared; the launch epoch below is a per-device call counter, so the flags of this call's
  // packets differ from everything earlier calls left there.
  e = cudaMemsetAsync(base + kOffSync, 0, nranks * kSyncStride, stream);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemsetAsync(flag pages)");
  // Copies from pageable memory are staged by the runtime before the call returns.
  e = cudaMemcpyAsync(base + kOffRankCtx, ctx, sizeof(RankCtx) * nranks, cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpyAsync(rank contexts)");
  e = cudaMemcpyAsync(base + kOffTbs, host_tbs, sizeof(DevTb) * num_tbs, cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpyAsync(threadblocks)");
  if (num_steps > 0) {
    e = cudaMemcpyAsync(base + kOffSteps, host_steps, sizeof(DevStep) * num_steps, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpyAsync(steps)");
  }

  ExecArgs a;
  memset(&a, 0, sizeof(a));
  a.tbs = reinterpret_cast<const DevTb*>(base + kOffTbs);
  a.steps = reinterpret_cast<const DevStep*>(base + kOffSteps);
  a.ranks = reinterpret_cast<const RankCtx*>(base + kOffRankCtx);
  a.chunk_elems = chunk_elems;
  a.tile_elems = tile;
  a.slot_bytes = slot_bytes;
  a.iterations = static_cast<int>(iterations);
  a.nranks = nranks;
  a.timeout_ns = 20ull * 1000 * 1000 * 1000;
  a.first_tb = 0;
  a.bufs_from_args = 0;
  a.epoch_base = epoch_base;
  a.wait_mode = 1;
  a.direct_mask = 7;            // all ranks live on this device: every buffer can be stored into directly
  for (int b = 0; b < 3; ++b) a.sym_off[b] = -1;
  e = launch_exec(a, dtype, proto, width, num_tbs, stream, true);
  if (e != cudaSuccess) return fail_cuda(e, "launch of the interpreter kernel");
  return MSCCL_NOALLOC_OK;
}

__attribute__((visibility("default"))) int msccl_exec_noalloc_status(int nranks, cudaStream_t stream) {
  g_last_error[0] = '\0';
  if (nranks < 1 || nranks > MSCCL_NOALLOC_MAX_RANKS) return -MSCCL_NOALLOC_BAD_ARGUMENT;
  unsigned char* base = nullptr;
  if (scratch_base(&base, nullptr) != MSCCL_NOALLOC_OK) return -MSCCL_NOALLOC_CUDA_ERROR;
  cudaError_t e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) { fail_cuda(e, "cudaStreamSynchronize"); return -MSCCL_NOALLOC_CUDA_ERROR; }
  for (int r = 0; r < nranks; ++r) {
    unsigned int code = 0;
    const SyncPage* page = reinterpret_cast<const SyncPage*>(base + kOffSync + r * kSyncStride);
    e = cudaMemcpy(&code, &page->status[0], sizeof(code), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) { fail_cuda(e, "cudaMemcpy(status)"); return -MSCCL_NOALLOC_CUDA_ERROR; }
    if (code != 0) return static_cast<int>(code);
  }
  return 0;
}

}  // extern "C"
