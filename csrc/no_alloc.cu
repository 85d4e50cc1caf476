// Allocation-free variant of the interpreter launch: see no_alloc.h for the contract.
#include "no_alloc.h"

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "msccl_device.h"

namespace msccl {
cudaError_t launch_exec(const ExecArgs& args, int dtype, int proto, int grid, cudaStream_t stream, bool cooperative);
int max_coresident_ctas(int dtype, int proto);
}  // namespace msccl

namespace {

using namespace msccl;

// Layout of the fixed array (offsets in bytes).
constexpr size_t kSyncStride = 64 * 1024;                       // one SyncPage per rank, padded
constexpr size_t kOffSync = 0;
constexpr size_t kOffRankCtx = kOffSync + MSCCL_NOALLOC_MAX_RANKS * kSyncStride;
constexpr size_t kOffTbs = kOffRankCtx + 4096;
constexpr size_t kOffSteps = kOffTbs + 8192;                    // 148 * 48 = 7104
constexpr size_t kOffFifo = kOffSteps + 81920;                  // 4096 * 20
constexpr size_t kOffScratch = kOffFifo + static_cast<size_t>(MSCCL_NOALLOC_MAX_RANKS) * MSCCL_NOALLOC_FIFO_PER_RANK;
constexpr size_t kEnd = kOffScratch + static_cast<size_t>(MSCCL_NOALLOC_MAX_RANKS) * MSCCL_NOALLOC_SCRATCH_PER_RANK;
static_assert(sizeof(SyncPage) <= kSyncStride, "sync page does not fit its slot");
static_assert(kEnd <= MSCCL_NOALLOC_BYTES, "fixed scratch array is too small for its layout");
static_assert(kOffFifo % 256 == 0 && kOffScratch % 256 == 0, "areas must stay 256-byte aligned");

// The scratch itself.  In host code this name is a handle for cudaGetSymbolAddress, not an address
// a kernel can use.
static __device__ __align__(256) unsigned char g_noalloc_scratch[MSCCL_NOALLOC_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
unsigned char* g_device_base[kMaxDevices] = {};
thread_local char g_last_error[256] = "";

int fail_cuda(cudaError_t e, const char* what) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
  return MSCCL_NOALLOC_CUDA_ERROR;
}

// Device address of the array on the current device; looked up once per device.
int scratch_base(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) {
    snprintf(g_last_error, sizeof(g_last_error), "device index %d outside the supported range", dev);
    return MSCCL_NOALLOC_BAD_ARGUMENT;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_device_base[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress");
    g_device_base[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_device_base[dev];
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
      chunk_elems <= 0 || slot_bytes <= 0 || max_cnt <= 0 || dtype < 0 || dtype > 2 || proto < 0 || proto > 1) {
    snprintf(g_last_error, sizeof(g_last_error), "null pointer or value out of range");
    return MSCCL_NOALLOC_BAD_ARGUMENT;
  }
  const long long elem = (dtype == DT_F32) ? 4 : 2;
  if ((chunk_elems * elem) % 16 != 0 || slot_bytes % 16 != 0) {
    snprintf(g_last_error, sizeof(g_last_error), "chunk and FIFO slot sizes must be multiples of 16 bytes");
    return MSCCL_NOALLOC_BAD_ARGUMENT;
  }
  if (nranks < 1 || nranks > MSCCL_NOALLOC_MAX_RANKS || num_tbs < 1 || num_tbs > MSCCL_NOALLOC_MAX_TBS ||
      num_steps < 0 || num_steps > MSCCL_NOALLOC_MAX_STEPS) {
    snprintf(g_last_error, sizeof(g_last_error), "program too large: %d ranks (max %d), %d threadblocks (max %d), %d steps (max %d)",
             nranks, MSCCL_NOALLOC_MAX_RANKS, num_tbs, MSCCL_NOALLOC_MAX_TBS, num_steps, MSCCL_NOALLOC_MAX_STEPS);
    return MSCCL_NOALLOC_TOO_LARGE;
  }
  // The plan was compiled for `slot_bytes` per FIFO slot; every connection's slots must lie inside
  // the fixed FIFO area of the receiving rank.
  const DevTb* tbs = static_cast<const DevTb*>(host_tbs);
  for (int i = 0; i < num_tbs; ++i) {
    const long long span = static_cast<long long>(kFifoSlots) * slot_bytes;
    if ((tbs[i].recv_peer >= 0 && tbs[i].recv_fifo_off + span > MSCCL_NOALLOC_FIFO_PER_RANK) ||
        (tbs[i].send_peer >= 0 && tbs[i].send_fifo_off + span > MSCCL_NOALLOC_FIFO_PER_RANK)) {
      snprintf(g_last_error, sizeof(g_last_error), "FIFO slots of %lld bytes do not fit the fixed %d-byte FIFO area", slot_bytes,
               MSCCL_NOALLOC_FIFO_PER_RANK);
      return MSCCL_NOALLOC_TOO_LARGE;
    }
    if (tbs[i].rank < 0 || tbs[i].rank >= nranks || tbs[i].send_peer >= nranks || tbs[i].recv_peer >= nranks) {
      snprintf(g_last_error, sizeof(g_last_error), "threadblock %d names a rank outside 0..%d", i, nranks - 1);
      return MSCCL_NOALLOC_BAD_ARGUMENT;
    }
  }
  for (int r = 0; r < nranks; ++r) {
    if (scratch_chunks[r] < 0 || static_cast<long long>(scratch_chunks[r]) * chunk_elems * elem > MSCCL_NOALLOC_SCRATCH_PER_RANK) {
      snprintf(g_last_error, sizeof(g_last_error), "rank %d needs %lld bytes of scratch, the fixed area has %d per rank", r,
               static_cast<long long>(scratch_chunks[r]) * chunk_elems * elem, MSCCL_NOALLOC_SCRATCH_PER_RANK);
      return MSCCL_NOALLOC_TOO_LARGE;
    }
    if (inputs[r] == nullptr || reinterpret_cast<uintptr_t>(inputs[r]) % 16 != 0 ||
        reinterpret_cast<uintptr_t>(outputs[r]) % 16 != 0) {
      snprintf(g_last_error, sizeof(g_last_error), "rank %d: input missing or a buffer is not 16-byte aligned", r);
      return MSCCL_NOALLOC_BAD_ARGUMENT;
    }
  }
  if (num_tbs > max_coresident_ctas(dtype, proto)) {
    snprintf(g_last_error, sizeof(g_last_error), "%d threadblocks cannot be co-resident on this device", num_tbs);
    return MSCCL_NOALLOC_TOO_LARGE;
  }

  unsigned char* base = nullptr;
  int rc = scratch_base(&base);
  if (rc != MSCCL_NOALLOC_OK) return rc;

  // Per-rank contexts, built on the host stack and copied into the array (no allocation).
  RankCtx ctx[MSCCL_NOALLOC_MAX_RANKS];
  memset(ctx, 0, sizeof(ctx));
  for (int r = 0; r < nranks; ++r) {
    ctx[r].sync = reinterpret_cast<SyncPage*>(base + kOffSync + r * kSyncStride);
    ctx[r].fifo = reinterpret_cast<char*>(base + kOffFifo + static_cast<size_t>(r) * MSCCL_NOALLOC_FIFO_PER_RANK);
    ctx[r].buf[BUF_INPUT] = const_cast<void*>(inputs[r]);
    ctx[r].buf[BUF_OUTPUT] = outputs[r];
    ctx[r].buf[BUF_SCRATCH] = base + kOffScratch + static_cast<size_t>(r) * MSCCL_NOALLOC_SCRATCH_PER_RANK;
  }
  cudaError_t e;
  // Flags and counters start from zero on every call: the array still holds the previous call's.
  e = cudaMemsetAsync(base + kOffSync, 0, nranks * kSyncStride, stream);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemsetAsync(flag pages)");
  // Pageable-memory copies are staged by the runtime before the call returns, so the host arrays
  // may be reused immediately.
  e = cudaMemcpyAsync(base + kOffRankCtx, ctx, sizeof(RankCtx) * nranks, cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpyAsync(rank contexts)");
  e = cudaMemcpyAsync(base + kOffTbs, host_tbs, sizeof(DevTb) * num_tbs, cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpyAsync(threadblocks)");
  if (num_steps > 0) {
    e = cudaMemcpyAsync(base + kOffSteps, host_steps, sizeof(DevStep) * num_steps, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpyAsync(steps)");
  }

  // Tile size: the largest step (max_cnt chunks) must fit one FIFO slot (half of it with LL).
  const long long payload = (proto == PROTO_SIMPLE) ? slot_bytes : slot_bytes / 2;
  const long long per_vec = 16 / elem;
  long long tile = payload / (static_cast<long long>(max_cnt) * elem) / per_vec * per_vec;
  if (tile <= 0) {
    snprintf(g_last_error, sizeof(g_last_error), "FIFO slot too small for steps of %d chunks", max_cnt);
    return MSCCL_NOALLOC_TOO_LARGE;
  }
  if (tile > chunk_elems) tile = chunk_elems;

  ExecArgs a;
  memset(&a, 0, sizeof(a));
  a.tbs = reinterpret_cast<const DevTb*>(base + kOffTbs);
  a.steps = reinterpret_cast<const DevStep*>(base + kOffSteps);
  a.ranks = reinterpret_cast<const RankCtx*>(base + kOffRankCtx);
  a.chunk_elems = chunk_elems;
  a.tile_elems = tile;
  a.slot_bytes = slot_bytes;
  a.iterations = static_cast<int>((chunk_elems + tile - 1) / tile);
  a.nranks = nranks;
  a.timeout_ns = 20ull * 1000 * 1000 * 1000;
  a.first_tb = 0;
  a.bufs_from_args = 0;
  e = launch_exec(a, dtype, proto, num_tbs, stream, true);
  if (e != cudaSuccess) return fail_cuda(e, "launch of the interpreter kernel");
  return MSCCL_NOALLOC_OK;
}

__attribute__((visibility("default"))) int msccl_exec_noalloc_status(int nranks, cudaStream_t stream) {
  g_last_error[0] = '\0';
  if (nranks < 1 || nranks > MSCCL_NOALLOC_MAX_RANKS) return -MSCCL_NOALLOC_BAD_ARGUMENT;
  unsigned char* base = nullptr;
  if (scratch_base(&base) != MSCCL_NOALLOC_OK) return -MSCCL_NOALLOC_CUDA_ERROR;
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
