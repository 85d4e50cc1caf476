/* Allocation-free entry point of the MSCCL-IR interpreter (single GPU, emulated ranks).
 *
 * This entry point has no counterpart in the reference (msccl-tools ships no runtime at all); it is
 * an addition of this library.
 *
 * Who it is for: code that must not, or cannot, allocate device memory at the time it wants to run
 * a collective program - a plugin called from inside another framework's memory-pool callback, a
 * process whose device memory is fully handed out to a caching allocator, or a service loop that
 * bans cudaMalloc / cudaFree after start-up because they synchronise the whole device.  The ordinary
 * executor path allocates its flag pages, FIFOs, plan arrays and scratch buffers with cudaMalloc /
 * torch; this one takes them from one fixed array that is part of the library image.
 *
 * What it does: runs one compiled MSCCL-IR program with all of its ranks emulated on the current
 * device (every <tb> of every rank is one CTA of a single cooperative launch), exactly like
 * Executor.run on an emulated communicator.  The caller passes the compiled program as host
 * arrays (the DevTb / DevStep records produced by msccl.runtime.plan.compile_plan) and one input
 * and one output device pointer per rank.  Everything else - flag pages, FIFOs, the program's
 * scratch buffers, the device copy of the plan - lives in a file-scope
 * `static __device__ __align__(256)` array of MSCCL_NOALLOC_BYTES bytes.  Every GPU that loads the
 * library holds that array until the process exits.
 *
 * Limits (requests beyond them are rejected with MSCCL_NOALLOC_TOO_LARGE):
 *   ranks <= 8, threadblocks <= 148 in total (128 per rank) and co-resident on the device,
 *   steps <= 4096 in total (4094 per threadblock),
 *   program scratch <= MSCCL_NOALLOC_SCRATCH_PER_RANK bytes per rank,
 *   FIFO area MSCCL_NOALLOC_FIFO_PER_RANK bytes per rank (tiles shrink to fit, the program just
 *   takes more iterations).
 * The tables are checked on the host before anything is enqueued: every index a threadblock or a
 * step names (ranks, step ranges, connections, dependencies, buffers, scratch offsets, FIFO slots)
 * must lie inside these limits, otherwise the call returns MSCCL_NOALLOC_BAD_ARGUMENT or
 * MSCCL_NOALLOC_TOO_LARGE and nothing has been copied or launched.
 *
 * First call on a device: looks up the device address of the array with cudaGetSymbolAddress (the
 * array's name is only a host-side handle, not a device pointer).  That lookup happens once per
 * device, with that device current, inside the first call on it; make that first call before any
 * stream capture is started.  No call ever uses cudaMalloc, cudaFree or an allocating library
 * routine.  Every call copies its tables from the caller's (pageable) host arrays with
 * cudaMemcpyAsync, which stages them before it returns; the status call synchronises the stream.
 *
 * Sharing: all calls on a device use the same array, which keeps whatever the previous call left.
 * Each call therefore clears the flag pages at its start (on the caller's stream), overwrites
 * the plan copy, and tags the packets of the flag-in-data protocols with a per-device call counter
 * so that nothing an earlier call left in the FIFO area can be mistaken for new data.  Two calls
 * whose kernels overlap on the GPU (different streams) race on the array; serialise them.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MSCCL_NOALLOC_MAX_RANKS 8
#define MSCCL_NOALLOC_MAX_TBS 148
#define MSCCL_NOALLOC_MAX_STEPS 4096
#define MSCCL_NOALLOC_FIFO_PER_RANK (512 * 1024)
#define MSCCL_NOALLOC_SCRATCH_PER_RANK (256 * 1024)
#define MSCCL_NOALLOC_BYTES (8 * 1024 * 1024)

enum msccl_noalloc_status {
  MSCCL_NOALLOC_OK = 0,
  MSCCL_NOALLOC_TOO_LARGE = 1,     /* a limit above is exceeded */
  MSCCL_NOALLOC_BAD_ARGUMENT = 2,  /* null pointer, unknown dtype/protocol, misaligned buffer, inconsistent table */
  MSCCL_NOALLOC_CUDA_ERROR = 3     /* a CUDA call failed; see msccl_noalloc_last_error() */
};

/* host_tbs / host_steps: num_tbs DevTb records (64 bytes each) and num_steps DevStep records
 * (32 bytes each) in host memory, compiled for ranks 0..nranks-1 with slot_bytes as the FIFO slot
 * size.  inputs / outputs: host arrays of nranks device pointers (outputs[r] may be null when rank
 * r's program never touches its output buffer, as in in-place programs); each buffer must hold
 * every chunk the program addresses in it.  scratch_chunks[r]: chunks of scratch rank r's program
 * uses.  dtype: 0 fp32, 1 bf16, 2 fp16.  proto: 0 Simple, 1 LL, 2 LL128.  Chunks that are not a
 * multiple of 16 bytes run on element-wide accesses (Simple and LL only).
 * The launch is asynchronous on `stream`; msccl_exec_noalloc_status reads the outcome. */
int msccl_exec_noalloc(const void* host_tbs, int num_tbs, const void* host_steps, int num_steps, int nranks,
                       const void* const* inputs, void* const* outputs, const int* scratch_chunks,
                       long long chunk_elems, long long slot_bytes, int max_cnt, int dtype, int proto,
                       cudaStream_t stream);

/* Synchronises `stream` and returns the kernel status word of the first rank that reported a
 * problem (0 = every rank finished; codes as in msccl_device.h StatusCode). */
int msccl_exec_noalloc_status(int nranks, cudaStream_t stream);

/* Text of the last error seen by this entry point on the calling thread ("" if none). */
const char* msccl_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
