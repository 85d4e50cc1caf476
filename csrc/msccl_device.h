// Plain-old-data contract between the host runtime and the sm_100a kernels.
//
// A compiled MSCCL-IR program ("plan") is three flat arrays in device memory: threadblock
// descriptors, steps, and per-rank contexts.  One CTA executes one <tb>.  In multi-process mode
// each process launches only its own rank's threadblocks and the rank contexts of peers hold
// pointers into peer memory mapped over NVLink; in single-process emulation all ranks live on
// one device and one cooperative launch runs the threadblocks of every rank.
//
// The reference hands this job to an external NCCL fork (msccl/autosynth/__init__.py:96-114);
// the step semantics below are the ones the XML implies (msccl/language/ir.py:69-83).
#pragma once
#include <cstdint>

namespace msccl {

enum StepType : uint8_t {
  ST_NOP = 0, ST_SEND, ST_RECV, ST_RCS, ST_RRS, ST_RRC, ST_RRCS, ST_CPY, ST_RE
};
enum BufId : uint8_t { BUF_INPUT = 0, BUF_OUTPUT = 1, BUF_SCRATCH = 2 };
enum Proto : int { PROTO_SIMPLE = 0, PROTO_LL = 1, PROTO_LL128 = 2 };
enum DType : int { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2 };

constexpr int kMaxRanks = 16;
constexpr int kMaxChannels = 128;
constexpr int kMaxConns = kMaxRanks * kMaxChannels;   // connection id = chan * kMaxRanks + peer
constexpr int kMaxTbsPerRank = 128;
constexpr int kFifoSlots = 4;                          // tiles in flight per connection
// recv_tail word: tiles produced in the low bits; bit kTailModeShift + (t % kFifoSlots) says whether tile t was stored
// straight into the receiver's buffer (1) or into FIFO slot t % kFifoSlots (0)
constexpr int kTailModeShift = 60;
constexpr unsigned long long kTailCountMask = (1ull << kTailModeShift) - 1;
constexpr int kExecThreads = 512;
constexpr int kMaxDirectCtas = 148;                     // CTAs of the direct (non-interpreted) kernels: one per SM at most
constexpr int kMaxBatch = 8;                            // local reduces fused into one multi-input add

// Error codes written to SyncPage::status[0]; 0 means success.
enum StatusCode : uint32_t {
  STATUS_OK = 0,
  STATUS_TIMEOUT_CREDIT = 1,    // sender waited for a free FIFO slot
  STATUS_TIMEOUT_DATA = 2,      // receiver waited for data
  STATUS_TIMEOUT_DEP = 3,       // waited on another threadblock of the same rank
  STATUS_TIMEOUT_DRAIN = 4,     // waited for the peer to consume the last tiles
  STATUS_ABORTED = 5,           // another threadblock of this rank gave up first
  STATUS_BOUNDS = 6,            // a step addressed memory outside its buffer
  STATUS_TIMEOUT_BARRIER = 7,
};

// One per rank, at the start of the rank's symmetric heap; peers write the flag arrays.
struct alignas(128) SyncPage {
  unsigned long long recv_tail[kMaxConns];   // written by the sending peer: tiles produced
  unsigned long long send_head[kMaxConns];   // written by the receiving peer: tiles consumed
  unsigned long long recv_seq[kMaxConns];    // local: tiles this rank has consumed so far
  unsigned long long send_seq[kMaxConns];    // local: tiles this rank has produced so far
  unsigned long long recv_posted[kMaxConns]; // written by the receiving peer: tiles it has opened for stores into its buffers
  unsigned long long progress[kMaxTbsPerRank];  // (epoch, iteration, step+1) of each threadblock
  // cross-rank barrier of the direct kernels, one lane per CTA: peers write [cta][their rank]
  unsigned long long cta_barrier[kMaxDirectCtas][kMaxRanks];
  unsigned long long cta_epoch[kMaxDirectCtas];  // local: barriers completed by each CTA lane
  unsigned long long ll_epoch;                   // local: one-shot LL launches completed
  unsigned long long exec_epoch;                 // local: interpreter launches completed
  unsigned int ll_done;                          // local: CTAs of the running one-shot launch that finished
  unsigned int exec_done;                        // local: CTAs of the running interpreter launch that finished
  unsigned int abort_flag;                      // local: set when any threadblock gives up
  unsigned int status[7];                       // code, rank, tb, step, iteration, aux0, aux1
};

// Step flags.  A send whose matching receive is `r` or `rcs` may store straight into the receiver's
// destination slot instead of the FIFO (the receiver then finds the data in place).  It does so for a tile
// when ExecArgs::direct_mask covers the receiving buffer and the receiver has already opened the slot;
// otherwise the tile takes the FIFO.  The sender says which in the upper bits of the tile counter.
enum StepFlags : uint8_t {
  SF_DIRECT_SEND = 1,   // the receiver's slot is (rbuf, roff) on the peer
  SF_DIRECT_RECV = 2,   // this receive may find its data already stored in (dstbuf, dstoff)
};

struct alignas(16) DevStep {    // 32 bytes, copied as two 16-byte vectors
  uint8_t type, srcbuf, dstbuf, hasdep;
  int16_t depid, deps;          // wait for threadblock depid (of this rank) to finish step deps; -1: none
  int32_t srcoff, dstoff, cnt;  // chunk units, aliases of in-place collectives already resolved
  uint8_t flags;                // StepFlags
  uint8_t rbuf;                 // SF_DIRECT_SEND: buffer of the matching receive on the peer
  uint8_t batch;                // >1: this and the next batch-1 steps (`re` into this step's dst, or `nop`) run as one
                                //     multi-input add with one store
  uint8_t pad0;
  int32_t roff;                 // SF_DIRECT_SEND: chunk offset of the matching receive on the peer
  uint16_t opens_after;         // receives of this threadblock whose slots may be opened once this step has completed
  uint16_t opens_before;        // receives opened by this (receive) step itself, after its dependency wait
};

struct alignas(16) DevTb {      // 64 bytes
  int16_t rank, tb_in_rank, send_peer, recv_peer;
  int32_t chan, nsteps, step_begin;
  int32_t tbs_in_rank;                    // threadblocks this rank runs in the plan
  int32_t send_conn, recv_conn;           // index into the flag arrays (-1: none)
  long long send_fifo_off, recv_fifo_off;  // byte offset of the connection's slots in the receiver's FIFO area
  // Opening receive slots for stores from the sender (see exec_kernel.cu).  Every receive step of an iteration is
  // opened exactly once, in step order: opens_at_start of them when the iteration begins, the others by the
  // opens_after / opens_before counts of the steps.  opens_at_start == nrecv means nothing on this GPU touches the
  // slots before the receives, and all iterations are opened when the kernel starts.
  int32_t opens_at_start;
  int32_t recv_bufmask;                   // bit b: some SF_DIRECT_RECV step of this threadblock lands in buffer b
  int32_t nrecv;                          // receive steps per iteration
  int32_t pad0;
};

// Per-rank addresses as seen from the launching process.
struct RankCtx {
  SyncPage* sync;        // rank's sync page (peer memory for other ranks)
  char* fifo;            // rank's FIFO area
  void* buf[3];          // input / output / scratch (only meaningful for ranks this process runs)
  long long buf_elems[3];
};

struct ExecArgs {
  const DevTb* tbs;
  const DevStep* steps;
  const RankCtx* ranks;
  long long chunk_elems;      // elements per chunk
  long long tile_elems;       // elements of each chunk processed per iteration
  long long slot_bytes;       // FIFO slot size
  int iterations;
  int nranks;
  unsigned long long timeout_ns;
  int first_tb;               // CTA b executes tbs[first_tb + b]
  int bufs_from_args;         // 1: use local_buf below (one rank per process); 0: ranks[rank].buf (emulation)
  void* local_buf[3];         // input / output / scratch of the launching rank
  long long local_elems[3];   // their sizes in elements (bounds of every step are checked against them)
  unsigned long long epoch_base;   // added to the launch epoch kept in the sync page (callers that clear the page
                                   // between launches pass a counter of their own so that flags never repeat)
  // Stores into a peer's buffers (SF_DIRECT_*).  One rank per process: buffer b of rank p is
  // peer_heap[p] + sym_off[b], valid when bit b of direct_mask is set (the tensor lies at the same offset of every
  // rank's symmetric heap).  Emulation: ranks[p].buf[b].
  char* peer_heap[kMaxRanks];
  long long sym_off[3];
  int direct_mask;
  int wait_mode;              // 0: warps pick up thread 0's verdict by polling shared memory; 1: at a CTA barrier
  // Optional step trace: 6 words per (threadblock, step): first start, last end, total ns waiting, moving (up to the
  // barrier that ends the step) and signalling; the sixth word is spare.
  unsigned long long* trace;
  int trace_steps;            // steps per threadblock the trace has room for
};

static_assert(sizeof(DevStep) == 32 && sizeof(DevTb) == 64, "layout shared with msccl/runtime/plan.py");

}  // namespace msccl
