// Python bindings of the native runtime (module msccl.runtime._msccl_native).
//
// The surface is pointer based on purpose: device addresses and streams cross the boundary as
// integers, so the module does not depend on PyTorch's C++ ABI and any tensor library that can
// hand out a device pointer can drive it.
#include <cuda_runtime.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "fused_tp.h"
#include "gemm_sm100.h"
#include "moe_a2a.h"
#include "msccl_device.h"
#include "symm_mem.h"

namespace py = pybind11;

namespace msccl {
cudaError_t launch_exec(const ExecArgs& args, int dtype, int proto, int width, int grid, cudaStream_t stream, bool cooperative);
int max_coresident_ctas(int dtype, int proto, int width);
cudaError_t launch_twoshot_allreduce(char* const* heap_bases, char* mc_base, long long offset, long long bytes, int dtype,
                                     int rank, int nranks, SyncPage* const* syncs, unsigned long long timeout_ns, int ctas,
                                     cudaStream_t stream, void* rs_out, bool pipelined);
cudaError_t launch_push(const void* src, bool same_src, char* const* heap_bases, char* mc_base, long long dst_offset,
                        long long block_bytes, int rank, int nranks, SyncPage* const* syncs, unsigned long long timeout_ns,
                        int ctas, cudaStream_t stream);
cudaError_t launch_oneshot(const void* in, void* out, char* const* staging, long long bytes, long long slot_bytes, int dtype,
                           int rank, int nranks, SyncPage* sync, unsigned long long timeout_ns, int ctas, int mode,
                           cudaStream_t stream);
}  // namespace msccl

namespace {

using msccl::SyncPage;

void check_rt(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + " failed: " + cudaGetErrorString(e));
}

cudaStream_t as_stream(uintptr_t s) { return reinterpret_cast<cudaStream_t>(s); }

uintptr_t device_malloc(size_t bytes, bool zero) {
  void* p = nullptr;
  check_rt(cudaMalloc(&p, bytes), "cudaMalloc");
  if (zero) check_rt(cudaMemset(p, 0, bytes), "cudaMemset");
  return reinterpret_cast<uintptr_t>(p);
}

void device_free(uintptr_t p) { cudaFree(reinterpret_cast<void*>(p)); }

void device_memset(uintptr_t p, int value, size_t bytes) {
  check_rt(cudaMemset(reinterpret_cast<void*>(p), value, bytes), "cudaMemset");
  check_rt(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
}

uintptr_t upload(const py::bytes& data) {
  std::string s = data;
  void* p = nullptr;
  check_rt(cudaMalloc(&p, s.size() ? s.size() : 16), "cudaMalloc");
  check_rt(cudaMemcpy(p, s.data(), s.size(), cudaMemcpyHostToDevice), "cudaMemcpy");
  return reinterpret_cast<uintptr_t>(p);
}

void upload_into(uintptr_t dst, const py::bytes& data, uintptr_t stream) {
  std::string s = data;
  check_rt(cudaMemcpyAsync(reinterpret_cast<void*>(dst), s.data(), s.size(), cudaMemcpyHostToDevice, as_stream(stream)),
           "cudaMemcpyAsync");
  check_rt(cudaStreamSynchronize(as_stream(stream)), "cudaStreamSynchronize");
}

py::bytes download(uintptr_t src, size_t bytes) {
  std::string s(bytes, '\0');
  check_rt(cudaMemcpy(s.data(), reinterpret_cast<void*>(src), bytes, cudaMemcpyDeviceToHost), "cudaMemcpy");
  return py::bytes(s);
}

// status words of a sync page: [code, rank, tb, step, iteration, aux0, aux1]
std::vector<unsigned int> read_status(uintptr_t sync_page) {
  std::vector<unsigned int> out(7);
  auto* page = reinterpret_cast<SyncPage*>(sync_page);
  check_rt(cudaMemcpy(out.data(), page->status, sizeof(unsigned int) * 7, cudaMemcpyDeviceToHost), "cudaMemcpy(status)");
  return out;
}

void clear_status(uintptr_t sync_page) {
  auto* page = reinterpret_cast<SyncPage*>(sync_page);
  check_rt(cudaMemset(&page->abort_flag, 0, sizeof(unsigned int) * 8), "cudaMemset(status)");
}

// One interpreter launch.  `geom` = [chunk_elems, tile_elems, slot_bytes, iterations, nranks, first_tb, grid, dtype, proto,
// width]; `bufs` = [in, out, scratch] pointers of the launching rank (one rank per process; empty in emulation, where the
// rank table carries them) and `elems` their sizes in elements; `peer_heaps` / `sym_off` / `direct_mask` describe which of
// the buffers lie at the same offset of every rank's symmetric heap (stores straight into a peer's buffer); `trace` is 0
// or a zeroed device array of grid x trace_steps x 6 words.
void launch(uintptr_t tbs, uintptr_t steps, uintptr_t ranks, const std::vector<long long>& geom, unsigned long long timeout_ns,
            uintptr_t stream, bool cooperative, const std::vector<uintptr_t>& bufs, const std::vector<long long>& elems,
            const std::vector<uintptr_t>& peer_heaps, const std::vector<long long>& sym_off, int direct_mask,
            unsigned long long epoch_base, uintptr_t trace, int trace_steps, int wait_mode) {
  if (geom.size() != 10) throw std::runtime_error("launch: geometry vector must have 10 entries");
  if (!bufs.empty() && (bufs.size() != 3 || elems.size() != 3)) throw std::runtime_error("launch: three buffers and three sizes");
  if (peer_heaps.size() > static_cast<size_t>(msccl::kMaxRanks) || (!sym_off.empty() && sym_off.size() != 3))
    throw std::runtime_error("launch: bad peer table");
  msccl::ExecArgs a;
  std::memset(&a, 0, sizeof(a));
  a.tbs = reinterpret_cast<const msccl::DevTb*>(tbs);
  a.steps = reinterpret_cast<const msccl::DevStep*>(steps);
  a.ranks = reinterpret_cast<const msccl::RankCtx*>(ranks);
  a.chunk_elems = geom[0];
  a.tile_elems = geom[1];
  a.slot_bytes = geom[2];
  a.iterations = static_cast<int>(geom[3]);
  a.nranks = static_cast<int>(geom[4]);
  a.timeout_ns = timeout_ns;
  a.first_tb = static_cast<int>(geom[5]);
  a.bufs_from_args = bufs.empty() ? 0 : 1;
  for (size_t b = 0; b < bufs.size(); ++b) {
    a.local_buf[b] = reinterpret_cast<void*>(bufs[b]);
    a.local_elems[b] = elems[b];
  }
  for (size_t r = 0; r < peer_heaps.size(); ++r) a.peer_heap[r] = reinterpret_cast<char*>(peer_heaps[r]);
  for (int b = 0; b < 3; ++b) a.sym_off[b] = sym_off.empty() ? -1 : sym_off[b];
  a.direct_mask = direct_mask;
  a.epoch_base = epoch_base;
  a.trace = reinterpret_cast<unsigned long long*>(trace);
  a.trace_steps = trace_steps;
  a.wait_mode = wait_mode;
  check_rt(msccl::launch_exec(a, static_cast<int>(geom[7]), static_cast<int>(geom[8]), static_cast<int>(geom[9]),
                              static_cast<int>(geom[6]), as_stream(stream), cooperative),
           "launch of the MSCCL-IR executor kernel");
}

py::dict layout() {
  py::dict d;
  d["sizeof_SyncPage"] = sizeof(SyncPage);
  d["sizeof_DevStep"] = sizeof(msccl::DevStep);
  d["sizeof_DevTb"] = sizeof(msccl::DevTb);
  d["sizeof_RankCtx"] = sizeof(msccl::RankCtx);
  d["kMaxRanks"] = msccl::kMaxRanks;
  d["kMaxChannels"] = msccl::kMaxChannels;
  d["kMaxTbsPerRank"] = msccl::kMaxTbsPerRank;
  d["kFifoSlots"] = msccl::kFifoSlots;
  d["kExecThreads"] = msccl::kExecThreads;
  d["kMaxBatch"] = msccl::kMaxBatch;
  d["kMaxDirectCtas"] = msccl::kMaxDirectCtas;
  return d;
}

py::dict vmm_create(int device, size_t size, size_t granularity) {
  msccl::VmmBlock b = msccl::vmm_create(device, size, granularity);
  py::dict d;
  d["ptr"] = reinterpret_cast<uintptr_t>(b.ptr);
  d["size"] = b.size;
  d["handle"] = b.handle;
  d["fd"] = b.fd;
  return d;
}

py::dict vmm_import(int device, int fd, size_t size, size_t granularity) {
  msccl::VmmBlock b = msccl::vmm_import(device, fd, size, granularity);
  py::dict d;
  d["ptr"] = reinterpret_cast<uintptr_t>(b.ptr);
  d["size"] = b.size;
  d["handle"] = b.handle;
  d["fd"] = b.fd;
  return d;
}

void vmm_release(uintptr_t ptr, size_t size, unsigned long long handle, int fd) {
  msccl::VmmBlock b;
  b.ptr = reinterpret_cast<void*>(ptr);
  b.size = size;
  b.handle = handle;
  b.fd = fd;
  msccl::vmm_release(b);
}

std::vector<SyncPage*> sync_list(const std::vector<uintptr_t>& v) {
  std::vector<SyncPage*> out;
  for (auto p : v) out.push_back(reinterpret_cast<SyncPage*>(p));
  return out;
}

}  // namespace

PYBIND11_MODULE(_msccl_native, m) {
  m.doc() = "Native runtime of the msccl B200 executor";
  m.def("layout", &layout);
  m.def("device_malloc", &device_malloc, py::arg("bytes"), py::arg("zero") = true);
  m.def("device_free", &device_free);
  m.def("device_memset", &device_memset);
  m.def("upload", &upload);
  m.def("upload_into", &upload_into);
  m.def("download", &download);
  m.def("read_status", &read_status);
  m.def("clear_status", &clear_status);
  m.def("launch", &launch, py::arg("tbs"), py::arg("steps"), py::arg("ranks"), py::arg("geom"), py::arg("timeout_ns"),
        py::arg("stream"), py::arg("cooperative"), py::arg("bufs") = std::vector<uintptr_t>(),
        py::arg("elems") = std::vector<long long>(), py::arg("peer_heaps") = std::vector<uintptr_t>(),
        py::arg("sym_off") = std::vector<long long>(), py::arg("direct_mask") = 0, py::arg("epoch_base") = 0ull,
        py::arg("trace") = 0, py::arg("trace_steps") = 0, py::arg("wait_mode") = 0);
  m.def("max_coresident_ctas", &msccl::max_coresident_ctas);

  m.def("vmm_granularity", &msccl::vmm_granularity);
  m.def("multicast_supported", &msccl::multicast_supported);
  m.def("vmm_create", &vmm_create);
  m.def("vmm_import", &vmm_import);
  m.def("vmm_release", &vmm_release);
  m.def("multicast_create", [](int n, size_t size) {
    int fd = -1;
    unsigned long long h = msccl::multicast_create(n, size, &fd);
    return py::make_tuple(h, fd);
  });
  m.def("multicast_import", &msccl::multicast_import);
  m.def("multicast_add_device", &msccl::multicast_add_device);
  m.def("multicast_bind", &msccl::multicast_bind);
  m.def("multicast_map", [](unsigned long long mc, size_t size, size_t gran, int dev) {
    return reinterpret_cast<uintptr_t>(msccl::multicast_map(mc, size, gran, dev));
  });
  m.def("multicast_unmap", [](uintptr_t p, size_t size, unsigned long long mc, int dev) {
    msccl::multicast_unmap(reinterpret_cast<void*>(p), size, mc, dev);
  });
  m.def("ipc_export", [](uintptr_t p) { return py::bytes(msccl::ipc_export(reinterpret_cast<void*>(p))); });
  m.def("ipc_import", [](const py::bytes& b) { return reinterpret_cast<uintptr_t>(msccl::ipc_import(std::string(b))); });
  m.def("ipc_close", [](uintptr_t p) { msccl::ipc_close(reinterpret_cast<void*>(p)); });
  m.def("fd_socket_open", &msccl::fd_socket_open);
  m.def("fd_socket_send", &msccl::fd_socket_send);
  m.def("fd_socket_recv", [](int sock) {
    int tag = -1;
    int fd = -1;
    {
      py::gil_scoped_release release;      // blocking receive; Python objects are built after re-acquiring
      fd = msccl::fd_socket_recv(sock, &tag);
    }
    return py::make_tuple(fd, tag);
  });
  m.def("fd_socket_close", &msccl::fd_socket_close);

  // D = epilogue(A[M,K] * B[N,K]^T) with the tcgen05 kernel; error_words: 4 ints of device memory (or 0).
  m.def("gemm_bf16", [](uintptr_t a, uintptr_t b, uintptr_t d, int M, int N, int K, int lda, int ldb, int ldd, int epilogue,
                         int bn, uintptr_t error_words, int max_ctas, uintptr_t stream) {
    check_rt(msccl::sm100::gemm_bf16(reinterpret_cast<const void*>(a), reinterpret_cast<const void*>(b),
                                     reinterpret_cast<void*>(d), M, N, K, lda, ldb, ldd, epilogue, bn,
                                     reinterpret_cast<int*>(error_words), max_ctas, as_stream(stream)),
             "launch of the tcgen05 GEMM kernel");
  });
  // The same product on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles).
  m.def("gemm_bf16_2cta", [](uintptr_t a, uintptr_t b, uintptr_t d, int M, int N, int K, int lda, int ldb, int ldd, int epilogue,
                              uintptr_t error_words, int max_pairs, uintptr_t stream) {
    check_rt(msccl::sm100::gemm_bf16_2cta(reinterpret_cast<const void*>(a), reinterpret_cast<const void*>(b),
                                          reinterpret_cast<void*>(d), M, N, K, lda, ldb, ldd, epilogue,
                                          reinterpret_cast<int*>(error_words), max_pairs, as_stream(stream)),
             "launch of the two-CTA tcgen05 GEMM kernel");
  });
  m.def("max_cta_pairs", [](int epilogue) { return msccl::sm100::max_cta_pairs(epilogue); });
  // D (bf16) = block-scaled e4m3 A[M,K] * B[N,K]^T; sfa / sfb: UE8M0 scales in 512-byte blocks per (128 rows, 128 K).
  m.def("gemm_mxfp8", [](uintptr_t a, uintptr_t sfa, uintptr_t b, uintptr_t sfb, uintptr_t d, int M, int N, int K, int lda,
                          int ldb, int ldd, uintptr_t error_words, int max_ctas, uintptr_t stream) {
    check_rt(msccl::sm100::gemm_mxfp8(reinterpret_cast<const void*>(a), reinterpret_cast<const void*>(sfa),
                                      reinterpret_cast<const void*>(b), reinterpret_cast<const void*>(sfb),
                                      reinterpret_cast<void*>(d), M, N, K, lda, ldb, ldd,
                                      reinterpret_cast<int*>(error_words), max_ctas, as_stream(stream)),
             "launch of the block-scaled fp8 GEMM kernel");
  });
  m.def("gemm_mxfp8_2cta", [](uintptr_t a, uintptr_t sfa, uintptr_t b, uintptr_t sfb, uintptr_t d, int M, int N, int K, int lda,
                               int ldb, int ldd, uintptr_t error_words, int max_pairs, uintptr_t stream) {
    check_rt(msccl::sm100::gemm_mxfp8_2cta(reinterpret_cast<const void*>(a), reinterpret_cast<const void*>(sfa),
                                           reinterpret_cast<const void*>(b), reinterpret_cast<const void*>(sfb),
                                           reinterpret_cast<void*>(d), M, N, K, lda, ldb, ldd,
                                           reinterpret_cast<int*>(error_words), max_pairs, as_stream(stream)),
             "launch of the two-CTA block-scaled fp8 GEMM kernel");
  });
  // Fused all-gather -> GEMM (epilogue 0: plain, 1: SwiGLU).  heap_ptrs: every rank's heap base in this process.
  m.def("ag_gemm", [](uintptr_t x_local, uintptr_t b, uintptr_t d, int rows_per_rank, int N, int K, int ldb, int ldd, int rank,
                       int nranks, int comm_ctas, uintptr_t heap_bases_dev, std::vector<uintptr_t> heap_ptrs, size_t off_fused,
                       uintptr_t mc_base, size_t gathered_off, size_t gathered_bytes, uintptr_t error_words, int epilogue,
                       int grid, int tuning, uintptr_t order, uintptr_t stream, bool pair) {
    msccl::sm100::AgGemmArgs g;
    std::memset(&g, 0, sizeof(g));
    g.x_local = reinterpret_cast<const void*>(x_local);
    g.b = reinterpret_cast<const void*>(b);
    g.d = reinterpret_cast<void*>(d);
    g.rows_per_rank = rows_per_rank; g.N = N; g.K = K; g.ldb = ldb; g.ldd = ldd;
    g.rank = rank; g.nranks = nranks; g.comm_ctas = comm_ctas; g.tuning = tuning;
    g.order = reinterpret_cast<const int*>(order);
    g.heap_bases = reinterpret_cast<char* const*>(heap_bases_dev);
    if (static_cast<int>(heap_ptrs.size()) != nranks || nranks > msccl::sm100::kFusedMaxRanks) throw std::runtime_error("bad rank count");
    for (int r = 0; r < nranks; ++r) {
      g.heap_bases_host[r] = reinterpret_cast<char*>(heap_ptrs[r]);
      g.pages[r] = reinterpret_cast<msccl::sm100::FusedPage*>(heap_ptrs[r] + off_fused);
    }
    g.mc_base = reinterpret_cast<char*>(mc_base);
    g.gathered_off = gathered_off;
    g.gathered_bytes = gathered_bytes;
    g.error_words = reinterpret_cast<int*>(error_words);
    if (pair) check_rt(msccl::sm100::launch_ag_gemm_2cta(g, epilogue, grid, as_stream(stream)), "launch of the fused all-gather GEMM kernel (CTA pairs)");
    else check_rt(msccl::sm100::launch_ag_gemm(g, epilogue, grid, as_stream(stream)), "launch of the fused all-gather GEMM kernel");
  }, py::arg("x_local"), py::arg("b"), py::arg("d"), py::arg("rows_per_rank"), py::arg("N"), py::arg("K"), py::arg("ldb"), py::arg("ldd"),
     py::arg("rank"), py::arg("nranks"), py::arg("comm_ctas"), py::arg("heap_bases_dev"), py::arg("heap_ptrs"), py::arg("off_fused"),
     py::arg("mc_base"), py::arg("gathered_off"), py::arg("gathered_bytes"), py::arg("error_words"), py::arg("epilogue"), py::arg("grid"),
     py::arg("tuning"), py::arg("order"), py::arg("stream"), py::arg("pair") = false);
  // Fused GEMM -> reduce-scatter.
  m.def("gemm_rs", [](uintptr_t a, uintptr_t b, uintptr_t out, int rows_per_rank, int N, int K, int lda, int ldb, int rank,
                       int nranks, uintptr_t heap_bases_dev, std::vector<uintptr_t> heap_ptrs, size_t off_fused, size_t partial_off,
                       uintptr_t error_words, int grid, uintptr_t order, uintptr_t reduce_order, int reduce_ctas,
                       uintptr_t stream, bool pair) {
    msccl::sm100::GemmRsArgs g;
    std::memset(&g, 0, sizeof(g));
    g.a = reinterpret_cast<const void*>(a);
    g.b = reinterpret_cast<const void*>(b);
    g.out = reinterpret_cast<void*>(out);
    g.rows_per_rank = rows_per_rank; g.N = N; g.K = K; g.lda = lda; g.ldb = ldb;
    g.rank = rank; g.nranks = nranks;
    g.heap_bases = reinterpret_cast<char* const*>(heap_bases_dev);
    if (static_cast<int>(heap_ptrs.size()) != nranks || nranks > msccl::sm100::kFusedMaxRanks) throw std::runtime_error("bad rank count");
    for (int r = 0; r < nranks; ++r) g.pages[r] = reinterpret_cast<msccl::sm100::FusedPage*>(heap_ptrs[r] + off_fused);
    g.partial_off = partial_off;
    g.error_words = reinterpret_cast<int*>(error_words);
    g.order = reinterpret_cast<const int*>(order);
    g.reduce_order = reinterpret_cast<const int*>(reduce_order);
    g.reduce_ctas = reduce_ctas;
    if (pair) check_rt(msccl::sm100::launch_gemm_rs_2cta(g, grid, as_stream(stream)), "launch of the fused GEMM reduce-scatter kernel (CTA pairs)");
    else check_rt(msccl::sm100::launch_gemm_rs(g, grid, as_stream(stream)), "launch of the fused GEMM reduce-scatter kernel");
  }, py::arg("a"), py::arg("b"), py::arg("out"), py::arg("rows_per_rank"), py::arg("N"), py::arg("K"), py::arg("lda"), py::arg("ldb"),
     py::arg("rank"), py::arg("nranks"), py::arg("heap_bases_dev"), py::arg("heap_ptrs"), py::arg("off_fused"), py::arg("partial_off"),
     py::arg("error_words"), py::arg("grid"), py::arg("order"), py::arg("reduce_order"), py::arg("reduce_ctas"), py::arg("stream"),
     py::arg("pair") = false);
  // The same two kernels on block-scaled fp8 operands (e4m3 values + packed UE8M0 scale blocks).
  m.def("ag_gemm_mxfp8", [](uintptr_t x_local, uintptr_t sf_local, uintptr_t b, uintptr_t sfb, uintptr_t d, int rows_per_rank, int N,
                             int K, int ldb, int ldd, int rank, int nranks, int comm_ctas, uintptr_t heap_bases_dev,
                             std::vector<uintptr_t> heap_ptrs, size_t off_fused, uintptr_t mc_base, size_t gathered_off,
                             size_t gathered_bytes, uintptr_t error_words, int epilogue, int grid, uintptr_t order, uintptr_t stream, bool pair) {
    msccl::sm100::AgGemmF8Args g;
    std::memset(&g, 0, sizeof(g));
    g.x_local = reinterpret_cast<const void*>(x_local);
    g.sf_local = reinterpret_cast<const void*>(sf_local);
    g.b = reinterpret_cast<const void*>(b);
    g.sfb = reinterpret_cast<const void*>(sfb);
    g.d = reinterpret_cast<void*>(d);
    g.rows_per_rank = rows_per_rank; g.N = N; g.K = K; g.ldb = ldb; g.ldd = ldd;
    g.rank = rank; g.nranks = nranks; g.comm_ctas = comm_ctas;
    g.order = reinterpret_cast<const int*>(order);
    g.heap_bases = reinterpret_cast<char* const*>(heap_bases_dev);
    if (static_cast<int>(heap_ptrs.size()) != nranks || nranks > msccl::sm100::kFusedMaxRanks) throw std::runtime_error("bad rank count");
    for (int r = 0; r < nranks; ++r) {
      g.heap_bases_host[r] = reinterpret_cast<char*>(heap_ptrs[r]);
      g.pages[r] = reinterpret_cast<msccl::sm100::FusedPage*>(heap_ptrs[r] + off_fused);
    }
    g.mc_base = reinterpret_cast<char*>(mc_base);
    g.gathered_off = gathered_off;
    g.gathered_bytes = gathered_bytes;
    g.error_words = reinterpret_cast<int*>(error_words);
    if (pair) check_rt(msccl::sm100::launch_ag_gemm_mxfp8_2cta(g, epilogue, grid, as_stream(stream)), "launch of the fused fp8 all-gather GEMM kernel (pairs)");
    else check_rt(msccl::sm100::launch_ag_gemm_mxfp8(g, epilogue, grid, as_stream(stream)), "launch of the fused fp8 all-gather GEMM kernel");
  });
  m.def("gemm_rs_mxfp8", [](uintptr_t a, uintptr_t sfa, uintptr_t b, uintptr_t sfb, uintptr_t out, int rows_per_rank, int N, int K,
                             int lda, int ldb, int rank, int nranks, uintptr_t heap_bases_dev, std::vector<uintptr_t> heap_ptrs,
                             size_t off_fused, size_t partial_off, uintptr_t error_words, int grid, uintptr_t order,
                             uintptr_t reduce_order, int reduce_ctas, uintptr_t stream, bool pair) {
    msccl::sm100::GemmRsF8Args g;
    std::memset(&g, 0, sizeof(g));
    g.a = reinterpret_cast<const void*>(a);
    g.sfa = reinterpret_cast<const void*>(sfa);
    g.b = reinterpret_cast<const void*>(b);
    g.sfb = reinterpret_cast<const void*>(sfb);
    g.out = reinterpret_cast<void*>(out);
    g.rows_per_rank = rows_per_rank; g.N = N; g.K = K; g.lda = lda; g.ldb = ldb;
    g.rank = rank; g.nranks = nranks;
    g.heap_bases = reinterpret_cast<char* const*>(heap_bases_dev);
    if (static_cast<int>(heap_ptrs.size()) != nranks || nranks > msccl::sm100::kFusedMaxRanks) throw std::runtime_error("bad rank count");
    for (int r = 0; r < nranks; ++r) g.pages[r] = reinterpret_cast<msccl::sm100::FusedPage*>(heap_ptrs[r] + off_fused);
    g.partial_off = partial_off;
    g.error_words = reinterpret_cast<int*>(error_words);
    g.order = reinterpret_cast<const int*>(order);
    g.reduce_order = reinterpret_cast<const int*>(reduce_order);
    g.reduce_ctas = reduce_ctas;
    if (pair) check_rt(msccl::sm100::launch_gemm_rs_mxfp8_2cta(g, grid, as_stream(stream)), "launch of the fused fp8 GEMM reduce-scatter kernel (pairs)");
    else check_rt(msccl::sm100::launch_gemm_rs_mxfp8(g, grid, as_stream(stream)), "launch of the fused fp8 GEMM reduce-scatter kernel");
  });
  m.def("sm_count", &msccl::sm100::sm_count);
  // bf16 [rows, K] -> e4m3 values and packed UE8M0 scale blocks (one pass)
  m.def("quantize_mxfp8", [](uintptr_t x, uintptr_t q, uintptr_t sf, int rows, int K, long long ldx, uintptr_t stream) {
    check_rt(msccl::sm100::quantize_mxfp8(reinterpret_cast<const void*>(x), reinterpret_cast<void*>(q), reinterpret_cast<void*>(sf),
                                          rows, K, ldx, as_stream(stream)),
             "launch of the MX quantisation kernel");
  });
  // Fused MoE: phase 0 = dispatch + grouped gate/up GEMM (SwiGLU), phase 1 = grouped down GEMM + combine.
  // geom = [rank, nranks, tokens, topk, hidden, ffn, num_experts, local_experts, cap, comm_ctas]
  // layout = [counts_off, meta_off, dispatch_off, combine_off, counts_parity, meta_parity, dispatch_parity, combine_parity]
  m.def("moe_phase", [](int phase, std::vector<int> geom, std::vector<size_t> layout, uintptr_t heap_bases_dev,
                         std::vector<uintptr_t> heap_ptrs, size_t off_fused, size_t moe_off, uintptr_t x, uintptr_t sorted_copy,
                         uintptr_t expert_start, uintptr_t copy_weight, uintptr_t w_gate_up, uintptr_t h, uintptr_t w_down,
                         uintptr_t y, uintptr_t error_words, int grid, uintptr_t stream, bool pair) {
    if (geom.size() != 10 || layout.size() != 8) throw std::runtime_error("bad geometry/layout vectors");
    msccl::sm100::MoeArgs g;
    std::memset(&g, 0, sizeof(g));
    g.rank = geom[0]; g.nranks = geom[1]; g.tokens = geom[2]; g.topk = geom[3]; g.hidden = geom[4]; g.ffn = geom[5];
    g.num_experts = geom[6]; g.local_experts = geom[7]; g.cap = geom[8]; g.comm_ctas = geom[9];
    if (static_cast<int>(heap_ptrs.size()) != g.nranks || g.nranks > msccl::sm100::kFusedMaxRanks) throw std::runtime_error("bad rank count");
    g.heap_bases = reinterpret_cast<char* const*>(heap_bases_dev);
    for (int r = 0; r < g.nranks; ++r) {
      g.heap_bases_host[r] = reinterpret_cast<char*>(heap_ptrs[r]);
      g.pages[r] = reinterpret_cast<msccl::sm100::FusedPage*>(heap_ptrs[r] + off_fused);
    }
    g.moe_off = moe_off;
    g.lay.counts_off = layout[0]; g.lay.meta_off = layout[1]; g.lay.dispatch_off = layout[2]; g.lay.combine_off = layout[3];
    g.lay.counts_parity = layout[4]; g.lay.meta_parity = layout[5]; g.lay.dispatch_parity = layout[6]; g.lay.combine_parity = layout[7];
    g.x = reinterpret_cast<const void*>(x);
    g.sorted_copy = reinterpret_cast<const int*>(sorted_copy);
    g.expert_start = reinterpret_cast<const int*>(expert_start);
    g.copy_weight = reinterpret_cast<const float*>(copy_weight);
    g.w_gate_up = reinterpret_cast<const void*>(w_gate_up);
    g.h = reinterpret_cast<void*>(h);
    g.w_down = reinterpret_cast<const void*>(w_down);
    g.y = reinterpret_cast<void*>(y);
    g.error_words = reinterpret_cast<int*>(error_words);
    if (pair) {
      if (phase == 0) check_rt(msccl::sm100::launch_moe_dispatch_gemm_2cta(g, grid, as_stream(stream)), "launch of the MoE dispatch kernel (pairs)");
      else check_rt(msccl::sm100::launch_moe_gemm_combine_2cta(g, grid, as_stream(stream)), "launch of the MoE combine kernel (pairs)");
    } else {
      if (phase == 0) check_rt(msccl::sm100::launch_moe_dispatch_gemm(g, grid, as_stream(stream)), "launch of the MoE dispatch kernel");
      else check_rt(msccl::sm100::launch_moe_gemm_combine(g, grid, as_stream(stream)), "launch of the MoE combine kernel");
    }
  }, py::arg("phase"), py::arg("geom"), py::arg("layout"), py::arg("heap_bases_dev"), py::arg("heap_ptrs"), py::arg("off_fused"),
     py::arg("moe_off"), py::arg("x"), py::arg("sorted_copy"), py::arg("expert_start"), py::arg("copy_weight"), py::arg("w_gate_up"),
     py::arg("h"), py::arg("w_down"), py::arg("y"), py::arg("error_words"), py::arg("grid"), py::arg("stream"), py::arg("pair") = false);
  // MoE routing on the device: top-k of the gate logits, and the stable sort of the token copies by expert.
  m.def("moe_topk", [](uintptr_t logits, int tokens, int experts, int k, uintptr_t out_experts, uintptr_t out_weights, uintptr_t stream) {
    check_rt(msccl::sm100::launch_moe_topk(reinterpret_cast<const float*>(logits), tokens, experts, k, reinterpret_cast<int*>(out_experts),
                                           reinterpret_cast<float*>(out_weights), as_stream(stream)), "launch of the MoE top-k kernel");
  });
  m.def("moe_sort", [](uintptr_t expert_of, int n, int experts, uintptr_t sorted_copy, uintptr_t expert_start, uintptr_t stream) {
    check_rt(msccl::sm100::launch_moe_sort(reinterpret_cast<const int*>(expert_of), n, experts, reinterpret_cast<int*>(sorted_copy),
                                           reinterpret_cast<int*>(expert_start), as_stream(stream)), "launch of the MoE sort kernel");
  });
  // In-place all-reduce of `bytes` at `offset` of every rank's symmetric heap.  mc_base = 0
  // selects peer loads/stores, otherwise the NVLink multicast window is used.
  m.def("twoshot_allreduce", [](uintptr_t heap_bases_dev, uintptr_t mc_base, long long offset, long long bytes, int dtype,
                                 int rank, int nranks, uintptr_t syncs_dev, unsigned long long timeout_ns, int ctas,
                                 uintptr_t stream, uintptr_t rs_out, bool pipelined) {
    check_rt(msccl::launch_twoshot_allreduce(reinterpret_cast<char* const*>(heap_bases_dev), reinterpret_cast<char*>(mc_base),
                                             offset, bytes, dtype, rank, nranks,
                                             reinterpret_cast<SyncPage* const*>(syncs_dev), timeout_ns, ctas, as_stream(stream),
                                             reinterpret_cast<void*>(rs_out), pipelined),
             "launch of the two-shot all-reduce kernel");
  }, py::arg("heap_bases"), py::arg("mc_base"), py::arg("offset"), py::arg("bytes"), py::arg("dtype"), py::arg("rank"),
     py::arg("nranks"), py::arg("syncs"), py::arg("timeout_ns"), py::arg("ctas"), py::arg("stream"), py::arg("rs_out") = 0,
     py::arg("pipelined") = false);
  // All-gather (same_src) or all-to-all: store this rank's block(s) into block `rank` of the buffer
  // at `dst_offset` of every rank's symmetric heap.  mc_base != 0 (all-gather only) uses multimem.st.
  m.def("push_blocks", [](uintptr_t src, bool same_src, uintptr_t heap_bases_dev, uintptr_t mc_base, long long dst_offset,
                           long long block_bytes, int rank, int nranks, uintptr_t syncs_dev, unsigned long long timeout_ns,
                           int ctas, uintptr_t stream) {
    check_rt(msccl::launch_push(reinterpret_cast<const void*>(src), same_src, reinterpret_cast<char* const*>(heap_bases_dev),
                                reinterpret_cast<char*>(mc_base), dst_offset, block_bytes, rank, nranks,
                                reinterpret_cast<SyncPage* const*>(syncs_dev), timeout_ns, ctas, as_stream(stream)),
             "launch of the push kernel");
  });
  // One-shot LL collectives through staging slots on every rank (any device memory).
  // mode: 0 all-reduce, 1 all-gather, 2 reduce-scatter, 3 all-to-all; `bytes` is the size of one block.
  m.def("oneshot", [](uintptr_t in, uintptr_t out, uintptr_t staging_dev, long long bytes, long long slot_bytes, int dtype,
                       int rank, int nranks, uintptr_t sync, unsigned long long timeout_ns, int ctas, int mode,
                       uintptr_t stream) {
    check_rt(msccl::launch_oneshot(reinterpret_cast<const void*>(in), reinterpret_cast<void*>(out),
                                   reinterpret_cast<char* const*>(staging_dev), bytes, slot_bytes, dtype, rank, nranks,
                                   reinterpret_cast<SyncPage*>(sync), timeout_ns, ctas, mode, as_stream(stream)),
             "launch of the one-shot LL kernel");
  });
  m.def("oneshot_allreduce", [](uintptr_t in, uintptr_t out, uintptr_t staging_dev, long long bytes, long long slot_bytes,
                                 int dtype, int rank, int nranks, uintptr_t sync, unsigned long long timeout_ns, int ctas,
                                 uintptr_t stream) {
    check_rt(msccl::launch_oneshot(reinterpret_cast<const void*>(in), reinterpret_cast<void*>(out),
                                   reinterpret_cast<char* const*>(staging_dev), bytes, slot_bytes, dtype, rank, nranks,
                                   reinterpret_cast<SyncPage*>(sync), timeout_ns, ctas, 0, as_stream(stream)),
             "launch of the one-shot all-reduce kernel");
  });
}
