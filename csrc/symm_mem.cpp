// Symmetric memory over NVLink for one-process-per-GPU jobs on a single NVSwitch box.
//
// Each rank allocates one physical block with the CUDA virtual-memory API, exports it as a POSIX
// file descriptor, and passes the descriptor to its peers over a Unix-domain socket
// (SCM_RIGHTS).  Every peer maps the block into its own address space, so kernels can store to
// and load from any rank's heap with ordinary pointers.  Optionally all blocks are bound to one
// NVLink multicast object, which gives the address window used by multimem.* instructions
// (in-switch reduction and broadcast).  A cudaIpc based path is kept for drivers where the
// descriptor export is not permitted.
//
// The driver API is reached through cudaGetDriverEntryPoint, so the module has no link-time
// dependency on libcuda and imports on machines without a GPU.
#include <cuda.h>
#include <cuda_runtime.h>
#include <errno.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "symm_mem.h"

namespace msccl {

namespace {

template <typename Fn> Fn driver_fn(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || p == nullptr || q != cudaDriverEntryPointSuccess)
    throw std::runtime_error(std::string("CUDA driver entry point not available: ") + name);
  return reinterpret_cast<Fn>(p);
}

void check(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return;
  static auto get_name = driver_fn<CUresult (*)(CUresult, const char**)>("cuGetErrorName");
  const char* name = "?";
  get_name(r, &name);
  throw std::runtime_error(std::string(what) + " failed: " + name + " (" + std::to_string(static_cast<int>(r)) + ")");
}

void check_rt(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + " failed: " + cudaGetErrorString(e));
}

size_t round_up(size_t v, size_t g) { return (v + g - 1) / g * g; }

CUmemAllocationProp local_prop(int device) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

void* map_handle(CUmemGenericAllocationHandle handle, size_t size, size_t granularity, int device) {
  static auto reserve = driver_fn<CUresult (*)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long)>("cuMemAddressReserve");
  static auto map = driver_fn<CUresult (*)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long)>("cuMemMap");
  static auto set_access = driver_fn<CUresult (*)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t)>("cuMemSetAccess");
  CUdeviceptr va = 0;
  check(reserve(&va, size, granularity, 0, 0), "cuMemAddressReserve");
  check(map(va, size, 0, handle, 0), "cuMemMap");
  CUmemAccessDesc access;
  memset(&access, 0, sizeof(access));
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  check(set_access(va, size, &access, 1), "cuMemSetAccess");
  return reinterpret_cast<void*>(va);
}

}  // namespace

// ------------------------------------------------------------------------- VMM blocks
size_t vmm_granularity(int device, bool multicast, int num_devices) {
  static auto gran = driver_fn<CUresult (*)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags)>("cuMemGetAllocationGranularity");
  CUmemAllocationProp prop = local_prop(device);
  size_t g = 0;
  check(gran(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
  if (multicast) {
    static auto mc_gran = driver_fn<CUresult (*)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags)>("cuMulticastGetGranularity");
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = num_devices;
    mp.size = g;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    check(mc_gran(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED), "cuMulticastGetGranularity");
    if (mg > g) g = mg;
  }
  return g;
}

bool multicast_supported(int device) {
  try {
    static auto get_attr = driver_fn<CUresult (*)(int*, CUdevice_attribute, CUdevice)>("cuDeviceGetAttribute");
    int v = 0;
    if (get_attr(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device) != CUDA_SUCCESS) return false;
    return v != 0;
  } catch (const std::exception&) {
    return false;
  }
}

VmmBlock vmm_create(int device, size_t size, size_t granularity) {
  static auto create = driver_fn<CUresult (*)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long)>("cuMemCreate");
  static auto do_export = driver_fn<CUresult (*)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long)>("cuMemExportToShareableHandle");
  VmmBlock b;
  b.size = round_up(size, granularity);
  b.granularity = granularity;
  CUmemAllocationProp prop = local_prop(device);
  CUmemGenericAllocationHandle h = 0;
  check(create(&h, b.size, &prop, 0), "cuMemCreate");
  b.handle = static_cast<unsigned long long>(h);
  int fd = -1;
  check(do_export(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
  b.fd = fd;
  b.ptr = map_handle(h, b.size, granularity, device);
  return b;
}

VmmBlock vmm_import(int device, int fd, size_t size, size_t granularity) {
  static auto do_import = driver_fn<CUresult (*)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType)>("cuMemImportFromShareableHandle");
  VmmBlock b;
  b.size = size;
  b.granularity = granularity;
  b.fd = fd;
  CUmemGenericAllocationHandle h = 0;
  check(do_import(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
        "cuMemImportFromShareableHandle");
  b.handle = static_cast<unsigned long long>(h);
  b.ptr = map_handle(h, size, granularity, device);
  return b;
}

void vmm_release(const VmmBlock& b) {
  static auto unmap = driver_fn<CUresult (*)(CUdeviceptr, size_t)>("cuMemUnmap");
  static auto free_va = driver_fn<CUresult (*)(CUdeviceptr, size_t)>("cuMemAddressFree");
  static auto release = driver_fn<CUresult (*)(CUmemGenericAllocationHandle)>("cuMemRelease");
  if (b.ptr != nullptr) {
    unmap(reinterpret_cast<CUdeviceptr>(b.ptr), b.size);
    free_va(reinterpret_cast<CUdeviceptr>(b.ptr), b.size);
  }
  if (b.handle != 0) release(static_cast<CUmemGenericAllocationHandle>(b.handle));
  if (b.fd >= 0) close(b.fd);
}

// -------------------------------------------------------------------------- multicast
unsigned long long multicast_create(int num_devices, size_t size, int* fd_out) {
  static auto create = driver_fn<CUresult (*)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*)>("cuMulticastCreate");
  static auto do_export = driver_fn<CUresult (*)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long)>("cuMemExportToShareableHandle");
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = num_devices;
  mp.size = size;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h = 0;
  check(create(&h, &mp), "cuMulticastCreate");
  int fd = -1;
  check(do_export(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle(multicast)");
  *fd_out = fd;
  return static_cast<unsigned long long>(h);
}

unsigned long long multicast_import(int fd) {
  static auto do_import = driver_fn<CUresult (*)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType)>("cuMemImportFromShareableHandle");
  CUmemGenericAllocationHandle h = 0;
  check(do_import(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
        "cuMemImportFromShareableHandle(multicast)");
  return static_cast<unsigned long long>(h);
}

void multicast_add_device(unsigned long long mc, int device) {
  static auto add = driver_fn<CUresult (*)(CUmemGenericAllocationHandle, CUdevice)>("cuMulticastAddDevice");
  check(add(static_cast<CUmemGenericAllocationHandle>(mc), device), "cuMulticastAddDevice");
}

void multicast_bind(unsigned long long mc, unsigned long long mem_handle, size_t size) {
  static auto bind = driver_fn<CUresult (*)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long)>("cuMulticastBindMem");
  check(bind(static_cast<CUmemGenericAllocationHandle>(mc), 0, static_cast<CUmemGenericAllocationHandle>(mem_handle), 0, size, 0),
        "cuMulticastBindMem");
}

void* multicast_map(unsigned long long mc, size_t size, size_t granularity, int device) {
  return map_handle(static_cast<CUmemGenericAllocationHandle>(mc), size, granularity, device);
}

void multicast_unmap(void* ptr, size_t size, unsigned long long mc, int device) {
  static auto unmap = driver_fn<CUresult (*)(CUdeviceptr, size_t)>("cuMemUnmap");
  static auto free_va = driver_fn<CUresult (*)(CUdeviceptr, size_t)>("cuMemAddressFree");
  static auto release = driver_fn<CUresult (*)(CUmemGenericAllocationHandle)>("cuMemRelease");
  if (ptr != nullptr) {
    unmap(reinterpret_cast<CUdeviceptr>(ptr), size);
    free_va(reinterpret_cast<CUdeviceptr>(ptr), size);
  }
  if (mc != 0) release(static_cast<CUmemGenericAllocationHandle>(mc));
}

// ------------------------------------------------------------------------------ cudaIpc
std::string ipc_export(void* ptr) {
  cudaIpcMemHandle_t h;
  check_rt(cudaIpcGetMemHandle(&h, ptr), "cudaIpcGetMemHandle");
  return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
}

void* ipc_import(const std::string& bytes) {
  if (bytes.size() != sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("bad IPC handle size");
  cudaIpcMemHandle_t h;
  memcpy(&h, bytes.data(), sizeof(h));
  void* p = nullptr;
  check_rt(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return p;
}

void ipc_close(void* ptr) { cudaIpcCloseMemHandle(ptr); }

// ----------------------------------------------------- descriptor passing (Unix sockets)
namespace {
sockaddr_un abstract_addr(const std::string& name, socklen_t* len) {
  sockaddr_un addr;
  memset(&addr, 0, sizeof(addr));
  addr.sun_family = AF_UNIX;
  if (name.size() + 1 >= sizeof(addr.sun_path)) throw std::runtime_error("socket name too long");
  memcpy(addr.sun_path + 1, name.data(), name.size());      // leading NUL: abstract namespace
  *len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + name.size());
  return addr;
}
}  // namespace

int fd_socket_open(const std::string& name) {
  int s = socket(AF_UNIX, SOCK_DGRAM, 0);
  if (s < 0) throw std::runtime_error(std::string("socket: ") + strerror(errno));
  socklen_t len;
  sockaddr_un addr = abstract_addr(name, &len);
  if (bind(s, reinterpret_cast<sockaddr*>(&addr), len) != 0) {
    int e = errno;
    close(s);
    throw std::runtime_error(std::string("bind ") + name + ": " + strerror(e));
  }
  timeval tv{60, 0};
  setsockopt(s, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  return s;
}

void fd_socket_send(int sock, const std::string& to, int fd, int tag) {
  socklen_t len;
  sockaddr_un addr = abstract_addr(to, &len);
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  iovec iov{&tag, sizeof(tag)};
  char control[CMSG_SPACE(sizeof(int))];
  memset(control, 0, sizeof(control));
  msg.msg_name = &addr;
  msg.msg_namelen = len;
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = control;
  msg.msg_controllen = sizeof(control);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  if (sendmsg(sock, &msg, 0) < 0) throw std::runtime_error(std::string("sendmsg to ") + to + ": " + strerror(errno));
}

int fd_socket_recv(int sock, int* tag_out) {
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  int tag = -1;
  iovec iov{&tag, sizeof(tag)};
  char control[CMSG_SPACE(sizeof(int))];
  memset(control, 0, sizeof(control));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = control;
  msg.msg_controllen = sizeof(control);
  if (recvmsg(sock, &msg, 0) < 0) throw std::runtime_error(std::string("recvmsg: ") + strerror(errno));
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (c == nullptr || c->cmsg_type != SCM_RIGHTS) throw std::runtime_error("message carried no file descriptor");
  int fd = -1;
  memcpy(&fd, CMSG_DATA(c), sizeof(int));
  *tag_out = tag;
  return fd;
}

void fd_socket_close(int sock) { close(sock); }

}  // namespace msccl
