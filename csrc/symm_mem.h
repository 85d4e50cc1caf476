// Host API of the symmetric-memory layer (see symm_mem.cpp).
#pragma once
#include <cstddef>
#include <string>

namespace msccl {

struct VmmBlock {
  void* ptr = nullptr;              // mapping in this process
  size_t size = 0;                  // rounded up to the granularity
  size_t granularity = 0;
  unsigned long long handle = 0;    // CUmemGenericAllocationHandle
  int fd = -1;                      // shareable descriptor (owner: exported; importer: received)
};

size_t vmm_granularity(int device, bool multicast, int num_devices);
bool multicast_supported(int device);
VmmBlock vmm_create(int device, size_t size, size_t granularity);
VmmBlock vmm_import(int device, int fd, size_t size, size_t granularity);
void vmm_release(const VmmBlock& block);

unsigned long long multicast_create(int num_devices, size_t size, int* fd_out);
unsigned long long multicast_import(int fd);
void multicast_add_device(unsigned long long mc, int device);
void multicast_bind(unsigned long long mc, unsigned long long mem_handle, size_t size);
void* multicast_map(unsigned long long mc, size_t size, size_t granularity, int device);
void multicast_unmap(void* ptr, size_t size, unsigned long long mc, int device);

std::string ipc_export(void* ptr);
void* ipc_import(const std::string& handle_bytes);
void ipc_close(void* ptr);

int fd_socket_open(const std::string& name);
void fd_socket_send(int sock, const std::string& to, int fd, int tag);
int fd_socket_recv(int sock, int* tag_out);
void fd_socket_close(int sock);

}  // namespace msccl
