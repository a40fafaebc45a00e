// Cross-process registration of KV-cache memory: the worker process exports a region of its
// GPU memory, the process that runs the engine opens it and gets a device pointer it can
// register.  This is the native form of the reference's CudaIPCWrapper + CudaTensorRegistry pair
// (python/pegaflow/ipc_wrapper.py:101-163, pegaflow-server/src/registry.rs:172-203), which does
// the same through torch's storage sharing on a dedicated Python thread of the server: here it
// is three C calls and no Python on the importing side.  Devices are identified by UUID, so the
// two processes may see different CUDA_VISIBLE_DEVICES orderings (ipc_wrapper.py:46-98).
#include <cuda_runtime.h>

#include <cstring>
#include <map>
#include <mutex>
#include <string>

#include "common.h"
#include "transfer.h"

namespace pf {
namespace {

// cuMemGetAddressRange through the runtime's driver entry point: the library does not link libcuda.
typedef int (*AddressRangeFn)(unsigned long long *base, size_t *size, unsigned long long ptr);

AddressRangeFn address_range_fn() {
  static AddressRangeFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &status) != cudaSuccess ||
        status != cudaDriverEntryPointSuccess)
      p = nullptr;
    cudaGetLastError();
    return reinterpret_cast<AddressRangeFn>(p);
  }();
  return fn;
}

void check(cudaError_t e, const char *what) {
  if (e != cudaSuccess) throw Error::storage(strf("%s failed: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e)));
}

int device_of_uuid(const uint8_t uuid[16]) {
  int count = 0;
  check(cudaGetDeviceCount(&count), "cudaGetDeviceCount");
  for (int d = 0; d < count; ++d) {
    cudaDeviceProp prop;
    check(cudaGetDeviceProperties(&prop, d), "cudaGetDeviceProperties");
    if (std::memcmp(prop.uuid.bytes, uuid, 16) == 0) return d;
  }
  throw Error::invalid("the exporting process's GPU (by UUID) is not visible to this process");
}

struct Mapping {
  char *base = nullptr;
  int device = 0;  // the device that was current when the handle was opened
  size_t users = 0;
};
std::mutex g_mu;
// One mapping per exported allocation and accessing device, keyed by the 64 handle bytes + device.
std::map<std::string, Mapping> g_open;

std::string mapping_key(const pf_ipc_region *region, int device) {
  std::string key(reinterpret_cast<const char *>(region->handle), sizeof region->handle);
  key.append(reinterpret_cast<const char *>(&device), sizeof device);
  return key;
}

// Opens (or reuses) the mapping of the region's allocation made with `device` current.  The driver
// ties an imported allocation to the context that opened it: kernels and copies of that device can
// use the pointer - over NVLink when the memory belongs to another GPU (peer access is switched on
// by the open, cudaIpcMemLazyEnablePeerAccess) - while another device of the same process cannot,
// even with peer access enabled afterwards.
constexpr int kOwnerKey = -1;  // pf_ipc_open: the mapping lives on the GPU that owns the memory

uint64_t open_on(const pf_ipc_region *region, int device, int key_device) {
  DeviceGuard on_device(device);
  const std::string key = mapping_key(region, key_device);
  std::lock_guard<std::mutex> g(g_mu);
  Mapping &m = g_open[key];
  if (!m.base) {
    cudaIpcMemHandle_t h;
    std::memcpy(&h, region->handle, sizeof h);
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      g_open.erase(key);
      check(e, "cudaIpcOpenMemHandle");
    }
    m.base = static_cast<char *>(p);
    m.device = device;
  }
  ++m.users;
  return (uint64_t)(uintptr_t)(m.base + region->offset);
}

void close_on(const pf_ipc_region *region, int key_device) {
  const std::string key = mapping_key(region, key_device);
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_open.find(key);
  if (it == g_open.end()) throw Error::invalid("ipc close: the region is not open");
  if (--it->second.users == 0) {
    DeviceGuard on_device(it->second.device);
    cudaError_t e = cudaIpcCloseMemHandle(it->second.base);
    g_open.erase(it);
    check(e, "cudaIpcCloseMemHandle");
  }
}

}  // namespace
}  // namespace pf

using namespace pf;

extern "C" {

int pf_ipc_export(uint64_t device_ptr, size_t nbytes, pf_ipc_region *out) {
  return guarded([&] {
    if (!out || !device_ptr || nbytes == 0) throw Error::invalid("ipc export: null pointer or empty region");
    cudaPointerAttributes attr;
    check(cudaPointerGetAttributes(&attr, reinterpret_cast<const void *>(device_ptr)), "cudaPointerGetAttributes");
    if (attr.type != cudaMemoryTypeDevice) throw Error::invalid("ipc export: not device memory");
    DeviceGuard on_device(attr.device);
    AddressRangeFn range = address_range_fn();
    if (!range) throw Error::cuda_init("cuMemGetAddressRange is not available from this driver");
    unsigned long long base = 0;
    size_t size = 0;
    if (range(&base, &size, device_ptr) != 0) throw Error::invalid("ipc export: the pointer is not inside a CUDA allocation");
    if (device_ptr + nbytes > base + size)
      throw Error::invalid(strf("ipc export: region of %zu bytes runs past its allocation (%zu bytes left)", nbytes,
                                (size_t)(base + size - device_ptr)));
    cudaIpcMemHandle_t h;
    check(cudaIpcGetMemHandle(&h, reinterpret_cast<void *>(base)), "cudaIpcGetMemHandle");
    static_assert(sizeof(h) == sizeof(out->handle), "handle size");
    std::memcpy(out->handle, &h, sizeof h);
    out->offset = device_ptr - base;
    out->nbytes = nbytes;
    cudaDeviceProp prop;
    check(cudaGetDeviceProperties(&prop, attr.device), "cudaGetDeviceProperties");
    std::memcpy(out->device_uuid, prop.uuid.bytes, 16);
  });
}

int pf_ipc_open(const pf_ipc_region *region, uint64_t *device_ptr, int *device_id) {
  return guarded([&] {
    if (!region || !device_ptr) throw Error::invalid("ipc open: null argument");
    const int device = device_of_uuid(region->device_uuid);
    *device_ptr = open_on(region, device, kOwnerKey);
    if (device_id) *device_id = device;
  });
}

int pf_ipc_close(const pf_ipc_region *region) {
  return guarded([&] {
    if (!region) throw Error::invalid("ipc close: null argument");
    close_on(region, kOwnerKey);
  });
}

int pf_ipc_open_for(const pf_ipc_region *region, int accessing_device, uint64_t *device_ptr, int *owner_device) {
  return guarded([&] {
    if (!region || !device_ptr) throw Error::invalid("ipc open: null argument");
    int count = 0;
    check(cudaGetDeviceCount(&count), "cudaGetDeviceCount");
    if (accessing_device < 0 || accessing_device >= count)
      throw Error::invalid(strf("ipc open: device %d out of range (%d devices)", accessing_device, count));
    const int owner = device_of_uuid(region->device_uuid);
    if (owner != accessing_device) {
      int can = 0;
      check(cudaDeviceCanAccessPeer(&can, accessing_device, owner), "cudaDeviceCanAccessPeer");
      if (!can) throw Error::cuda_init(strf("device %d cannot access device %d", accessing_device, owner));
    }
    *device_ptr = open_on(region, accessing_device, accessing_device);
    if (owner_device) *owner_device = owner;
  });
}

int pf_ipc_close_for(const pf_ipc_region *region, int accessing_device) {
  return guarded([&] {
    if (!region) throw Error::invalid("ipc close: null argument");
    if (accessing_device < 0) throw Error::invalid("ipc close: device out of range");
    close_on(region, accessing_device);
  });
}

}  // extern "C"
