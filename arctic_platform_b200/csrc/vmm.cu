// Virtual-memory-management arena: device buffers whose address survives giving the physical memory back, and
// whose physical memory can be handed to another process of the node as a file descriptor.
//
// Two uses.  (1) Symmetric buffers without a framework in between: every rank allocates a buffer, exports it as a
// POSIX file descriptor, the ranks pass the descriptors over Unix sockets (Python side), and each rank maps its
// peers' memory into its own address space -- the per-rank pointer table the peer-load / peer-store kernels take.
// (2) Sleep / wake with stable addresses: release() gives the physical pages back to the driver and keeps the
// address range reserved; remap() puts fresh pages under the same addresses, so CUDA graphs and pointer tables
// recorded before the sleep stay valid.  (The reference gets (2) from vLLM's cumem allocator and (1) from NCCL /
// CUDA IPC inside its engines.)
//
// Only driver calls are used, resolved through cudaGetDriverEntryPoint, so the library has no link-time dependency
// on libcuda and still loads on a machine without a GPU.  Every function returns 0 or a CUresult / negative code;
// nothing here launches a kernel.
#include "host_utils.cuh"

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace apb {
namespace {

struct Driver {
  CUresult (*GetGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*Create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*Release)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*AddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*AddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*Map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*Unmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*SetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*Export)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*Import)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  bool ok = false;
};

template <typename F>
bool resolve(const char* name, F* out) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p)
    return false;
  *out = reinterpret_cast<F>(p);
  return true;
}

Driver* driver() {
  static Driver d;
  static bool tried = false;
  if (!tried) {
    tried = true;
    d.ok = resolve("cuMemGetAllocationGranularity", &d.GetGranularity) && resolve("cuMemCreate", &d.Create) &&
           resolve("cuMemRelease", &d.Release) && resolve("cuMemAddressReserve", &d.AddressReserve) &&
           resolve("cuMemAddressFree", &d.AddressFree) && resolve("cuMemMap", &d.Map) &&
           resolve("cuMemUnmap", &d.Unmap) && resolve("cuMemSetAccess", &d.SetAccess) &&
           resolve("cuMemExportToShareableHandle", &d.Export) &&
           resolve("cuMemImportFromShareableHandle", &d.Import);
  }
  return d.ok ? &d : nullptr;
}

constexpr int kNoDriver = -10;     // no usable CUDA driver (CPU-only machine)
constexpr int kBadArg = -11;

CUmemAllocationProp device_prop(int device) {
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

int grant_access(Driver* d, CUdeviceptr va, size_t bytes, int device) {
  CUmemAccessDesc acc = {};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  return static_cast<int>(d->SetAccess(va, bytes, &acc, 1));
}

}  // namespace
}  // namespace apb

extern "C" {

// Smallest size the driver maps on `device`; every size below is rounded up to a multiple of it.
int apb_vmm_granularity(int device, size_t* out) {
  using namespace apb;
  Driver* d = driver();
  if (!d) return kNoDriver;
  if (!out || device < 0) return kBadArg;
  CUmemAllocationProp prop = device_prop(device);
  return static_cast<int>(d->GetGranularity(out, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM));
}

// Reserves an address range of `bytes` (rounded up, returned in *padded), backs it with new physical memory on
// `device` and makes it readable and writable from `device`.
int apb_vmm_alloc(int device, size_t bytes, void** va_out, size_t* padded_out, unsigned long long* handle_out) {
  using namespace apb;
  Driver* d = driver();
  if (!d) return kNoDriver;
  if (!va_out || !padded_out || !handle_out || bytes == 0 || device < 0) return kBadArg;
  size_t gran = 0;
  CUmemAllocationProp prop = device_prop(device);
  CUresult r = d->GetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  if (gran == 0) return kBadArg;
  const size_t padded = (bytes + gran - 1) / gran * gran;
  CUmemGenericAllocationHandle h = 0;
  r = d->Create(&h, padded, &prop, 0);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  CUdeviceptr va = 0;
  r = d->AddressReserve(&va, padded, gran, 0, 0);
  if (r != CUDA_SUCCESS) {
    d->Release(h);
    return static_cast<int>(r);
  }
  r = d->Map(va, padded, 0, h, 0);
  if (r == CUDA_SUCCESS) r = static_cast<CUresult>(grant_access(d, va, padded, device));
  if (r != CUDA_SUCCESS) {
    d->Unmap(va, padded);
    d->AddressFree(va, padded);
    d->Release(h);
    return static_cast<int>(r);
  }
  *va_out = reinterpret_cast<void*>(va);
  *padded_out = padded;
  *handle_out = static_cast<unsigned long long>(h);
  return 0;
}

// The physical allocation as a file descriptor another process of this node can import.  The caller owns the
// descriptor (close it after it has been sent).
int apb_vmm_export_fd(unsigned long long handle, int* fd_out) {
  using namespace apb;
  Driver* d = driver();
  if (!d) return kNoDriver;
  if (!fd_out || handle == 0) return kBadArg;
  int fd = -1;
  CUresult r = d->Export(&fd, static_cast<CUmemGenericAllocationHandle>(handle), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  *fd_out = fd;
  return 0;
}

// Maps the allocation behind a received descriptor (of `padded` bytes, as reported by the exporter) into this
// process and makes it accessible from `device`.  The memory stays where the exporter put it; access from another
// GPU goes over NVLink.
int apb_vmm_import_fd(int device, int fd, size_t padded, void** va_out, unsigned long long* handle_out) {
  using namespace apb;
  Driver* d = driver();
  if (!d) return kNoDriver;
  if (!va_out || !handle_out || fd < 0 || padded == 0 || device < 0) return kBadArg;
  CUmemGenericAllocationHandle h = 0;
  CUresult r = d->Import(&h, reinterpret_cast<void*>(static_cast<intptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  CUdeviceptr va = 0;
  r = d->AddressReserve(&va, padded, 0, 0, 0);
  if (r != CUDA_SUCCESS) {
    d->Release(h);
    return static_cast<int>(r);
  }
  r = d->Map(va, padded, 0, h, 0);
  if (r == CUDA_SUCCESS) r = static_cast<CUresult>(grant_access(d, va, padded, device));
  if (r != CUDA_SUCCESS) {
    d->Unmap(va, padded);
    d->AddressFree(va, padded);
    d->Release(h);
    return static_cast<int>(r);
  }
  *va_out = reinterpret_cast<void*>(va);
  *handle_out = static_cast<unsigned long long>(h);
  return 0;
}

// Gives the physical memory back and keeps the addresses reserved (sleep).  The contents are lost.
int apb_vmm_release_physical(void* va, size_t padded, unsigned long long handle) {
  using namespace apb;
  Driver* d = driver();
  if (!d) return kNoDriver;
  if (!va || padded == 0 || handle == 0) return kBadArg;
  CUresult r = d->Unmap(reinterpret_cast<CUdeviceptr>(va), padded);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  return static_cast<int>(d->Release(static_cast<CUmemGenericAllocationHandle>(handle)));
}

// Puts new physical memory under a range that release_physical() emptied (wake).  Contents are undefined.
int apb_vmm_remap(int device, void* va, size_t padded, unsigned long long* handle_out) {
  using namespace apb;
  Driver* d = driver();
  if (!d) return kNoDriver;
  if (!va || padded == 0 || !handle_out || device < 0) return kBadArg;
  CUmemAllocationProp prop = device_prop(device);
  CUmemGenericAllocationHandle h = 0;
  CUresult r = d->Create(&h, padded, &prop, 0);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  const CUdeviceptr p = reinterpret_cast<CUdeviceptr>(va);
  r = d->Map(p, padded, 0, h, 0);
  if (r == CUDA_SUCCESS) r = static_cast<CUresult>(grant_access(d, p, padded, device));
  if (r != CUDA_SUCCESS) {
    d->Unmap(p, padded);
    d->Release(h);
    return static_cast<int>(r);
  }
  *handle_out = static_cast<unsigned long long>(h);
  return 0;
}

// Unmaps, releases and frees the address range.  `handle` may be 0 for a range whose memory was already released.
int apb_vmm_free(void* va, size_t padded, unsigned long long handle) {
  using namespace apb;
  Driver* d = driver();
  if (!d) return kNoDriver;
  if (!va || padded == 0) return kBadArg;
  const CUdeviceptr p = reinterpret_cast<CUdeviceptr>(va);
  int rc = 0;
  if (handle != 0) {
    CUresult r = d->Unmap(p, padded);
    if (r != CUDA_SUCCESS) rc = static_cast<int>(r);
    r = d->Release(static_cast<CUmemGenericAllocationHandle>(handle));
    if (r != CUDA_SUCCESS && rc == 0) rc = static_cast<int>(r);
  }
  CUresult r = d->AddressFree(p, padded);
  if (r != CUDA_SUCCESS && rc == 0) rc = static_cast<int>(r);
  return rc;
}
}
