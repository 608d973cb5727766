#include "segments.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <sstream>

#include "comm.h"

namespace pccl {

namespace {

template <typename Fn>
Fn driver_fn(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
    cudaGetLastError();
    throw Error(std::string("CUDA driver entry point not available: ") + name);
  }
  return reinterpret_cast<Fn>(p);
}
#define DRV(name) driver_fn<decltype(&name)>(#name)

void check_drv(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return;
  const char* s = nullptr;
  try {
    DRV(cuGetErrorString)(r, &s);
  } catch (...) {
  }
  std::ostringstream os;
  os << "CUDA driver error " << (int)r << " (" << (s ? s : "?") << ") in " << what;
  throw Error(os.str());
}
#define PCCL_DRV(call, ...) check_drv(DRV(call)(__VA_ARGS__), #call)

uint64_t round_up(uint64_t v, uint64_t g) { return (v + g - 1) / g * g; }

CUmemAllocationProp device_prop(int device) {
  CUmemAllocationProp prop;
  std::memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

void map_rw(CUdeviceptr* va, uint64_t bytes, uint64_t gran, CUmemGenericAllocationHandle h, int device) {
  PCCL_DRV(cuMemAddressReserve, va, bytes, gran, 0, 0);
  CUresult r = DRV(cuMemMap)(*va, bytes, 0, h, 0);
  if (r != CUDA_SUCCESS) {
    DRV(cuMemAddressFree)(*va, bytes);
    check_drv(r, "cuMemMap");
  }
  CUmemAccessDesc acc;
  std::memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = DRV(cuMemSetAccess)(*va, bytes, &acc, 1);
  if (r != CUDA_SUCCESS) {
    DRV(cuMemUnmap)(*va, bytes);
    DRV(cuMemAddressFree)(*va, bytes);
    check_drv(r, "cuMemSetAccess");
  }
}

}  // namespace

// ------------------------------------------------------------------ IpcSegment
IpcSegment::IpcSegment(int device, uint64_t bytes) : device_(device), bytes_(bytes), owner_(true) {
  PCCL_CUDA(cudaSetDevice(device));
  void* p = nullptr;
  PCCL_CUDA(cudaMalloc(&p, bytes));
  PCCL_CUDA(cudaMemset(p, 0, bytes));
  PCCL_CUDA(cudaDeviceSynchronize());
  ptr_ = (uint64_t)p;
}

IpcSegment::IpcSegment(int device, const std::string& handle, uint64_t bytes) : device_(device), bytes_(bytes) {
  if (handle.size() != sizeof(cudaIpcMemHandle_t)) throw Error("IPC handle has the wrong length");
  PCCL_CUDA(cudaSetDevice(device));
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle.data(), sizeof(h));
  void* p = nullptr;
  PCCL_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  ptr_ = (uint64_t)p;
}

std::string IpcSegment::handle() const {
  if (!owner_) throw Error("only the owning process can export an IPC handle");
  cudaIpcMemHandle_t h;
  PCCL_CUDA(cudaIpcGetMemHandle(&h, (void*)ptr_));
  return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
}

void IpcSegment::close() {
  if (ptr_ == 0) return;
  if (owner_) cudaFree((void*)ptr_);
  else cudaIpcCloseMemHandle((void*)ptr_);
  ptr_ = 0;
}

IpcSegment::~IpcSegment() { close(); }

// ------------------------------------------------------------------ VmmSegment
VmmSegment::VmmSegment(int device, uint64_t bytes, int world_for_multicast) : device_(device), owner_(true) {
  PCCL_CUDA(cudaSetDevice(device));
  PCCL_CUDA(cudaFree(nullptr));  // make sure the primary context exists
  CUmemAllocationProp prop = device_prop(device);
  size_t gran = 0;
  PCCL_DRV(cuMemGetAllocationGranularity, &gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (world_for_multicast > 1 && multicast_supported(device)) {
    CUmulticastObjectProp mp;
    std::memset(&mp, 0, sizeof(mp));
    mp.numDevices = (unsigned)world_for_multicast;
    mp.size = round_up(bytes, gran);
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mgran = 0;
    if (DRV(cuMulticastGetGranularity)(&mgran, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mgran > 0)
      gran = std::max(gran, mgran);
  }
  bytes_ = round_up(bytes, gran);
  CUmemGenericAllocationHandle h;
  PCCL_DRV(cuMemCreate, &h, bytes_, &prop, 0);
  handle_ = h;
  CUdeviceptr va = 0;
  try {
    map_rw(&va, bytes_, gran, h, device);
  } catch (...) {
    DRV(cuMemRelease)(h);
    handle_ = 0;
    throw;
  }
  ptr_ = (uint64_t)va;
  mapped_ = true;
  PCCL_CUDA(cudaMemset((void*)ptr_, 0, bytes_));
  PCCL_CUDA(cudaDeviceSynchronize());
}

VmmSegment::VmmSegment(int device, int fd, uint64_t bytes) : device_(device), bytes_(bytes) {
  PCCL_CUDA(cudaSetDevice(device));
  PCCL_CUDA(cudaFree(nullptr));
  CUmemGenericAllocationHandle h;
  CUresult r = DRV(cuMemImportFromShareableHandle)(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  ::close(fd);
  check_drv(r, "cuMemImportFromShareableHandle");
  handle_ = h;
  CUmemAllocationProp prop = device_prop(device);
  size_t gran = 0;
  PCCL_DRV(cuMemGetAllocationGranularity, &gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  CUdeviceptr va = 0;
  try {
    map_rw(&va, bytes_, gran, h, device);
  } catch (...) {
    DRV(cuMemRelease)(h);
    handle_ = 0;
    throw;
  }
  ptr_ = (uint64_t)va;
  mapped_ = true;
}

int VmmSegment::export_fd() {
  if (!owner_) throw Error("only the owning process exports its segment");
  int fd = -1;
  PCCL_DRV(cuMemExportToShareableHandle, (void*)&fd, (CUmemGenericAllocationHandle)handle_,
           CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  return fd;
}

bool VmmSegment::multicast_supported(int device) {
  try {
    int v = 0;
    CUdevice dev;
    if (DRV(cuDeviceGet)(&dev, device) != CUDA_SUCCESS) return false;
    if (DRV(cuDeviceGetAttribute)(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return false;
    return v != 0;
  } catch (const Error&) {
    return false;
  }
}

int VmmSegment::multicast_create(int world) {
  CUmulticastObjectProp mp;
  std::memset(&mp, 0, sizeof(mp));
  mp.numDevices = (unsigned)world;
  mp.size = bytes_;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle mc;
  PCCL_DRV(cuMulticastCreate, &mc, &mp);
  mc_handle_ = mc;
  mc_have_ = true;
  int fd = -1;
  PCCL_DRV(cuMemExportToShareableHandle, (void*)&fd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  return fd;
}

void VmmSegment::multicast_import(int fd) {
  CUmemGenericAllocationHandle mc;
  CUresult r = DRV(cuMemImportFromShareableHandle)(&mc, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  ::close(fd);
  check_drv(r, "cuMemImportFromShareableHandle(multicast)");
  mc_handle_ = mc;
  mc_have_ = true;
}

void VmmSegment::multicast_add_device() {
  if (!mc_have_) throw Error("no multicast object");
  CUdevice dev;
  PCCL_DRV(cuDeviceGet, &dev, device_);
  PCCL_DRV(cuMulticastAddDevice, (CUmemGenericAllocationHandle)mc_handle_, dev);
}

uint64_t VmmSegment::multicast_bind_and_map() {
  if (!mc_have_) throw Error("no multicast object");
  PCCL_DRV(cuMulticastBindMem, (CUmemGenericAllocationHandle)mc_handle_, 0, (CUmemGenericAllocationHandle)handle_, 0,
           bytes_, 0);
  mc_bound_ = true;
  CUmemAllocationProp prop = device_prop(device_);
  size_t gran = 0;
  PCCL_DRV(cuMemGetAllocationGranularity, &gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  CUdeviceptr va = 0;
  map_rw(&va, bytes_, gran, (CUmemGenericAllocationHandle)mc_handle_, device_);
  mc_ptr_ = (uint64_t)va;
  return mc_ptr_;
}

void VmmSegment::multicast_release() {
  if (mc_ptr_ != 0) {
    DRV(cuMemUnmap)((CUdeviceptr)mc_ptr_, bytes_);
    DRV(cuMemAddressFree)((CUdeviceptr)mc_ptr_, bytes_);
    mc_ptr_ = 0;
  }
  if (mc_bound_) {
    CUdevice dev;
    if (DRV(cuDeviceGet)(&dev, device_) == CUDA_SUCCESS)
      DRV(cuMulticastUnbind)((CUmemGenericAllocationHandle)mc_handle_, dev, 0, bytes_);
    mc_bound_ = false;
  }
  if (mc_have_) {
    DRV(cuMemRelease)((CUmemGenericAllocationHandle)mc_handle_);
    mc_have_ = false;
  }
}

void VmmSegment::close() {
  try {
    if (mc_have_ || mc_ptr_ != 0) {
      cudaDeviceSynchronize();
      multicast_release();
    }
    if (mapped_) {
      DRV(cuMemUnmap)((CUdeviceptr)ptr_, bytes_);
      DRV(cuMemAddressFree)((CUdeviceptr)ptr_, bytes_);
      mapped_ = false;
      ptr_ = 0;
    }
    if (handle_ != 0) {
      DRV(cuMemRelease)((CUmemGenericAllocationHandle)handle_);
      handle_ = 0;
    }
  } catch (const Error&) {
    // teardown at interpreter exit: the driver may already be gone
  }
}

VmmSegment::~VmmSegment() { close(); }

}  // namespace pccl
