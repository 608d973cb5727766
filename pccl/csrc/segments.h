// Device memory that other processes on the same NVSwitch domain can map.
//
// Two ways to obtain it, tried in this order by the Python bootstrap:
//   VmmSegment  cuMemCreate + POSIX file-descriptor export.  The descriptor travels to the
//               peers over a unix socket (SCM_RIGHTS, done in Python); peers import and map
//               it.  Only this kind can be bound to an NVLS multicast object.
//   IpcSegment  cudaMalloc + cudaIpcGetMemHandle.  The 64-byte handle travels through the
//               torch.distributed store.
// The reference needs neither: GPU-aware MPI moved the bytes (pccl/src/all_gather.cpp:61-63).
//
// The driver API is reached through cudaGetDriverEntryPoint so that the extension loads
// on machines without libcuda (CPU-only test runs).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace pccl {

class IpcSegment {
 public:
  // Owner side: allocate `bytes` (zero-filled) on `device`.
  IpcSegment(int device, uint64_t bytes);
  // Peer side: map a handle produced by another process.
  IpcSegment(int device, const std::string& handle, uint64_t bytes);
  ~IpcSegment();
  IpcSegment(const IpcSegment&) = delete;
  IpcSegment& operator=(const IpcSegment&) = delete;
  uint64_t ptr() const { return ptr_; }
  uint64_t bytes() const { return bytes_; }
  std::string handle() const;   // 64 raw bytes
  void close();

 private:
  int device_;
  uint64_t ptr_ = 0, bytes_ = 0;
  bool owner_ = false;
};

class VmmSegment {
 public:
  // Owner side.  `bytes` is rounded up to the allocation (and multicast) granularity.
  VmmSegment(int device, uint64_t bytes, int world_for_multicast);
  // Peer side: import a received file descriptor (consumed: closed after the import).
  VmmSegment(int device, int fd, uint64_t bytes);
  ~VmmSegment();
  VmmSegment(const VmmSegment&) = delete;
  VmmSegment& operator=(const VmmSegment&) = delete;
  uint64_t ptr() const { return ptr_; }
  uint64_t bytes() const { return bytes_; }
  int export_fd();              // a new descriptor per call; the caller closes it
  void close();

  // ---- NVLS multicast over the owner segments of all ranks
  static bool multicast_supported(int device);
  // Rank 0 creates the object and exports it; the others import the descriptor.
  int multicast_create(int world);          // returns an fd to ship to the peers
  void multicast_import(int fd);
  void multicast_add_device();              // every rank, before anyone binds
  uint64_t multicast_bind_and_map();        // every rank, after all have added; returns the multicast VA
  void multicast_release();

 private:
  int device_;
  uint64_t ptr_ = 0, bytes_ = 0;
  unsigned long long handle_ = 0;
  bool mapped_ = false, owner_ = false;
  unsigned long long mc_handle_ = 0;
  uint64_t mc_ptr_ = 0;
  bool mc_bound_ = false, mc_have_ = false;
};

}  // namespace pccl
