// Symmetric heap: every rank allocates one identically laid-out region and maps
// every peer's region into its own address space, so a peer's byte at offset x
// is addressable as peer_base[r] + x from device code.
//
// Layout of one rank's region (all parts reachable by every peer):
//   [ data : data_bytes ][ signals : 65536 x u32 ][ control : 4 MiB ]
// Allocation uses the CUDA virtual-memory API so that the physical handle can be
// exported as a file descriptor (for peers) and bound to a multicast object
// (NVLS).  In-process clusters of virtual ranks use the same allocator without
// export.  (The reference carves workspace out of the tail of a 1 GiB buffer
// and has 4096 signal slots: csrc/engine/memory_layout.cc:8-138,
// include/common/config.h:8-35, csrc/plugins/cuda/cuda_device.cc:103-216.)
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "../executors/sm100/program.h"
#include "cuda_driver.h"

namespace pccl {

struct HeapLayout {
  size_t data_bytes = 0;
  size_t signal_offset = 0;     // from region base
  size_t control_offset = 0;
  size_t total_bytes = 0;       // multiple of the allocation granularity
  static constexpr size_t kControlBytes = 4u << 20;
  static HeapLayout make(size_t data_bytes, size_t granularity);
};

// One mapped region (own or a peer's).
struct Mapping {
  CUmemGenericAllocationHandle handle = 0;
  CUdeviceptr base = 0;
  size_t bytes = 0;
  bool mapped = false;
};

class SymmetricHeap {
 public:
  SymmetricHeap() = default;
  ~SymmetricHeap();
  SymmetricHeap(const SymmetricHeap&) = delete;
  SymmetricHeap& operator=(const SymmetricHeap&) = delete;

  // Allocate this rank's region on `device`.  `shareable` requests a handle type
  // that can be exported as a POSIX fd.
  void allocate(int device, size_t data_bytes, bool shareable);
  void release();
  bool allocated() const { return own_.mapped; }

  int export_fd() const;                       // caller owns the returned fd
  // Map a peer's region from its exported fd (takes ownership of fd).  The
  // peer must have allocated with the same data_bytes.
  void map_peer(int rank, int fd);
  // In-process peers: alias another heap of the same process.
  void alias_peer(int rank, const SymmetricHeap& other);

  const HeapLayout& layout() const { return layout_; }
  int device() const { return device_; }
  uint8_t* base(int rank) const;
  uint8_t* data(int rank) const { return base(rank); }
  uint32_t* signals(int rank) const { return reinterpret_cast<uint32_t*>(base(rank) + layout_.signal_offset); }
  uint8_t* control(int rank) const { return base(rank) + layout_.control_offset; }
  void set_self(int rank) { self_ = rank; if (static_cast<int>(peers_.size()) <= rank) peers_.resize(rank + 1); }
  int self() const { return self_; }
  bool has_peer(int rank) const;
  CUmemGenericAllocationHandle own_handle() const { return own_.handle; }

  // Bump allocator inside this rank's control area (never freed; reset with the heap).
  uint8_t* control_alloc(size_t bytes, size_t align = 128);

  // --- NVLS ------------------------------------------------------------------------------
  static bool multicast_supported(int device);
  // Rank 0: create the multicast object for `world` devices; returns an fd to publish.
  int multicast_create(int world);
  void multicast_import(int fd);               // other ranks (takes ownership of fd)
  void multicast_add_device();                 // every rank, before any bind
  void multicast_bind_and_map();               // every rank, after all ranks added their device
  void multicast_release();
  uint8_t* mc_base() const { return reinterpret_cast<uint8_t*>(mc_.base); }
  bool multicast_ready() const { return mc_.mapped; }

 private:
  int device_ = -1;
  int self_ = 0;
  size_t granularity_ = 0;
  HeapLayout layout_;
  Mapping own_;
  std::vector<Mapping> peers_;          // indexed by rank; own slot unused
  std::vector<const SymmetricHeap*> aliases_;
  size_t control_used_ = 0;
  Mapping mc_;
  size_t mc_bytes_ = 0;
  bool mc_bound_ = false;
};

}  // namespace pccl
