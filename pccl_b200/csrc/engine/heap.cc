#include "heap.h"

#include <unistd.h>

namespace pccl {

namespace {
size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

CUmemAllocationProp alloc_prop(int device, bool shareable) {
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = shareable ? CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR : CU_MEM_HANDLE_TYPE_NONE;
  return prop;
}

void grant_access(CUdeviceptr base, size_t bytes, int device) {
  CUmemAccessDesc access{};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  PCCL_CU(DriverApi::get().cuMemSetAccess(base, bytes, &access, 1));
}
}  // namespace

HeapLayout HeapLayout::make(size_t data_bytes, size_t granularity) {
  HeapLayout l;
  l.data_bytes = round_up(data_bytes, 4096);
  l.signal_offset = l.data_bytes;
  l.control_offset = l.signal_offset + round_up(static_cast<size_t>(kSignalSlots) * sizeof(uint32_t), 4096);
  l.total_bytes = round_up(l.control_offset + kControlBytes, granularity);
  return l;
}

SymmetricHeap::~SymmetricHeap() {
  try { release(); } catch (...) {}
}

void SymmetricHeap::allocate(int device, size_t data_bytes, bool shareable) {
  PCCL_CHECK(!own_.mapped, "symmetric heap already allocated");
  const DriverApi& cu = DriverApi::get();
  device_ = device;
  PCCL_CUDA(cudaSetDevice(device));
  PCCL_CUDA(cudaFree(nullptr));   // make sure the primary context exists
  CUmemAllocationProp prop = alloc_prop(device, shareable);
  PCCL_CU(cu.cuMemGetAllocationGranularity(&granularity_, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  if (multicast_supported(device)) {
    // Multicast binding wants its own (possibly coarser) granularity.
    CUmulticastObjectProp mp{};
    mp.numDevices = 2;
    mp.size = granularity_;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (cu.cuMulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > granularity_)
      granularity_ = mg;
  }
  layout_ = HeapLayout::make(data_bytes, granularity_);
  own_.bytes = layout_.total_bytes;
  PCCL_CU(cu.cuMemCreate(&own_.handle, own_.bytes, &prop, 0));
  PCCL_CU(cu.cuMemAddressReserve(&own_.base, own_.bytes, granularity_, 0, 0));
  PCCL_CU(cu.cuMemMap(own_.base, own_.bytes, 0, own_.handle, 0));
  grant_access(own_.base, own_.bytes, device);
  own_.mapped = true;
  control_used_ = 0;
  // Signals and control start from zero.
  PCCL_CUDA(cudaMemset(reinterpret_cast<void*>(own_.base + layout_.signal_offset), 0,
                       layout_.total_bytes - layout_.signal_offset));
}

void SymmetricHeap::release() {
  multicast_release();
  if (device_ < 0) return;
  const DriverApi& cu = DriverApi::get();
  auto drop = [&](Mapping& m) {
    if (!m.mapped) return;
    cu.cuMemUnmap(m.base, m.bytes);
    cu.cuMemAddressFree(m.base, m.bytes);
    cu.cuMemRelease(m.handle);
    m = Mapping{};
  };
  for (auto& p : peers_) drop(p);
  peers_.clear();
  aliases_.clear();
  drop(own_);
  device_ = -1;
}

int SymmetricHeap::export_fd() const {
  PCCL_CHECK(own_.mapped, "symmetric heap not allocated");
  int fd = -1;
  PCCL_CU(DriverApi::get().cuMemExportToShareableHandle(&fd, own_.handle,
                                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  return fd;
}

void SymmetricHeap::map_peer(int rank, int fd) {
  PCCL_CHECK(own_.mapped, "allocate the local heap before mapping peers");
  PCCL_CHECK(rank >= 0 && rank < kMaxRanks, "peer rank " << rank << " out of range");
  const DriverApi& cu = DriverApi::get();
  if (static_cast<int>(peers_.size()) <= rank) peers_.resize(rank + 1);
  Mapping& m = peers_[rank];
  PCCL_CHECK(!m.mapped, "peer " << rank << " already mapped");
  m.bytes = layout_.total_bytes;
  CUresult r = cu.cuMemImportFromShareableHandle(&m.handle, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                                 CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  close(fd);
  PCCL_CHECK(r == CUDA_SUCCESS, "importing rank " << rank << "'s heap failed: " << cu.error_string(r));
  PCCL_CU(cu.cuMemAddressReserve(&m.base, m.bytes, granularity_, 0, 0));
  PCCL_CU(cu.cuMemMap(m.base, m.bytes, 0, m.handle, 0));
  grant_access(m.base, m.bytes, device_);
  m.mapped = true;
}

void SymmetricHeap::alias_peer(int rank, const SymmetricHeap& other) {
  PCCL_CHECK(other.layout_.total_bytes == layout_.total_bytes, "in-process peers must share one layout");
  if (static_cast<int>(aliases_.size()) <= rank) aliases_.resize(rank + 1, nullptr);
  aliases_[rank] = &other;
}

bool SymmetricHeap::has_peer(int rank) const {
  if (rank == self_) return own_.mapped;
  if (rank < static_cast<int>(aliases_.size()) && aliases_[rank]) return true;
  return rank >= 0 && rank < static_cast<int>(peers_.size()) && peers_[rank].mapped;
}

uint8_t* SymmetricHeap::base(int rank) const {
  if (rank == self_) return reinterpret_cast<uint8_t*>(own_.base);
  if (rank < static_cast<int>(aliases_.size()) && aliases_[rank])
    return reinterpret_cast<uint8_t*>(aliases_[rank]->own_.base);
  PCCL_CHECK(rank >= 0 && rank < static_cast<int>(peers_.size()) && peers_[rank].mapped,
             "rank " << rank << "'s heap is not mapped (was its endpoint exchanged?)");
  return reinterpret_cast<uint8_t*>(peers_[rank].base);
}

uint8_t* SymmetricHeap::control_alloc(size_t bytes, size_t align) {
  size_t at = round_up(control_used_, align);
  PCCL_CHECK(at + bytes <= HeapLayout::kControlBytes, "control area exhausted (" << at + bytes << " bytes)");
  control_used_ = at + bytes;
  return control(self_) + at;
}

// ---- NVLS --------------------------------------------------------------------------------------

bool SymmetricHeap::multicast_supported(int device) {
  try {
    const DriverApi& cu = DriverApi::get();
    CUdevice dev;
    if (cu.cuDeviceGet(&dev, device) != CUDA_SUCCESS) return false;
    int flag = 0;
    if (cu.cuDeviceGetAttribute(&flag, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return false;
    return flag != 0;
  } catch (const Error&) {
    return false;
  }
}

int SymmetricHeap::multicast_create(int world) {
  const DriverApi& cu = DriverApi::get();
  CUmulticastObjectProp prop{};
  prop.numDevices = static_cast<unsigned>(world);
  prop.size = layout_.total_bytes;
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  PCCL_CU(cu.cuMulticastCreate(&mc_.handle, &prop));
  mc_bytes_ = layout_.total_bytes;
  int fd = -1;
  PCCL_CU(cu.cuMemExportToShareableHandle(&fd, mc_.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  return fd;
}

void SymmetricHeap::multicast_import(int fd) {
  const DriverApi& cu = DriverApi::get();
  CUresult r = cu.cuMemImportFromShareableHandle(&mc_.handle, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                                 CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  close(fd);
  PCCL_CHECK(r == CUDA_SUCCESS, "importing the multicast object failed: " << cu.error_string(r));
  mc_bytes_ = layout_.total_bytes;
}

void SymmetricHeap::multicast_add_device() {
  const DriverApi& cu = DriverApi::get();
  CUdevice dev;
  PCCL_CU(cu.cuDeviceGet(&dev, device_));
  PCCL_CU(cu.cuMulticastAddDevice(mc_.handle, dev));
}

void SymmetricHeap::multicast_bind_and_map() {
  const DriverApi& cu = DriverApi::get();
  PCCL_CU(cu.cuMulticastBindMem(mc_.handle, 0, own_.handle, 0, mc_bytes_, 0));
  mc_bound_ = true;
  mc_.bytes = mc_bytes_;
  PCCL_CU(cu.cuMemAddressReserve(&mc_.base, mc_.bytes, granularity_, 0, 0));
  PCCL_CU(cu.cuMemMap(mc_.base, mc_.bytes, 0, mc_.handle, 0));
  grant_access(mc_.base, mc_.bytes, device_);
  mc_.mapped = true;
}

void SymmetricHeap::multicast_release() {
  if (mc_.handle == 0) return;
  const DriverApi& cu = DriverApi::get();
  if (mc_.mapped) {
    cu.cuMemUnmap(mc_.base, mc_.bytes);
    cu.cuMemAddressFree(mc_.base, mc_.bytes);
  }
  if (mc_bound_) {
    CUdevice dev;
    if (cu.cuDeviceGet(&dev, device_) == CUDA_SUCCESS) cu.cuMulticastUnbind(mc_.handle, dev, 0, mc_bytes_);
  }
  cu.cuMemRelease(mc_.handle);
  mc_ = Mapping{};
  mc_bound_ = false;
}

}  // namespace pccl
