#include "cuda_driver.h"

#include <mutex>

namespace pccl {

namespace {
template <class Fn>
void resolve(const char* name, Fn* out) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult status;
  cudaError_t err = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &status);
  if (err != cudaSuccess || status != cudaDriverEntryPointSuccess || fn == nullptr) {
    (void)cudaGetLastError();
    throw Error(std::string("CUDA driver entry point '") + name + "' is unavailable: " +
                (err != cudaSuccess ? cudaGetErrorString(err) : "symbol not found"));
  }
  *out = reinterpret_cast<Fn>(fn);
}
}  // namespace

const DriverApi& DriverApi::get() {
  static DriverApi api;
  static std::once_flag once;
  std::call_once(once, [] {
#define PCCL_RESOLVE(NAME) resolve(#NAME, &api.NAME)
    PCCL_RESOLVE(cuGetErrorString);
    PCCL_RESOLVE(cuDeviceGet);
    PCCL_RESOLVE(cuDeviceGetAttribute);
    PCCL_RESOLVE(cuMemGetAllocationGranularity);
    PCCL_RESOLVE(cuMemCreate);
    PCCL_RESOLVE(cuMemRelease);
    PCCL_RESOLVE(cuMemAddressReserve);
    PCCL_RESOLVE(cuMemAddressFree);
    PCCL_RESOLVE(cuMemMap);
    PCCL_RESOLVE(cuMemUnmap);
    PCCL_RESOLVE(cuMemSetAccess);
    PCCL_RESOLVE(cuMemExportToShareableHandle);
    PCCL_RESOLVE(cuMemImportFromShareableHandle);
    PCCL_RESOLVE(cuMulticastCreate);
    PCCL_RESOLVE(cuMulticastAddDevice);
    PCCL_RESOLVE(cuMulticastBindMem);
    PCCL_RESOLVE(cuMulticastUnbind);
    PCCL_RESOLVE(cuMulticastGetGranularity);
    PCCL_RESOLVE(cuTensorMapEncodeTiled);
#undef PCCL_RESOLVE
  });
  return api;
}

std::string DriverApi::error_string(CUresult r) const {
  const char* text = nullptr;
  if (cuGetErrorString(r, &text) == CUDA_SUCCESS && text) return text;
  return "CUresult " + std::to_string(static_cast<int>(r));
}

}  // namespace pccl
