// CUDA driver entry points resolved at run time through the runtime
// (cudaGetDriverEntryPoint), so the extension neither links libcuda nor fails
// to load on a machine without a driver.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <string>

#include "../common/util.h"

namespace pccl {

struct DriverApi {
  CUresult (*cuGetErrorString)(CUresult, const char**);
  CUresult (*cuDeviceGet)(CUdevice*, int);
  CUresult (*cuDeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  CUresult (*cuMemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*cuMemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*cuMemRelease)(CUmemGenericAllocationHandle);
  CUresult (*cuMemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*cuMemAddressFree)(CUdeviceptr, size_t);
  CUresult (*cuMemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*cuMemUnmap)(CUdeviceptr, size_t);
  CUresult (*cuMemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*cuMemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*cuMemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*cuMulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*cuMulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*cuMulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
  CUresult (*cuMulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*cuMulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
  CUresult (*cuTensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                     CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                     CUtensorMapFloatOOBfill);

  // Resolved once per process; throws pccl::Error if the driver is unavailable.
  static const DriverApi& get();
  std::string error_string(CUresult r) const;
};

#define PCCL_CU(CALL)                                                                         \
  do {                                                                                        \
    CUresult pccl_cu_r = (CALL);                                                              \
    if (pccl_cu_r != CUDA_SUCCESS)                                                            \
      throw ::pccl::Error(std::string(#CALL) + " failed: " +                                  \
                          ::pccl::DriverApi::get().error_string(pccl_cu_r));                  \
  } while (0)

#define PCCL_CUDA(CALL)                                                                       \
  do {                                                                                        \
    cudaError_t pccl_rt_r = (CALL);                                                           \
    if (pccl_rt_r != cudaSuccess)                                                             \
      throw ::pccl::Error(std::string(#CALL) + " failed: " + cudaGetErrorString(pccl_rt_r));  \
  } while (0)

}  // namespace pccl
