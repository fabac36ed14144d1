// Sharing device buffers between the ranks (one process per GPU) of one box, for the
// column-parallel exchange of the decode GEMV: a rank exports the allocation that holds its
// exchange buffer, the peers map it and from then on store into it over NVLink from their
// own kernels. Plain CUDA IPC; nothing here launches a kernel.
#include <cuda.h>

#include <cstring>

#include "common.cuh"

using namespace b200lut;

namespace {

typedef CUresult (*AddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

AddressRangeFn address_range_fn() {
  static AddressRangeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<AddressRangeFn>(p);
  }();
  return fn;
}

}  // namespace

extern "C" int b200lut_peer_export(const void* ptr, unsigned char handle[64], int64_t* offset) {
  B200LUT_REQUIRE(ptr && handle && offset, B200LUT_ERR_INVALID, "null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  B200LUT_CUDA_OK(cudaFree(nullptr));   // make sure the context exists
  AddressRangeFn range = address_range_fn();
  B200LUT_REQUIRE(range, B200LUT_ERR_CUDA, "driver entry cuMemGetAddressRange not found");
  CUdeviceptr base = 0;
  size_t size = 0;
  B200LUT_REQUIRE(range(&base, &size, CUdeviceptr(uintptr_t(ptr))) == CUDA_SUCCESS,
                  B200LUT_ERR_INVALID, "pointer is not inside a device allocation");
  cudaIpcMemHandle_t h;
  B200LUT_CUDA_OK(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(uintptr_t(base))));
  memcpy(handle, &h, 64);
  *offset = int64_t(uintptr_t(ptr) - uintptr_t(base));
  return B200LUT_OK;
}

extern "C" int b200lut_peer_open(const unsigned char handle[64], void** base) {
  B200LUT_REQUIRE(handle && base, B200LUT_ERR_INVALID, "null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  B200LUT_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *base = p;
  return B200LUT_OK;
}

extern "C" int b200lut_peer_close(void* base) {
  B200LUT_REQUIRE(base, B200LUT_ERR_INVALID, "null argument");
  B200LUT_CUDA_OK(cudaIpcCloseMemHandle(base));
  return B200LUT_OK;
}
