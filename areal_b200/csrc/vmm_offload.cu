// Device buffers that can give their physical memory back and get it again at the
// SAME virtual address (CUDA virtual memory management): tensors, TMA descriptors,
// captured graphs and peer tables that point into the buffer stay valid across an
// offload / onload cycle. Used for colocated training + rollout on one GPU: the idle
// side releases HBM (optionally parking the contents in pinned host memory).
//
// Counterpart of the reference's dependency torch_memory_saver
// (areal/engine/fsdp_engine.py offload / onload; areal/utils/offload.py).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>
#include <unordered_map>

#include "common/host_utils.h"

namespace b200 {
namespace {

struct DrvApi {
  CUresult (*memCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*memRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*memAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*memAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*memMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*memUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*memSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*memGetGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  bool ok = false;
};

template <class F>
bool load_sym(const char* name, F*& fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p)
    return false;
  fn = reinterpret_cast<F*>(p);
  return true;
}

DrvApi& drv() {
  static DrvApi api = [] {
    DrvApi a;
    a.ok = load_sym("cuMemCreate", a.memCreate) && load_sym("cuMemRelease", a.memRelease) &&
           load_sym("cuMemAddressReserve", a.memAddressReserve) && load_sym("cuMemAddressFree", a.memAddressFree) &&
           load_sym("cuMemMap", a.memMap) && load_sym("cuMemUnmap", a.memUnmap) &&
           load_sym("cuMemSetAccess", a.memSetAccess) &&
           load_sym("cuMemGetAllocationGranularity", a.memGetGranularity);
    return a;
  }();
  return api;
}

struct Region {
  size_t bytes = 0;  // padded to the allocation granularity
  int device = 0;
  CUmemGenericAllocationHandle handle = 0;
  bool resident = false;
  void* host_copy = nullptr;  // pinned, present only while offloaded with preserve
};

std::mutex g_mu;
std::unordered_map<uintptr_t, Region> g_regions;

CUmemAllocationProp prop_for(int device) {
  CUmemAllocationProp p{};
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  return p;
}

int map_physical(Region& r, CUdeviceptr va) {
  DrvApi& d = drv();
  CUmemAllocationProp p = prop_for(r.device);
  if (d.memCreate(&r.handle, r.bytes, &p, 0) != CUDA_SUCCESS) return -2;  // out of memory
  if (d.memMap(va, r.bytes, 0, r.handle, 0) != CUDA_SUCCESS) {
    d.memRelease(r.handle);
    return -3;
  }
  CUmemAccessDesc acc{};
  acc.location = p.location;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (d.memSetAccess(va, r.bytes, &acc, 1) != CUDA_SUCCESS) {
    d.memUnmap(va, r.bytes);
    d.memRelease(r.handle);
    return -4;
  }
  r.resident = true;
  return 0;
}

}  // namespace
}  // namespace b200

extern "C" {

// Returns the device pointer (0 on failure). The buffer is resident and uninitialised.
void* b200_vmm_alloc(size_t bytes) {
  using namespace b200;
  DrvApi& d = drv();
  if (!d.ok || bytes == 0) return nullptr;
  Region r;
  if (cudaGetDevice(&r.device) != cudaSuccess) return nullptr;
  cudaFree(0);
  CUmemAllocationProp p = prop_for(r.device);
  size_t gran = 0;
  if (d.memGetGranularity(&gran, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || gran == 0) return nullptr;
  r.bytes = (bytes + gran - 1) / gran * gran;
  CUdeviceptr va = 0;
  if (d.memAddressReserve(&va, r.bytes, gran, 0, 0) != CUDA_SUCCESS) return nullptr;
  if (map_physical(r, va) != 0) {
    d.memAddressFree(va, r.bytes);
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  g_regions[static_cast<uintptr_t>(va)] = r;
  return reinterpret_cast<void*>(va);
}

// Releases the physical memory; the address range stays reserved. With preserve != 0 the
// contents are parked in pinned host memory first. The caller has synchronised every
// stream that uses the buffer.
int b200_vmm_offload(void* ptr, int preserve) {
  using namespace b200;
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_regions.find(reinterpret_cast<uintptr_t>(ptr));
  if (it == g_regions.end()) return -1;
  Region& r = it->second;
  if (!r.resident) return 0;
  if (preserve) {
    if (!r.host_copy) B200_CHECK(cudaMallocHost(&r.host_copy, r.bytes));
    B200_CHECK(cudaMemcpy(r.host_copy, ptr, r.bytes, cudaMemcpyDeviceToHost));
  } else {
    B200_CHECK(cudaDeviceSynchronize());
  }
  DrvApi& d = drv();
  if (d.memUnmap(reinterpret_cast<CUdeviceptr>(ptr), r.bytes) != CUDA_SUCCESS) return -5;
  d.memRelease(r.handle);
  r.resident = false;
  return 0;
}

// Maps fresh physical memory at the same address; restores parked contents (else zero-fills).
int b200_vmm_onload(void* ptr) {
  using namespace b200;
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_regions.find(reinterpret_cast<uintptr_t>(ptr));
  if (it == g_regions.end()) return -1;
  Region& r = it->second;
  if (r.resident) return 0;
  int rc = map_physical(r, reinterpret_cast<CUdeviceptr>(ptr));
  if (rc) return rc;
  if (r.host_copy) {
    B200_CHECK(cudaMemcpy(ptr, r.host_copy, r.bytes, cudaMemcpyHostToDevice));
    cudaFreeHost(r.host_copy);
    r.host_copy = nullptr;
  } else {
    B200_CHECK(cudaMemset(ptr, 0, r.bytes));
  }
  return 0;
}

int b200_vmm_is_resident(void* ptr) {
  using namespace b200;
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_regions.find(reinterpret_cast<uintptr_t>(ptr));
  return it == g_regions.end() ? -1 : (it->second.resident ? 1 : 0);
}

int b200_vmm_free(void* ptr) {
  using namespace b200;
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_regions.find(reinterpret_cast<uintptr_t>(ptr));
  if (it == g_regions.end()) return -1;
  Region& r = it->second;
  DrvApi& d = drv();
  if (r.resident) {
    cudaDeviceSynchronize();
    d.memUnmap(reinterpret_cast<CUdeviceptr>(ptr), r.bytes);
    d.memRelease(r.handle);
  }
  if (r.host_copy) cudaFreeHost(r.host_copy);
  d.memAddressFree(reinterpret_cast<CUdeviceptr>(ptr), r.bytes);
  g_regions.erase(it);
  return 0;
}

}  // extern "C"
