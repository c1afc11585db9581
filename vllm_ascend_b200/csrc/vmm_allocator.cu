// Sleep-mode allocator on the CUDA virtual memory management API.
//
// Every allocation reserves a virtual address range and maps freshly created
// physical memory into it.  "Sleeping" unmaps and releases the physical memory
// while the virtual range stays reserved, so that after wake-up the same
// addresses are valid again (weights, KV cache and captured graphs keep their
// pointers).  Allocations carry the tag that was current when they were made
// ("weights", "kv_cache", ...), so the Python side can decide per tag whether
// the contents are backed up to host memory first.
//
// Parity: csrc/camem_allocator.cpp:49-346 of the reference (aclrtReserveMemAddress /
// aclrtMallocPhysical / aclrtMapMem) and vllm_ascend/device_allocator/camem.py.
// The malloc/free entry points have the signature torch's CUDAPluggableAllocator
// expects.  Driver entry points are resolved at run time, so the library loads
// on machines without a GPU driver.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

#define B200_API extern "C" __attribute__((visibility("default")))

namespace {

struct Driver {
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*,
                                          CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr,
                                unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*,
                        unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle,
                     unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  bool ok = false;
};

template <typename F>
bool resolve(const char* name, F& fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess || !p)
    return false;
  fn = reinterpret_cast<F>(p);
  return true;
}

Driver& drv() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    d.ok = resolve("cuMemGetAllocationGranularity", d.MemGetAllocationGranularity) &&
           resolve("cuMemAddressReserve", d.MemAddressReserve) &&
           resolve("cuMemAddressFree", d.MemAddressFree) &&
           resolve("cuMemCreate", d.MemCreate) && resolve("cuMemRelease", d.MemRelease) &&
           resolve("cuMemMap", d.MemMap) && resolve("cuMemUnmap", d.MemUnmap) &&
           resolve("cuMemSetAccess", d.MemSetAccess);
  });
  return d;
}

struct Alloc {
  size_t size = 0;          // mapped (granularity-aligned) size
  size_t requested = 0;
  int device = 0;
  CUmemGenericAllocationHandle handle = 0;
  bool mapped = false;
  std::string tag;
};

std::mutex g_mu;
std::map<uintptr_t, Alloc> g_allocs;
std::string g_tag = "default";
int g_last_error = 0;

CUmemAllocationProp make_prop(int device) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  return prop;
}

int create_and_map(int device, CUdeviceptr va, size_t size, CUmemGenericAllocationHandle* h) {
  Driver& d = drv();
  CUmemAllocationProp prop = make_prop(device);
  CUresult r = d.MemCreate(h, size, &prop, 0);
  if (r != CUDA_SUCCESS) return (int)r;
  r = d.MemMap(va, size, 0, *h, 0);
  if (r != CUDA_SUCCESS) {
    d.MemRelease(*h);
    return (int)r;
  }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = d.MemSetAccess(va, size, &acc, 1);
  if (r != CUDA_SUCCESS) {
    d.MemUnmap(va, size);
    d.MemRelease(*h);
    return (int)r;
  }
  return 0;
}

}  // namespace

// ---- torch pluggable-allocator entry points
B200_API void* b200_vmm_malloc(ssize_t size, int device, cudaStream_t /*stream*/) {
  Driver& d = drv();
  if (!d.ok || size <= 0) {
    g_last_error = -1;
    return nullptr;
  }
  cudaSetDevice(device);
  cudaFree(0);   // make sure the primary context exists on this thread
  CUmemAllocationProp prop = make_prop(device);
  size_t gran = 0;
  CUresult r = d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM);
  if (r != CUDA_SUCCESS || gran == 0) {
    g_last_error = (int)r;
    return nullptr;
  }
  const size_t aligned = ((size_t)size + gran - 1) / gran * gran;
  CUdeviceptr va = 0;
  r = d.MemAddressReserve(&va, aligned, gran, 0, 0);
  if (r != CUDA_SUCCESS) {
    g_last_error = (int)r;
    return nullptr;
  }
  CUmemGenericAllocationHandle h = 0;
  int rc = create_and_map(device, va, aligned, &h);
  if (rc) {
    d.MemAddressFree(va, aligned);
    g_last_error = rc;
    return nullptr;
  }
  std::lock_guard<std::mutex> g(g_mu);
  Alloc a;
  a.size = aligned;
  a.requested = (size_t)size;
  a.device = device;
  a.handle = h;
  a.mapped = true;
  a.tag = g_tag;
  g_allocs[(uintptr_t)va] = a;
  return (void*)va;
}

B200_API void b200_vmm_free(void* ptr, ssize_t /*size*/, int /*device*/, cudaStream_t /*stream*/) {
  Driver& d = drv();
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_allocs.find((uintptr_t)ptr);
  if (it == g_allocs.end()) return;
  Alloc& a = it->second;
  if (a.mapped) {
    d.MemUnmap((CUdeviceptr)ptr, a.size);
    d.MemRelease(a.handle);
  }
  d.MemAddressFree((CUdeviceptr)ptr, a.size);
  g_allocs.erase(it);
}

// ---- control surface used by device_allocator/vmm.py
B200_API int b200_vmm_available() { return drv().ok ? 1 : 0; }
B200_API int b200_vmm_last_error() { return g_last_error; }

B200_API void b200_vmm_set_tag(const char* tag) {
  std::lock_guard<std::mutex> g(g_mu);
  g_tag = tag ? tag : "default";
}

B200_API int b200_vmm_num_allocs() {
  std::lock_guard<std::mutex> g(g_mu);
  return (int)g_allocs.size();
}

// Fills parallel arrays (capacity n); returns the number written.
B200_API int b200_vmm_list(int n, uint64_t* ptrs, uint64_t* sizes, int* mapped, char* tags,
                           int tag_stride) {
  std::lock_guard<std::mutex> g(g_mu);
  int i = 0;
  for (auto& kv : g_allocs) {
    if (i >= n) break;
    ptrs[i] = (uint64_t)kv.first;
    sizes[i] = (uint64_t)kv.second.size;
    mapped[i] = kv.second.mapped ? 1 : 0;
    strncpy(tags + (size_t)i * tag_stride, kv.second.tag.c_str(), tag_stride - 1);
    tags[(size_t)i * tag_stride + tag_stride - 1] = 0;
    i++;
  }
  return i;
}

// Unmap + release the physical memory behind ptr, keep the virtual range.
B200_API int b200_vmm_unmap_and_release(void* ptr) {
  Driver& d = drv();
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_allocs.find((uintptr_t)ptr);
  if (it == g_allocs.end()) return -2;
  Alloc& a = it->second;
  if (!a.mapped) return 0;
  CUresult r = d.MemUnmap((CUdeviceptr)ptr, a.size);
  if (r != CUDA_SUCCESS) return (int)r;
  r = d.MemRelease(a.handle);
  if (r != CUDA_SUCCESS) return (int)r;
  a.mapped = false;
  a.handle = 0;
  return 0;
}

// Create new physical memory and map it at the same virtual address.
B200_API int b200_vmm_create_and_map(void* ptr) {
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_allocs.find((uintptr_t)ptr);
  if (it == g_allocs.end()) return -2;
  Alloc& a = it->second;
  if (a.mapped) return 0;
  cudaSetDevice(a.device);
  int rc = create_and_map(a.device, (CUdeviceptr)ptr, a.size, &a.handle);
  if (rc) return rc;
  a.mapped = true;
  return 0;
}

B200_API int b200_vmm_memcpy(void* dst, const void* src, uint64_t bytes, int to_host) {
  cudaError_t e = cudaMemcpy(dst, src, (size_t)bytes,
                             to_host ? cudaMemcpyDeviceToHost : cudaMemcpyHostToDevice);
  return (int)e;
}
