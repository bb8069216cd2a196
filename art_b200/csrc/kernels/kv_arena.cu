// Virtual-memory arena for the KV cache (and other large buffers whose physical memory comes and goes).
//
// A fixed virtual address range is reserved once (cuMemAddressReserve); physical chunks are created and mapped on
// demand (cuMemCreate + cuMemMap + cuMemSetAccess) and can be unmapped and released again while the addresses stay
// valid.  That is what lets the rollout engine give its KV memory to the trainer ("sleep") and take it back without
// invalidating the pointers baked into captured CUDA graphs or into the block tables.
//
// Counterpart in the reference: the CuMemAllocator-based sleep mode it patches into the inference library, which
// copies the KV arena to the host and unmaps it (src/art/local/vllm.py:148-231; raw cudaMemcpy at :199-201,223-227).
// Driver entry points are resolved through the runtime (no link-time dependency on libcuda).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

#include "host_utils.h"

namespace artb {

struct DriverVmm {
  CUresult (*getGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*addressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*addressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*setAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  bool ok = false;
};

static void* entry(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return p;
}

static const DriverVmm& vmm() {
  static DriverVmm d;
  static bool tried = false;
  if (!tried) {
    tried = true;
    d.getGranularity = reinterpret_cast<decltype(d.getGranularity)>(entry("cuMemGetAllocationGranularity"));
    d.addressReserve = reinterpret_cast<decltype(d.addressReserve)>(entry("cuMemAddressReserve"));
    d.addressFree = reinterpret_cast<decltype(d.addressFree)>(entry("cuMemAddressFree"));
    d.create = reinterpret_cast<decltype(d.create)>(entry("cuMemCreate"));
    d.release = reinterpret_cast<decltype(d.release)>(entry("cuMemRelease"));
    d.map = reinterpret_cast<decltype(d.map)>(entry("cuMemMap"));
    d.unmap = reinterpret_cast<decltype(d.unmap)>(entry("cuMemUnmap"));
    d.setAccess = reinterpret_cast<decltype(d.setAccess)>(entry("cuMemSetAccess"));
    d.ok = d.getGranularity && d.addressReserve && d.addressFree && d.create && d.release && d.map && d.unmap &&
           d.setAccess;
  }
  return d;
}

struct Arena {
  int device = 0;
  size_t chunk = 0;          // physical chunk size (multiple of the allocation granularity)
  size_t reserved = 0;       // bytes of virtual address space
  CUdeviceptr base = 0;
  std::vector<CUmemGenericAllocationHandle> handles;   // one per chunk, 0 = not mapped
  size_t mapped_chunks = 0;
};

}  // namespace artb

using namespace artb;

// Reserve `reserve_bytes` of address space on the current device; physical memory is handled in chunks of about
// `chunk_bytes` (rounded up to the allocation granularity, typically 2 MiB).  Returns nullptr on failure.
ARTB_EXPORT void* artb_arena_create(size_t reserve_bytes, size_t chunk_bytes) {
  const DriverVmm& d = vmm();
  if (!d.ok || reserve_bytes == 0) return nullptr;
  cudaFree(nullptr);   // make sure the primary context exists
  auto* a = new Arena();
  cudaGetDevice(&a->device);
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = a->device;
  size_t gran = 0;
  if (d.getGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || gran == 0) {
    delete a;
    return nullptr;
  }
  if (chunk_bytes < gran) chunk_bytes = gran;
  a->chunk = (chunk_bytes + gran - 1) / gran * gran;
  a->reserved = (reserve_bytes + a->chunk - 1) / a->chunk * a->chunk;
  if (d.addressReserve(&a->base, a->reserved, a->chunk, 0, 0) != CUDA_SUCCESS) {
    delete a;
    return nullptr;
  }
  a->handles.assign(a->reserved / a->chunk, 0);
  return a;
}

ARTB_EXPORT uint64_t artb_arena_base(void* h) { return static_cast<uint64_t>(static_cast<Arena*>(h)->base); }
ARTB_EXPORT size_t artb_arena_chunk(void* h) { return static_cast<Arena*>(h)->chunk; }
ARTB_EXPORT size_t artb_arena_reserved(void* h) { return static_cast<Arena*>(h)->reserved; }
ARTB_EXPORT size_t artb_arena_mapped_bytes(void* h) {
  auto* a = static_cast<Arena*>(h);
  return a->mapped_chunks * a->chunk;
}

// Back [offset, offset + bytes) with physical memory (chunks already mapped are left alone).  0 on success; on
// failure (e.g. out of memory) the chunks mapped by this call are rolled back and a positive CUresult is returned.
ARTB_EXPORT int artb_arena_map(void* h, size_t offset, size_t bytes) {
  auto* a = static_cast<Arena*>(h);
  const DriverVmm& d = vmm();
  if (!a || bytes == 0 || offset + bytes > a->reserved) return ERR_BAD_SHAPE;
  const size_t c0 = offset / a->chunk, c1 = (offset + bytes + a->chunk - 1) / a->chunk;
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = a->device;
  CUmemAccessDesc acc = {};
  acc.location = prop.location;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  std::vector<size_t> done;
  CUresult r = CUDA_SUCCESS;
  for (size_t c = c0; c < c1 && r == CUDA_SUCCESS; ++c) {
    if (a->handles[c]) continue;
    CUmemGenericAllocationHandle hd = 0;
    r = d.create(&hd, a->chunk, &prop, 0);
    if (r != CUDA_SUCCESS) break;
    r = d.map(a->base + c * a->chunk, a->chunk, 0, hd, 0);
    if (r == CUDA_SUCCESS) r = d.setAccess(a->base + c * a->chunk, a->chunk, &acc, 1);
    if (r != CUDA_SUCCESS) {
      d.unmap(a->base + c * a->chunk, a->chunk);
      d.release(hd);
      break;
    }
    a->handles[c] = hd;
    a->mapped_chunks++;
    done.push_back(c);
  }
  if (r != CUDA_SUCCESS) {
    for (size_t c : done) {
      d.unmap(a->base + c * a->chunk, a->chunk);
      d.release(a->handles[c]);
      a->handles[c] = 0;
      a->mapped_chunks--;
    }
    return static_cast<int>(r);
  }
  return 0;
}

// Return the physical memory of every chunk fully inside [offset, offset + bytes) to the driver; addresses stay
// reserved.  The caller must have synchronised all work that touches the range.
ARTB_EXPORT int artb_arena_unmap(void* h, size_t offset, size_t bytes) {
  auto* a = static_cast<Arena*>(h);
  const DriverVmm& d = vmm();
  if (!a || offset + bytes > a->reserved) return ERR_BAD_SHAPE;
  const size_t c0 = (offset + a->chunk - 1) / a->chunk, c1 = (offset + bytes) / a->chunk;
  for (size_t c = c0; c < c1; ++c) {
    if (!a->handles[c]) continue;
    d.unmap(a->base + c * a->chunk, a->chunk);
    d.release(a->handles[c]);
    a->handles[c] = 0;
    a->mapped_chunks--;
  }
  return 0;
}

ARTB_EXPORT void artb_arena_destroy(void* h) {
  auto* a = static_cast<Arena*>(h);
  if (!a) return;
  const DriverVmm& d = vmm();
  cudaDeviceSynchronize();
  for (size_t c = 0; c < a->handles.size(); ++c)
    if (a->handles[c]) {
      d.unmap(a->base + c * a->chunk, a->chunk);
      d.release(a->handles[c]);
    }
  d.addressFree(a->base, a->reserved);
  delete a;
}
