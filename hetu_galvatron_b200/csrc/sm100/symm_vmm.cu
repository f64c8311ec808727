// Symmetric (peer-mapped) device memory through the CUDA virtual-memory-management API: the allocator behind the
// peer-memory kernels when HG_SYMM_ALLOC=vmm (the default allocator is torch.distributed._symmetric_memory).
//
// Every rank of a single-node group
//   1. creates a physical allocation that can be exported as a POSIX file descriptor (cuMemCreate +
//      cuMemExportToShareableHandle);
//   2. hands (pid, fd) to its peers through the Python layer (an all-gather of two integers; the peers duplicate
//      the descriptor with pidfd_getfd, so no socket plumbing is needed);
//   3. imports the peers' allocations (cuMemImportFromShareableHandle), reserves one virtual range per rank and maps
//      them (cuMemAddressReserve / cuMemMap / cuMemSetAccess for the local device).
// The result is the same thing the kernels get from the default allocator: one device pointer per rank, all valid on
// this GPU, pointer[me] being the local buffer.  Peer memory is then touched only by plain loads and stores in the
// kernels; nothing here launches a kernel or issues a TMA copy.
//
// The driver API is reached through cudaGetDriverEntryPoint, so the library needs no link against libcuda.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <mutex>

namespace {

struct Drv {
  CUresult (*memCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*memRelease)(CUmemGenericAllocationHandle);
  CUresult (*memExport)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*memImport)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*memGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*addrReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*addrFree)(CUdeviceptr, size_t);
  CUresult (*memMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*memUnmap)(CUdeviceptr, size_t);
  CUresult (*memSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  bool ok = false;
};

Drv g_drv;
std::mutex g_mu;

template <typename F>
bool entry(const char* name, F& fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return false;
  fn = reinterpret_cast<F>(p);
  return true;
}

bool load_driver() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_drv.ok) return true;
  cudaFree(nullptr);  // a current context on this thread
  Drv d;
  bool ok = entry("cuMemCreate", d.memCreate) && entry("cuMemRelease", d.memRelease) &&
            entry("cuMemExportToShareableHandle", d.memExport) && entry("cuMemImportFromShareableHandle", d.memImport) &&
            entry("cuMemGetAllocationGranularity", d.memGranularity) && entry("cuMemAddressReserve", d.addrReserve) &&
            entry("cuMemAddressFree", d.addrFree) && entry("cuMemMap", d.memMap) && entry("cuMemUnmap", d.memUnmap) &&
            entry("cuMemSetAccess", d.memSetAccess);
  if (ok) {
    g_drv = d;
    g_drv.ok = true;
  }
  return ok;
}

CUmemAllocationProp prop_for(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

int err(CUresult r) { return r == CUDA_SUCCESS ? 0 : -(1000 + int(r)); }

}  // namespace

extern "C" {

// Size that an allocation of `bytes` really takes on `device` (a multiple of the allocation granularity), or < 0.
long long hg_vmm_padded_size(long long bytes, int device) {
  if (bytes <= 0 || !load_driver()) return -1;
  CUmemAllocationProp p = prop_for(device);
  size_t g = 0;
  CUresult r = g_drv.memGranularity(&g, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS || g == 0) return err(r) ? err(r) : -1;
  return (long long)(((size_t)bytes + g - 1) / g * g);
}

// Create this rank's physical allocation of `padded` bytes (from hg_vmm_padded_size) on `device` and export it.
// handle_out: opaque 64-bit handle for hg_vmm_map / hg_vmm_release; fd_out: the descriptor the peers duplicate.
int hg_vmm_create(long long padded, int device, unsigned long long* handle_out, int* fd_out) {
  if (!load_driver() || padded <= 0 || handle_out == nullptr || fd_out == nullptr) return -1;
  CUmemAllocationProp p = prop_for(device);
  CUmemGenericAllocationHandle h;
  CUresult r = g_drv.memCreate(&h, (size_t)padded, &p, 0);
  if (r != CUDA_SUCCESS) return err(r);
  int fd = -1;
  r = g_drv.memExport(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    g_drv.memRelease(h);
    return err(r);
  }
  *handle_out = (unsigned long long)h;
  *fd_out = fd;
  return 0;
}

// Import a peer's allocation from a descriptor that is valid in THIS process.
int hg_vmm_import(int fd, unsigned long long* handle_out) {
  if (!load_driver() || handle_out == nullptr) return -1;
  CUmemGenericAllocationHandle h;
  CUresult r = g_drv.memImport(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return err(r);
  *handle_out = (unsigned long long)h;
  return 0;
}

// Map `t` allocations of `padded` bytes each (handles[r] = rank r's, handles[me] the local one) into this process for
// access from `device`; ptrs_out[r] receives the device pointer of rank r's buffer.
int hg_vmm_map(const unsigned long long* handles, int t, long long padded, int device, void** ptrs_out) {
  if (!load_driver() || t < 1 || t > 64 || padded <= 0) return -1;
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (int r = 0; r < t; ++r) {
    CUdeviceptr va = 0;
    CUresult e = g_drv.addrReserve(&va, (size_t)padded, 0, 0, 0);
    if (e != CUDA_SUCCESS) return err(e);
    e = g_drv.memMap(va, (size_t)padded, 0, (CUmemGenericAllocationHandle)handles[r], 0);
    if (e != CUDA_SUCCESS) {
      g_drv.addrFree(va, (size_t)padded);
      return err(e);
    }
    e = g_drv.memSetAccess(va, (size_t)padded, &acc, 1);
    if (e != CUDA_SUCCESS) {
      g_drv.memUnmap(va, (size_t)padded);
      g_drv.addrFree(va, (size_t)padded);
      return err(e);
    }
    ptrs_out[r] = reinterpret_cast<void*>(va);
  }
  return 0;
}

// Undo hg_vmm_map for one pointer and drop the reference on its allocation.
int hg_vmm_unmap_release(void* ptr, long long padded, unsigned long long handle) {
  if (!load_driver()) return -1;
  CUdeviceptr va = reinterpret_cast<CUdeviceptr>(ptr);
  CUresult a = g_drv.memUnmap(va, (size_t)padded);
  CUresult b = g_drv.addrFree(va, (size_t)padded);
  CUresult c = g_drv.memRelease((CUmemGenericAllocationHandle)handle);
  return err(a) ? err(a) : (err(b) ? err(b) : err(c));
}

}  // extern "C"
