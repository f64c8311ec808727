// Host-side runtime of the kernel library: per-device status word, tensor-map encoding through
// the driver entry point, and small C-ABI utilities used by the Python layer.
#include <mutex>

#include "sm100_common.cuh"

namespace hg_host {

static std::mutex g_mu;
static int* g_status[64] = {nullptr};
static EncodeTiledFn g_encode = nullptr;

int* status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_status[dev] == nullptr) {
    int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    g_status[dev] = p;
  }
  return g_status[dev];
}

// cuTensorMapEncodeTiled is a driver call and needs a current context on the calling thread; threads
// that have only been handed work by another thread (autograd's backward workers) may not have bound
// the primary context yet, so bind it once per thread through the runtime.
static void ensure_context_on_this_thread() {
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

EncodeTiledFn get_encode_fn() {
  ensure_context_on_this_thread();
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  return g_encode;
}

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return -2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, HG_TMAP_LP, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(1000 + int(r));
}

int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1,
                      uint64_t stride2, uint32_t box0, uint32_t box1, uint32_t box2) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return -2;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1 * 2, stride2 * 2};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, HG_TMAP_LP, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(1000 + int(r));
}

}  // namespace hg_host

extern "C" {

// Reads (and optionally clears) the device status word.  Synchronises the device.
int hg_read_status(int clear) {
  int* p = hg_host::status_ptr();
  if (p == nullptr) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (clear && v != 0) cudaMemset(p, 0, sizeof(int));
  return v;
}

// Device address of the status word (lets a test or a fused kernel's host side poll it).
void* hg_status_address() { return hg_host::status_ptr(); }

int hg_library_version() { return 100; }

}  // extern "C"
