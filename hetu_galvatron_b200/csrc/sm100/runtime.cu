// Host-side runtime of the kernel library: per-device status word, tensor-map encoding through
// the driver entry point, and small C-ABI utilities used by the Python layer.
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "sm100_common.cuh"

namespace hg_host {

int encode_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                   uint32_t box_cols);

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

// ---------------------------------------------------------------------------------------------------------------
// Tensor-map cache.  A tensor map is a pure function of (base address, extents, strides, box): a training step
// encodes the same few hundred of them again and again (every GEMM two, every attention call three or four), each a
// driver call.  A small direct-mapped table per host thread (the autograd engine launches the backward from its own
// threads, so no lock is needed) returns the 128-byte descriptor of a key seen before.  A cached entry never goes
// stale: it names addresses, not allocations, and the same address with the same geometry gives the same descriptor.
// ---------------------------------------------------------------------------------------------------------------
namespace {

struct TmapKey {
  uint64_t v[8];
  bool operator==(const TmapKey& o) const { return memcmp(v, o.v, sizeof(v)) == 0; }
};
struct TmapEntry {
  TmapKey key;
  CUtensorMap map;
  bool valid;
};
constexpr int kTmapSlots = 2048;   // power of two

TmapEntry* tmap_table() {
  static thread_local TmapEntry* table = nullptr;
  if (table == nullptr) table = static_cast<TmapEntry*>(calloc(kTmapSlots, sizeof(TmapEntry)));   // lives as long as the thread
  return table;
}
inline uint32_t tmap_slot(const TmapKey& k) {
  uint64_t h = 0x9E3779B97F4A7C15ull;
  for (int i = 0; i < 8; ++i) {
    h ^= k.v[i] + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
  }
  return uint32_t(h ^ (h >> 29)) & (kTmapSlots - 1);
}

}  // namespace

const CUtensorMap* tmap_cache_find(const uint64_t (&key)[8]) {
  TmapEntry* t = tmap_table();
  if (t == nullptr) return nullptr;
  TmapKey k;
  memcpy(k.v, key, sizeof(k.v));
  TmapEntry& e = t[tmap_slot(k)];
  return (e.valid && e.key == k) ? &e.map : nullptr;
}
void tmap_cache_store(const uint64_t (&key)[8], const CUtensorMap& map) {
  TmapEntry* t = tmap_table();
  if (t == nullptr) return;
  TmapKey k;
  memcpy(k.v, key, sizeof(k.v));
  TmapEntry& e = t[tmap_slot(k)];
  e.key = k;
  e.map = map;
  e.valid = true;
}

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols) {
  const uint64_t key[8] = {2, uint64_t(reinterpret_cast<uintptr_t>(base)), rows, cols, ld,
                           (uint64_t(box_rows) << 32) | box_cols, 0, 0};
  if (const CUtensorMap* hit = tmap_cache_find(key)) {
    *out = *hit;
    return 0;
  }
  const int rc = encode_tmap_2d(out, base, rows, cols, ld, box_rows, box_cols);
  if (rc == 0) tmap_cache_store(key, *out);
  return rc;
}

int encode_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                   uint32_t box_cols) {
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
