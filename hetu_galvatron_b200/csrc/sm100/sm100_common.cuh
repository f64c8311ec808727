// Blackwell (sm_100a) device primitives shared by every kernel of this library:
// mbarrier, TMA (cp.async.bulk.tensor, never with cluster multicast), tcgen05
// (TMEM alloc, UMMA issue/commit, TMEM loads) and the shared-memory / instruction
// descriptor encoders.  All waits are bounded: a wait that runs out records a code
// in a device status word and returns false so that the kernel can unwind (release
// TMEM, return) instead of spinning forever.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// ---------------------------------------------------------------------------
// The 16-bit storage type of every kernel.  The regular build works on bfloat16; compiled with -DHG_HALF the same
// sources work on IEEE half (libhg_sm100_fp16.so, loaded for `mixed_precision: fp16` models).  Accumulation,
// softmax, normalisation statistics and optimizer state are fp32 in both builds.
// ---------------------------------------------------------------------------
#ifdef HG_HALF
typedef __half hg_lp_t;
typedef __half2 hg_lp2_t;
#define HG_TMAP_LP CU_TENSOR_MAP_DATA_TYPE_FLOAT16
__device__ __forceinline__ float hg_lp2f(hg_lp_t x) { return __half2float(x); }
__device__ __forceinline__ hg_lp_t hg_f2lp(float x) { return __float2half_rn(x); }
__device__ __forceinline__ hg_lp2_t hg_ff2lp2(float lo, float hi) { return __floats2half2_rn(lo, hi); }
__device__ __forceinline__ float2 hg_lp22ff(hg_lp2_t v) { return __half22float2(v); }
#else
typedef __nv_bfloat16 hg_lp_t;
typedef __nv_bfloat162 hg_lp2_t;
#define HG_TMAP_LP CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
__device__ __forceinline__ float hg_lp2f(hg_lp_t x) { return __bfloat162float(x); }
__device__ __forceinline__ hg_lp_t hg_f2lp(float x) { return __float2bfloat16(x); }
__device__ __forceinline__ hg_lp2_t hg_ff2lp2(float lo, float hi) { return __floats2bfloat162_rn(lo, hi); }
__device__ __forceinline__ float2 hg_lp22ff(hg_lp2_t v) { return __bfloat1622float2(v); }
#endif
// two packed 16-bit values of a 32-bit word -> two floats
__device__ __forceinline__ float2 hg_unpack2(uint32_t w) { return hg_lp22ff(*reinterpret_cast<hg_lp2_t*>(&w)); }

namespace hg {

// ---------------------------------------------------------------------------
// Status word shared by all kernels of the library (0 == healthy).
// ---------------------------------------------------------------------------
enum StatusCode : int {
  kOk = 0,
  kTimeoutSmemFull = 1,
  kTimeoutSmemEmpty = 2,
  kTimeoutTmemFull = 3,
  kTimeoutTmemEmpty = 4,
  kTimeoutPeerFlag = 5,
  kBadArgument = 6,
  kTimeoutOther = 7,
};

// Kernels receive the status word's device address as an argument (one word per
// device, owned by runtime.cu); the first failure wins.
__device__ __forceinline__ void set_status(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

// Debug build (-DHG_DEBUG_BOUNDS, libhg_sm100_debug.so): every index a kernel derives from its arguments (tile
// coordinates, row ranges of expert segments, peer indices, rows of peer buffers) is checked before the access it
// feeds; a failed check records kBadArgument in the status word and the access is skipped (no trap, no fault).
// In the regular build the checks compile to nothing.
#ifdef HG_DEBUG_BOUNDS
#define HG_BOUNDS_OK(cond, status) ((cond) ? true : (::hg::set_status((status), ::hg::kBadArgument), false))
#else
#define HG_BOUNDS_OK(cond, status) (true)
#endif

// Every spin wait is bounded in wall-clock time (the global nanosecond timer), not in iterations:
// one mbarrier.try_wait may itself block for a hardware-defined slice of time.
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s
constexpr uint32_t kSpinLimit = 1u << 22;          // iteration cap of the flag polls that also sleep

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---------------------------------------------------------------------------
// Small helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n"
      ".reg .b32 rx;\n"
      ".reg .pred px;\n"
      "elect.sync rx|px, %1;\n"
      "@px mov.s32 %0, 1;\n"
      "}\n"
      : "+r"(pred)
      : "r"(0xFFFFFFFFu));
  return pred;
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One arrival for the whole (converged) warp: the lanes meet first, so what each of them did before the call is
// ordered before the arrival that lane 0 makes.  The barrier counts warps, not threads: 32 arrivals on one
// shared-memory word serialise, and a barrier that every softmax thread hits several times per step pays for it.
__device__ __forceinline__ void mbar_arrive_warp(uint64_t* bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and records `code`) when the limit is reached.
// `abort` (optional, shared memory) lets a sibling role that already gave up cut the wait short.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code,
                                          volatile int* abort = nullptr) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 128; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (abort != nullptr && *abort) return false;
    if (globaltimer_ns() - t0 > kWaitLimitNs) break;
  }
  set_status(status, code);
  return false;
}

// Warp-collective bounded wait: every lane waits, the verdict is made uniform so that the warp never
// diverges around the .sync.aligned tcgen05 instructions that follow.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, int* status, int code,
                                               volatile int* abort = nullptr) {
  const bool ok = mbar_wait(bar, parity, status, code, abort);
  return __all_sync(0xffffffffu, ok);
}

// ---------------------------------------------------------------------------
// Proxy fences
// ---------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------
// TMA (tiled bulk tensor copies; loads complete on an mbarrier)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05: tensor memory and UMMA
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier once every previously issued tcgen05.mma of this thread retired.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], bf16/fp16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor for 128-byte-swizzled tiles (the layout TMA
// writes with CU_TENSOR_MAP_SWIZZLE_128B when the box's inner extent is 128 bytes).
//   K-major operand : rows of 128 B (64 bf16 along K); groups of 8 rows are 1024 B
//                     apart (SBO); LBO is unused.  Advance K by adding bytes>>4 to
//                     the start-address field (32 B per UMMA_K = 16).
//   MN-major operand: rows of 128 B (64 bf16 along M/N), one row per K index; groups
//                     of 8 K-rows are SBO = 1024 B apart; the next 64-wide M/N slab
//                     starts LBO bytes further.  Advance K by 16 rows = 2048 B.
constexpr uint64_t kDescSw128 = (uint64_t(1) << 46) | (uint64_t(2) << 61);
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return kDescSw128 | uint64_t((saddr & 0x3FFFF) >> 4) | (uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16) |
         (uint64_t((sbo_bytes >> 4) & 0x3FFF) << 32);
}

// Instruction descriptor of kind::f16 with fp32 accumulation; A / B format 1 = bf16, 0 = f16 (the build's 16-bit type).
#ifdef HG_HALF
constexpr uint32_t kIdescLpFormat = 0u;
#else
constexpr uint32_t kIdescLpFormat = 1u;
#endif
__host__ __device__ constexpr uint32_t make_idesc_lp(int m, int n, bool a_mn_major, bool b_mn_major) {
  return (1u << 4)                  // D format: f32
         | (kIdescLpFormat << 7)    // A format
         | (kIdescLpFormat << 10)   // B format
         | (uint32_t(a_mn_major) << 15) | (uint32_t(b_mn_major) << 16) | (uint32_t(n >> 3) << 17) |
         (uint32_t(m >> 4) << 24);
}

// TMEM -> registers: this thread's lane (row), 32 / 16 / 8 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Byte offset of 16-byte chunk `chunk16` (0..7) of row `row` inside a 128B-swizzled
// tile whose rows are 128 bytes (tile base 1024-byte aligned).
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t chunk16) {
  return row * 128u + ((chunk16 ^ (row & 7u)) << 4);
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  hg_lp2_t v = hg_ff2lp2(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace hg

// ---------------------------------------------------------------------------
// Host side: tensor-map encoding through the driver entry point (no -lcuda).
// ---------------------------------------------------------------------------
namespace hg_host {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn();

// Device address of the current device's status word (allocated on first use).
int* status_ptr();

// rank-2 bf16 tensor [rows, cols] with row pitch `ld` elements; box = [box_rows, box_cols]; 128B swizzle.
// Returns 0 on success.
// Per-thread cache of encoded tensor maps, keyed by eight words that determine the descriptor (runtime.cu).
const CUtensorMap* tmap_cache_find(const uint64_t (&key)[8]);
void tmap_cache_store(const uint64_t (&key)[8], const CUtensorMap& map);
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols);
// rank-3 bf16 tensor [d2, d1, d0] (d0 innermost) with strides in elements.
int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1,
                      uint64_t stride2, uint32_t box0, uint32_t box1, uint32_t box2);

}  // namespace hg_host
