// bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2 with a 256 x 256 x 64 tile per two-SM cluster.
//
// Compared with the one-CTA kernel (gemm.cu, 128 x 256 tile per SM) each SM stages only half of the B tile: the
// pair's MMA reads A rows [0,128) / [128,256) from the two CTAs' shared memory and the two halves of B's N range
// from both, so a 128 x 256 slice of the output costs 32 KB of operand traffic per k-block per SM instead of 48 KB,
// and six stages fit where four did.
//
// Roles per CTA (192 threads): warp 0 TMA producer (the warp walks the loop, one elected lane issues), warp 1 TMEM allocator (+ UMMA issuer in the leader
// CTA only: the warp walks the loop, one elected lane issues), warps 2-5 epilogue.  Barriers (same shared-memory offsets in both CTAs):
//   full[s]        leader only; the leader's producer arrives with the byte count of BOTH CTAs' loads, every load
//                  (from either CTA) completes its bytes on the leader's barrier
//   empty[s]       both CTAs; signalled by tcgen05.commit with a cluster mask covering the pair
//   tmem_full[a]   both CTAs; same mechanism, once per tile
//   tmem_empty[a]  leader only; all 256 epilogue threads of the pair arrive (the peer's through its cluster address)
// Every wait is bounded (2 s); a CTA that gives up raises its abort flag and the status word, its partner runs into
// its own limit, and both still meet at the final cluster barrier and free their tensor memory.
// No operand load uses cluster multicast: each CTA loads exactly the bytes it alone needs.
#include <cstdlib>
#include <mutex>

#include "gemm2_core.cuh"

namespace hg {
namespace gemm2 {

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  Smem2 s = carve2(smem_raw);
  const int warp = threadIdx.x >> 5;
  const uint32_t rank = cluster_ctarank();
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
#pragma unroll
    for (int i = 0; i < STAGES2; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.tmem_full[i], 1);
      mbar_init(&s.tmem_empty[i], 2 * EPI_WARPS * 32);
    }
    *s.abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(s.tmem_base, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers exist before anything arrives on them remotely
  tc_fence_after();
  const uint32_t tmem_base = *s.tmem_base;

  if (warp == 0) {
    producer2<A_MN, B_MN>(&tmA, &tmB, p, s, rank, pair, pairs, num_tiles);
  } else if (warp == 1) {
    if (rank == 0) mma2<A_MN, B_MN>(p, s, tmem_base, pair, pairs, num_tiles);
  } else {
    epilogue2(p, s, tmem_base, rank, pair, pairs, num_tiles);
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees tensor memory or leaves while its partner may still touch it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm2
}  // namespace hg

using namespace hg::gemm;
using namespace hg::gemm2;

namespace {

// Scratch of the tail split: partial tiles and arrival counters, one set per (device, stream) for up to four
// streams per device (a launch on a fifth stream runs without the split).  Allocated on first use, never freed.
constexpr int kSplitMaxUnits = 128;                 // >= number of CTA pairs
struct SplitScratch {
  cudaStream_t stream;
  float* ws;
  int* flags;
};
SplitScratch g_split[64][4] = {};
std::mutex g_split_mu;

bool split_scratch(cudaStream_t st, float** ws, int** flags) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  std::lock_guard<std::mutex> lk(g_split_mu);
  for (int i = 0; i < 4; ++i) {
    SplitScratch& e = g_split[dev][i];
    if (e.ws != nullptr && e.stream != st) continue;
    if (e.ws == nullptr) {
      void* p = nullptr;
      if (cudaMalloc(&p, size_t(kSplitMaxUnits) * kSplitTileFloats * sizeof(float) + kSplitMaxUnits * sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return false;
      }
      e.ws = static_cast<float*>(p);
      e.flags = reinterpret_cast<int*>(e.ws + size_t(kSplitMaxUnits) * kSplitTileFloats);
      e.stream = st;
    }
    *ws = e.ws;
    *flags = e.flags;
    return true;
  }
  return false;
}

// HG_GEMM_SPLIT_TAIL=1 switches the tail split on, 0 off.
constexpr int kSplitDefault = 0;
bool split_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("HG_GEMM_SPLIT_TAIL");
    on = (e == nullptr || e[0] == 0) ? kSplitDefault : (e[0] != '0');
  }
  return on != 0;
}

}  // namespace

template <bool A_MN, bool B_MN>
static int launch2(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p_in, int want_pairs, cudaStream_t st) {
  Params p = p_in;
  static int max_pairs = -1;
  auto k = gemm2_bf16_kernel<A_MN, B_MN>;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = SMEM2_BYTES;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (max_pairs < 0) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2_BYTES);
    if (e != cudaSuccess) return int(e);
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cfg.gridDim = dim3(unsigned(sms / 2 * 2), 1, 1);
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, k, &cfg);
    if (e != cudaSuccess) return int(e);
    if (n <= 0) return -2;
    max_pairs = n;
  }
  const int pairs = want_pairs < max_pairs ? want_pairs : max_pairs;
  cfg.gridDim = dim3(unsigned(2 * pairs), 1, 1);
  // Last wave partly filled: let several pairs share each of its tiles (see Params::split_s).
  p.split_s = 0;
  const int tiles = p.tiles_m * p.tiles_n, num_kb = (p.K + BK - 1) / BK;
  const int full = tiles / pairs, tail = tiles - full * pairs;
  if (split_enabled() && p.k_ranges == nullptr && p.ready == nullptr && full >= 1 && tail >= 1 && pairs <= kSplitMaxUnits) {
    int s = pairs / tail;
    if (s > 4) s = 4;
    if (s > num_kb / 8) s = num_kb / 8;
    if (s >= 2 && split_scratch(st, &p.split_ws, &p.split_flags)) {
      p.split_s = s;
      p.split_tail_begin = full * pairs;
      cudaError_t me = cudaMemsetAsync(p.split_flags, 0, size_t(tail) * s * sizeof(int), st);
      if (me != cudaSuccess) return int(me);
    }
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, k, ta, tb, p);
  return int(e);
}

extern "C" {

// Same contract as hg_gemm_bf16 (gemm.cu), computed by CTA pairs.  Returns -2 when the device cannot co-schedule a
// pair of these CTAs (the caller then uses the one-CTA kernel).
int hg_gemm2_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb,
                  int ldc, int a_mn, int b_mn, int out_mode, int max_ctas, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -1;
  CUtensorMap ta, tb;
  int rc;
  if (a_mn) rc = hg_host::make_tmap_2d_bf16(&ta, A, K, M, lda, 64, 64);
  else      rc = hg_host::make_tmap_2d_bf16(&ta, A, M, K, lda, BM, 64);
  if (rc) return rc;
  if (b_mn) rc = hg_host::make_tmap_2d_bf16(&tb, B, K, N, ldb, 64, 64);
  else      rc = hg_host::make_tmap_2d_bf16(&tb, B, N, K, ldb, HALF_N, 64);
  if (rc) return rc;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.C = C;
  p.bias = reinterpret_cast<const hg_lp_t*>(bias);
  p.out_mode = out_mode;
  p.tiles_m = (M + CM - 1) / CM;
  p.tiles_n = (N + BN - 1) / BN;
  p.group_m = 4;
  p.status = hg_host::status_ptr();
  p.ready = nullptr; p.rows_per_flag = 1; p.ready_target = 0; p.m_tile_shift = 0;
  p.k_ranges = nullptr; p.groups = 1; p.c_group_stride = 0;
  int pairs = p.tiles_m * p.tiles_n;
  if (max_ctas > 1 && max_ctas / 2 < pairs) pairs = max_ctas / 2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a_mn && b_mn) return launch2<true, true>(ta, tb, p, pairs, st);
  if (a_mn) return launch2<true, false>(ta, tb, p, pairs, st);
  if (b_mn) return launch2<false, true>(ta, tb, p, pairs, st);
  return launch2<false, false>(ta, tb, p, pairs, st);
}

}  // extern "C"
