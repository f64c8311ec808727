// Plain (single-GPU) entry points of the tcgen05 GEMM: dense, batched-by-offset and the
// grouped (per-expert) variant used by the MoE expert MLPs.
#include "gemm_core.cuh"

namespace hg {
namespace gemm {

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  SmemLayout s = carve(smem_raw);
  const int warp = threadIdx.x >> 5;
  const int num_tiles = p.tiles_m * p.tiles_n * p.groups;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    init_barriers(s);
  }
  if (warp == 1) {
    tmem_alloc(s.tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s.tmem_base;

  if (warp == 0) {
    producer_loop<A_MN, B_MN>(&tmA, &tmB, p, s, blockIdx.x, gridDim.x, num_tiles);  // whole warp, one elected issuer
  } else if (warp == 1) {
    mma_loop<A_MN, B_MN>(p, s, tmem_base, blockIdx.x, gridDim.x, num_tiles);  // whole warp, one elected issuer
  } else {
    epilogue_loop(p, s, tmem_base, blockIdx.x, gridDim.x, num_tiles);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Grouped GEMM: G independent problems that share N and K (and B's leading dimension) but have
// their own row range [row_start[g], row_start[g+1]) of A and C, and their own B matrix
// (B + g * b_group_stride).  One launch; tiles are enumerated group by group on the device from
// the row offsets, so the host never reads the routing result.
struct GroupedParams {
  Params base;
  const int* row_start;  // [G+1], device
  int G;
  int b_group_rows;      // rows of one group's B in the stacked tensor map (N for K-major, K for N-major)
};

template <bool B_MN>
__global__ void __launch_bounds__(192, 1)
grouped_gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const GroupedParams gp) {
  // Implementation note: each CTA walks the global tile list; a tile is (group, tm, tn).  A is K-major
  // [sum_rows, K]; rows past the group's end are masked in the epilogue (their products are discarded).
  extern __shared__ uint8_t smem_raw[];
  SmemLayout s = carve(smem_raw);
  const Params& p = gp.base;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    init_barriers(s);
  }
  if (warp == 1) {
    tmem_alloc(s.tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s.tmem_base;
  const int num_kb = (p.K + BK - 1) / BK;
  const int tiles_n = p.tiles_n;

  // Every role walks the same tile sequence: for g in groups, for tile in tiles(g) (n fastest).
  auto for_each_tile = [&](auto&& fn) {
    int counter = 0;
    for (int g = 0; g < gp.G; ++g) {
      const int r0 = gp.row_start[g], r1 = gp.row_start[g + 1];
      // an expert's row range must lie inside the operand and not run backwards (checked in the debug build)
      if (!HG_BOUNDS_OK(r0 >= 0 && r1 >= r0 && r1 <= p.M, p.status)) return;
      const int tm_cnt = (r1 - r0 + BM - 1) / BM;
      const int cnt = tm_cnt * tiles_n;
      // tiles of this group owned by this CTA: global index = counter + t
      int t = (int(blockIdx.x) - counter % int(gridDim.x) + int(gridDim.x)) % int(gridDim.x);
      for (; t < cnt; t += gridDim.x) {
        const int tm = t / tiles_n, tn = t % tiles_n;
        if (!fn(g, r0 + tm * BM, r1, tn * BN)) return;
      }
      counter += cnt;
    }
  };

  if (warp == 0) {
    // the whole warp walks the tile list; one elected lane issues the copies (see producer_loop in gemm_core.cuh)
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    const bool issuer = elect_one() != 0;
    for_each_tile([&](int g, int m0, int m_end, int n0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait_warp(&s.empty[stage], phase ^ 1, p.status, kTimeoutSmemEmpty, s.abort)) { ok = false; return false; }
        uint8_t* sa = s.a + stage * A_STAGE_BYTES;
        uint8_t* sb = s.b + stage * B_STAGE_BYTES;
        const int k0 = kb * BK;
        if (issuer) {
          mbar_expect_tx(&s.full[stage], A_STAGE_BYTES + B_STAGE_BYTES);
          tma_load_2d(sa, &tmA, &s.full[stage], k0, m0);
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * SLAB_BYTES, &tmB, &s.full[stage], n0 + j * 64, g * gp.b_group_rows + k0);
          } else {
            tma_load_2d(sb, &tmB, &s.full[stage], k0, g * gp.b_group_rows + n0);
          }
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      return true;
    });
    if (!ok) *s.abort = 1;
  } else if (warp == 1) {
    // the whole warp walks the tile list; one elected lane issues the MMAs (see mma_loop in gemm_core.cuh)
    constexpr uint32_t idesc = make_idesc_lp(BM, BN, false, B_MN);
    constexpr uint32_t b_lbo = B_MN ? SLAB_BYTES : 16, b_kadv = B_MN ? 2048 : 32;
    uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
    bool ok = true;
    const bool issuer = elect_one() != 0;
    for_each_tile([&](int, int, int, int) {
      if (!mbar_wait_warp(&s.tmem_empty[acc], acc_phase ^ 1, p.status, kTimeoutTmemEmpty, s.abort)) { ok = false; return false; }
      tc_fence_after();
      const uint32_t d = tmem_base + acc * BN;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait_warp(&s.full[stage], phase, p.status, kTimeoutSmemFull, s.abort)) { ok = false; return false; }
        tc_fence_after();
        const uint32_t sa = smem_u32(s.a + stage * A_STAGE_BYTES);
        const uint32_t sb = smem_u32(s.b + stage * B_STAGE_BYTES);
        if (issuer) {
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16_ss(d, make_smem_desc(sa + k * 32, 16, 1024), make_smem_desc(sb + k * b_kadv, b_lbo, 1024), idesc,
                        (kb | k) != 0);
          umma_commit(&s.empty[stage]);
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (issuer) umma_commit(&s.tmem_full[acc]);
      __syncwarp();
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      return true;
    });
    if (!ok) *s.abort = 1;
  } else {
    const int wq = warp & 3;
    const uint32_t lane_off = uint32_t(wq * 32) << 16;
    uint32_t acc = 0, acc_phase = 0;
    for_each_tile([&](int, int m0, int m_end, int n0) {
      if (!mbar_wait_warp(&s.tmem_full[acc], acc_phase, p.status, kTimeoutTmemFull, s.abort)) { *s.abort = 1; return false; }
      tc_fence_after();
      const int row = m0 + wq * 32 + lane_id();
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r0[32];
        tmem_ld32(tmem_base + lane_off + acc * BN + c * 32, r0);
        tmem_ld_wait();
        if (row < m_end && n0 + c * 32 < p.N) store_row_chunk(p, row, n0 + c * 32, r0);
      }
      tc_fence_before();
      mbar_arrive(&s.tmem_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      return true;
    });
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm
}  // namespace hg

// ------------------------------------------------------------------------------------------------
// Host launchers (C ABI; called from Python through ctypes with raw device pointers)
// ------------------------------------------------------------------------------------------------
using namespace hg::gemm;

static int g_num_sms = 0;
static int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_num_sms;
}

template <bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, int grid, cudaStream_t st) {
  static bool configured = false;
  auto k = gemm_bf16_kernel<A_MN, B_MN>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return int(e);
    configured = true;
  }
  k<<<grid, 192, SMEM_BYTES, st>>>(ta, tb, p);
  return int(cudaGetLastError());
}

extern "C" {

// C[M,N] = op(A) x op(B) with fp32 accumulation.
//   a_mn == 0 : A is [M,K] row-major with pitch lda;  a_mn == 1 : A is [K,M] row-major.
//   b_mn == 0 : B is [N,K] row-major with pitch ldb;  b_mn == 1 : B is [K,N] row-major.
//   out_mode  : see hg::gemm::OutMode.  Pitches are in elements and must be multiples of 8.
// Returns 0 on success, a CUDA error code or -1 (bad argument) otherwise.
int hg_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb,
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
  else      rc = hg_host::make_tmap_2d_bf16(&tb, B, N, K, ldb, BN, 64);
  if (rc) return rc;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.C = C;
  p.bias = reinterpret_cast<const hg_lp_t*>(bias);
  p.out_mode = out_mode;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.group_m = 8;
  p.status = hg_host::status_ptr();
  p.ready = nullptr; p.rows_per_flag = 1; p.ready_target = 0; p.m_tile_shift = 0;
  p.k_ranges = nullptr; p.groups = 1; p.c_group_stride = 0;
  int grid = p.tiles_m * p.tiles_n;
  int cap = num_sms();
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  if (grid > cap) grid = cap;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a_mn && b_mn) return launch<true, true>(ta, tb, p, grid, st);
  if (a_mn) return launch<true, false>(ta, tb, p, grid, st);
  if (b_mn) return launch<false, true>(ta, tb, p, grid, st);
  return launch<false, false>(ta, tb, p, grid, st);
}

// Grouped GEMM over G row ranges of A/C (row_start is a device array of G+1 ints, ascending):
//   C[r0:r1, :] = A[r0:r1, :] x op(B_g),  B_g = B + g * (b_mn ? K : N) rows of the stacked B.
//   A is [total_rows, K] row-major (K-major); B stacked [G*N, K] (b_mn == 0) or [G*K, N] (b_mn == 1).
//   `max_rows` is the host-known upper bound of total rows (the size of A's first dimension).
int hg_grouped_gemm_bf16(const void* A, const void* B, void* C, const void* row_start, int G, int max_rows, int N,
                         int K, int lda, int ldb, int ldc, int b_mn, int out_mode, void* stream) {
  if (G <= 0 || max_rows <= 0) return 0;
  if ((lda & 7) || (ldb & 7)) return -1;
  CUtensorMap ta, tb;
  int rc = hg_host::make_tmap_2d_bf16(&ta, A, max_rows, K, lda, BM, 64);
  if (rc) return rc;
  if (b_mn) rc = hg_host::make_tmap_2d_bf16(&tb, B, uint64_t(G) * K, N, ldb, 64, 64);
  else      rc = hg_host::make_tmap_2d_bf16(&tb, B, uint64_t(G) * N, K, ldb, BN, 64);
  if (rc) return rc;
  GroupedParams gp{};
  Params& p = gp.base;
  p.M = max_rows; p.N = N; p.K = K; p.ldc = ldc; p.C = C; p.bias = nullptr; p.out_mode = out_mode;
  p.tiles_m = 0; p.tiles_n = (N + BN - 1) / BN; p.group_m = 1; p.status = hg_host::status_ptr();
  gp.row_start = reinterpret_cast<const int*>(row_start);
  gp.G = G;
  gp.b_group_rows = b_mn ? K : N;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  static bool cfg[2] = {false, false};
  if (b_mn) {
    auto k = grouped_gemm_bf16_kernel<true>;
    if (!cfg[1]) { cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES); cfg[1] = true; }
    k<<<num_sms(), 192, SMEM_BYTES, st>>>(ta, tb, gp);
  } else {
    auto k = grouped_gemm_bf16_kernel<false>;
    if (!cfg[0]) { cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES); cfg[0] = true; }
    k<<<num_sms(), 192, SMEM_BYTES, st>>>(ta, tb, gp);
  }
  return int(cudaGetLastError());
}

// Self-test of the bounded waits: runs a small GEMM whose A-row gate is never opened.  The producer gives
// up after the wait limit, records kTimeoutPeerFlag in the status word, the other roles unwind, TMEM is
// released and the launch returns normally.  Returns 0 when the kernel came back and the context is healthy.
int hg_gemm_gated_selftest(void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int M = 256, N = 256, K = 128;
  void *A = nullptr, *B = nullptr, *C = nullptr, *flags = nullptr;
  if (cudaMalloc(&A, M * K * 2) || cudaMalloc(&B, N * K * 2) || cudaMalloc(&C, M * N * 2) || cudaMalloc(&flags, 64))
    return -4;
  cudaMemsetAsync(A, 0, M * K * 2, st);
  cudaMemsetAsync(B, 0, N * K * 2, st);
  cudaMemsetAsync(flags, 0, 64, st);
  CUtensorMap ta, tb;
  int rc = hg_host::make_tmap_2d_bf16(&ta, A, M, K, K, BM, 64);
  if (!rc) rc = hg_host::make_tmap_2d_bf16(&tb, B, N, K, K, BN, 64);
  if (!rc) {
    Params p{};
    p.M = M; p.N = N; p.K = K; p.ldc = N; p.C = C; p.out_mode = kOutBf16;
    p.tiles_m = 2; p.tiles_n = 1; p.group_m = 8; p.status = hg_host::status_ptr();
    p.ready = reinterpret_cast<const int*>(flags); p.rows_per_flag = 128; p.ready_target = 1;
    p.groups = 1;
    rc = launch<false, false>(ta, tb, p, 2, st);
    if (!rc) rc = int(cudaStreamSynchronize(st));
  }
  cudaFree(A); cudaFree(B); cudaFree(C); cudaFree(flags);
  return rc;
}

// Grouped weight gradient: out[g] (+)= dy[seg_g]^T x[seg_g], out fp32 [G, N, K] contiguous.
//   dy: [rows, N], x: [rows, K] (row-major); row_start: device int[G+1], every boundary a multiple of 64.
int hg_grouped_wgrad_bf16(const void* dy, const void* x, void* out, const void* row_start, int G, int rows, int N,
                          int K, int lddy, int ldx, int out_mode, int max_ctas, void* stream) {
  if (G <= 0 || rows <= 0) return 0;
  if ((lddy & 7) || (ldx & 7)) return -1;
  CUtensorMap ta, tb;
  int rc = hg_host::make_tmap_2d_bf16(&ta, dy, rows, N, lddy, 64, 64);
  if (rc) return rc;
  rc = hg_host::make_tmap_2d_bf16(&tb, x, rows, K, ldx, 64, 64);
  if (rc) return rc;
  Params p{};
  p.M = N; p.N = K; p.K = rows; p.ldc = K; p.C = out; p.bias = nullptr; p.out_mode = out_mode;
  p.tiles_m = (N + BM - 1) / BM; p.tiles_n = (K + BN - 1) / BN; p.group_m = 8;
  p.status = hg_host::status_ptr();
  p.ready = nullptr; p.rows_per_flag = 1; p.ready_target = 0; p.m_tile_shift = 0;
  p.k_ranges = reinterpret_cast<const int*>(row_start); p.groups = G; p.c_group_stride = (long long)N * K;
  int grid = p.tiles_m * p.tiles_n * G;
  int cap = num_sms();
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  if (grid > cap) grid = cap;
  // the kernel derives its tile count from tiles_m * tiles_n * groups
  return launch<true, true>(ta, tb, p, grid, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
