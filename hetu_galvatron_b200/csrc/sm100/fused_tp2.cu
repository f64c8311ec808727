// Fused tensor-parallel kernels on the CTA-pair tile (tcgen05.mma.cta_group::2, 256 x 256 x 64 per two-SM cluster):
// the same two operations as fused_tp.cu, with the same cross-rank protocol, built on gemm2_core.cuh.
//
//   all-gather -> column GEMM   : the communication warps (two per CTA, in both CTAs of every pair) pull the peers'
//                                 activation slabs with plain 16-byte peer loads into this GPU's gathered buffer and
//                                 count arrivals per 128-row block; each CTA's TMA producer waits for the block that
//                                 holds ITS 128 rows of the pair's tile.  Tiles of the local slab run first.
//   row GEMM -> reduce-scatter  : each CTA's epilogue stores its 128 x 256 partial (bf16, wire layout) into the
//                                 staging area of the rank that owns those rows and raises the tile's flag; after
//                                 its last tile every CTA reduces tiles of its own slab in fp32.
//
// Every tensor map covers local memory only and no load uses cluster multicast; peer memory is touched by plain
// ld / st.  Every wait is bounded and reports through the status word; a CTA that gives up sets its abort flag, its
// partner runs into its own limit, both meet at the final cluster barrier and free their tensor memory.
//
// Replaces the NCCL all-gather / reduce-scatter + library GEMM sequences of
// galvatron/core/runtime/tensor_parallel/layers.py:289-303, :320-376, :925-980.
#include "gemm2_core.cuh"

namespace hg {
namespace fused2 {

using namespace hg::gemm;
using namespace hg::gemm2;

constexpr int kMaxRanks = 8;
constexpr int kThreads2 = 256;  // 6 GEMM warps + 2 communication warps per CTA
constexpr int kSubRows = 8;     // rows per all-gather sub-block
constexpr int kInFlight = 16;   // independent 16-byte loads per communication thread

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void comm_bar() { asm volatile("bar.sync 1, 64;" ::: "memory"); }
__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

__device__ __forceinline__ bool wait_flag_sys(const int* flag, int target, int* status, volatile int* abort) {
  const uint64_t t0 = globaltimer_ns();
  while (ld_acquire_sys(flag) < target) {
    if ((abort != nullptr && *abort) || globaltimer_ns() - t0 > kWaitLimitNs) {
      set_status(status, kTimeoutPeerFlag);
      return false;
    }
    __nanosleep(100);
  }
  return true;
}

__device__ __forceinline__ void pair_prologue(const CUtensorMap* tmA, const CUtensorMap* tmB, const Smem2& s, int warp) {
  if (threadIdx.x == 0) {
    tma_prefetch_desc(tmA);
    tma_prefetch_desc(tmB);
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
    s.abort[0] = 0;
    s.abort[1] = 0;
    s.abort[2] = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(s.tmem_base, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
}

__device__ __forceinline__ void pair_epilogue_sync(uint32_t tmem_base, int warp) {
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------
// all-gather -> GEMM
// ------------------------------------------------------------------------------------------------
struct AgParams {
  const uint4* src[kMaxRanks];   // every rank's staging slab (src[me] is local)
  int* signal[kMaxRanks];        // signal[p]: rank p's "data ready" slots (int[kMaxRanks]); we write slot `me`
  int* my_signal;                // our own slots: my_signal[p] >= epoch once rank p's slab may be read
  uint4* gathered;               // local [t * slab_rows, K] buffer the GEMM reads
  int* block_ready;              // local arrival counters, one per 128-row block of `gathered`
  int t, me, epoch;
  int slab_rows;                 // rows per rank (multiple of 256)
  int row_vec;                   // uint4 per row (K * 2 / 16)
};

template <bool B_MN>
__global__ void __launch_bounds__(kThreads2, 1)
ag_gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p,
                const AgParams ag) {
  extern __shared__ uint8_t smem_raw[];
  Smem2 s = carve2(smem_raw);
  const int warp = threadIdx.x >> 5;
  const uint32_t rank = cluster_ctarank();
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  pair_prologue(&tmA, &tmB, s, warp);
  const uint32_t tmem_base = *s.tmem_base;

  if (warp == 0) {
    producer2<false, B_MN>(&tmA, &tmB, p, s, rank, pair, pairs, num_tiles);
  } else if (warp == 1) {
    if (rank == 0) mma2<false, B_MN>(p, s, tmem_base, pair, pairs, num_tiles);
  } else if (warp < 6) {
    epilogue2(p, s, tmem_base, rank, pair, pairs, num_tiles);
  } else {
    // ---- communication warps: 64 threads of every CTA ----------------------------------------------
    const int tid = threadIdx.x - 6 * 32;
    if (blockIdx.x == 0 && tid == 0) {
      // our slab was written by earlier work of this stream: publish it to every peer
      __threadfence_system();
      for (int q = 0; q < ag.t; ++q)
        if (q != ag.me) st_release_sys(ag.signal[q] + ag.me, ag.epoch);
    }
    // Sub-blocks of kSubRows rows are spread over every CTA with kInFlight independent 16-byte loads per thread
    // (NVLink needs on the order of 2 MB in flight chip-wide).  A 128-row block is ready once all of its
    // sub-blocks have arrived (arrival counter, zeroed by the host before the call).
    const int subs_per_slab = ag.slab_rows / kSubRows;
    const int total_subs = subs_per_slab * ag.t;
    const size_t sub_vec = size_t(kSubRows) * ag.row_vec;
    volatile int* comm_go = s.abort + 1;  // written by comm thread 0 between barriers: a uniform verdict
    for (int i = blockIdx.x; i < total_subs; i += gridDim.x) {
      const int hop = i / subs_per_slab;                // 0 = our own slab, then the ring of peers
      const int q = (ag.me + hop) % ag.t;
      const int j = i - hop * subs_per_slab;
      if (tid == 0) {
        bool ok = !*s.abort;
        if (ok && q != ag.me) ok = wait_flag_sys(ag.my_signal + q, ag.epoch, p.status, s.abort);
        if (!ok) *s.abort = 1;
        *comm_go = ok ? 1 : 0;
      }
      comm_bar();
      if (!*comm_go) break;
      const uint4* src = ag.src[q] + size_t(j) * sub_vec;
      uint4* dst = ag.gathered + (size_t(q) * subs_per_slab + j) * sub_vec;
      for (size_t v0 = tid; v0 < sub_vec; v0 += 64 * kInFlight) {
        uint4 buf[kInFlight];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u)
          if (v0 + size_t(u) * 64 < sub_vec) buf[u] = src[v0 + size_t(u) * 64];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u)
          if (v0 + size_t(u) * 64 < sub_vec) dst[v0 + size_t(u) * 64] = buf[u];
      }
      __threadfence();
      comm_bar();
      if (tid == 0) {
        int* ctr = ag.block_ready + (q * ag.slab_rows + j * kSubRows) / BM;
        asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(ctr) : "memory");
      }
    }
  }
  pair_epilogue_sync(tmem_base, warp);
}

// ------------------------------------------------------------------------------------------------
// GEMM -> reduce-scatter
// ------------------------------------------------------------------------------------------------
struct RsParams {
  hg_lp_t* stage[kMaxRanks];  // stage[d]: rank d's staging area [t][tiles_per_slab][128 x 256 bf16]; we write block `me`
  int* flags[kMaxRanks];            // flags[d]: rank d's tile flags [t][tiles_per_slab]; we write row `me`
  const hg_lp_t* my_stage;
  int* my_flags;
  hg_lp_t* out;               // [slab_rows, N] reduced result (local)
  int ldo;
  int t, me, epoch;
  int slab_rows;
  int tiles_per_slab;               // (slab_rows / 128) * tiles_n: staging granularity is one CTA's 128 x 256 block
};

__device__ __forceinline__ void rs_epilogue2(const Params& p, const RsParams& rs, const Smem2& s, uint32_t tmem_base,
                                             uint32_t rank, int first, int step, int num_tiles) {
  const int wq = (threadIdx.x >> 5) & 3;
  const uint32_t lane_off = uint32_t(wq * 32) << 16;
  const int etid = threadIdx.x - 64;  // 0..127
  uint32_t acc = 0, acc_phase = 0;
  volatile int* epi_go = s.abort + 2;  // written by epilogue thread 0 between barriers: a uniform verdict
  bool alive = true;
  for (int tile = first; tile < num_tiles; tile += step) {
    int tm, tn;
    tile_coords(p, tile, tm, tn);
    const int m0 = tm * CM + int(rank) * BM;           // this CTA's 128 rows of the pair's tile
    const int d = m0 / rs.slab_rows;                   // owner of those rows
    const int mblk = (m0 - d * rs.slab_rows) / BM;
    if (alive && !mbar_wait_warp(&s.tmem_full[acc], acc_phase, p.status, kTimeoutTmemFull, s.abort)) {
      *s.abort = 1;
      alive = false;
    }
    if (alive) {
      tc_fence_after();
      // wire layout of a block: [32-column chunk][8-column group][row] x 16 bytes, so that the 32 lanes of a warp
      // (32 consecutive rows) write 512 contiguous bytes per store instruction
      const int tile_in_slab = mblk * p.tiles_n + tn;
      uint4* tile_base = reinterpret_cast<uint4*>(rs.stage[d]) +
                         (size_t(rs.me) * rs.tiles_per_slab + tile_in_slab) * (BM * BN / 8);
      const int row_in_tile = wq * 32 + int(lane_id());
#pragma unroll 1
      for (int c = 0; c < BN / 32; c += 2) {
        uint32_t r0[32], r1[32];
        tmem_ld32(tmem_base + lane_off + acc * BN + c * 32, r0);
        tmem_ld32(tmem_base + lane_off + acc * BN + (c + 1) * 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 u, w;
          u.x = pack_bf16(__uint_as_float(r0[g * 8 + 0]), __uint_as_float(r0[g * 8 + 1]));
          u.y = pack_bf16(__uint_as_float(r0[g * 8 + 2]), __uint_as_float(r0[g * 8 + 3]));
          u.z = pack_bf16(__uint_as_float(r0[g * 8 + 4]), __uint_as_float(r0[g * 8 + 5]));
          u.w = pack_bf16(__uint_as_float(r0[g * 8 + 6]), __uint_as_float(r0[g * 8 + 7]));
          w.x = pack_bf16(__uint_as_float(r1[g * 8 + 0]), __uint_as_float(r1[g * 8 + 1]));
          w.y = pack_bf16(__uint_as_float(r1[g * 8 + 2]), __uint_as_float(r1[g * 8 + 3]));
          w.z = pack_bf16(__uint_as_float(r1[g * 8 + 4]), __uint_as_float(r1[g * 8 + 5]));
          w.w = pack_bf16(__uint_as_float(r1[g * 8 + 6]), __uint_as_float(r1[g * 8 + 7]));
          tile_base[(c * 4 + g) * BM + row_in_tile] = u;
          tile_base[((c + 1) * 4 + g) * BM + row_in_tile] = w;
        }
      }
      tc_fence_before();
      // the accumulator buffer is free again once all 256 epilogue threads of the pair have read it
      if (rank == 0) mbar_arrive(&s.tmem_empty[acc]);
      else mbar_arrive_cluster(map_to_cta(smem_u32(&s.tmem_empty[acc]), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      __threadfence_system();
    }
    // the four epilogue warps agree on going on before the block is published to its owner
    epi_bar();
    if (etid == 0) *epi_go = *s.abort ? 0 : 1;
    epi_bar();
    if (!*epi_go) break;
    if (etid == 0) st_release_sys(rs.flags[d] + rs.me * rs.tiles_per_slab + mblk * p.tiles_n + tn, rs.epoch);
  }
}

// Reduce the t partials of the blocks of our own slab (fp32 accumulation, bf16 result).
__device__ __forceinline__ void rs_reduce2(const Params& p, const RsParams& rs, const Smem2& s) {
  const int etid = threadIdx.x - 64;
  volatile int* epi_go = s.abort + 2;
  for (int tile = blockIdx.x; tile < rs.tiles_per_slab; tile += gridDim.x) {
    const int mblk = tile / p.tiles_n, tn = tile - mblk * p.tiles_n;
    if (etid < rs.t && !wait_flag_sys(rs.my_flags + etid * rs.tiles_per_slab + tile, rs.epoch, p.status, s.abort))
      *s.abort = 1;
    epi_bar();
    if (etid == 0) *epi_go = *s.abort ? 0 : 1;
    epi_bar();
    if (!*epi_go) return;
    const int n0 = tn * BN;
    const int groups = min(BN, p.N - n0) >> 3;          // valid 8-column groups of this block
    constexpr int kV = 4;                               // vectors per thread per step: t * kV loads in flight
    const size_t tile_vecs = BM * BN / 8;
    const uint4* my = reinterpret_cast<const uint4*>(rs.my_stage);
    for (int v0 = etid; v0 < groups * BM; v0 += 128 * kV) {
      uint4 part[kMaxRanks][kV];
#pragma unroll
      for (int src = 0; src < kMaxRanks; ++src)
        if (src < rs.t) {
          const uint4* base = my + (size_t(src) * rs.tiles_per_slab + tile) * tile_vecs;
#pragma unroll
          for (int u = 0; u < kV; ++u)
            if (v0 + u * 128 < groups * BM) part[src][u] = base[v0 + u * 128];
        }
#pragma unroll
      for (int u = 0; u < kV; ++u) {
        const int v = v0 + u * 128;
        if (v >= groups * BM) continue;
        float accv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) accv[i] = 0.f;
#pragma unroll
        for (int src = 0; src < kMaxRanks; ++src)
          if (src < rs.t) {
            const hg_lp2_t* h = reinterpret_cast<const hg_lp2_t*>(&part[src][u]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = hg_lp22ff(h[i]);
              accv[2 * i] += f.x;
              accv[2 * i + 1] += f.y;
            }
          }
        uint4 o;
        o.x = pack_bf16(accv[0], accv[1]);
        o.y = pack_bf16(accv[2], accv[3]);
        o.z = pack_bf16(accv[4], accv[5]);
        o.w = pack_bf16(accv[6], accv[7]);
        const int grp = v / BM, r = v - grp * BM;       // staging index = group * 128 + row
        *reinterpret_cast<uint4*>(rs.out + size_t(mblk * BM + r) * rs.ldo + n0 + grp * 8) = o;
      }
    }
  }
}

template <bool B_MN>
__global__ void __launch_bounds__(kThreads2, 1)
gemm_rs2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p,
                const RsParams rs) {
  extern __shared__ uint8_t smem_raw[];
  Smem2 s = carve2(smem_raw);
  const int warp = threadIdx.x >> 5;
  const uint32_t rank = cluster_ctarank();
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  pair_prologue(&tmA, &tmB, s, warp);
  const uint32_t tmem_base = *s.tmem_base;

  if (warp == 0) {
    producer2<false, B_MN>(&tmA, &tmB, p, s, rank, pair, pairs, num_tiles);
  } else if (warp == 1) {
    if (rank == 0) mma2<false, B_MN>(p, s, tmem_base, pair, pairs, num_tiles);
  } else if (warp < 6) {
    rs_epilogue2(p, rs, s, tmem_base, rank, pair, pairs, num_tiles);
    if (!*s.abort) rs_reduce2(p, rs, s);
  }
  pair_epilogue_sync(tmem_base, warp);
}

}  // namespace fused2
}  // namespace hg

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
using namespace hg::gemm;
using namespace hg::gemm2;
using namespace hg::fused2;

namespace {

// Launch `k` as clusters of two CTAs, at most `want_pairs` of them and never more than can be resident together
// (the communication warps of every CTA and the flags they publish are part of every tile's dependency chain).
template <typename K, typename X>
int launch_pairs(K k, int& max_pairs, const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, const X& x,
                 int want_pairs, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kThreads2, 1, 1);
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
  return int(cudaLaunchKernelEx(&cfg, k, ta, tb, p, x));
}

}  // namespace

extern "C" {

// CTA-pair form of hg_ag_gemm_bf16 (fused_tp.cu): same arguments and workspace, slab_rows a multiple of 256.
// Returns -2 when the device cannot co-schedule a pair of these CTAs.
int hg_ag_gemm2_bf16(const void* const* src_ptrs, void* const* signal_ptrs, void* gathered, void* block_ready,
                     const void* B, void* C, const void* bias, int t, int me, int epoch, int slab_rows, int N, int K,
                     int ldb, int ldc, int b_mn, int out_mode, void* stream) {
  if (t < 1 || t > kMaxRanks || slab_rows % CM || (K & 7) || (ldb & 7)) return -1;
  const int M = t * slab_rows;
  CUtensorMap ta, tb;
  int rc = hg_host::make_tmap_2d_bf16(&ta, gathered, M, K, K, BM, 64);
  if (rc) return rc;
  rc = b_mn ? hg_host::make_tmap_2d_bf16(&tb, B, K, N, ldb, 64, 64) : hg_host::make_tmap_2d_bf16(&tb, B, N, K, ldb, HALF_N, 64);
  if (rc) return rc;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.C = C; p.bias = reinterpret_cast<const hg_lp_t*>(bias);
  p.out_mode = out_mode; p.tiles_m = M / CM; p.tiles_n = (N + BN - 1) / BN; p.group_m = 4;
  p.status = hg_host::status_ptr();
  p.ready = reinterpret_cast<const int*>(block_ready); p.rows_per_flag = BM; p.ready_target = BM / kSubRows;
  p.m_tile_shift = me * (slab_rows / CM);               // the slab we already own first
  p.k_ranges = nullptr; p.groups = 1; p.c_group_stride = 0;
  AgParams ag{};
  for (int i = 0; i < t; ++i) {
    ag.src[i] = reinterpret_cast<const uint4*>(src_ptrs[i]);
    ag.signal[i] = reinterpret_cast<int*>(signal_ptrs[i]);
  }
  ag.my_signal = ag.signal[me];
  ag.gathered = reinterpret_cast<uint4*>(gathered);
  ag.block_ready = reinterpret_cast<int*>(block_ready);
  ag.t = t; ag.me = me; ag.epoch = epoch; ag.slab_rows = slab_rows; ag.row_vec = K * 2 / 16;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  static int max_pairs[2] = {-1, -1};
  const int pairs = p.tiles_m * p.tiles_n;
  if (b_mn) return launch_pairs(ag_gemm2_kernel<true>, max_pairs[1], ta, tb, p, ag, pairs, st);
  return launch_pairs(ag_gemm2_kernel<false>, max_pairs[0], ta, tb, p, ag, pairs, st);
}

// CTA-pair form of hg_gemm_rs_bf16 (fused_tp.cu): same arguments and workspace, slab_rows a multiple of 256.
int hg_gemm_rs2_bf16(const void* A, const void* B, void* out, void* const* stage_ptrs, void* const* flag_ptrs, int t,
                     int me, int epoch, int slab_rows, int N, int K, int lda, int ldb, int ldo, int b_mn, void* stream) {
  if (t < 1 || t > kMaxRanks || slab_rows % CM || (lda & 7) || (ldb & 7) || (N & 7)) return -1;
  const int M = t * slab_rows;
  CUtensorMap ta, tb;
  int rc = hg_host::make_tmap_2d_bf16(&ta, A, M, K, lda, BM, 64);
  if (rc) return rc;
  rc = b_mn ? hg_host::make_tmap_2d_bf16(&tb, B, K, N, ldb, 64, 64) : hg_host::make_tmap_2d_bf16(&tb, B, N, K, ldb, HALF_N, 64);
  if (rc) return rc;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.ldc = N; p.C = nullptr; p.bias = nullptr; p.out_mode = kOutBf16;
  p.tiles_m = M / CM; p.tiles_n = (N + BN - 1) / BN; p.group_m = 4; p.status = hg_host::status_ptr();
  p.ready = nullptr; p.rows_per_flag = 1; p.ready_target = 0;
  p.m_tile_shift = ((me + 1) % t) * (slab_rows / CM);   // peers' slabs first, our own last
  p.k_ranges = nullptr; p.groups = 1; p.c_group_stride = 0;
  RsParams rs{};
  for (int i = 0; i < t; ++i) {
    rs.stage[i] = reinterpret_cast<hg_lp_t*>(stage_ptrs[i]);
    rs.flags[i] = reinterpret_cast<int*>(flag_ptrs[i]);
  }
  rs.my_stage = rs.stage[me]; rs.my_flags = rs.flags[me];
  rs.out = reinterpret_cast<hg_lp_t*>(out); rs.ldo = ldo;
  rs.t = t; rs.me = me; rs.epoch = epoch; rs.slab_rows = slab_rows;
  rs.tiles_per_slab = (slab_rows / BM) * p.tiles_n;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  static int max_pairs[2] = {-1, -1};
  const int pairs = p.tiles_m * p.tiles_n;
  if (b_mn) return launch_pairs(gemm_rs2_kernel<true>, max_pairs[1], ta, tb, p, rs, pairs, st);
  return launch_pairs(gemm_rs2_kernel<false>, max_pairs[0], ta, tb, p, rs, pairs, st);
}

}  // extern "C"
