// Device-side building blocks of the CTA-pair (tcgen05.mma.cta_group::2) bf16 GEMM: shared-memory layout, pair
// primitives, TMA producer, UMMA issuer and the row-coalescing epilogue.  Used by gemm2.cu (plain GEMM) and
// fused_tp2.cu (all-gather -> GEMM and GEMM -> reduce-scatter over peer memory on the same tile).
#pragma once
#include "gemm_core.cuh"

namespace hg {
namespace gemm2 {

using namespace hg::gemm;

constexpr int CM = 256;                       // rows of the pair's tile
constexpr int HALF_N = BN / 2;                // B rows staged by one CTA
constexpr int STAGES2 = 6;
constexpr int A2_BYTES = BM * BK * 2;         // 16 KB
constexpr int B2_BYTES = HALF_N * BK * 2;     // 16 KB
constexpr int EPI_STAGE_FLOATS = 32 * 33;     // one 32 x 32 fp32 block per epilogue warp, rows padded to 33 words
constexpr int SMEM2_BYTES = STAGES2 * (A2_BYTES + B2_BYTES) + 1024 + 256 + EPI_WARPS * EPI_STAGE_FLOATS * 4;
constexpr uint16_t kPairMask = 0x3;

struct Smem2 {
  uint8_t* a;
  uint8_t* b;
  uint64_t* full;
  uint64_t* empty;
  uint64_t* tmem_full;
  uint64_t* tmem_empty;
  uint32_t* tmem_base;
  volatile int* abort;
  float* epi_stage;
};

__device__ __forceinline__ Smem2 carve2(uint8_t* raw) {
  Smem2 s;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  s.a = base;
  s.b = base + STAGES2 * A2_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + STAGES2 * (A2_BYTES + B2_BYTES));
  s.full = bars;
  s.empty = bars + STAGES2;
  s.tmem_full = bars + 2 * STAGES2;
  s.tmem_empty = bars + 2 * STAGES2 + 2;
  s.tmem_base = reinterpret_cast<uint32_t*>(bars + 2 * STAGES2 + 4);
  s.abort = reinterpret_cast<volatile int*>(s.tmem_base + 1);
  s.epi_stage = reinterpret_cast<float*>(base + STAGES2 * (A2_BYTES + B2_BYTES) + 256);
  return s;
}

// ---- cluster / pair primitives -------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `local_addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tile load into this CTA's shared memory; the bytes complete on the barrier at `bar_cluster_addr`
// (the leader's).  No multicast: the destination is this CTA only.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int c0,
                                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in every CTA of `mask` once the issued MMAs retired.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(mask)
      : "memory");
}

// ---- work units -------------------------------------------------------------------------------------------------
// Pair `first` of `step` walks tiles first, first + step, ...; with the tail split on, every pair has the same number
// of whole tiles (split_tail_begin / step) and the first (tail tiles x split_s) pairs one slice of a tail tile after them.
struct Unit {
  int tile, kb0, kb1, slice;
};
constexpr int kSplitTileFloats = CM * BN;
__device__ __forceinline__ int unit_count(const Params& p, int first, int step, int num_tiles) {
  if (p.split_s > 1) return p.split_tail_begin / step + (first < (num_tiles - p.split_tail_begin) * p.split_s ? 1 : 0);
  return first < num_tiles ? (num_tiles - first + step - 1) / step : 0;
}
__device__ __forceinline__ Unit unit_at(const Params& p, int first, int step, int u, int num_kb) {
  Unit w;
  if (p.split_s > 1 && u == p.split_tail_begin / step) {
    w.tile = p.split_tail_begin + first / p.split_s;
    w.slice = first % p.split_s;
    w.kb0 = num_kb * w.slice / p.split_s;
    w.kb1 = num_kb * (w.slice + 1) / p.split_s;
  } else {
    w.tile = first + u * step;
    w.slice = 0;
    w.kb0 = 0;
    w.kb1 = num_kb;
  }
  return w;
}

// ---- roles ------------------------------------------------------------------------------------------------------
template <bool A_MN, bool B_MN>
__device__ __forceinline__ void producer2(const CUtensorMap* tmA, const CUtensorMap* tmB, const Params& p, const Smem2& s,
                                          uint32_t rank, int first, int step, int num_tiles) {
  uint32_t stage = 0, phase = 0;
  bool issued[STAGES2];
  uint32_t issued_parity[STAGES2];
#pragma unroll
  for (int i = 0; i < STAGES2; ++i) { issued[i] = false; issued_parity[i] = 0; }
  const int num_kb = (p.K + BK - 1) / BK;
  bool ok = true;
  const bool issuer = elect_one() != 0;   // the warp walks the loop together; only this lane issues the copies
  const int n_units = unit_count(p, first, step, num_tiles);
  for (int u = 0; ok && u < n_units; ++u) {
    const Unit w = unit_at(p, first, step, u, num_kb);
    int tm, tn;
    tile_coords(p, w.tile, tm, tn);
    const int m0 = tm * CM + int(rank) * BM;
    const int n0 = tn * BN + int(rank) * HALF_N;
    if (p.ready != nullptr) {
      // readiness gate on this CTA's 128 A rows (all-gather fused variant): one lane polls, bounded, and the verdict
      // is made warp-uniform; the rows were written with ordinary stores, TMA reads through the async proxy
      const int f0 = m0 / p.rows_per_flag;
      const int f1 = (min(m0 + BM, p.M) - 1) / p.rows_per_flag;
      int landed = 1;
      if (lane_id() == 0) {
        for (int f = f0; landed && f <= f1; ++f) {
          const uint64_t t0 = globaltimer_ns();
          while (ld_acquire_sys(p.ready + f) < p.ready_target) {
            if (*s.abort || globaltimer_ns() - t0 > kWaitLimitNs) {
              set_status(p.status, kTimeoutPeerFlag);
              landed = 0;
              break;
            }
            __nanosleep(64);
          }
        }
      }
      landed = __shfl_sync(0xffffffffu, landed, 0);
      __syncwarp();
      if (!landed) { ok = false; break; }
      asm volatile("fence.proxy.async.global;" ::: "memory");
    }
    for (int kb = w.kb0; kb < w.kb1; ++kb) {
      if (!mbar_wait_warp(&s.empty[stage], phase ^ 1, p.status, kTimeoutSmemEmpty, s.abort)) { ok = false; break; }
      const uint32_t bar = map_to_cta(smem_u32(&s.full[stage]), 0);
      uint8_t* sa = s.a + stage * A2_BYTES;
      uint8_t* sb = s.b + stage * B2_BYTES;
      const int k0 = kb * BK;
      if (issuer) {
        if (rank == 0) mbar_expect_tx(&s.full[stage], 2 * (A2_BYTES + B2_BYTES));
        if (A_MN) {
#pragma unroll
          for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * SLAB_BYTES, tmA, bar, m0 + j * 64, k0);
        } else {
          tma_load_2d_pair(sa, tmA, bar, k0, m0);
        }
        if (B_MN) {
#pragma unroll
          for (int j = 0; j < HALF_N / 64; ++j) tma_load_2d_pair(sb + j * SLAB_BYTES, tmB, bar, n0 + j * 64, k0);
        } else {
          tma_load_2d_pair(sb, tmB, bar, k0, n0);
        }
      }
      __syncwarp();
      issued[stage] = true;
      issued_parity[stage] = phase;
      if (++stage == STAGES2) { stage = 0; phase ^= 1; }
    }
  }
  if (!ok) {
    *s.abort = 1;
    if (rank == 0) {
      // the leader can see its own copies land; give them a bounded moment before shared memory is released
#pragma unroll
      for (int i = 0; i < STAGES2; ++i)
        if (issued[i])
          for (uint32_t spin = 0; spin < (1u << 16); ++spin)
            if (mbar_try_wait(&s.full[i], issued_parity[i])) break;
    } else {
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);  // 2 ms: far longer than a tile load
    }
  }
}

template <bool A_MN, bool B_MN>
__device__ __forceinline__ void mma2(const Params& p, const Smem2& s, uint32_t tmem_base, int first, int step,
                                     int num_tiles) {
  constexpr uint32_t idesc = make_idesc_lp(CM, BN, A_MN, B_MN);
  constexpr uint32_t a_lbo = A_MN ? SLAB_BYTES : 16, a_sbo = 1024, a_kadv = A_MN ? 2048 : 32;
  constexpr uint32_t b_lbo = B_MN ? SLAB_BYTES : 16, b_sbo = 1024, b_kadv = B_MN ? 2048 : 32;
  const int num_kb = (p.K + BK - 1) / BK;
  uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
  bool ok = true;
  const bool issuer = elect_one() != 0;   // the warp walks the loop together; only this lane issues (see gemm_core.cuh)
  const int n_units = unit_count(p, first, step, num_tiles);
  for (int u = 0; ok && u < n_units; ++u) {
    const Unit w = unit_at(p, first, step, u, num_kb);
    if (!mbar_wait_warp(&s.tmem_empty[acc], acc_phase ^ 1, p.status, kTimeoutTmemEmpty, s.abort)) { ok = false; break; }
    tc_fence_after();
    const uint32_t d = tmem_base + acc * BN;
    for (int kb = w.kb0; kb < w.kb1; ++kb) {
      if (!mbar_wait_warp(&s.full[stage], phase, p.status, kTimeoutSmemFull, s.abort)) { ok = false; break; }
      tc_fence_after();
      const uint32_t sa = smem_u32(s.a + stage * A2_BYTES);
      const uint32_t sb = smem_u32(s.b + stage * B2_BYTES);
      if (issuer) {
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint64_t da = make_smem_desc(sa + k * a_kadv, a_lbo, a_sbo);
          const uint64_t db = make_smem_desc(sb + k * b_kadv, b_lbo, b_sbo);
          umma_f16_ss_pair(d, da, db, idesc, ((kb - w.kb0) | k) != 0);
        }
        umma_commit_pair(&s.empty[stage], kPairMask);
      }
      __syncwarp();
      if (++stage == STAGES2) { stage = 0; phase ^= 1; }
    }
    if (!ok) break;
    if (issuer) umma_commit_pair(&s.tmem_full[acc], kPairMask);
    __syncwarp();
    if (++acc == 2) { acc = 0; acc_phase ^= 1; }
  }
  if (!ok) *s.abort = 1;
}

// Epilogue: tcgen05.ld hands every thread one accumulator ROW (32 consecutive columns), but a row per thread is the
// wrong shape for global memory: a warp's 16-byte accesses land in 32 different rows and fill only half of every
// 32-byte sector (138 MB of L2 writes for a 67 MB result, and twice that again for the read-modify-write of the
// fp32 accumulate mode).  Each warp therefore turns its 32 x 32 block through shared memory and touches global
// memory one row at a time, 32 lanes on 32 consecutive columns: whole sectors only.
// `part` (optional): the other slices' partial sums of this 32 x 32 block, slice k at part + k * kSplitTileFloats,
// rows 256 floats apart, already offset to this lane's column; they are added in slice order before anything else.
__device__ __forceinline__ void store_block_rows(const Params& p, float* stg, int row0, int col0,
                                                 const float* part = nullptr, int nparts = 0) {
  const int lane = int(lane_id());
  if (part != nullptr) {
    for (int k = 0; k < nparts; ++k) {
      float add[32];
#pragma unroll
      for (int r = 0; r < 32; ++r) add[r] = __ldcg(part + size_t(k) * kSplitTileFloats + r * BN);
#pragma unroll
      for (int r = 0; r < 32; ++r) stg[r * 33 + lane] += add[r];
    }
  }
  const int col = col0 + lane;
  if (!HG_BOUNDS_OK(row0 >= 0 && row0 < p.M && col0 >= 0 && col0 < p.N, p.status)) return;
  if (col >= p.N) return;
  const float bias = p.bias != nullptr ? hg_lp2f(p.bias[col]) : 0.f;
  const int rows = min(32, p.M - row0);
  if (p.out_mode == kOutBf16 || p.out_mode == kOutBf16Acc) {
    hg_lp_t* c = reinterpret_cast<hg_lp_t*>(p.C) + size_t(row0) * p.ldc + col;
    float old[32];
    if (p.out_mode == kOutBf16Acc) {   // all 32 loads in flight before the first use
#pragma unroll
      for (int r = 0; r < 32; ++r) old[r] = r < rows ? hg_lp2f(c[size_t(r) * p.ldc]) : 0.f;
    } else {
#pragma unroll
      for (int r = 0; r < 32; ++r) old[r] = 0.f;
    }
#pragma unroll
    for (int r = 0; r < 32; ++r)
      if (r < rows) c[size_t(r) * p.ldc] = hg_f2lp(stg[r * 33 + lane] + bias + old[r]);
  } else {
    float* c = reinterpret_cast<float*>(p.C) + size_t(row0) * p.ldc + col;
    float old[32];
    if (p.out_mode == kOutF32Acc) {
#pragma unroll
      for (int r = 0; r < 32; ++r) old[r] = r < rows ? c[size_t(r) * p.ldc] : 0.f;
    } else {
#pragma unroll
      for (int r = 0; r < 32; ++r) old[r] = 0.f;
    }
#pragma unroll
    for (int r = 0; r < 32; ++r)
      if (r < rows) c[size_t(r) * p.ldc] = stg[r * 33 + lane] + bias + old[r];
  }
}

__device__ __forceinline__ void epilogue2(const Params& p, const Smem2& s, uint32_t tmem_base, uint32_t rank, int first,
                                          int step, int num_tiles) {
  const int wq = (threadIdx.x >> 5) & 3;
  const int lane = int(lane_id());
  const uint32_t lane_off = uint32_t(wq * 32) << 16;
  float* stg = s.epi_stage + wq * EPI_STAGE_FLOATS;
  uint32_t acc = 0, acc_phase = 0;
  const int num_kb = (p.K + BK - 1) / BK;
  const int n_units = unit_count(p, first, step, num_tiles);
  for (int u = 0; u < n_units; ++u) {
    const Unit w = unit_at(p, first, step, u, num_kb);
    const int tile = w.tile;
    int tm, tn;
    tile_coords(p, tile, tm, tn);
    const int row0 = tm * CM + int(rank) * BM + wq * 32;   // first of this warp's 32 rows
    const int n0 = tn * BN;
    // a tail tile shared with other pairs: where this pair's partial goes, or where the others' are
    const bool shared_tile = p.split_s > 1 && tile >= p.split_tail_begin;
    const int tail_idx = tile - p.split_tail_begin;
    const int in_row = int(rank) * BM + wq * 32;           // this warp's first row inside the 256 x 256 tile
    float* ws_mine = nullptr;
    const float* ws_others = nullptr;
    if (shared_tile) {
      float* ws_tile = p.split_ws + size_t(tail_idx) * (p.split_s - 1) * kSplitTileFloats;
      if (w.slice > 0) ws_mine = ws_tile + size_t(w.slice - 1) * kSplitTileFloats;
      else ws_others = ws_tile;
    }
    if (!mbar_wait_warp(&s.tmem_full[acc], acc_phase, p.status, kTimeoutTmemFull, s.abort)) {
      *s.abort = 1;
      break;
    }
    tc_fence_after();
    if (ws_others != nullptr) {
      // every epilogue warp of the other slices' pairs (8 each) has stored its part: bounded wait, one lane polls
      int landed = 1;
      if (lane == 0) {
        for (int k = 1; landed && k < p.split_s; ++k) {
          const int* flag = p.split_flags + tail_idx * p.split_s + k;
          const uint64_t t0 = globaltimer_ns();
          while (ld_acquire_gpu(flag) < 2 * EPI_WARPS) {
            if (*s.abort || globaltimer_ns() - t0 > kWaitLimitNs) {
              set_status(p.status, kTimeoutPeerFlag);
              landed = 0;
              break;
            }
            __nanosleep(64);
          }
        }
      }
      landed = __shfl_sync(0xffffffffu, landed, 0);
      if (!landed) {
        *s.abort = 1;
        break;
      }
    }
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r0[32];
      tmem_ld32(tmem_base + lane_off + acc * BN + c * 32, r0);
      tmem_ld_wait();
      if (ws_mine != nullptr) {
        // partial tile: row r of this thread's lane = tile row in_row + lane, 32 consecutive floats
        float* dst = ws_mine + size_t(in_row + lane) * BN + c * 32;
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          __stcg(reinterpret_cast<float4*>(dst + i), make_float4(__uint_as_float(r0[i]), __uint_as_float(r0[i + 1]),
                                                                 __uint_as_float(r0[i + 2]), __uint_as_float(r0[i + 3])));
      } else if (row0 < p.M && n0 + c * 32 < p.N) {   // warp-uniform
#pragma unroll
        for (int i = 0; i < 32; ++i) stg[lane * 33 + i] = __uint_as_float(r0[i]);   // bank (lane + i) % 32: no conflicts
        __syncwarp();
        store_block_rows(p, stg, row0, n0 + c * 32,
                         ws_others ? ws_others + size_t(in_row) * BN + c * 32 + lane : nullptr, p.split_s - 1);
        __syncwarp();
      }
    }
    if (ws_mine != nullptr) {
      __threadfence();
      __syncwarp();
      if (lane == 0) atomicAdd(p.split_flags + tail_idx * p.split_s + w.slice, 1);
    }
    tc_fence_before();
    // the accumulator buffer is free again once all 256 epilogue threads of the pair have read it
    if (rank == 0) mbar_arrive(&s.tmem_empty[acc]);
    else mbar_arrive_cluster(map_to_cta(smem_u32(&s.tmem_empty[acc]), 0));
    if (++acc == 2) { acc = 0; acc_phase ^= 1; }
  }
}


}  // namespace gemm2
}  // namespace hg
