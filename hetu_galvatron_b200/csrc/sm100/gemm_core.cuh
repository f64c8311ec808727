// Persistent, warp-specialised bf16 GEMM for sm_100a built on tcgen05.mma with the
// fp32 accumulator in tensor memory and TMA-fed, 128B-swizzled operand tiles.
//
//   C[M,N] (+)= op(A) * op(B)^T-style contraction over K, fp32 accumulate.
//
// CTA tile 128 x 256 x 64, one CTA per SM, grid = min(#tiles, #SMs).
//   warp 0      : TMA producer (one lane), 4-stage ring of {A 16 KB, B 32 KB}
//   warp 1      : TMEM allocator + UMMA issuer (one lane), 128x256x16 instructions,
//                 two 256-column accumulators so the epilogue of tile i overlaps
//                 the main loop of tile i+1
//   warps 2..5  : epilogue; warp w owns TMEM lanes 32*(w%4).. and converts / stores
//                 its 32 rows
//   warps 6..7  : (fused variants only) communication warps
//
// Operand majorness is a template parameter so that forward (A K-major, B K-major),
// dgrad (A K-major, B N-major) and wgrad (A M-major, B N-major) all read the
// tensors as PyTorch stores them, without a transpose pass.
//
// This replaces the library GEMM call sites of the reference's tensor-parallel
// linear layers (galvatron/core/runtime/tensor_parallel/layers.py:300,342,414).
#pragma once
#include "sm100_common.cuh"

namespace hg {
namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int SLAB_BYTES = 64 * BK * 2;     // one 64x64 MN-major box, 8 KB
constexpr int TMEM_COLS = 512;
constexpr int EPI_WARPS = 4;
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 1024 /*align*/ + 256 /*barriers*/;

enum OutMode : int {
  kOutBf16 = 0,      // C = acc (bf16)
  kOutF32 = 1,       // C = acc (fp32)
  kOutF32Acc = 2,    // C += acc (fp32)   (weight-gradient accumulation)
  kOutBf16Acc = 3,   // C = C + acc (bf16)
};

struct Params {
  int M, N, K;
  int ldc;
  void* C;
  const hg_lp_t* bias;  // optional, per output column
  int out_mode;
  int tiles_m, tiles_n;
  int group_m;                // tile-order swizzle: rows of tiles walked together for L2 reuse
  int* status;
  // Optional readiness gate on A rows (used by the all-gather fused variant): the producer
  // waits until ready[m0 / rows_per_flag] >= ready_target before loading A rows starting at m0.
  const int* ready;
  int rows_per_flag;
  int ready_target;
  // Optional row rotation: tile-row order starts at `m_tile_shift` (so that every rank begins
  // with the slab it already owns).
  int m_tile_shift;
  // Optional grouped contraction (per-expert weight gradients): tile list = groups x tiles_m x tiles_n;
  // group g contracts over K rows [k_ranges[g], k_ranges[g+1]) and writes C + g * c_group_stride.
  const int* k_ranges;
  int groups;
  long long c_group_stride;
  // Optional split of the last, partly filled wave (CTA-pair kernel only): tiles from `split_tail_begin` on are each
  // computed by `split_s` pairs, every pair taking a contiguous share of the k-blocks.  Slices 1.. leave their fp32
  // partial tile in `split_ws` (256 x 256 floats per (tail tile, slice - 1)) and count their eight epilogue warps into
  // `split_flags[tail tile * split_s + slice]`; slice 0 waits for them (bounded) and adds the partials in slice order,
  // so the result does not depend on timing.  split_s < 2: off.
  int split_s;
  int split_tail_begin;
  float* split_ws;
  int* split_flags;
};

struct TileInfo {
  int m0, n0, k_start, num_kb;
  long long c_off;
};

__device__ __forceinline__ void tile_coords(const Params& p, int tile, int& tm, int& tn);

__device__ __forceinline__ TileInfo tile_info(const Params& p, int tile) {
  TileInfo t;
  int tm, tn;
  if (p.k_ranges == nullptr) {
    tile_coords(p, tile, tm, tn);
    t.k_start = 0;
    t.num_kb = (p.K + BK - 1) / BK;
    t.c_off = 0;
  } else {
    const int per = p.tiles_m * p.tiles_n;
    const int g = tile / per;
    tile_coords(p, tile - g * per, tm, tn);
    t.k_start = p.k_ranges[g];
    t.num_kb = (p.k_ranges[g + 1] - t.k_start + BK - 1) / BK;
    t.c_off = (long long)g * p.c_group_stride;
  }
  t.m0 = tm * BM;
  t.n0 = tn * BN;
  return t;
}

__device__ __forceinline__ void tile_coords(const Params& p, int tile, int& tm, int& tn) {
  const int per_group = p.group_m * p.tiles_n;
  const int g = tile / per_group;
  const int first_m = g * p.group_m;
  const int gsize = min(p.tiles_m - first_m, p.group_m);
  const int r = tile - g * per_group;
  tm = first_m + (r % gsize);
  tn = r / gsize;
  if (p.m_tile_shift) tm = (tm + p.m_tile_shift) % p.tiles_m;
}

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct SmemLayout {
  uint8_t* a;
  uint8_t* b;
  uint64_t* full;
  uint64_t* empty;
  uint64_t* tmem_full;
  uint64_t* tmem_empty;
  uint32_t* tmem_base;
  volatile int* abort;
};

__device__ __forceinline__ SmemLayout carve(uint8_t* raw) {
  SmemLayout s;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  s.a = base;
  s.b = base + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES));
  s.full = bars;
  s.empty = bars + STAGES;
  s.tmem_full = bars + 2 * STAGES;
  s.tmem_empty = bars + 2 * STAGES + 2;
  s.tmem_base = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  s.abort = reinterpret_cast<volatile int*>(s.tmem_base + 1);
  return s;
}

// ---- producer: the whole warp walks the loop, one elected lane issues the copies ------------------------
// (same reason as for the MMA issuer below: a lane that branched away from its warp pays on the order of a
// hundred cycles per TMA instruction, which made the M/N-major layouts, with their four loads per stage,
// producer-bound)
template <bool A_MN, bool B_MN>
__device__ __forceinline__ void producer_loop(const CUtensorMap* tmA, const CUtensorMap* tmB, const Params& p,
                                              const SmemLayout& s, int first_tile, int tile_step, int num_tiles) {
  uint32_t stage = 0, phase = 0;
  uint32_t issued_parity[STAGES];
  bool issued[STAGES];
#pragma unroll
  for (int i = 0; i < STAGES; ++i) { issued[i] = false; issued_parity[i] = 0; }
  bool ok = true;
  const bool issuer = elect_one() != 0;
  for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
    const TileInfo ti = tile_info(p, tile);
    const int m0 = ti.m0, n0 = ti.n0, num_kb = ti.num_kb;
    if (p.ready != nullptr && num_kb > 0) {
      // all rows of this tile must have landed: check the flags of its first and last row
      const int f0 = m0 / p.rows_per_flag;
      const int f1 = (min(m0 + BM, p.M) - 1) / p.rows_per_flag;
      int landed = 1;
      if (lane_id() == 0) {  // one lane polls; the verdict is made warp-uniform below
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
      // the rows were written with ordinary stores (generic proxy); TMA reads through the async proxy
      asm volatile("fence.proxy.async.global;" ::: "memory");
    }
    for (int kb = 0; kb < num_kb; ++kb) {
      if (!mbar_wait_warp(&s.empty[stage], phase ^ 1, p.status, kTimeoutSmemEmpty, s.abort)) { ok = false; break; }
      uint8_t* sa = s.a + stage * A_STAGE_BYTES;
      uint8_t* sb = s.b + stage * B_STAGE_BYTES;
      const int k0 = ti.k_start + kb * BK;
      if (issuer) {
        mbar_expect_tx(&s.full[stage], A_STAGE_BYTES + B_STAGE_BYTES);
        if (A_MN) {
#pragma unroll
          for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * SLAB_BYTES, tmA, &s.full[stage], m0 + j * 64, k0);
        } else {
          tma_load_2d(sa, tmA, &s.full[stage], k0, m0);
        }
        if (B_MN) {
#pragma unroll
          for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * SLAB_BYTES, tmB, &s.full[stage], n0 + j * 64, k0);
        } else {
          tma_load_2d(sb, tmB, &s.full[stage], k0, n0);
        }
      }
      __syncwarp();
      issued[stage] = true;
      issued_parity[stage] = phase;
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
  }
  if (!ok) {
    *s.abort = 1;
    // let our own bulk copies land before the CTA's shared memory is released
#pragma unroll
    for (int i = 0; i < STAGES; ++i)
      if (issued[i]) {
        for (uint32_t spin = 0; spin < (1u << 16); ++spin)
          if (mbar_try_wait(&s.full[i], issued_parity[i])) break;
      }
  }
}

// ---- UMMA issuer: the whole warp walks the loop, one elected lane issues --------------------------------
// Every lane executes the waits and the stage arithmetic, so addresses and descriptors stay warp-uniform, and only
// the tcgen05.mma / tcgen05.commit instructions are predicated on the elected lane.  Issuing from a lane that had
// branched away from its warp cost about 115 cycles of that lane per MMA (measured: the tensor pipe idled at
// 76 % busy with no memory traffic at all); issued this way the same loop keeps the pipe above 97 % busy.
template <bool A_MN, bool B_MN>
__device__ __forceinline__ void mma_loop(const Params& p, const SmemLayout& s, uint32_t tmem_base, int first_tile,
                                         int tile_step, int num_tiles) {
  constexpr uint32_t idesc = make_idesc_lp(BM, BN, A_MN, B_MN);
  // K-major: 8-row groups 1024 B apart, K advance 32 B.  MN-major: 64-wide slabs SLAB_BYTES apart (LBO),
  // 8-row K groups 1024 B apart (SBO), K advance 16 rows * 128 B.
  constexpr uint32_t a_lbo = A_MN ? SLAB_BYTES : 16, a_sbo = 1024, a_kadv = A_MN ? 2048 : 32;
  constexpr uint32_t b_lbo = B_MN ? SLAB_BYTES : 16, b_sbo = 1024, b_kadv = B_MN ? 2048 : 32;
  uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
  bool ok = true;
  const bool issuer = elect_one() != 0;
  for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
    const int num_kb = tile_info(p, tile).num_kb;
    if (num_kb == 0) continue;  // empty group: nothing to contract, the epilogue handles the output
    if (!mbar_wait_warp(&s.tmem_empty[acc], acc_phase ^ 1, p.status, kTimeoutTmemEmpty, s.abort)) { ok = false; break; }
    tc_fence_after();
    const uint32_t d = tmem_base + acc * BN;
    for (int kb = 0; kb < num_kb; ++kb) {
      if (!mbar_wait_warp(&s.full[stage], phase, p.status, kTimeoutSmemFull, s.abort)) { ok = false; break; }
      tc_fence_after();
      const uint32_t sa = smem_u32(s.a + stage * A_STAGE_BYTES);
      const uint32_t sb = smem_u32(s.b + stage * B_STAGE_BYTES);
      if (issuer) {
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint64_t da = make_smem_desc(sa + k * a_kadv, a_lbo, a_sbo);
          const uint64_t db = make_smem_desc(sb + k * b_kadv, b_lbo, b_sbo);
          umma_f16_ss(d, da, db, idesc, (kb | k) != 0);
        }
        umma_commit(&s.empty[stage]);
      }
      __syncwarp();
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
    if (!ok) break;
    if (issuer) umma_commit(&s.tmem_full[acc]);
    __syncwarp();
    if (++acc == 2) { acc = 0; acc_phase ^= 1; }
  }
  if (!ok) *s.abort = 1;
}

// ---- epilogue: 4 warps, thread == accumulator row ------------------------------------------------
__device__ __forceinline__ void store_row_chunk(const Params& p, int row, int col0, const uint32_t (&r)[32],
                                                long long c_off = 0) {
  // 32 consecutive output columns of one row
  if (!HG_BOUNDS_OK(row >= 0 && row < p.M && col0 >= 0 && col0 < p.N && c_off >= 0, p.status)) return;
  const bool full = (col0 + 32 <= p.N);
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
  if (p.bias != nullptr) {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (full || col0 + i < p.N) v[i] += hg_lp2f(p.bias[col0 + i]);
  }
  const size_t off = size_t(c_off) + size_t(row) * p.ldc + col0;
  if (p.out_mode == kOutBf16 || p.out_mode == kOutBf16Acc) {
    hg_lp_t* c = reinterpret_cast<hg_lp_t*>(p.C) + off;
    const bool vec = full && ((reinterpret_cast<uintptr_t>(c) & 15) == 0);
    if (vec) {
      uint4* c4 = reinterpret_cast<uint4*>(c);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (p.out_mode == kOutBf16Acc) {
          uint4 old = c4[q];
          const hg_lp2_t* o2 = reinterpret_cast<const hg_lp2_t*>(&old);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = hg_lp22ff(o2[j]);
            v[q * 8 + 2 * j] += f.x;
            v[q * 8 + 2 * j + 1] += f.y;
          }
        }
        uint4 o;
        o.x = pack_bf16(v[q * 8 + 0], v[q * 8 + 1]);
        o.y = pack_bf16(v[q * 8 + 2], v[q * 8 + 3]);
        o.z = pack_bf16(v[q * 8 + 4], v[q * 8 + 5]);
        o.w = pack_bf16(v[q * 8 + 6], v[q * 8 + 7]);
        c4[q] = o;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) {
          float x = v[i];
          if (p.out_mode == kOutBf16Acc) x += hg_lp2f(c[i]);
          c[i] = hg_f2lp(x);
        }
    }
  } else {
    float* c = reinterpret_cast<float*>(p.C) + off;
    const bool vec = full && ((reinterpret_cast<uintptr_t>(c) & 15) == 0);
    if (vec) {
      float4* c4 = reinterpret_cast<float4*>(c);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
        if (p.out_mode == kOutF32Acc) {
          float4 old = c4[q];
          o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        c4[q] = o;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) c[i] = (p.out_mode == kOutF32Acc) ? c[i] + v[i] : v[i];
    }
  }
}

__device__ __forceinline__ void epilogue_loop(const Params& p, const SmemLayout& s, uint32_t tmem_base, int first_tile,
                                              int tile_step, int num_tiles) {
  const int wq = (threadIdx.x >> 5) & 3;  // TMEM lane quarter this warp may read
  const uint32_t lane_off = uint32_t(wq * 32) << 16;
  uint32_t acc = 0, acc_phase = 0;
  for (int tile = first_tile; tile < num_tiles; tile += tile_step) {
    const TileInfo ti = tile_info(p, tile);
    const int row = ti.m0 + wq * 32 + lane_id();
    const int n0 = ti.n0;
    if (ti.num_kb == 0) {
      // empty contraction: the result is zero (or unchanged for the accumulating modes)
      if (p.out_mode == kOutBf16 || p.out_mode == kOutF32) {
        uint32_t z[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) z[i] = 0u;
        if (row < p.M)
          for (int c = 0; c < BN / 32; ++c)
            if (n0 + c * 32 < p.N) store_row_chunk(p, row, n0 + c * 32, z, ti.c_off);
      }
      continue;
    }
    if (!mbar_wait_warp(&s.tmem_full[acc], acc_phase, p.status, kTimeoutTmemFull, s.abort)) {
      *s.abort = 1;
      break;
    }
    tc_fence_after();
#pragma unroll 1
    for (int c = 0; c < BN / 32; c += 2) {
      uint32_t r0[32], r1[32];
      tmem_ld32(tmem_base + lane_off + acc * BN + c * 32, r0);
      tmem_ld32(tmem_base + lane_off + acc * BN + (c + 1) * 32, r1);
      tmem_ld_wait();
      if (row < p.M) {
        if (n0 + c * 32 < p.N) store_row_chunk(p, row, n0 + c * 32, r0, ti.c_off);
        if (n0 + (c + 1) * 32 < p.N) store_row_chunk(p, row, n0 + (c + 1) * 32, r1, ti.c_off);
      }
    }
    tc_fence_before();
    mbar_arrive(&s.tmem_empty[acc]);
    if (++acc == 2) { acc = 0; acc_phase ^= 1; }
  }
}

__device__ __forceinline__ void init_barriers(const SmemLayout& s) {
#pragma unroll
  for (int i = 0; i < STAGES; ++i) {
    mbar_init(&s.full[i], 1);
    mbar_init(&s.empty[i], 1);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    mbar_init(&s.tmem_full[i], 1);
    mbar_init(&s.tmem_empty[i], EPI_WARPS * 32);
  }
  *s.abort = 0;
  mbar_fence_init();
}

}  // namespace gemm
}  // namespace hg
