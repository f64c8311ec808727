// Flash attention for sm_100a on tcgen05 / TMEM: forward (O, LSE), and a two-kernel backward
// (dK,dV per key block; dQ per query block) that recomputes the scores.  Causal or full, GQA,
// head dim 64 or 128, arbitrary (s, b, head) strides so that Q/K/V are read straight out of the
// packed QKV projection and O is written in [tokens, heads*hd] layout for the output projection.
//
// Every score-like product runs as  tcgen05.mma (SS, both operands K-major, TMA-loaded),
// accumulators live in TMEM, each softmax thread owns one accumulator row (tcgen05.ld 32x32b),
// probabilities go back to shared memory as the bf16 K-major A operand of the second product,
// whose B operand is the same TMA tile of V / dO / Q / K read through an MN-major descriptor.
//
// Replaces flash_attn_varlen_func / _flash_attn_forward / _flash_attn_backward as called from
// galvatron/core/runtime/transformer/attention_impl.py:55-111,587-616,696-727.
#include <type_traits>

#include "sm100_common.cuh"

namespace hg {
namespace attn {

constexpr int kThreads = 192;  // warp 0: TMA, warp 1: UMMA, warps 2-5: softmax / epilogue
// Backward kernels: two softmax warpgroups (warps 2-5 and 6-9).  Thread == accumulator row in both; warpgroup g owns
// columns [32g, 32g+32) of every 64-column score step, which halves the exp2 / FMA work per thread so that the
// score pipeline keeps up with the tensor core.  (TMEM lanes a warp may touch are 32*(warp%4)..: warps w and w+4
// share a lane quarter.)
constexpr int kBwdThreads = 320;
constexpr int kBwdSoftmaxThreads = 256;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// 2^x on the special-function unit: one instruction, results below 2^-126 flush to zero, 2^-inf = 0.
// (exp2f() wraps the same instruction in range handling that costs several more per element, and the score
// loops below run it tens of thousands of times per step.)
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x on the FMA pipe, for x <= 0 (probabilities): x is split by the add-a-large-constant rounding trick into an
// integer n (left in the low mantissa bits of t) and f in [-0.5, 0.5]; 2^f is a degree-3 near-minimax polynomial
// (maximum relative error 7.5e-5, a fiftieth of the bf16 rounding the result gets next) and n goes straight into
// the exponent field.  Nine FMA / integer instructions against one on the special-function unit, which delivers
// far fewer results per clock: giving a share of the elements to this path takes the exp2 unit off the critical path.
// Inputs below -126 (masked entries, -inf) give exactly 0, as the flushing hardware instruction does.
__device__ __forceinline__ float ex2_poly(float x) {
  const float xc = fmaxf(x, -126.f);
  const float t = xc + 12582912.f;         // 1.5 * 2^23
  const float f = xc - (t - 12582912.f);
  float r = fmaf(f, 0.05517165f, 0.24261113f);
  r = fmaf(r, f, 0.69326097f);
  r = fmaf(r, f, 0.99992806f);
  r = __int_as_float(__float_as_int(r) + (__float_as_int(t) << 23));
  return x < -126.f ? 0.f : r;
}
// Softmax warpgroups of the 128-query dK/dV kernel (2 or 4).
#ifndef HG_DKV_WARPGROUPS
#define HG_DKV_WARPGROUPS 4
#endif
constexpr int kDkvWarpgroups = HG_DKV_WARPGROUPS;
// Softmax warpgroups of the 128-key dQ kernel (2 or 4).
#ifndef HG_DQ_WARPGROUPS
#define HG_DQ_WARPGROUPS 4
#endif
constexpr int kDqWarpgroups = HG_DQ_WARPGROUPS;
// How many of every four exponentials of the two-tile forward kernel take ex2_poly instead of the special-function unit
// (its two softmax warpgroups run at the same time and share that unit).
#ifndef HG_FWD_POLY_OF_4
#define HG_FWD_POLY_OF_4 0
#endif
// How many of every four probabilities of the 128-query dK/dV kernel take ex2_poly instead of the special-function unit.
#ifndef HG_DKV_POLY_OF_4
#define HG_DKV_POLY_OF_4 0
#endif

// Per-role cycle counts of CTA (0, 0, 0), for builds with -DHG_ATTN_TIMING: where a step's time goes (waiting for the
// other role, or working).  Lane 0 of the first softmax warp writes words 16..20 of the device status buffer
// (steps, wait for S^T, probabilities, wait for dP^T, dS^T and stores), lane 0 of the MMA warp words 24..28 (steps, wait
// for free S^T columns, wait for P^T, wait for dS^T, time spent issuing).  The dQ kernel reports in words 40..44 and
// 48..52: softmax (steps, wait for S, loads, arithmetic, dS store), MMA (steps, S + dP issue including
// its waits, wait for dS, dQ issue).  The counts are clock64() differences; nothing is compiled in without
// the define.
#ifdef HG_ATTN_TIMING
#define HG_DKV_TIMERS(a, b, c, d) long long a = 0, b = 0, c = 0, d = 0
#define HG_DKV_TICK(t) long long t = clock64()
#define HG_DKV_TOCK(acc, t)          \
  do {                               \
    const long long now_ = clock64(); \
    acc += now_ - t;                 \
    t = now_;                        \
  } while (0)
#define HG_DKV_REPORT(off, n, a, b, c, d)                                                                   \
  do {                                                                                                      \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane_id() == 0 && (warp == 1 || warp == 2)) { \
      p.status[16 + off] = n;                                                                               \
      p.status[17 + off] = int(a);                                                                          \
      p.status[18 + off] = int(b);                                                                          \
      p.status[19 + off] = int(c);                                                                          \
      p.status[20 + off] = int(d);                                                                          \
    }                                                                                                       \
  } while (0)
#else
#define HG_DKV_TIMERS(a, b, c, d)
#define HG_DKV_TICK(t)
#define HG_DKV_TOCK(acc, t)
#define HG_DKV_REPORT(off, n, a, b, c, d)
#endif

// Head -> slot mapping inside the (possibly packed) tensor:  slot = (h / qpg) * gs + (h % qpg) * hs + off
struct SlotMap {
  int gs, hs, off;
  __device__ __forceinline__ int slot(int h, int qpg) const { return (h / qpg) * gs + (h % qpg) * hs + off; }
};

struct FwdParams {
  int Sq, Skv, B, nheads, qpg;  // qpg = query heads per kv head
  int causal;
  int q_pos0, k_pos0;           // global positions of row 0 / key 0 (ring / context-parallel steps)
  float scale;                  // softmax scale (1/sqrt(hd))
  SlotMap qmap, kmap, vmap;
  hg_lp_t* O;             // element (s, b, h, d) at O + s*o_ss + b*o_sb + h*hd + d
  int64_t o_ss, o_sb;
  float* LSE;                   // [B, nheads, Sq]
  int* status;
};

// K-major operand: `rows` x (64*slabs) bf16 stored as slabs of [rows x 128 B]; descriptor for k-step kk.
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t base, int rows, int kk) {
  return make_smem_desc(base + (kk >> 2) * rows * 128 + (kk & 3) * 32, 16, 1024);
}
// The same buffer viewed as an MN-major operand (MN = the 64*slabs columns, K = rows); k-step kk = rows 16kk..
__device__ __forceinline__ uint64_t mnmajor_desc(uint32_t base, int rows, int kk) {
  return make_smem_desc(base + kk * 2048, rows * 128, 1024);
}

// =================================================================================================
// Forward
// =================================================================================================
template <int HD>
struct FwdSmem {
  static constexpr int kQ = 128 * HD * 2;
  static constexpr int kKV = 128 * HD * 2;
  static constexpr int kP = 128 * 128 * 2;
  static constexpr int kTotal = kQ + 4 * kKV + kP + 1024 + 256;
};

template <int HD>
__global__ void __launch_bounds__(kThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = base;
  uint8_t* sK = sQ + FwdSmem<HD>::kQ;              // 2 stages
  uint8_t* sV = sK + 2 * FwdSmem<HD>::kKV;         // 2 stages
  uint8_t* sP = sV + 2 * FwdSmem<HD>::kKV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + FwdSmem<HD>::kP);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // 2
  uint64_t* s_empty = bars + 11;    // 2
  uint64_t* p_full = bars + 13;     // 1
  uint64_t* o_done = bars + 14;     // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int qb = gridDim.x - 1 - blockIdx.x;  // heavy (late) query blocks first under a causal mask
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = qb * 128;

  // key blocks this query block attends to
  int kv_len = p.Skv;
  if (p.causal) {
    const int last = p.q_pos0 + q0 + 127 - p.k_pos0;  // last visible key index for the last row
    kv_len = min(p.Skv, last + 1);
  }
  const int n_kv = kv_len > 0 ? (kv_len + 127) / 128 : 0;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);     // one arrival per softmax warp (mbar_arrive_warp)
    }
    mbar_init(p_full, 4);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS[2] = {tmem, tmem + 128};
  const uint32_t tO = tmem + 256;

  const int qslot = p.qmap.slot(h, p.qpg), kslot = p.kmap.slot(h, p.qpg), vslot = p.vmap.slot(h, p.qpg);

  if (warp == 0) {
    if (n_kv > 0) {
      // the whole warp walks the loop, one elected lane issues the copies (see producer_loop in gemm_core.cuh)
      const bool issuer = elect_one() != 0;
      if (issuer) mbar_expect_tx(q_full, FwdSmem<HD>::kQ);
#pragma unroll
      for (int j = 0; j < HD / 64; ++j) if (issuer) tma_load_4d(sQ + j * 128 * 128, &tmQ, q_full, j * 64, qslot, q0, b);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait_warp(&k_empty[st], ph ^ 1, p.status, kTimeoutSmemEmpty, abort_flag)) { *abort_flag = 1; break; }
        if (issuer) mbar_expect_tx(&k_full[st], FwdSmem<HD>::kKV);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          if (issuer) tma_load_4d(sK + st * FwdSmem<HD>::kKV + c * 128 * 128, &tmK, &k_full[st], c * 64, kslot, j * 128, b);
        if (!mbar_wait_warp(&v_empty[st], ph ^ 1, p.status, kTimeoutSmemEmpty, abort_flag)) { *abort_flag = 1; break; }
        if (issuer) mbar_expect_tx(&v_full[st], FwdSmem<HD>::kKV);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          if (issuer) tma_load_4d(sV + st * FwdSmem<HD>::kKV + c * 128 * 128, &tmV, &v_full[st], c * 64, vslot, j * 128, b);
      }
    }
  } else if (warp == 1) {
    if (n_kv > 0) {
      // the whole warp walks the loop, one elected lane issues (see mma_loop in gemm_core.cuh)
      const bool issuer = elect_one() != 0;
      constexpr uint32_t idesc_s = make_idesc_lp(128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc_lp(128, HD, false, true);
      const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);
      bool ok = mbar_wait_warp(q_full, 0, p.status, kTimeoutSmemFull, abort_flag);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait_warp(&k_full[st], ph, p.status, kTimeoutSmemFull, abort_flag)) return false;
        if (!mbar_wait_warp(&s_empty[st], ph ^ 1, p.status, kTimeoutTmemEmpty, abort_flag)) return false;
        tc_fence_after();
        const uint32_t aK = smem_u32(sK + st * FwdSmem<HD>::kKV);
        if (issuer) {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk)
            umma_f16_ss(tS[st], kmajor_desc(aQ, 128, kk), kmajor_desc(aK, 128, kk), idesc_s, kk != 0);
          umma_commit(&s_full[st]);
          umma_commit(&k_empty[st]);
        }
        __syncwarp();
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; ok && j < n_kv; ++j) {
        if (j + 1 < n_kv) { ok = issue_s(j + 1); if (!ok) break; }
        const int st = j & 1;
        if (!mbar_wait_warp(p_full, j & 1, p.status, kTimeoutOther, abort_flag)) { ok = false; break; }
        if (!mbar_wait_warp(&v_full[st], (j >> 1) & 1, p.status, kTimeoutSmemFull, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t aV = smem_u32(sV + st * FwdSmem<HD>::kKV);
        if (issuer) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_f16_ss(tO, kmajor_desc(aP, 128, kk), mnmajor_desc(aV, 128, kk), idesc_o, (j | kk) != 0);
          umma_commit(&v_empty[st]);
          umma_commit(o_done);
        }
        __syncwarp();
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    // ---- softmax: thread == query row ----
    const int wq = warp & 3;
    const int row = wq * 32 + lane_id();
    const uint32_t lane_off = uint32_t(wq * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    const int q_pos = p.q_pos0 + q0 + row;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int st = j & 1;
      if (!mbar_wait_warp(&s_full[st], (j >> 1) & 1, p.status, kTimeoutTmemFull, abort_flag)) { ok = false; break; }
      tc_fence_after();
      float s[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tS[st] + lane_off + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(r[i]);
      }
      tc_fence_before();
      mbar_arrive_warp(&s_empty[st]);
      // masking (only blocks that cross the diagonal or the ragged end need it)
      const int k_base = p.k_pos0 + j * 128;
      const bool need_mask = (p.causal && (k_base + 127 > p.q_pos0 + q0)) || (j * 128 + 128 > p.Skv);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          const bool dead = (j * 128 + i >= p.Skv) || (p.causal && (k_base + i > q_pos));
          if (dead) s[i] = -INFINITY;
        }
      }
      float mx4[4] = {s[0], s[1], s[2], s[3]};   // four chains: a single one is 127 dependent instructions long
#pragma unroll
      for (int i = 4; i < 128; i += 4) {
        mx4[0] = fmaxf(mx4[0], s[i]); mx4[1] = fmaxf(mx4[1], s[i + 1]);
        mx4[2] = fmaxf(mx4[2], s[i + 2]); mx4[3] = fmaxf(mx4[3], s[i + 3]);
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx *= sl2;
      // lazy rescale: keep the running reference max unless the new max exceeds it by more than 2^8
      float alpha = 1.f;
      bool rescale = false;
      if (mx > m_used + 8.f) {
        alpha = (m_used == -INFINITY) ? 0.f : ex2(m_used - mx);
        m_used = mx;
        rescale = (j > 0);
      }
      const float nmref = (m_used == -INFINITY) ? 0.f : -m_used;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 128; i += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          s[i + u] = ex2(fmaf(s[i + u], sl2, nmref));
          sum4[u] += s[i + u];
        }
      }
      l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      if (j > 0) {
        if (!mbar_wait_warp(o_done, (j - 1) & 1, p.status, kTimeoutOther, abort_flag)) { ok = false; break; }
        tc_fence_after();
      }
      if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tO + lane_off + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(tO + lane_off + c * 32, r);
        }
        tmem_st_wait();
      }
      // P -> shared memory, bf16, 128B-swizzled K-major (two 64-column slabs)
#pragma unroll
      for (int cc = 0; cc < 16; ++cc) {
        uint4 u;
        u.x = pack_bf16(s[cc * 8 + 0], s[cc * 8 + 1]);
        u.y = pack_bf16(s[cc * 8 + 2], s[cc * 8 + 3]);
        u.z = pack_bf16(s[cc * 8 + 4], s[cc * 8 + 5]);
        u.w = pack_bf16(s[cc * 8 + 6], s[cc * 8 + 7]);
        *reinterpret_cast<uint4*>(sP + (cc >> 3) * 128 * 128 + sw128_offset(row, cc & 7)) = u;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive_warp(p_full);
    }
    // ---- epilogue: O / l -> global, LSE ----
    const int srow = q0 + row;
    if (n_kv == 0) {
      if (srow < p.Sq) {
        hg_lp_t* o = p.O + int64_t(srow) * p.o_ss + int64_t(b) * p.o_sb + h * HD;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) reinterpret_cast<uint4*>(o)[i] = make_uint4(0, 0, 0, 0);
        p.LSE[(size_t(b) * p.nheads + h) * p.Sq + srow] = -INFINITY;
      }
    } else if (ok && !*abort_flag && mbar_wait_warp(o_done, (n_kv - 1) & 1, p.status, kTimeoutOther, abort_flag)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tO + lane_off + c * 32, r);
        tmem_ld_wait();
        if (srow < p.Sq) {
          hg_lp_t* o = p.O + int64_t(srow) * p.o_ss + int64_t(b) * p.o_sb + h * HD + c * 32;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack_bf16(__uint_as_float(r[q * 8 + 0]) * inv, __uint_as_float(r[q * 8 + 1]) * inv);
            u.y = pack_bf16(__uint_as_float(r[q * 8 + 2]) * inv, __uint_as_float(r[q * 8 + 3]) * inv);
            u.z = pack_bf16(__uint_as_float(r[q * 8 + 4]) * inv, __uint_as_float(r[q * 8 + 5]) * inv);
            u.w = pack_bf16(__uint_as_float(r[q * 8 + 6]) * inv, __uint_as_float(r[q * 8 + 7]) * inv);
            reinterpret_cast<uint4*>(o)[q] = u;
          }
        }
      }
      if (srow < p.Sq)
        p.LSE[(size_t(b) * p.nheads + h) * p.Sq + srow] = (l > 0.f) ? (m_used + log2f(l)) * kLn2 : -INFINITY;
    } else {
      *abort_flag = 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// =================================================================================================
// Forward with two query tiles per CTA and P in tensor memory (head dim 128).
// In the one-tile kernel a scheduler hosts a single softmax warp, so every latency of its step (the loads from tensor
// memory, the maximum, the exp2 / convert chains) is exposed, and the tensor core idles while the softmax of its only
// tile runs.  Here a CTA owns 256 queries as two tiles of 128, one softmax warpgroup per tile: while one tile's
// threads work on their scores, the tensor core runs the other tile's products, and every scheduler has two softmax
// warps to switch between.  P never goes through shared memory: the threads store it, packed, over the first 64 of
// the 128 S columns they have just read, and the PV product takes its A operand from tensor memory.
//
// Tensor memory (512 columns): S of tile 0 / 1 at 0 / 128, O of tile 0 / 1 at 256 / 384.  Per tile the order is
// S(j) -> softmax(j) -> P(j) -> PV(j) -> S(j+1): S(j+1) overwrites the columns PV(j) reads, and the tensor core
// executes in issue order, so the MMA warp issues PV(t, j) and S(t, j+1) back to back when P(t, j) is stored.
// K and V stages are shared by the two tiles; a stage is released after the last product that reads it.
// =================================================================================================
template <int HD>
struct Fwd2Smem {
  static constexpr int kQ = 128 * HD * 2;     // one query tile
  static constexpr int kKV = 128 * HD * 2;    // one stage of K or V
  static constexpr int kTotal = 2 * kQ + 4 * kKV + 1024 + 256;
};

template <int HD>
__global__ void __launch_bounds__(320, 1)
flash_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  static_assert(HD == 128, "the two-tile forward is written for head dim 128");
  extern __shared__ uint8_t smem_raw[];
  using L = Fwd2Smem<HD>;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = base;                     // 2 tiles
  uint8_t* sK = sQ + 2 * L::kQ;           // 2 stages
  uint8_t* sV = sK + 2 * L::kKV;          // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * L::kKV);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // 2 (per tile)
  uint64_t* p_full = bars + 11;     // 2 (per tile)
  uint64_t* o_done = bars + 13;     // 2 (per tile)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int qb = gridDim.x - 1 - blockIdx.x;  // heavy (late) query blocks first under a causal mask
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = qb * 256;

  // key blocks each tile attends to (tile 1 never fewer than tile 0)
  int n_kv_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    int kv_len = p.Skv;
    if (p.causal) kv_len = min(p.Skv, p.q_pos0 + q0 + t * 128 + 127 - p.k_pos0 + 1);
    n_kv_t[t] = (kv_len > 0 && q0 + t * 128 < p.Sq) ? (kv_len + 127) / 128 : 0;
  }
  const int n_kv = max(n_kv_t[0], n_kv_t[1]);

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);      // one arrival per softmax warp of the tile (mbar_arrive_warp)
      mbar_init(&o_done[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS[2] = {tmem, tmem + 128};
  const uint32_t tO[2] = {tmem + 256, tmem + 384};

  const int qslot = p.qmap.slot(h, p.qpg), kslot = p.kmap.slot(h, p.qpg), vslot = p.vmap.slot(h, p.qpg);

  if (warp == 0) {
    if (n_kv > 0) {
      // the whole warp walks the loop, one elected lane issues the copies (see producer_loop in gemm_core.cuh)
      const bool issuer = elect_one() != 0;
      if (issuer) mbar_expect_tx(q_full, 2 * L::kQ);   // rows past the end of the tensor arrive as zeros
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          if (issuer) tma_load_4d(sQ + t * L::kQ + c * 128 * 128, &tmQ, q_full, c * 64, qslot, q0 + t * 128, b);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait_warp(&k_empty[st], ph ^ 1, p.status, kTimeoutSmemEmpty, abort_flag)) { *abort_flag = 1; break; }
        if (issuer) mbar_expect_tx(&k_full[st], L::kKV);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          if (issuer) tma_load_4d(sK + st * L::kKV + c * 128 * 128, &tmK, &k_full[st], c * 64, kslot, j * 128, b);
        if (!mbar_wait_warp(&v_empty[st], ph ^ 1, p.status, kTimeoutSmemEmpty, abort_flag)) { *abort_flag = 1; break; }
        if (issuer) mbar_expect_tx(&v_full[st], L::kKV);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          if (issuer) tma_load_4d(sV + st * L::kKV + c * 128 * 128, &tmV, &v_full[st], c * 64, vslot, j * 128, b);
      }
    }
  } else if (warp == 1) {
    if (n_kv > 0) {
      // the whole warp walks the loop, one elected lane issues (see mma_loop in gemm_core.cuh)
      const bool issuer = elect_one() != 0;
      constexpr uint32_t idesc_s = make_idesc_lp(128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc_lp(128, HD, false, true);
      bool ok = mbar_wait_warp(q_full, 0, p.status, kTimeoutSmemFull, abort_flag);
      // the last tile (in issue order) that has a step j: it releases the K / V stage of that step
      auto last_user = [&](int j) -> int { return j < n_kv_t[1] ? 1 : 0; };
      auto issue_s = [&](int t, int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait_warp(&k_full[st], (j >> 1) & 1, p.status, kTimeoutSmemFull, abort_flag)) return false;
        tc_fence_after();
        const uint32_t aQ = smem_u32(sQ + t * L::kQ), aK = smem_u32(sK + st * L::kKV);
        if (issuer) {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk)
            umma_f16_ss(tS[t], kmajor_desc(aQ, 128, kk), kmajor_desc(aK, 128, kk), idesc_s, kk != 0);
          umma_commit(&s_full[t]);
          if (t == last_user(j)) umma_commit(&k_empty[st]);
        }
        __syncwarp();
        return true;
      };
#pragma unroll
      for (int t = 0; t < 2; ++t)
        if (ok && n_kv_t[t] > 0) ok = issue_s(t, 0);
      HG_DKV_TIMERS(tm_wait_p0, tm_wait_p1, tm_issue, tm_unused);
      HG_DKV_TICK(t0);
      for (int j = 0; ok && j < n_kv; ++j) {
        const int st = j & 1;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (!ok || j >= n_kv_t[t]) continue;
          if (!mbar_wait_warp(&p_full[t], j & 1, p.status, kTimeoutOther, abort_flag)) { ok = false; break; }
          if (t == 0) { HG_DKV_TOCK(tm_wait_p0, t0); } else { HG_DKV_TOCK(tm_wait_p1, t0); }
          if (!mbar_wait_warp(&v_full[st], (j >> 1) & 1, p.status, kTimeoutSmemFull, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t aV = smem_u32(sV + st * L::kKV);
          if (issuer) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)   // k-step kk = keys 16kk..16kk+15 = 8 packed columns of P
              umma_f16_ts(tO[t], tS[t] + kk * 8, mnmajor_desc(aV, 128, kk), idesc_o, (j | kk) != 0);
            if (t == last_user(j)) umma_commit(&v_empty[st]);
            if (j + 1 >= n_kv_t[t]) umma_commit(&o_done[t]);
          }
          __syncwarp();
          if (j + 1 < n_kv_t[t]) ok = issue_s(t, j + 1);
          HG_DKV_TOCK(tm_issue, t0);
        }
      }
      HG_DKV_REPORT(8, n_kv, tm_wait_p0, tm_wait_p1, tm_issue, tm_unused);
      if (!ok) *abort_flag = 1;
    }
  } else {
    // ---- softmax: one warpgroup per tile, thread == query row ----
    const int t = (warp - 2) >> 2;
    const int wq = warp & 3;
    const int row = wq * 32 + lane_id();
    const uint32_t lane_off = uint32_t(wq * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    const int qt0 = q0 + t * 128;
    const int q_pos = p.q_pos0 + qt0 + row;
    const int my_kv = n_kv_t[t];
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    HG_DKV_TIMERS(tm_wait_s, tm_ld, tm_math, tm_st);
    for (int j = 0; j < my_kv; ++j) {
      HG_DKV_TICK(t0);
      if (!mbar_wait_warp(&s_full[t], j & 1, p.status, kTimeoutTmemFull, abort_flag)) { ok = false; break; }
      tc_fence_after();
      HG_DKV_TOCK(tm_wait_s, t0);
      float s[128];
      {
        uint32_t r[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tS[t] + lane_off + c * 32, r[c]);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(r[c][i]);
      }
      HG_DKV_TOCK(tm_ld, t0);
      // masking (only blocks that cross the diagonal or the ragged end need it)
      const int k_base = p.k_pos0 + j * 128;
      const bool need_mask = (p.causal && (k_base + 127 > p.q_pos0 + qt0)) || (j * 128 + 128 > p.Skv);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          const bool dead = (j * 128 + i >= p.Skv) || (p.causal && (k_base + i > q_pos));
          if (dead) s[i] = -INFINITY;
        }
      }
      float mx4[4] = {s[0], s[1], s[2], s[3]};   // four chains: a single one is 127 dependent instructions long
#pragma unroll
      for (int i = 4; i < 128; i += 4) {
        mx4[0] = fmaxf(mx4[0], s[i]); mx4[1] = fmaxf(mx4[1], s[i + 1]);
        mx4[2] = fmaxf(mx4[2], s[i + 2]); mx4[3] = fmaxf(mx4[3], s[i + 3]);
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx *= sl2;
      // lazy rescale: keep the running reference max unless the new max exceeds it by more than 2^8
      float alpha = 1.f;
      bool rescale = false;
      if (mx > m_used + 8.f) {
        alpha = (m_used == -INFINITY) ? 0.f : ex2(m_used - mx);
        m_used = mx;
        rescale = (j > 0);
      }
      const float nmref = (m_used == -INFINITY) ? 0.f : -m_used;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[64];
#pragma unroll
      for (int i = 0; i < 128; i += 4) {
        float e[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float x = fmaf(s[i + u], sl2, nmref);
          e[u] = (u < HG_FWD_POLY_OF_4) ? ex2_poly(x) : ex2(x);
          sum4[u] += e[u];
        }
        pk[i >> 1] = pack_bf16(e[0], e[1]);
        pk[(i >> 1) + 1] = pack_bf16(e[2], e[3]);
      }
      l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      HG_DKV_TOCK(tm_math, t0);
      // S(t, j) was issued after PV(t, j-1), and the tensor core executes in order: O holds steps 0..j-1 by now
      if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tO[t] + lane_off + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(tO[t] + lane_off + c * 32, r);
        }
      }
      // P, packed, over the first 64 of this row's S columns
      {
        const uint32_t(&lo)[32] = *reinterpret_cast<const uint32_t(*)[32]>(&pk[0]);
        const uint32_t(&hi)[32] = *reinterpret_cast<const uint32_t(*)[32]>(&pk[32]);
        tmem_st32(tS[t] + lane_off, lo);
        tmem_st32(tS[t] + lane_off + 32, hi);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive_warp(&p_full[t]);
      HG_DKV_TOCK(tm_st, t0);
    }
    if (t == 0) { HG_DKV_REPORT(0, my_kv, tm_wait_s, tm_ld, tm_math, tm_st); }
    // ---- epilogue: O / l -> global, LSE ----
    const int srow = qt0 + row;
    if (my_kv == 0) {
      if (srow < p.Sq) {
        hg_lp_t* o = p.O + int64_t(srow) * p.o_ss + int64_t(b) * p.o_sb + h * HD;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) reinterpret_cast<uint4*>(o)[i] = make_uint4(0, 0, 0, 0);
        p.LSE[(size_t(b) * p.nheads + h) * p.Sq + srow] = -INFINITY;
      }
    } else if (ok && !*abort_flag && mbar_wait_warp(&o_done[t], 0, p.status, kTimeoutOther, abort_flag)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tO[t] + lane_off + c * 32, r);
        tmem_ld_wait();
        if (srow < p.Sq) {
          hg_lp_t* o = p.O + int64_t(srow) * p.o_ss + int64_t(b) * p.o_sb + h * HD + c * 32;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack_bf16(__uint_as_float(r[q * 8 + 0]) * inv, __uint_as_float(r[q * 8 + 1]) * inv);
            u.y = pack_bf16(__uint_as_float(r[q * 8 + 2]) * inv, __uint_as_float(r[q * 8 + 3]) * inv);
            u.z = pack_bf16(__uint_as_float(r[q * 8 + 4]) * inv, __uint_as_float(r[q * 8 + 5]) * inv);
            u.w = pack_bf16(__uint_as_float(r[q * 8 + 6]) * inv, __uint_as_float(r[q * 8 + 7]) * inv);
            reinterpret_cast<uint4*>(o)[q] = u;
          }
        }
      }
      if (srow < p.Sq)
        p.LSE[(size_t(b) * p.nheads + h) * p.Sq + srow] = (l > 0.f) ? (m_used + log2f(l)) * kLn2 : -INFINITY;
    } else {
      *abort_flag = 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// =================================================================================================
// Backward, part 0:  D[b,h,s] = sum_d dO * O
// =================================================================================================
__global__ void attn_bwd_dot_kernel(const hg_lp_t* __restrict__ O, const hg_lp_t* __restrict__ dO,
                                    int64_t ss, int64_t sb, int64_t dss, int64_t dsb, int S, int B, int nheads, int hd,
                                    float* __restrict__ D) {
  // one warp per (s, b, h)
  const int64_t total = int64_t(S) * B * nheads;
  const int64_t gw = (blockIdx.x * int64_t(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= total) return;
  const int h = int(gw % nheads);
  const int b = int((gw / nheads) % B);
  const int s = int(gw / (int64_t(nheads) * B));
  const hg_lp_t* o = O + s * ss + b * sb + h * hd;
  const hg_lp_t* d = dO + s * dss + b * dsb + h * hd;
  float acc = 0.f;
  for (int i = lane * 2; i < hd; i += 64) {
    const float2 a = hg_lp22ff(*reinterpret_cast<const hg_lp2_t*>(o + i));
    const float2 c = hg_lp22ff(*reinterpret_cast<const hg_lp2_t*>(d + i));
    acc += a.x * c.x + a.y * c.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) D[(size_t(b) * nheads + h) * S + s] = acc;
}

// =================================================================================================
// Backward parameters (shared by the dK/dV and the dQ kernels)
// =================================================================================================
struct BwdParams {
  int Sq, Skv, B, nheads, qpg;
  int causal;
  int q_pos0, k_pos0;
  float scale;
  SlotMap qmap, kmap, vmap, domap;  // dO uses slot = h (gs = qpg, hs = 1, off = 0)
  const float* LSE;                 // [B, nheads, Sq]
  const float* D;                   // [B, nheads, Sq]
  // outputs: element (s, b, slot, d) at base + s*ss + b*sb + slot*hd + d
  hg_lp_t* dQ; int64_t dq_ss, dq_sb; SlotMap dqmap;
  hg_lp_t* dK; int64_t dk_ss, dk_sb; SlotMap dkmap;
  hg_lp_t* dV; int64_t dv_ss, dv_sb; SlotMap dvmap;
  int* status;
};

// =================================================================================================
// Backward, part 1: one CTA per (key block of 128, kv head, batch); loops over the query heads of the
// group and over 64-row query steps.  Thread == key row.
//   S^T = K Q^T, dP^T = V dO^T  (M = 128 keys, N = 64 queries)
//   P^T = exp2(S^T*c - lse), dS^T = P^T * (dP^T - D)
//   dV += P^T dO, dK += dS^T Q   (A from shared memory written by the threads; B = the dO / Q tile, MN-major)
// =================================================================================================
template <int HD>
struct DkvSmem {
  static constexpr int kKV = 128 * HD * 2;     // resident K or V
  static constexpr int kQD = 64 * HD * 2;      // one stage of Q or dO
  static constexpr int kQDStages = 3;          // a stage is held from its S^T product to its dK product, i.e. for more
                                               // than a step: with two stages every load was waited for in full
  static constexpr int kPT = 128 * 64 * 2;     // one P^T or dS^T buffer (two of each: written for step i+1 while step i is multiplied)
  static constexpr int kStats = 2 * 2 * 64 * 4;  // lse2/D, double buffered
  static constexpr int kTotal = 2 * kKV + 2 * kQDStages * kQD + 4 * kPT + kStats + 1024 + 256;
};

template <int HD>
__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                     const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = base;
  uint8_t* sV = sK + DkvSmem<HD>::kKV;
  constexpr int NQ = DkvSmem<HD>::kQDStages;
  uint8_t* sQ = sV + DkvSmem<HD>::kKV;            // NQ stages
  uint8_t* sDO = sQ + NQ * DkvSmem<HD>::kQD;      // NQ stages
  uint8_t* sPT = sDO + NQ * DkvSmem<HD>::kQD;
  uint8_t* sDST = sPT + 2 * DkvSmem<HD>::kPT;
  float* sStats = reinterpret_cast<float*>(sDST + 2 * DkvSmem<HD>::kPT);  // [2][2][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sStats) + DkvSmem<HD>::kStats);
  uint64_t* kv_full = bars;        // 1
  uint64_t* qd_full = bars + 1;    // 3
  uint64_t* qd_empty = bars + 4;   // 3
  uint64_t* st_full = bars + 7;    // 2
  uint64_t* st_empty = bars + 9;   // 2
  uint64_t* pds_full = bars + 11;  // 2
  uint64_t* pds_empty = bars + 13; // 2
  uint64_t* stats_full = bars + 15; // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int kb = blockIdx.x, g = blockIdx.y, b = blockIdx.z;  // g = kv head
  const int k0 = kb * 128;
  // first query row that can see this key block
  int q_first = 0;
  if (p.causal) q_first = max(0, p.k_pos0 + k0 - p.q_pos0);
  const int qs0 = (q_first / 64);                       // first 64-row query step
  const int n_qs = (p.Sq + 63) / 64;
  const int steps_per_head = max(0, n_qs - qs0);
  const int n_it = steps_per_head * p.qpg;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
    mbar_init(kv_full, 1);
    for (int i = 0; i < NQ; ++i) {
      mbar_init(&qd_full[i], 1);
      mbar_init(&qd_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&st_full[i], 1);
      mbar_init(&st_empty[i], kBwdSoftmaxThreads);
      mbar_init(&pds_full[i], kBwdSoftmaxThreads);
      mbar_init(&pds_empty[i], 1);
    }
    mbar_init(&stats_full[0], kBwdSoftmaxThreads);
    mbar_init(&stats_full[1], kBwdSoftmaxThreads);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // columns: S^T[0] 0..63, dP^T[0] 64..127, S^T[1] 128..191, dP^T[1] 192..255, dV 256.., dK 384..
  const uint32_t tST[2] = {tmem, tmem + 128};
  const uint32_t tDPT[2] = {tmem + 64, tmem + 192};
  const uint32_t tDV = tmem + 256, tDK = tmem + 384;

  const int h0 = g * p.qpg;  // first query head of the group
  const int kslot = p.kmap.slot(h0, p.qpg), vslot = p.vmap.slot(h0, p.qpg);

  if (warp == 0) {
    if (n_it > 0) {
      // the whole warp walks the loop, one elected lane issues the copies (see producer_loop in gemm_core.cuh)
      const bool issuer = elect_one() != 0;
      if (issuer) mbar_expect_tx(kv_full, 2 * DkvSmem<HD>::kKV);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
        if (issuer) tma_load_4d(sK + c * 128 * 128, &tmK, kv_full, c * 64, kslot, k0, b);
        if (issuer) tma_load_4d(sV + c * 128 * 128, &tmV, kv_full, c * 64, vslot, k0, b);
      }
      int st = 0;            // ring slot and its phase, and the (head, query step) of the iteration
      uint32_t ph = 0;
      int h = h0, qs = qs0;
      for (int it = 0; it < n_it; ++it) {
        const int qrow = qs * 64;
        if (!mbar_wait_warp(&qd_empty[st], ph ^ 1, p.status, kTimeoutSmemEmpty, abort_flag)) { *abort_flag = 1; break; }
        if (issuer) mbar_expect_tx(&qd_full[st], 2 * DkvSmem<HD>::kQD);
        const int qslot = p.qmap.slot(h, p.qpg), doslot = p.domap.slot(h, p.qpg);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) {
          if (issuer) tma_load_4d(sQ + st * DkvSmem<HD>::kQD + c * 64 * 128, &tmQ, &qd_full[st], c * 64, qslot, qrow, b);
          if (issuer) tma_load_4d(sDO + st * DkvSmem<HD>::kQD + c * 64 * 128, &tmDO, &qd_full[st], c * 64, doslot, qrow, b);
        }
        if (++st == NQ) { st = 0; ph ^= 1; }
        if (++qs == n_qs) { qs = qs0; ++h; }
      }
    }
  } else if (warp == 1) {
    if (n_it > 0) {
      // the whole warp walks the loop, one elected lane issues (see mma_loop in gemm_core.cuh)
      const bool issuer = elect_one() != 0;
      constexpr uint32_t idesc_st = make_idesc_lp(128, 64, false, false);
      constexpr uint32_t idesc_acc = make_idesc_lp(128, HD, false, true);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aPT = smem_u32(sPT), aDST = smem_u32(sDST);
      bool ok = mbar_wait_warp(kv_full, 0, p.status, kTimeoutSmemFull, abort_flag);
      int qs_s = 0, qs_d = 0;          // Q / dO ring slot of the next S^T issue and of the next dV / dK issue
      uint32_t qph_s = 0;
      auto issue_st = [&](int it) -> bool {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait_warp(&qd_full[qs_s], qph_s, p.status, kTimeoutSmemFull, abort_flag)) return false;
        if (!mbar_wait_warp(&st_empty[st], ph ^ 1, p.status, kTimeoutTmemEmpty, abort_flag)) return false;
        tc_fence_after();
        const uint32_t aQ = smem_u32(sQ + qs_s * DkvSmem<HD>::kQD), aDO = smem_u32(sDO + qs_s * DkvSmem<HD>::kQD);
        if (++qs_s == NQ) { qs_s = 0; qph_s ^= 1; }
        if (issuer) {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk)
            umma_f16_ss(tST[st], kmajor_desc(aK, 128, kk), kmajor_desc(aQ, 64, kk), idesc_st, kk != 0);
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk)
            umma_f16_ss(tDPT[st], kmajor_desc(aV, 128, kk), kmajor_desc(aDO, 64, kk), idesc_st, kk != 0);
          umma_commit(&st_full[st]);
        }
        __syncwarp();
        return true;
      };
      if (ok) ok = issue_st(0);
      for (int it = 0; ok && it < n_it; ++it) {
        if (it + 1 < n_it) { ok = issue_st(it + 1); if (!ok) break; }
        const int st = it & 1;
        if (!mbar_wait_warp(&pds_full[st], (it >> 1) & 1, p.status, kTimeoutOther, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t aQ = smem_u32(sQ + qs_d * DkvSmem<HD>::kQD), aDO = smem_u32(sDO + qs_d * DkvSmem<HD>::kQD);
        const uint32_t aPTs = aPT + st * DkvSmem<HD>::kPT, aDSTs = aDST + st * DkvSmem<HD>::kPT;
        if (issuer) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16_ss(tDV, kmajor_desc(aPTs, 128, kk), mnmajor_desc(aDO, 64, kk), idesc_acc, (it | kk) != 0);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16_ss(tDK, kmajor_desc(aDSTs, 128, kk), mnmajor_desc(aQ, 64, kk), idesc_acc, (it | kk) != 0);
          umma_commit(&qd_empty[qs_d]);
          umma_commit(&pds_empty[st]);
        }
        __syncwarp();
        if (++qs_d == NQ) qs_d = 0;
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    const int wq = warp & 3;
    const int half = (warp - 2) >> 2;     // which 32 of the step's 64 query columns this warpgroup owns
    const int c0 = half * 32;
    const int row = wq * 32 + lane_id();  // key row inside the block
    const int tid = threadIdx.x - 64;     // 0..255 among the softmax threads
    const uint32_t lane_off = uint32_t(wq * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    const int k_pos = p.k_pos0 + k0 + row;
    const bool k_valid = (k0 + row) < p.Skv;
    bool ok = true;
    // Per-query statistics (-LSE * log2 e and D) of a step, fetched one step ahead so that the global-memory
    // latency is hidden behind the previous step's work: thread t < 64 carries -lse2 of query t, 64 <= t < 128 D.
    int ld_h = h0, ld_qs = qs0, ld_it = 0;   // (head, query step) of the next statistics fetch; no division in the loop
    auto load_stat = [&]() -> float {
      float v = 0.f;
      if (tid < 128 && ld_it < n_it) {
        const int q = ld_qs * 64 + (tid & 63);
        if (q >= p.Sq) {
          v = (tid < 64) ? INFINITY : 0.f;    // rows past the end: -inf after scaling, 2^-inf = 0
        } else {
          const float* src = (tid < 64) ? p.LSE : p.D;
          v = src[(size_t(b) * p.nheads + ld_h) * p.Sq + q];   // raw; scaled by stat_scale when it is stored, so
        }                                                        // that nothing waits for the load here
      }
      ++ld_it;
      if (++ld_qs == n_qs) { ld_qs = qs0; ++ld_h; }
      return v;
    };
    const float stat_scale = (tid < 64) ? -kLog2e : 1.f;   // -LSE * log2 e for the first 64 threads, D as it is
    float stat_next = load_stat();
    if (n_it > 0) {
      if (tid < 128) sStats[tid] = stat_next * stat_scale;
      mbar_arrive(&stats_full[0]);
      stat_next = load_stat();
    }
    int cur_qs = qs0;
    for (int it = 0; it < n_it; ++it) {
      const int st = it & 1;
      const int qrow = cur_qs * 64;
      if (++cur_qs == n_qs) cur_qs = qs0;
      if (!mbar_wait_warp(&stats_full[st], (it >> 1) & 1, p.status, kTimeoutOther, abort_flag)) { ok = false; break; }
      if (!mbar_wait_warp(&st_full[st], (it >> 1) & 1, p.status, kTimeoutTmemFull, abort_flag)) { ok = false; break; }
      tc_fence_after();
      float pt[32], ds[32];
      {
        uint32_t r0[32], r1[32];
        tmem_ld32(tST[st] + lane_off + c0, r0);
        tmem_ld32(tDPT[st] + lane_off + c0, r1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) { pt[i] = __uint_as_float(r0[i]); ds[i] = __uint_as_float(r1[i]); }
      }
      tc_fence_before();
      mbar_arrive(&st_empty[st]);
      {
        const float4* nl4 = reinterpret_cast<const float4*>(sStats + st * 128 + c0);   // -lse2
        const float4* dd4 = nl4 + 16;                                                  // D
        // only steps that touch the diagonal, or a key block with rows past the end, need the mask
        const bool need_mask = !k_valid || (p.causal && (p.q_pos0 + qrow < p.k_pos0 + k0 + 127));
        const int q_base = p.q_pos0 + qrow + c0;
        if (!need_mask) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 nl = nl4[i >> 2], dd = dd4[i >> 2];
            const float nlv[4] = {nl.x, nl.y, nl.z, nl.w}, ddv[4] = {dd.x, dd.y, dd.z, dd.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              pt[i + u] = ex2(fmaf(pt[i + u], sl2, nlv[u]));
              ds[i + u] = pt[i + u] * (ds[i + u] - ddv[u]);   // in the same loop: these overlap with the exp2 unit
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 nl = nl4[i >> 2], dd = dd4[i >> 2];
            const float nlv[4] = {nl.x, nl.y, nl.z, nl.w}, ddv[4] = {dd.x, dd.y, dd.z, dd.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const bool dead = !k_valid || (p.causal && k_pos > q_base + i + u);
              pt[i + u] = dead ? 0.f : ex2(fmaf(pt[i + u], sl2, nlv[u]));
              ds[i + u] = pt[i + u] * (ds[i + u] - ddv[u]);
            }
          }
        }
      }
      // the next step's statistics go to the other buffer: every thread is past its reads of that buffer (they
      // all arrived on this step's stats barrier after finishing the previous step)
      if (it + 1 < n_it) {
        if (tid < 128) sStats[(st ^ 1) * 128 + tid] = stat_next * stat_scale;
        mbar_arrive(&stats_full[st ^ 1]);
        stat_next = load_stat();
      }
      if (it >= 2) {   // these buffers were last read by the dV / dK products of step it-2
        if (!mbar_wait_warp(&pds_empty[st], ((it >> 1) & 1) ^ 1, p.status, kTimeoutOther, abort_flag)) { ok = false; break; }
      }
      uint8_t* sPTs = sPT + st * DkvSmem<HD>::kPT;
      uint8_t* sDSTs = sDST + st * DkvSmem<HD>::kPT;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint4 u, w;
        u.x = pack_bf16(pt[cc * 8 + 0], pt[cc * 8 + 1]); u.y = pack_bf16(pt[cc * 8 + 2], pt[cc * 8 + 3]);
        u.z = pack_bf16(pt[cc * 8 + 4], pt[cc * 8 + 5]); u.w = pack_bf16(pt[cc * 8 + 6], pt[cc * 8 + 7]);
        w.x = pack_bf16(ds[cc * 8 + 0], ds[cc * 8 + 1]); w.y = pack_bf16(ds[cc * 8 + 2], ds[cc * 8 + 3]);
        w.z = pack_bf16(ds[cc * 8 + 4], ds[cc * 8 + 5]); w.w = pack_bf16(ds[cc * 8 + 6], ds[cc * 8 + 7]);
        *reinterpret_cast<uint4*>(sPTs + sw128_offset(row, half * 4 + cc)) = u;
        *reinterpret_cast<uint4*>(sDSTs + sw128_offset(row, half * 4 + cc)) = w;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&pds_full[st]);
    }
    // ---- epilogue ----
    const int krow = k0 + row;
    const int dkslot = p.dkmap.slot(h0, p.qpg), dvslot = p.dvmap.slot(h0, p.qpg);
    hg_lp_t* dk = p.dK + int64_t(krow) * p.dk_ss + int64_t(b) * p.dk_sb + int64_t(dkslot) * HD;
    hg_lp_t* dv = p.dV + int64_t(krow) * p.dv_ss + int64_t(b) * p.dv_sb + int64_t(dvslot) * HD;
    if (n_it == 0) {
      if (krow < p.Skv) {
#pragma unroll
        for (int i = half; i < HD / 8; i += 2) {
          reinterpret_cast<uint4*>(dk)[i] = make_uint4(0, 0, 0, 0);
          reinterpret_cast<uint4*>(dv)[i] = make_uint4(0, 0, 0, 0);
        }
      }
    } else if (ok && !*abort_flag &&
               mbar_wait_warp(&pds_empty[(n_it - 1) & 1], ((n_it - 1) >> 1) & 1, p.status, kTimeoutOther, abort_flag)) {
      tc_fence_after();
#pragma unroll
      for (int c = half; c < HD / 32; c += 2) {   // the two warpgroups take alternate 32-column chunks
        uint32_t r0[32], r1[32];
        tmem_ld32(tDV + lane_off + c * 32, r0);
        tmem_ld32(tDK + lane_off + c * 32, r1);
        tmem_ld_wait();
        if (krow < p.Skv) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u, w;
            u.x = pack_bf16(__uint_as_float(r0[q * 8 + 0]), __uint_as_float(r0[q * 8 + 1]));
            u.y = pack_bf16(__uint_as_float(r0[q * 8 + 2]), __uint_as_float(r0[q * 8 + 3]));
            u.z = pack_bf16(__uint_as_float(r0[q * 8 + 4]), __uint_as_float(r0[q * 8 + 5]));
            u.w = pack_bf16(__uint_as_float(r0[q * 8 + 6]), __uint_as_float(r0[q * 8 + 7]));
            w.x = pack_bf16(__uint_as_float(r1[q * 8 + 0]) * p.scale, __uint_as_float(r1[q * 8 + 1]) * p.scale);
            w.y = pack_bf16(__uint_as_float(r1[q * 8 + 2]) * p.scale, __uint_as_float(r1[q * 8 + 3]) * p.scale);
            w.z = pack_bf16(__uint_as_float(r1[q * 8 + 4]) * p.scale, __uint_as_float(r1[q * 8 + 5]) * p.scale);
            w.w = pack_bf16(__uint_as_float(r1[q * 8 + 6]) * p.scale, __uint_as_float(r1[q * 8 + 7]) * p.scale);
            reinterpret_cast<uint4*>(dv + c * 32)[q] = u;
            reinterpret_cast<uint4*>(dk + c * 32)[q] = w;
          }
        }
      }
    } else {
      *abort_flag = 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// =================================================================================================
// Backward, part 1 with 128-query steps and the probabilities kept in tensor memory (head dim 128).
// The 64-query version issues its score products with N = 64, which occupy the tensor core as long as N = 128 would,
// and stages P^T / dS^T through 64 KB of shared memory.  Here a step covers 128 queries:
//   S^T = K Q^T and dP^T = V dO^T are 128 x 128 products (8 MMAs each);
//   the softmax threads turn them into P^T = exp2(S^T c - lse) and dS^T = P^T (dP^T - D) and store both back into
//   tensor memory as packed 16-bit pairs;
//   dV += P^T dO and dK += dS^T Q take their A operand from tensor memory (8 MMAs each, K = 128 queries).
// Per 128 queries that is 32 MMAs instead of 48, no shared-memory traffic from the softmax threads, and the 64 KB
// of staging buffers become Q / dO ring slots (three of Q, two of dO: a Q tile lives from its S^T product to its
// dK product, a dO tile from dP^T to dV).
//
// Tensor memory (512 columns): S^T 0..127, dP^T 128..255, dV 256..383, dK 384..511.  A softmax thread (one key row,
// the 128 / NWG query columns of its warpgroup) loads its S^T values and releases the S^T columns at once, so that
// S^T of the next step is computed while this step's exponentials run; once dP^T has arrived it loads its dP^T
// values and then owns those columns: the packed P^T goes over their first half, the packed dS^T over the second.
// The tensor core executes MMAs in issue order, which makes the reuse safe: dP^T(i+1) is issued after dV(i) and
// dK(i), the readers of P^T(i) and dS^T(i).  Per step the MMA warp issues S^T(i+1) when the S^T(i) columns are
// free, dV(i) when P^T(i) is stored, dK(i) and dP^T(i+1) when dS^T(i) is stored.
// =================================================================================================

template <int HD>
struct Dkv128Smem {
  static constexpr int kKV = 128 * HD * 2;       // resident K or V
  static constexpr int kQD = 128 * HD * 2;       // one Q or dO tile
  static constexpr int kQStages = 3;
  static constexpr int kDOStages = 2;
  static constexpr int kStats = 2 * 2 * 128 * 4;  // -lse*log2e and D of a step, double buffered
  static constexpr int kBars = 256;
  static constexpr int kUsed = 2 * kKV + (kQStages + kDOStages) * kQD + kStats + kBars;
  static constexpr int kTotal = 232448;          // everything a CTA can have; the 1024-byte alignment of the tiles comes out of the rest
};

// NWG softmax warpgroups (2 or 4): thread == key row, warpgroup g owns query columns [g * 128 / NWG, (g + 1) * 128 / NWG)
// of every step.  Four warpgroups put four warps on every scheduler, which is what keeps the exp2 unit and the FMA
// pipe busy through the latencies of the loads from tensor memory and of the dependent exp2 / convert chains.
template <int HD, int NWG>
__global__ void __launch_bounds__(64 + 128 * NWG, 1)
flash_bwd_dkv128_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                        const BwdParams p) {
  static_assert(HD == 128, "the 128-query dK/dV kernel is written for head dim 128");
  static_assert(NWG == 2 || NWG == 4, "two or four softmax warpgroups");
  constexpr int kSoftmaxWarps = 4 * NWG;
  constexpr int CPT = 128 / NWG;               // query columns per thread and step
  extern __shared__ uint8_t smem_raw[];
  using L = Dkv128Smem<HD>;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if (base + L::kUsed > smem_raw + L::kTotal) {   // the same for every thread: nothing has been set up yet
    if (threadIdx.x == 0) set_status(p.status, kTimeoutOther);
    return;
  }
  uint8_t* sK = base;
  uint8_t* sV = sK + L::kKV;
  constexpr int NQ = L::kQStages, ND = L::kDOStages;
  uint8_t* sQ = sV + L::kKV;                 // NQ tiles
  uint8_t* sDO = sQ + NQ * L::kQD;           // ND tiles
  float* sStats = reinterpret_cast<float*>(sDO + ND * L::kQD);   // [2][256]: 128 x -lse2, 128 x D
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sStats) + L::kStats);
  uint64_t* kv_full = bars;          // 1
  uint64_t* q_full = bars + 1;       // 3
  uint64_t* q_empty = bars + 4;      // 3
  uint64_t* do_full = bars + 7;      // 2
  uint64_t* do_empty = bars + 9;     // 2
  uint64_t* st_full = bars + 11;     // S^T of a step is in tensor memory
  uint64_t* dpt_full = bars + 12;    // dP^T of a step is in tensor memory
  uint64_t* p_full = bars + 13;      // every thread has stored its part of P^T
  uint64_t* ds_full = bars + 14;     // every thread has stored its part of dS^T
  uint64_t* acc_full = bars + 15;    // the last dK product has completed
  uint64_t* stats_full = bars + 16;  // 2
  uint64_t* x_free = bars + 18;      // every thread has loaded its S^T values: the S^T columns may be overwritten
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int kb = blockIdx.x, g = blockIdx.y, b = blockIdx.z;  // g = kv head
  const int k0 = kb * 128;
  int q_first = 0;                                            // first query row that can see this key block
  if (p.causal) q_first = max(0, p.k_pos0 + k0 - p.q_pos0);
  const int qs0 = q_first / 128;                              // first 128-row query step
  const int n_qs = (p.Sq + 127) / 128;
  const int steps_per_head = max(0, n_qs - qs0);
  const int n_it = steps_per_head * p.qpg;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
    mbar_init(kv_full, 1);
    for (int i = 0; i < NQ; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); }
    for (int i = 0; i < ND; ++i) { mbar_init(&do_full[i], 1); mbar_init(&do_empty[i], 1); }
    mbar_init(st_full, 1);
    mbar_init(dpt_full, 1);
    mbar_init(p_full, kSoftmaxWarps);       // one arrival per softmax warp (mbar_arrive_warp)
    mbar_init(ds_full, kSoftmaxWarps);
    mbar_init(x_free, kSoftmaxWarps);
    mbar_init(acc_full, 1);
    mbar_init(&stats_full[0], kSoftmaxWarps);
    mbar_init(&stats_full[1], kSoftmaxWarps);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tST = tmem, tDPT = tmem + 128, tDV = tmem + 256, tDK = tmem + 384;

  const int h0 = g * p.qpg;  // first query head of the group
  const int kslot = p.kmap.slot(h0, p.qpg), vslot = p.vmap.slot(h0, p.qpg);

  if (warp == 0) {
    if (n_it > 0) {
      // the whole warp walks the loop, one elected lane issues the copies (see producer_loop in gemm_core.cuh)
      const bool issuer = elect_one() != 0;
      if (issuer) mbar_expect_tx(kv_full, 2 * L::kKV);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
        if (issuer) tma_load_4d(sK + c * 128 * 128, &tmK, kv_full, c * 64, kslot, k0, b);
        if (issuer) tma_load_4d(sV + c * 128 * 128, &tmV, kv_full, c * 64, vslot, k0, b);
      }
      int qs_slot = 0, ds_slot = 0;
      uint32_t qph = 0, dph = 0;
      int h = h0, qs = qs0;
      for (int it = 0; it < n_it; ++it) {
        const int qrow = qs * 128;
        const int qslot = p.qmap.slot(h, p.qpg), doslot = p.domap.slot(h, p.qpg);
        if (!mbar_wait_warp(&q_empty[qs_slot], qph ^ 1, p.status, kTimeoutSmemEmpty, abort_flag)) { *abort_flag = 1; break; }
        if (issuer) mbar_expect_tx(&q_full[qs_slot], L::kQD);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          if (issuer) tma_load_4d(sQ + qs_slot * L::kQD + c * 128 * 128, &tmQ, &q_full[qs_slot], c * 64, qslot, qrow, b);
        if (!mbar_wait_warp(&do_empty[ds_slot], dph ^ 1, p.status, kTimeoutSmemEmpty, abort_flag)) { *abort_flag = 1; break; }
        if (issuer) mbar_expect_tx(&do_full[ds_slot], L::kQD);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          if (issuer) tma_load_4d(sDO + ds_slot * L::kQD + c * 128 * 128, &tmDO, &do_full[ds_slot], c * 64, doslot, qrow, b);
        if (++qs_slot == NQ) { qs_slot = 0; qph ^= 1; }
        if (++ds_slot == ND) { ds_slot = 0; dph ^= 1; }
        if (++qs == n_qs) { qs = qs0; ++h; }
      }
    }
  } else if (warp == 1) {
    if (n_it > 0) {
      // the whole warp walks the loop, one elected lane issues (see mma_loop in gemm_core.cuh)
      const bool issuer = elect_one() != 0;
      constexpr uint32_t idesc_st = make_idesc_lp(128, 128, false, false);
      constexpr uint32_t idesc_acc = make_idesc_lp(128, HD, false, true);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ0 = smem_u32(sQ), aDO0 = smem_u32(sDO);
      // queries 16kk.. belong to warpgroup 16kk / CPT; its packed P^T values start at the first of its CPT columns of
      // the dP^T range, its packed dS^T values CPT / 2 columns further
      auto packed_col = [](int kk) -> uint32_t { return uint32_t((16 * kk / CPT) * CPT + (16 * kk % CPT) / 2); };
      // ring positions: Q / dO tile of the next S^T / dP^T issue, and of the next dK / dV issue
      int q_s = 0, q_k = 0, d_p = 0, d_v = 0;
      uint32_t qph_s = 0, dph_p = 0;
      auto issue_st = [&]() -> bool {     // S^T of the next step
        if (!mbar_wait_warp(&q_full[q_s], qph_s, p.status, kTimeoutSmemFull, abort_flag)) return false;
        tc_fence_after();
        const uint32_t aQ = aQ0 + q_s * L::kQD;
        if (issuer) {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk)
            umma_f16_ss(tST, kmajor_desc(aK, 128, kk), kmajor_desc(aQ, 128, kk), idesc_st, kk != 0);
          umma_commit(st_full);
        }
        __syncwarp();
        if (++q_s == NQ) { q_s = 0; qph_s ^= 1; }
        return true;
      };
      auto issue_dpt = [&]() -> bool {    // dP^T of the next step
        if (!mbar_wait_warp(&do_full[d_p], dph_p, p.status, kTimeoutSmemFull, abort_flag)) return false;
        tc_fence_after();
        const uint32_t aDO = aDO0 + d_p * L::kQD;
        if (issuer) {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk)
            umma_f16_ss(tDPT, kmajor_desc(aV, 128, kk), kmajor_desc(aDO, 128, kk), idesc_st, kk != 0);
          umma_commit(dpt_full);
        }
        __syncwarp();
        if (++d_p == ND) { d_p = 0; dph_p ^= 1; }
        return true;
      };
      bool ok = mbar_wait_warp(kv_full, 0, p.status, kTimeoutSmemFull, abort_flag);
      if (ok) ok = issue_st();
      if (ok) ok = issue_dpt();
      HG_DKV_TIMERS(tm_wait_x, tm_wait_p, tm_wait_ds, tm_issue);
      for (int it = 0; ok && it < n_it; ++it) {
        const uint32_t ph = it & 1;
        HG_DKV_TICK(t0);
        // ---- S^T(it+1), as soon as the S^T(it) values are in the threads' registers
        if (!mbar_wait_warp(x_free, ph, p.status, kTimeoutOther, abort_flag)) { ok = false; break; }
        tc_fence_after();
        HG_DKV_TOCK(tm_wait_x, t0);
        if (it + 1 < n_it) { ok = issue_st(); if (!ok) break; }
        HG_DKV_TOCK(tm_issue, t0);
        // ---- dV(it)
        if (!mbar_wait_warp(p_full, ph, p.status, kTimeoutOther, abort_flag)) { ok = false; break; }
        tc_fence_after();
        HG_DKV_TOCK(tm_wait_p, t0);
        if (issuer) {
          const uint32_t aDO = aDO0 + d_v * L::kQD;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)     // k-step kk = queries 16kk..16kk+15 = 8 packed columns of their warpgroup's range
            umma_f16_ts(tDV, tDPT + packed_col(kk), mnmajor_desc(aDO, 128, kk), idesc_acc, (it | kk) != 0);
          umma_commit(&do_empty[d_v]);
        }
        __syncwarp();
        if (++d_v == ND) d_v = 0;
        HG_DKV_TOCK(tm_issue, t0);
        // ---- dK(it), then dP^T(it+1) over the columns dV and dK have just read
        if (!mbar_wait_warp(ds_full, ph, p.status, kTimeoutOther, abort_flag)) { ok = false; break; }
        tc_fence_after();
        HG_DKV_TOCK(tm_wait_ds, t0);
        if (issuer) {
          const uint32_t aQ = aQ0 + q_k * L::kQD;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_f16_ts(tDK, tDPT + CPT / 2 + packed_col(kk), mnmajor_desc(aQ, 128, kk), idesc_acc, (it | kk) != 0);
          umma_commit(&q_empty[q_k]);
        }
        __syncwarp();
        if (++q_k == NQ) q_k = 0;
        if (it + 1 < n_it) { ok = issue_dpt(); if (!ok) break; }
        HG_DKV_TOCK(tm_issue, t0);
      }
      HG_DKV_REPORT(8, n_it, tm_wait_x, tm_wait_p, tm_wait_ds, tm_issue);
      if (ok && issuer) umma_commit(acc_full);
      __syncwarp();
      if (!ok) *abort_flag = 1;
    }
  } else {
    const int wq = warp & 3;
    const int half = (warp - 2) >> 2;     // warpgroup: which CPT of the step's 128 query columns these threads own
    const int c0 = half * CPT;
    const int row = wq * 32 + lane_id();  // key row inside the block
    const int tid = threadIdx.x - 64;     // 0..128*NWG-1 among the softmax threads; the first 256 carry the statistics
    const uint32_t lane_off = uint32_t(wq * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    const int k_pos = p.k_pos0 + k0 + row;
    const bool k_valid = (k0 + row) < p.Skv;
    bool ok = true;
    // Per-query statistics of a step, fetched one step ahead: thread t < 128 carries -lse * log2 e of query t of the
    // step, thread 128 + t carries D of query t.
    int ld_h = h0, ld_qs = qs0, ld_it = 0;
    auto load_stat = [&]() -> float {
      float v = 0.f;
      if (tid < 256 && ld_it < n_it) {
        const int q = ld_qs * 128 + (tid & 127);
        if (q >= p.Sq) {
          v = (tid < 128) ? INFINITY : 0.f;    // rows past the end: -inf after scaling, 2^-inf = 0
        } else {
          const float* src = (tid < 128) ? p.LSE : p.D;
          v = src[(size_t(b) * p.nheads + ld_h) * p.Sq + q];
        }
      }
      ++ld_it;
      if (++ld_qs == n_qs) { ld_qs = qs0; ++ld_h; }
      return v;
    };
    const float stat_scale = (tid < 128) ? -kLog2e : 1.f;
    float stat_next = load_stat();
    if (n_it > 0) {
      if (tid < 256) sStats[tid] = stat_next * stat_scale;
      mbar_arrive_warp(&stats_full[0]);
      stat_next = load_stat();
    }
    int cur_qs = qs0;
    HG_DKV_TIMERS(tm_wait_a, tm_a, tm_wait_b, tm_b);
    for (int it = 0; it < n_it; ++it) {
      const int sb = it & 1;
      const uint32_t ph = it & 1;
      HG_DKV_TICK(t0);
      const int qrow = cur_qs * 128;
      if (++cur_qs == n_qs) cur_qs = qs0;
      const float* st = sStats + sb * 256;
      uint32_t pp[CPT / 2];               // this thread's probabilities, packed, kept for the second phase
      // ---------------- S^T -> probabilities (kept in registers; the S^T columns are released at once)
      if (!mbar_wait_warp(&stats_full[sb], (it >> 1) & 1, p.status, kTimeoutOther, abort_flag)) { ok = false; break; }
      if (!mbar_wait_warp(st_full, ph, p.status, kTimeoutTmemFull, abort_flag)) { ok = false; break; }
      tc_fence_after();
      HG_DKV_TOCK(tm_wait_a, t0);
      {
        // only steps that touch the diagonal, or a key block with rows past the end, need the mask
        const bool need_mask = !k_valid || (p.causal && (p.q_pos0 + qrow < p.k_pos0 + k0 + 127));
        uint32_t rr[CPT / 32][32];
#pragma unroll
        for (int hh = 0; hh < CPT / 32; ++hh) tmem_ld32(tST + lane_off + c0 + hh * 32, rr[hh]);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive_warp(x_free);
        // The masked and the plain form are two straight-line bodies: a branch inside the element loop would cut it
        // into sixteen basic blocks, and the compiler schedules (overlaps the loads, FMAs and exp2 of different
        // elements) only inside one.
        auto probabilities = [&](auto masked) {
#pragma unroll
          for (int hh = 0; hh < CPT / 32; ++hh) {
            const uint32_t(&r)[32] = rr[hh];
            const float4* nl4 = reinterpret_cast<const float4*>(st + c0 + hh * 32);
            const int q_base = p.q_pos0 + qrow + c0 + hh * 32;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float4 nl = nl4[i >> 2];
              const float nlv[4] = {nl.x, nl.y, nl.z, nl.w};
              float e[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const float x = fmaf(__uint_as_float(r[i + u]), sl2, nlv[u]);
                e[u] = (u < HG_DKV_POLY_OF_4) ? ex2_poly(x) : ex2(x);
                if (decltype(masked)::value && (!k_valid || (p.causal && k_pos > q_base + i + u))) e[u] = 0.f;
              }
              pp[hh * 16 + (i >> 1)] = pack_bf16(e[0], e[1]);
              pp[hh * 16 + (i >> 1) + 1] = pack_bf16(e[2], e[3]);
            }
          }
        };
        if (need_mask) probabilities(std::true_type{});
        else probabilities(std::false_type{});
      }
      HG_DKV_TOCK(tm_a, t0);
      // ---------------- dP^T -> dS^T; P^T and dS^T go, packed, over this thread's own dP^T columns
      if (!mbar_wait_warp(dpt_full, ph, p.status, kTimeoutTmemFull, abort_flag)) { ok = false; break; }
      tc_fence_after();
      HG_DKV_TOCK(tm_wait_b, t0);
      {
        uint32_t dsp[CPT / 2];
        uint32_t rr[CPT / 32][32];
#pragma unroll
        for (int hh = 0; hh < CPT / 32; ++hh) tmem_ld32(tDPT + lane_off + c0 + hh * 32, rr[hh]);
        tmem_ld_wait();
        if constexpr (CPT == 64) tmem_st32(tDPT + lane_off + c0, pp);
        else tmem_st16(tDPT + lane_off + c0, pp);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive_warp(p_full);
#pragma unroll
        for (int hh = 0; hh < CPT / 32; ++hh) {
          const uint32_t(&r)[32] = rr[hh];
          const float4* dd4 = reinterpret_cast<const float4*>(st + 128 + c0 + hh * 32);
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 dd = dd4[i >> 2];
            const float2 p01 = hg_unpack2(pp[hh * 16 + (i >> 1)]), p23 = hg_unpack2(pp[hh * 16 + (i >> 1) + 1]);
            dsp[hh * 16 + (i >> 1)] = pack_bf16(p01.x * (__uint_as_float(r[i]) - dd.x),
                                                 p01.y * (__uint_as_float(r[i + 1]) - dd.y));
            dsp[hh * 16 + (i >> 1) + 1] = pack_bf16(p23.x * (__uint_as_float(r[i + 2]) - dd.z),
                                                     p23.y * (__uint_as_float(r[i + 3]) - dd.w));
          }
        }
        if constexpr (CPT == 64) tmem_st32(tDPT + lane_off + c0 + CPT / 2, dsp);
        else tmem_st16(tDPT + lane_off + c0 + CPT / 2, dsp);
      }
      // the next step's statistics go to the other buffer: its last readers were the second phases of step it-1,
      // and every thread finished that before it arrived on this step's statistics barrier
      if (it + 1 < n_it) {
        if (tid < 256) sStats[(sb ^ 1) * 256 + tid] = stat_next * stat_scale;
        mbar_arrive_warp(&stats_full[sb ^ 1]);
        stat_next = load_stat();
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive_warp(ds_full);
      HG_DKV_TOCK(tm_b, t0);
    }
    HG_DKV_REPORT(0, n_it, tm_wait_a, tm_a, tm_wait_b, tm_b);
    // ---- epilogue ----
    const int krow = k0 + row;
    const int dkslot = p.dkmap.slot(h0, p.qpg), dvslot = p.dvmap.slot(h0, p.qpg);
    hg_lp_t* dk = p.dK + int64_t(krow) * p.dk_ss + int64_t(b) * p.dk_sb + int64_t(dkslot) * HD;
    hg_lp_t* dv = p.dV + int64_t(krow) * p.dv_ss + int64_t(b) * p.dv_sb + int64_t(dvslot) * HD;
    if (n_it == 0) {
      if (krow < p.Skv) {
#pragma unroll
        for (int i = half; i < HD / 8; i += NWG) {
          reinterpret_cast<uint4*>(dk)[i] = make_uint4(0, 0, 0, 0);
          reinterpret_cast<uint4*>(dv)[i] = make_uint4(0, 0, 0, 0);
        }
      }
    } else if (ok && !*abort_flag && mbar_wait_warp(acc_full, 0, p.status, kTimeoutOther, abort_flag)) {
      tc_fence_after();
#pragma unroll
      for (int c = half; c < HD / 32; c += NWG) {   // the warpgroups take alternate 32-column chunks
        uint32_t r0[32], r1[32];
        tmem_ld32(tDV + lane_off + c * 32, r0);
        tmem_ld32(tDK + lane_off + c * 32, r1);
        tmem_ld_wait();
        if (krow < p.Skv) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u, w;
            u.x = pack_bf16(__uint_as_float(r0[q * 8 + 0]), __uint_as_float(r0[q * 8 + 1]));
            u.y = pack_bf16(__uint_as_float(r0[q * 8 + 2]), __uint_as_float(r0[q * 8 + 3]));
            u.z = pack_bf16(__uint_as_float(r0[q * 8 + 4]), __uint_as_float(r0[q * 8 + 5]));
            u.w = pack_bf16(__uint_as_float(r0[q * 8 + 6]), __uint_as_float(r0[q * 8 + 7]));
            w.x = pack_bf16(__uint_as_float(r1[q * 8 + 0]) * p.scale, __uint_as_float(r1[q * 8 + 1]) * p.scale);
            w.y = pack_bf16(__uint_as_float(r1[q * 8 + 2]) * p.scale, __uint_as_float(r1[q * 8 + 3]) * p.scale);
            w.z = pack_bf16(__uint_as_float(r1[q * 8 + 4]) * p.scale, __uint_as_float(r1[q * 8 + 5]) * p.scale);
            w.w = pack_bf16(__uint_as_float(r1[q * 8 + 6]) * p.scale, __uint_as_float(r1[q * 8 + 7]) * p.scale);
            reinterpret_cast<uint4*>(dv + c * 32)[q] = u;
            reinterpret_cast<uint4*>(dk + c * 32)[q] = w;
          }
        }
      }
    } else {
      *abort_flag = 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// =================================================================================================
// Backward, part 2: one CTA per (query block of 128, head, batch); loops over 64-row key steps.
// Thread == query row.   S = Q K^T, dP = dO V^T (N = 64);  dS = P * (dP - D);  dQ += dS K
// =================================================================================================
template <int HD>
struct DqSmem {
  static constexpr int kQ = 128 * HD * 2;     // resident Q or dO
  static constexpr int kKV = 64 * HD * 2;     // one stage of K or V
  static constexpr int kDS = 128 * 64 * 2;    // one dS buffer (two are kept so that step i+1 is written while step i is multiplied)
  static constexpr int kTotal = 2 * kQ + 4 * kKV + 2 * kDS + 1024 + 256;
};

template <int HD>
__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = base;
  uint8_t* sDO = sQ + DqSmem<HD>::kQ;
  uint8_t* sK = sDO + DqSmem<HD>::kQ;            // 2 stages
  uint8_t* sV = sK + 2 * DqSmem<HD>::kKV;        // 2 stages
  uint8_t* sDS = sV + 2 * DqSmem<HD>::kKV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + 2 * DqSmem<HD>::kDS);
  uint64_t* qdo_full = bars;       // 1
  uint64_t* kv_full = bars + 1;    // 2
  uint64_t* kv_empty = bars + 3;   // 2
  uint64_t* s_full = bars + 5;     // 2
  uint64_t* s_empty = bars + 7;    // 2
  uint64_t* ds_full = bars + 9;    // 2
  uint64_t* ds_empty = bars + 11;  // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int qb = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = qb * 128;
  int kv_len = p.Skv;
  if (p.causal) kv_len = min(p.Skv, p.q_pos0 + q0 + 127 - p.k_pos0 + 1);
  const int n_it = kv_len > 0 ? (kv_len + 63) / 64 : 0;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
    mbar_init(qdo_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], kBwdSoftmaxThreads);
      mbar_init(&ds_full[i], kBwdSoftmaxThreads);
      mbar_init(&ds_empty[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS[2] = {tmem, tmem + 128};
  const uint32_t tDP[2] = {tmem + 64, tmem + 192};
  const uint32_t tDQ = tmem + 256;

  const int qslot = p.qmap.slot(h, p.qpg), kslot = p.kmap.slot(h, p.qpg), vslot = p.vmap.slot(h, p.qpg),
            doslot = p.domap.slot(h, p.qpg);

  if (warp == 0) {
    if (n_it > 0) {
      // the whole warp walks the loop, one elected lane issues the copies (see producer_loop in gemm_core.cuh)
      const bool issuer = elect_one() != 0;
      if (issuer) mbar_expect_tx(qdo_full, 2 * DqSmem<HD>::kQ);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
        if (issuer) tma_load_4d(sQ + c * 128 * 128, &tmQ, qdo_full, c * 64, qslot, q0, b);
        if (issuer) tma_load_4d(sDO + c * 128 * 128, &tmDO, qdo_full, c * 64, doslot, q0, b);
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it & 1;
        if (!mbar_wait_warp(&kv_empty[st], ((it >> 1) & 1) ^ 1, p.status, kTimeoutSmemEmpty, abort_flag)) { *abort_flag = 1; break; }
        if (issuer) mbar_expect_tx(&kv_full[st], 2 * DqSmem<HD>::kKV);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) {
          if (issuer) tma_load_4d(sK + st * DqSmem<HD>::kKV + c * 64 * 128, &tmK, &kv_full[st], c * 64, kslot, it * 64, b);
          if (issuer) tma_load_4d(sV + st * DqSmem<HD>::kKV + c * 64 * 128, &tmV, &kv_full[st], c * 64, vslot, it * 64, b);
        }
      }
    }
  } else if (warp == 1) {
    if (n_it > 0) {
      // the whole warp walks the loop, one elected lane issues (see mma_loop in gemm_core.cuh)
      const bool issuer = elect_one() != 0;
      constexpr uint32_t idesc_s = make_idesc_lp(128, 64, false, false);
      constexpr uint32_t idesc_dq = make_idesc_lp(128, HD, false, true);
      const uint32_t aQ = smem_u32(sQ), aDO = smem_u32(sDO), aDS = smem_u32(sDS);
      bool ok = mbar_wait_warp(qdo_full, 0, p.status, kTimeoutSmemFull, abort_flag);
      auto issue_s = [&](int it) -> bool {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait_warp(&kv_full[st], ph, p.status, kTimeoutSmemFull, abort_flag)) return false;
        if (!mbar_wait_warp(&s_empty[st], ph ^ 1, p.status, kTimeoutTmemEmpty, abort_flag)) return false;
        tc_fence_after();
        const uint32_t aK = smem_u32(sK + st * DqSmem<HD>::kKV), aV = smem_u32(sV + st * DqSmem<HD>::kKV);
        if (issuer) {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk)
            umma_f16_ss(tS[st], kmajor_desc(aQ, 128, kk), kmajor_desc(aK, 64, kk), idesc_s, kk != 0);
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk)
            umma_f16_ss(tDP[st], kmajor_desc(aDO, 128, kk), kmajor_desc(aV, 64, kk), idesc_s, kk != 0);
          umma_commit(&s_full[st]);
        }
        __syncwarp();
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int it = 0; ok && it < n_it; ++it) {
        if (it + 1 < n_it) { ok = issue_s(it + 1); if (!ok) break; }
        const int st = it & 1;
        if (!mbar_wait_warp(&ds_full[st], (it >> 1) & 1, p.status, kTimeoutOther, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t aK = smem_u32(sK + st * DqSmem<HD>::kKV);
        const uint32_t aDSs = aDS + st * DqSmem<HD>::kDS;
        if (issuer) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16_ss(tDQ, kmajor_desc(aDSs, 128, kk), mnmajor_desc(aK, 64, kk), idesc_dq, (it | kk) != 0);
          umma_commit(&kv_empty[st]);
          umma_commit(&ds_empty[st]);
        }
        __syncwarp();
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    const int wq = warp & 3;
    const int half = (warp - 2) >> 2;     // which 32 of the step's 64 key columns this warpgroup owns
    const int c0 = half * 32;
    const int row = wq * 32 + lane_id();
    const uint32_t lane_off = uint32_t(wq * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    const int srow = q0 + row;
    const int q_pos = p.q_pos0 + srow;
    float lse2 = INFINITY, dsum = 0.f;
    if (srow < p.Sq) {
      const size_t idx = (size_t(b) * p.nheads + h) * p.Sq + srow;
      lse2 = p.LSE[idx] * kLog2e;
      dsum = p.D[idx];
    }
    const float nlse2 = -lse2;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int st = it & 1;
      if (!mbar_wait_warp(&s_full[st], (it >> 1) & 1, p.status, kTimeoutTmemFull, abort_flag)) { ok = false; break; }
      tc_fence_after();
      float ds[32];
      {
        float sv[32];
        {
          uint32_t r0[32], r1[32];
          tmem_ld32(tS[st] + lane_off + c0, r0);
          tmem_ld32(tDP[st] + lane_off + c0, r1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) { sv[i] = __uint_as_float(r0[i]); ds[i] = __uint_as_float(r1[i]); }
        }
        tc_fence_before();
        mbar_arrive(&s_empty[st]);
        const int kbase = it * 64 + c0;
        const bool need_mask = (p.causal && (p.k_pos0 + kbase + 31 > p.q_pos0 + q0)) || (kbase + 32 > p.Skv);
        if (!need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) ds[i] = ex2(fmaf(sv[i], sl2, nlse2)) * (ds[i] - dsum);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const bool dead = (kbase + i >= p.Skv) || (p.causal && (p.k_pos0 + kbase + i > q_pos));
            ds[i] = dead ? 0.f : ex2(fmaf(sv[i], sl2, nlse2)) * (ds[i] - dsum);
          }
        }
      }
      if (it >= 2) {   // this buffer was last read by the dQ product of step it-2
        if (!mbar_wait_warp(&ds_empty[st], ((it >> 1) & 1) ^ 1, p.status, kTimeoutOther, abort_flag)) { ok = false; break; }
      }
      uint8_t* sDSs = sDS + st * DqSmem<HD>::kDS;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint4 w;
        w.x = pack_bf16(ds[cc * 8 + 0], ds[cc * 8 + 1]); w.y = pack_bf16(ds[cc * 8 + 2], ds[cc * 8 + 3]);
        w.z = pack_bf16(ds[cc * 8 + 4], ds[cc * 8 + 5]); w.w = pack_bf16(ds[cc * 8 + 6], ds[cc * 8 + 7]);
        *reinterpret_cast<uint4*>(sDSs + sw128_offset(row, half * 4 + cc)) = w;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&ds_full[st]);
    }
    const int dqslot = p.dqmap.slot(h, p.qpg);
    hg_lp_t* dq = p.dQ + int64_t(srow) * p.dq_ss + int64_t(b) * p.dq_sb + int64_t(dqslot) * HD;
    if (n_it == 0) {
      if (srow < p.Sq) {
#pragma unroll
        for (int i = half; i < HD / 8; i += 2) reinterpret_cast<uint4*>(dq)[i] = make_uint4(0, 0, 0, 0);
      }
    } else if (ok && !*abort_flag &&
               mbar_wait_warp(&ds_empty[(n_it - 1) & 1], ((n_it - 1) >> 1) & 1, p.status, kTimeoutOther, abort_flag)) {
      tc_fence_after();
#pragma unroll
      for (int c = half; c < HD / 32; c += 2) {   // the two warpgroups take alternate 32-column chunks
        uint32_t r[32];
        tmem_ld32(tDQ + lane_off + c * 32, r);
        tmem_ld_wait();
        if (srow < p.Sq) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack_bf16(__uint_as_float(r[q * 8 + 0]) * p.scale, __uint_as_float(r[q * 8 + 1]) * p.scale);
            u.y = pack_bf16(__uint_as_float(r[q * 8 + 2]) * p.scale, __uint_as_float(r[q * 8 + 3]) * p.scale);
            u.z = pack_bf16(__uint_as_float(r[q * 8 + 4]) * p.scale, __uint_as_float(r[q * 8 + 5]) * p.scale);
            u.w = pack_bf16(__uint_as_float(r[q * 8 + 6]) * p.scale, __uint_as_float(r[q * 8 + 7]) * p.scale);
            reinterpret_cast<uint4*>(dq + c * 32)[q] = u;
          }
        }
      }
    } else {
      *abort_flag = 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}


// =================================================================================================
// Backward, part 2 with 128-key steps (head dim 128).  A tcgen05.mma of shape 128 x N x 16 occupies the tensor core
// for the same time whatever N <= 256 is, so the score products are issued with N = 128 instead of 64: per 128 keys
// the kernel issues 24 MMAs (8 S, 8 dP, 8 dQ) where the 64-key version issues 40.  Shared memory holds three K
// stages and one V stage of 128 rows (128 KB) and Q and dO (64 KB); tensor memory holds one S / dP pair (256 columns),
// dQ (128) and two dS buffers (64 columns each): the softmax threads store dS there as packed 16-bit pairs and the
// dQ product takes it as its A operand, so nothing of a step goes through shared memory.  The S and dP products of
// step i+1 are issued as soon as the softmax threads have loaded step i into registers, so they overlap the
// arithmetic.  NWG softmax warpgroups (2 or 4): thread == query row, warpgroup g owns key columns
// [g * 128 / NWG, (g + 1) * 128 / NWG) of every step; four warpgroups put four warps on every scheduler, which is
// what covers the latencies of the tensor-memory loads and of the exp2 / convert chains.
// =================================================================================================
template <int HD>
struct Dq128Smem {
  static constexpr int kQ = 128 * HD * 2;      // resident Q or dO
  static constexpr int kKV = 128 * HD * 2;     // one stage of K or V
  // K is read by the first and by the last product of a step (S = Q K^T, dQ += dS K), so a K slot is held for more
  // than a step: three slots let the load of step i+2 start while step i is still being multiplied.  V is read by
  // dP = dO V^T only, early in the step, so one slot suffices: its reload has the rest of the step to land.
  static constexpr int kKStages = 3;
  static constexpr int kTotal = 2 * kQ + (kKStages + 1) * kKV + 1024 + 256;
};

template <int HD, int NWG>
__global__ void __launch_bounds__(64 + 128 * NWG, 1)
flash_bwd_dq128_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                       const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  using L = Dq128Smem<HD>;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = base;
  uint8_t* sDO = sQ + L::kQ;
  constexpr int NK = L::kKStages;
  uint8_t* sK = sDO + L::kQ;            // NK stages
  uint8_t* sV = sK + NK * L::kKV;       // 1 stage
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + L::kKV);
  static_assert(NWG == 2 || NWG == 4, "two or four softmax warpgroups");
  constexpr int kSoftmaxWarps = 4 * NWG;
  constexpr int CPT = 128 / NWG;        // key columns per thread and step
  uint64_t* qdo_full = bars;       // 1
  uint64_t* k_full = bars + 1;     // 3
  uint64_t* k_empty = bars + 4;    // 3
  uint64_t* v_full = bars + 7;     // 1
  uint64_t* v_empty = bars + 8;    // 1
  uint64_t* s_full = bars + 9;     // 1
  uint64_t* s_empty = bars + 10;   // 1
  uint64_t* ds_full = bars + 11;   // 1
  uint64_t* ds_empty = bars + 12;  // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int qb = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = qb * 128;
  int kv_len = p.Skv;
  if (p.causal) kv_len = min(p.Skv, p.q_pos0 + q0 + 127 - p.k_pos0 + 1);
  const int n_it = kv_len > 0 ? (kv_len + 127) / 128 : 0;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
    mbar_init(qdo_full, 1);
    for (int i = 0; i < NK; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(s_empty, kSoftmaxWarps);   // one arrival per softmax warp (mbar_arrive_warp)
    mbar_init(ds_full, kSoftmaxWarps);
    mbar_init(&ds_empty[0], 1);
    mbar_init(&ds_empty[1], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tDP = tmem + 128, tDQ = tmem + 256;
  const uint32_t tDS[2] = {tmem + 384, tmem + 448};   // packed dS, step parity

  const int qslot = p.qmap.slot(h, p.qpg), kslot = p.kmap.slot(h, p.qpg), vslot = p.vmap.slot(h, p.qpg),
            doslot = p.domap.slot(h, p.qpg);

  if (warp == 0) {
    if (n_it > 0) {
      // the whole warp walks the loop, one elected lane issues the copies (see producer_loop in gemm_core.cuh)
      const bool issuer = elect_one() != 0;
      if (issuer) mbar_expect_tx(qdo_full, 2 * L::kQ);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
        if (issuer) tma_load_4d(sQ + c * 128 * 128, &tmQ, qdo_full, c * 64, qslot, q0, b);
        if (issuer) tma_load_4d(sDO + c * 128 * 128, &tmDO, qdo_full, c * 64, doslot, q0, b);
      }
      int ks = 0;
      uint32_t kph = 0;
      for (int it = 0; it < n_it; ++it) {
        if (!mbar_wait_warp(&k_empty[ks], kph ^ 1, p.status, kTimeoutSmemEmpty, abort_flag)) { *abort_flag = 1; break; }
        if (issuer) mbar_expect_tx(&k_full[ks], L::kKV);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          if (issuer) tma_load_4d(sK + ks * L::kKV + c * 128 * 128, &tmK, &k_full[ks], c * 64, kslot, it * 128, b);
        if (!mbar_wait_warp(v_empty, (it & 1) ^ 1, p.status, kTimeoutSmemEmpty, abort_flag)) { *abort_flag = 1; break; }
        if (issuer) mbar_expect_tx(v_full, L::kKV);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          if (issuer) tma_load_4d(sV + c * 128 * 128, &tmV, v_full, c * 64, vslot, it * 128, b);
        if (++ks == NK) { ks = 0; kph ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (n_it > 0) {
      // the whole warp walks the loop, one elected lane issues (see mma_loop in gemm_core.cuh)
      const bool issuer = elect_one() != 0;
      constexpr uint32_t idesc_s = make_idesc_lp(128, 128, false, false);
      constexpr uint32_t idesc_dq = make_idesc_lp(128, HD, false, true);
      const uint32_t aQ = smem_u32(sQ), aDO = smem_u32(sDO);
      bool ok = mbar_wait_warp(qdo_full, 0, p.status, kTimeoutSmemFull, abort_flag);
      int ks_s = 0, ks_d = 0;          // K slot of the next S issue and of the next dQ issue
      uint32_t kph_s = 0;
      const uint32_t aV = smem_u32(sV);
      auto issue_s = [&](int it) -> bool {
        if (!mbar_wait_warp(&k_full[ks_s], kph_s, p.status, kTimeoutSmemFull, abort_flag)) return false;
        if (!mbar_wait_warp(s_empty, (it & 1) ^ 1, p.status, kTimeoutTmemEmpty, abort_flag)) return false;
        tc_fence_after();
        const uint32_t aK = smem_u32(sK + ks_s * L::kKV);
        if (issuer) {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk)
            umma_f16_ss(tS, kmajor_desc(aQ, 128, kk), kmajor_desc(aK, 128, kk), idesc_s, kk != 0);
        }
        __syncwarp();
        if (!mbar_wait_warp(v_full, it & 1, p.status, kTimeoutSmemFull, abort_flag)) return false;
        tc_fence_after();
        if (issuer) {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk)
            umma_f16_ss(tDP, kmajor_desc(aDO, 128, kk), kmajor_desc(aV, 128, kk), idesc_s, kk != 0);
          umma_commit(v_empty);
          umma_commit(s_full);
        }
        __syncwarp();
        if (++ks_s == NK) { ks_s = 0; kph_s ^= 1; }
        return true;
      };
      if (ok) ok = issue_s(0);
      HG_DKV_TIMERS(tm_s, tm_wait_ds, tm_dq, tm_unused);
      for (int it = 0; ok && it < n_it; ++it) {
        HG_DKV_TICK(t0);
        if (it + 1 < n_it) { ok = issue_s(it + 1); if (!ok) break; }
        HG_DKV_TOCK(tm_s, t0);
        if (!mbar_wait_warp(ds_full, it & 1, p.status, kTimeoutOther, abort_flag)) { ok = false; break; }
        tc_fence_after();
        HG_DKV_TOCK(tm_wait_ds, t0);
        const uint32_t aK = smem_u32(sK + ks_d * L::kKV);
        if (issuer) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)   // k-step kk = keys 16kk..16kk+15 = 8 packed columns
            umma_f16_ts(tDQ, tDS[it & 1] + kk * 8, mnmajor_desc(aK, 128, kk), idesc_dq, (it | kk) != 0);
          umma_commit(&k_empty[ks_d]);
          umma_commit(&ds_empty[it & 1]);
        }
        __syncwarp();
        if (++ks_d == NK) ks_d = 0;
        HG_DKV_TOCK(tm_dq, t0);
      }
      HG_DKV_REPORT(32, n_it, tm_s, tm_wait_ds, tm_dq, tm_unused);
      if (!ok) *abort_flag = 1;
    }
  } else {
    const int wq = warp & 3;
    const int half = (warp - 2) >> 2;     // warpgroup: which CPT of the step's 128 key columns these threads own
    const int c0 = half * CPT;
    const int row = wq * 32 + lane_id();
    const uint32_t lane_off = uint32_t(wq * 32) << 16;
    const float sl2 = p.scale * kLog2e;
    const int srow = q0 + row;
    const int q_pos = p.q_pos0 + srow;
    float lse2 = INFINITY, dsum = 0.f;
    if (srow < p.Sq) {
      const size_t idx = (size_t(b) * p.nheads + h) * p.Sq + srow;
      lse2 = p.LSE[idx] * kLog2e;
      dsum = p.D[idx];
    }
    const float nlse2 = -lse2;
    bool ok = true;
    HG_DKV_TIMERS(tm_wait_s, tm_ld, tm_math, tm_st);
    for (int it = 0; it < n_it; ++it) {
      HG_DKV_TICK(t0);
      if (!mbar_wait_warp(s_full, it & 1, p.status, kTimeoutTmemFull, abort_flag)) { ok = false; break; }
      tc_fence_after();
      HG_DKV_TOCK(tm_wait_s, t0);
      float ds[CPT];
      {
        float sv[CPT];
#pragma unroll
        for (int c = 0; c < CPT / 32; ++c) {
          uint32_t r0[32], r1[32];
          tmem_ld32(tS + lane_off + c0 + c * 32, r0);
          tmem_ld32(tDP + lane_off + c0 + c * 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) { sv[c * 32 + i] = __uint_as_float(r0[i]); ds[c * 32 + i] = __uint_as_float(r1[i]); }
        }
        tc_fence_before();
        mbar_arrive_warp(s_empty);
        HG_DKV_TOCK(tm_ld, t0);
        const int kbase = it * 128 + c0;
        const bool need_mask = (p.causal && (p.k_pos0 + kbase + CPT - 1 > p.q_pos0 + q0)) || (kbase + CPT > p.Skv);
        if (!need_mask) {
#pragma unroll
          for (int i = 0; i < CPT; ++i) ds[i] = ex2(fmaf(sv[i], sl2, nlse2)) * (ds[i] - dsum);
        } else {
#pragma unroll
          for (int i = 0; i < CPT; ++i) {
            const bool dead = (kbase + i >= p.Skv) || (p.causal && (p.k_pos0 + kbase + i > q_pos));
            ds[i] = dead ? 0.f : ex2(fmaf(sv[i], sl2, nlse2)) * (ds[i] - dsum);
          }
        }
      }
      HG_DKV_TOCK(tm_math, t0);
      if (it >= 2) {   // this dS buffer was last read by the dQ product of step it-2
        if (!mbar_wait_warp(&ds_empty[it & 1], ((it >> 1) & 1) ^ 1, p.status, kTimeoutOther, abort_flag)) { ok = false; break; }
        tc_fence_after();
      }
      {
        uint32_t w[CPT / 2];
#pragma unroll
        for (int i = 0; i < CPT / 2; ++i) w[i] = pack_bf16(ds[2 * i], ds[2 * i + 1]);
        if constexpr (CPT == 64) tmem_st32(tDS[it & 1] + lane_off + half * (CPT / 2), w);
        else tmem_st16(tDS[it & 1] + lane_off + half * (CPT / 2), w);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive_warp(ds_full);
      HG_DKV_TOCK(tm_st, t0);
    }
    HG_DKV_REPORT(24, n_it, tm_wait_s, tm_ld, tm_math, tm_st);
    const int dqslot = p.dqmap.slot(h, p.qpg);
    hg_lp_t* dq = p.dQ + int64_t(srow) * p.dq_ss + int64_t(b) * p.dq_sb + int64_t(dqslot) * HD;
    if (n_it == 0) {
      if (srow < p.Sq) {
#pragma unroll
        for (int i = half; i < HD / 8; i += NWG) reinterpret_cast<uint4*>(dq)[i] = make_uint4(0, 0, 0, 0);
      }
    } else if (ok && !*abort_flag &&
               mbar_wait_warp(&ds_empty[(n_it - 1) & 1], ((n_it - 1) >> 1) & 1, p.status, kTimeoutOther, abort_flag)) {
      tc_fence_after();
#pragma unroll
      for (int c = half; c < HD / 32; c += NWG) {
        uint32_t r[32];
        tmem_ld32(tDQ + lane_off + c * 32, r);
        tmem_ld_wait();
        if (srow < p.Sq) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 u;
            u.x = pack_bf16(__uint_as_float(r[q * 8 + 0]) * p.scale, __uint_as_float(r[q * 8 + 1]) * p.scale);
            u.y = pack_bf16(__uint_as_float(r[q * 8 + 2]) * p.scale, __uint_as_float(r[q * 8 + 3]) * p.scale);
            u.z = pack_bf16(__uint_as_float(r[q * 8 + 4]) * p.scale, __uint_as_float(r[q * 8 + 5]) * p.scale);
            u.w = pack_bf16(__uint_as_float(r[q * 8 + 6]) * p.scale, __uint_as_float(r[q * 8 + 7]) * p.scale);
            reinterpret_cast<uint4*>(dq + c * 32)[q] = u;
          }
        }
      }
    } else {
      *abort_flag = 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace attn
}  // namespace hg

// ------------------------------------------------------------------------------------------------
// Host launchers
// ------------------------------------------------------------------------------------------------
using namespace hg::attn;

namespace {

// 4-D tensor map over (d, slot, s, b) of a bf16 tensor whose element (s, b, slot, d) sits at
// base + s*ss + b*sb + slot*hd + d.  Box = (64, 1, box_rows, 1).
int make_map(CUtensorMap* out, const void* base, int hd, int slots, int S, int B, int64_t ss, int64_t sb,
             int box_rows) {
  const uint64_t key[8] = {4, uint64_t(reinterpret_cast<uintptr_t>(base)), (uint64_t(uint32_t(hd)) << 32) | uint32_t(slots),
                           (uint64_t(uint32_t(S)) << 32) | uint32_t(B), uint64_t(ss), uint64_t(sb), uint64_t(box_rows), 0};
  if (const CUtensorMap* hit = hg_host::tmap_cache_find(key)) {
    *out = *hit;
    return 0;
  }
  auto enc = hg_host::get_encode_fn();
  if (enc == nullptr) return -2;
  cuuint64_t dims[4] = {cuuint64_t(hd), cuuint64_t(slots), cuuint64_t(S), cuuint64_t(B)};
  cuuint64_t strides[3] = {cuuint64_t(hd) * 2, cuuint64_t(ss) * 2, cuuint64_t(sb) * 2};
  cuuint32_t box[4] = {64, 1, cuuint32_t(box_rows), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (B == 1) strides[2] = strides[1] * cuuint64_t(S);  // any legal value; the coordinate is always 0
  CUresult r = enc(out, HG_TMAP_LP, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) hg_host::tmap_cache_store(key, *out);
  return r == CUDA_SUCCESS ? 0 : -(1000 + int(r));
}

// dK/dV kernel for head dim 128: 0 = 128-query steps with P^T / dS^T in tensor memory, 1 = 64-query steps staged
// through shared memory (kept for head dim 64 and for side-by-side timing).
int g_dkv_variant = 0;
// Forward kernel for head dim 128: 0 = two query tiles per CTA with P in tensor memory (sequences longer than one
// tile), 1 = one tile per CTA with P staged in shared memory (also what head dim 64 and single-tile calls use).
int g_fwd_variant = 0;

template <typename K>
int set_smem(K kernel, int bytes) {
  return int(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
}

}  // namespace

extern "C" {

// Tensor descriptor passed from Python: base pointer, strides (elements) over s and b, number of head
// slots in a token row, and the head->slot map (gs, hs, off).
struct HgAttnTensor {
  void* ptr;
  long long ss, sb;
  int slots;
  int gs, hs, off;
};

int hg_flash_fwd(const HgAttnTensor* q, const HgAttnTensor* k, const HgAttnTensor* v, const HgAttnTensor* o,
                 void* lse, int Sq, int Skv, int B, int nheads, int nkv, int hd, int causal, int q_pos0, int k_pos0,
                 float scale, void* stream) {
  if (hd != 64 && hd != 128) return -1;
  if (Sq <= 0 || Skv <= 0 || B <= 0) return 0;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_map(&tq, q->ptr, hd, q->slots, Sq, B, q->ss, q->sb, 128))) return rc;
  if ((rc = make_map(&tk, k->ptr, hd, k->slots, Skv, B, k->ss, k->sb, 128))) return rc;
  if ((rc = make_map(&tv, v->ptr, hd, v->slots, Skv, B, v->ss, v->sb, 128))) return rc;
  FwdParams p{};
  p.Sq = Sq; p.Skv = Skv; p.B = B; p.nheads = nheads; p.qpg = nheads / nkv; p.causal = causal;
  p.q_pos0 = q_pos0; p.k_pos0 = k_pos0; p.scale = scale;
  p.qmap = {q->gs, q->hs, q->off}; p.kmap = {k->gs, k->hs, k->off}; p.vmap = {v->gs, v->hs, v->off};
  p.O = reinterpret_cast<hg_lp_t*>(o->ptr); p.o_ss = o->ss; p.o_sb = o->sb;
  p.LSE = reinterpret_cast<float*>(lse);
  p.status = hg_host::status_ptr();
  dim3 grid((Sq + 127) / 128, nheads, B);
  cudaStream_t st = (cudaStream_t)stream;
  if (hd == 128 && Sq > 128 && g_fwd_variant == 0) {   // two query tiles per CTA, P in tensor memory
    static bool cfg = false;
    if (!cfg) { if ((rc = set_smem(flash_fwd2_kernel<128>, Fwd2Smem<128>::kTotal))) return rc; cfg = true; }
    dim3 grid2((Sq + 255) / 256, nheads, B);
    flash_fwd2_kernel<128><<<grid2, 320, Fwd2Smem<128>::kTotal, st>>>(tq, tk, tv, p);
  } else if (hd == 128) {
    static bool cfg = false;
    if (!cfg) { if ((rc = set_smem(flash_fwd_kernel<128>, FwdSmem<128>::kTotal))) return rc; cfg = true; }
    flash_fwd_kernel<128><<<grid, kThreads, FwdSmem<128>::kTotal, st>>>(tq, tk, tv, p);
  } else {
    static bool cfg = false;
    if (!cfg) { if ((rc = set_smem(flash_fwd_kernel<64>, FwdSmem<64>::kTotal))) return rc; cfg = true; }
    flash_fwd_kernel<64><<<grid, kThreads, FwdSmem<64>::kTotal, st>>>(tq, tk, tv, p);
  }
  return int(cudaGetLastError());
}

// Selects the forward kernel used for head dim 128 (see g_fwd_variant); returns the previous value.
int hg_attn_set_fwd_variant(int v) {
  const int old = g_fwd_variant;
  g_fwd_variant = v ? 1 : 0;
  return old;
}

// Selects the dK/dV kernel used for head dim 128 (see g_dkv_variant); returns the previous value.
int hg_attn_set_dkv_variant(int v) {
  const int old = g_dkv_variant;
  g_dkv_variant = v ? 1 : 0;
  return old;
}

// dsum: scratch [B, nheads, Sq] fp32 (filled here with rowsum(dO*O)).
int hg_flash_bwd(const HgAttnTensor* q, const HgAttnTensor* k, const HgAttnTensor* v, const HgAttnTensor* o,
                 const HgAttnTensor* d_o, const void* lse, void* dsum, const HgAttnTensor* dq, const HgAttnTensor* dk,
                 const HgAttnTensor* dv, int Sq, int Skv, int B, int nheads, int nkv, int hd, int causal, int q_pos0,
                 int k_pos0, float scale, void* stream) {
  if (hd != 64 && hd != 128) return -1;
  if (Sq <= 0 || Skv <= 0 || B <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  int rc;
  {
    const int64_t warps = int64_t(Sq) * B * nheads;
    const int blocks = int((warps * 32 + 255) / 256);
    attn_bwd_dot_kernel<<<blocks, 256, 0, st>>>((const hg_lp_t*)o->ptr, (const hg_lp_t*)d_o->ptr, o->ss,
                                                o->sb, d_o->ss, d_o->sb, Sq, B, nheads, hd, (float*)dsum);
  }
  BwdParams p{};
  p.Sq = Sq; p.Skv = Skv; p.B = B; p.nheads = nheads; p.qpg = nheads / nkv; p.causal = causal;
  p.q_pos0 = q_pos0; p.k_pos0 = k_pos0; p.scale = scale;
  p.qmap = {q->gs, q->hs, q->off}; p.kmap = {k->gs, k->hs, k->off}; p.vmap = {v->gs, v->hs, v->off};
  p.domap = {d_o->gs, d_o->hs, d_o->off};
  p.LSE = (const float*)lse; p.D = (const float*)dsum;
  p.dQ = (hg_lp_t*)dq->ptr; p.dq_ss = dq->ss; p.dq_sb = dq->sb; p.dqmap = {dq->gs, dq->hs, dq->off};
  p.dK = (hg_lp_t*)dk->ptr; p.dk_ss = dk->ss; p.dk_sb = dk->sb; p.dkmap = {dk->gs, dk->hs, dk->off};
  p.dV = (hg_lp_t*)dv->ptr; p.dv_ss = dv->ss; p.dv_sb = dv->sb; p.dvmap = {dv->gs, dv->hs, dv->off};
  p.status = hg_host::status_ptr();
  {
    CUtensorMap tq, tk, tv, tdo;
    const bool wide = (hd == 128) && g_dkv_variant == 0;   // 128-query steps, P^T / dS^T in tensor memory
    const int q_rows = wide ? 128 : 64;
    if ((rc = make_map(&tq, q->ptr, hd, q->slots, Sq, B, q->ss, q->sb, q_rows))) return rc;
    if ((rc = make_map(&tk, k->ptr, hd, k->slots, Skv, B, k->ss, k->sb, 128))) return rc;
    if ((rc = make_map(&tv, v->ptr, hd, v->slots, Skv, B, v->ss, v->sb, 128))) return rc;
    if ((rc = make_map(&tdo, d_o->ptr, hd, d_o->slots, Sq, B, d_o->ss, d_o->sb, q_rows))) return rc;
    dim3 grid((Skv + 127) / 128, nkv, B);
    if (wide) {
      static bool cfg = false;
      if (!cfg) { if ((rc = set_smem(flash_bwd_dkv128_kernel<128, kDkvWarpgroups>, Dkv128Smem<128>::kTotal))) return rc; cfg = true; }
      flash_bwd_dkv128_kernel<128, kDkvWarpgroups><<<grid, 64 + 128 * kDkvWarpgroups, Dkv128Smem<128>::kTotal, st>>>(tq, tk, tv, tdo, p);
    } else if (hd == 128) {
      static bool cfg = false;
      if (!cfg) { if ((rc = set_smem(flash_bwd_dkv_kernel<128>, DkvSmem<128>::kTotal))) return rc; cfg = true; }
      flash_bwd_dkv_kernel<128><<<grid, kBwdThreads, DkvSmem<128>::kTotal, st>>>(tq, tk, tv, tdo, p);
    } else {
      static bool cfg = false;
      if (!cfg) { if ((rc = set_smem(flash_bwd_dkv_kernel<64>, DkvSmem<64>::kTotal))) return rc; cfg = true; }
      flash_bwd_dkv_kernel<64><<<grid, kBwdThreads, DkvSmem<64>::kTotal, st>>>(tq, tk, tv, tdo, p);
    }
  }
  {
    CUtensorMap tq, tk, tv, tdo;
    const int kv_rows = (hd == 128) ? 128 : 64;   // keys per step of the dQ kernel
    if ((rc = make_map(&tq, q->ptr, hd, q->slots, Sq, B, q->ss, q->sb, 128))) return rc;
    if ((rc = make_map(&tk, k->ptr, hd, k->slots, Skv, B, k->ss, k->sb, kv_rows))) return rc;
    if ((rc = make_map(&tv, v->ptr, hd, v->slots, Skv, B, v->ss, v->sb, kv_rows))) return rc;
    if ((rc = make_map(&tdo, d_o->ptr, hd, d_o->slots, Sq, B, d_o->ss, d_o->sb, 128))) return rc;
    dim3 grid((Sq + 127) / 128, nheads, B);
    if (hd == 128) {
      static bool cfg = false;
      if (!cfg) { if ((rc = set_smem(flash_bwd_dq128_kernel<128, kDqWarpgroups>, Dq128Smem<128>::kTotal))) return rc; cfg = true; }
      flash_bwd_dq128_kernel<128, kDqWarpgroups><<<grid, 64 + 128 * kDqWarpgroups, Dq128Smem<128>::kTotal, st>>>(tq, tk, tv, tdo, p);
    } else {
      static bool cfg = false;
      if (!cfg) { if ((rc = set_smem(flash_bwd_dq_kernel<64>, DqSmem<64>::kTotal))) return rc; cfg = true; }
      flash_bwd_dq_kernel<64><<<grid, kBwdThreads, DqSmem<64>::kTotal, st>>>(tq, tk, tv, tdo, p);
    }
  }
  return int(cudaGetLastError());
}

}  // extern "C"
