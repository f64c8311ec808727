// ZeRO data-parallel hot path over NVLink peer memory: two kernels that replace
// "NCCL reduce-scatter -> AdamW -> NCCL all-gather" on the flat gradient / parameter buffers of a wrap unit.
//
//   zero_reduce_scatter_kernel   out[i] = sum_r grad_r[me*S + i]          every rank's fp32 gradient buffer is read
//                                                                          through its peer mapping (16-byte loads,
//                                                                          all ranks' loads of an element group in
//                                                                          flight together)
//   zero_adamw_allgather_kernel  AdamW on this rank's shard (fp32 master weights and moments), then the updated
//                                bf16 values are stored straight into every rank's parameter buffer at this
//                                shard's offset (16-byte peer stores) -- the all-gather happens in the epilogue
//
// The fp32-wire reduce-scatter and the AdamW kernel never wait on another GPU: the callers order them against the
// peers' work with stream-ordered collectives (a one-element all-reduce before the first and after the second).
// The bf16-wire reduce-scatter carries its own rendezvous: it publishes "my staged gradients are complete" in every
// peer's signal slots and waits, with a 2-second limit that reports through the status word, for the peers' signals
// of the same epoch, so a whole unit's reduction is two launches (round, reduce) with no library collective.
// Buffers that peers touch must come from one symmetric allocation per rank.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "peer_rendezvous.cuh"

namespace {

constexpr int kMaxPeers = 8;
constexpr int kThreads = 256;

struct PeerPtrs {
  void* p[kMaxPeers];
};

struct AdamHyper {
  float lr, beta1, beta2, eps, weight_decay, bias1, bias2;
};

inline int grid_for(long long groups) {
  long long g = (groups + kThreads - 1) / kThreads;
  const long long cap = 148LL * 8;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return int(g);
}

// n4 = number of float4 groups of the shard.  T is the rank count (compile-time so that all T loads of a group are
// issued before the first add).
template <int T>
__global__ void __launch_bounds__(kThreads)
zero_reduce_scatter_kernel(PeerPtrs grads, int me, long long shard_floats, long long n4, float4* __restrict__ out) {
  const float4* src[T];
#pragma unroll
  for (int r = 0; r < T; ++r) {
    src[r] = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + me * shard_floats);
  }
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (; i + stride < n4; i += 2 * stride) {
    float4 a[T], b[T];
#pragma unroll
    for (int r = 0; r < T; ++r) a[r] = __ldcs(src[r] + i);
#pragma unroll
    for (int r = 0; r < T; ++r) b[r] = __ldcs(src[r] + i + stride);
    // fixed summation order (rank 0, 1, ...): deterministic
    float4 sa = make_float4(0.f, 0.f, 0.f, 0.f), sb = sa;
#pragma unroll
    for (int r = 0; r < T; ++r) {
      sa.x += a[r].x; sa.y += a[r].y; sa.z += a[r].z; sa.w += a[r].w;
      sb.x += b[r].x; sb.y += b[r].y; sb.z += b[r].z; sb.w += b[r].w;
    }
    out[i] = sa;
    out[i + stride] = sb;
  }
  for (; i < n4; i += stride) {
    float4 a[T];
#pragma unroll
    for (int r = 0; r < T; ++r) a[r] = __ldcs(src[r] + i);
    float4 sa = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < T; ++r) {
      sa.x += a[r].x; sa.y += a[r].y; sa.z += a[r].z; sa.w += a[r].w;
    }
    out[i] = sa;
  }
}


// bf16-on-the-wire variant (the reference's default, reduce_in_fp32 = false): every rank first rounds its fp32
// gradient buffer into a bf16 staging buffer (symmetric memory); this kernel then sums, in fp32 and in rank order,
// the peers' bf16 slices (16-byte loads of 8 values: half the NVLink bytes of the fp32 kernel) and this rank's own
// slice taken from the fp32 buffer, unrounded.  n8 = number of 8-element groups of the shard.  With kAcc the
// result is added to `out` (running shard of the per-micro-batch reduction mode).  U groups per thread and
// iteration keep (T - 1) * U peer loads of 16 bytes in flight per thread.
template <int T, bool kAcc, int U>
__global__ void __launch_bounds__(kThreads)
zero_reduce_scatter_bf16wire_kernel(PeerPtrs staged, const float* __restrict__ own, int me, long long shard_elems,
                                    long long n8, float4* __restrict__ out, hg::Rendezvous rv) {
  if (!hg::rendezvous(rv)) return;
  const uint4* src[T];
#pragma unroll
  for (int r = 0; r < T; ++r) {
    src[r] = reinterpret_cast<const uint4*>(reinterpret_cast<const hg_lp_t*>(staged.p[r]) + me * shard_elems);
  }
  const float4* mine = reinterpret_cast<const float4*>(own + me * shard_elems);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < n8; i0 += U * stride) {
    uint4 a[U][T];
    float4 m0[U], m1[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < n8) {
#pragma unroll
        for (int r = 0; r < T; ++r)
          if (r != me) a[u][r] = __ldcs(src[r] + i);
        m0[u] = __ldcs(mine + 2 * i);
        m1[u] = __ldcs(mine + 2 * i + 1);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= n8) continue;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < T; ++r) {   // fixed summation order (rank 0, 1, ...): deterministic
        if (r == me) {
          acc[0] += m0[u].x; acc[1] += m0[u].y; acc[2] += m0[u].z; acc[3] += m0[u].w;
          acc[4] += m1[u].x; acc[5] += m1[u].y; acc[6] += m1[u].z; acc[7] += m1[u].w;
        } else {
          const uint32_t w[4] = {a[u][r].x, a[u][r].y, a[u][r].z, a[u][r].w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 f = hg_unpack2(w[k]);
            acc[2 * k] += f.x;
            acc[2 * k + 1] += f.y;
          }
        }
      }
      float4 o0 = make_float4(acc[0], acc[1], acc[2], acc[3]), o1 = make_float4(acc[4], acc[5], acc[6], acc[7]);
      if (kAcc) {
        const float4 p0 = out[2 * i], p1 = out[2 * i + 1];
        o0.x += p0.x; o0.y += p0.y; o0.z += p0.z; o0.w += p0.w;
        o1.x += p1.x; o1.y += p1.y; o1.z += p1.z; o1.w += p1.w;
      }
      out[2 * i] = o0;
      out[2 * i + 1] = o1;
    }
  }
}

// out[i] += x[i] on float4 groups (running shard of the per-micro-batch reduction mode, fp32 wire).
__global__ void __launch_bounds__(kThreads) add_inplace_kernel(float4* __restrict__ out, const float4* __restrict__ x, long long n4) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 a = out[i];
    const float4 b = __ldcs(x + i);
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    out[i] = a;
  }
}

__device__ __forceinline__ float adam_one(float& p, float g, float& m, float& v, const AdamHyper& a, float step,
                                          float inv_b2) {
  m = a.beta1 * m + (1.f - a.beta1) * g;
  v = a.beta2 * v + (1.f - a.beta2) * g * g;
  p -= a.lr * a.weight_decay * p;
  p -= step * m / (sqrtf(v) * inv_b2 + a.eps);
  return p;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  hg_lp2_t h = hg_ff2lp2(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// n8 = number of 8-element groups of the shard.  `params.p[r]` is rank r's bf16 parameter buffer; the shard's
// values land at element offset `dst_off` in each of the `t_out` buffers.
__global__ void __launch_bounds__(kThreads)
zero_adamw_allgather_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                            float* __restrict__ v, PeerPtrs params, int t_out, long long dst_off, long long n8,
                            AdamHyper a, const float* __restrict__ gscale, const int* __restrict__ skip) {
  if (skip != nullptr && *skip != 0) return;
  const float gs = gscale ? *gscale : 1.f;
  const float step = a.lr / a.bias1;
  const float inv_b2 = rsqrtf(a.bias2);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += stride) {
    float4 pv[2], gv[2], mv[2], vv[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      pv[h] = reinterpret_cast<const float4*>(p)[2 * i + h];
      gv[h] = __ldcs(reinterpret_cast<const float4*>(g) + 2 * i + h);
      mv[h] = reinterpret_cast<const float4*>(m)[2 * i + h];
      vv[h] = reinterpret_cast<const float4*>(v)[2 * i + h];
    }
    uint4 packed;
    uint32_t w[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float x0 = adam_one(pv[h].x, gv[h].x * gs, mv[h].x, vv[h].x, a, step, inv_b2);
      const float x1 = adam_one(pv[h].y, gv[h].y * gs, mv[h].y, vv[h].y, a, step, inv_b2);
      const float x2 = adam_one(pv[h].z, gv[h].z * gs, mv[h].z, vv[h].z, a, step, inv_b2);
      const float x3 = adam_one(pv[h].w, gv[h].w * gs, mv[h].w, vv[h].w, a, step, inv_b2);
      w[2 * h] = pack2(x0, x1);
      w[2 * h + 1] = pack2(x2, x3);
      reinterpret_cast<float4*>(p)[2 * i + h] = pv[h];
      reinterpret_cast<float4*>(m)[2 * i + h] = mv[h];
      reinterpret_cast<float4*>(v)[2 * i + h] = vv[h];
    }
    packed = make_uint4(w[0], w[1], w[2], w[3]);
    for (int r = 0; r < t_out; ++r) {
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<hg_lp_t*>(params.p[r]) + dst_off) + i;
      *dst = packed;
    }
  }
  // peer stores must be visible system-wide before the kernel is reported complete to the ordering collective
  __threadfence_system();
}

}  // namespace

extern "C" {

// grads[r]: rank r's fp32 gradient buffer (t * shard_floats elements, peer-mapped).  out: this rank's reduced shard.
// shard_floats must be a multiple of 4 and every buffer 16-byte aligned.
int hg_zero_reduce_scatter_capped(void* const* grads, int t, int me, long long shard_floats, void* out, int max_ctas,
                                  void* stream);
int hg_zero_reduce_scatter(void* const* grads, int t, int me, long long shard_floats, void* out, void* stream) {
  return hg_zero_reduce_scatter_capped(grads, t, me, shard_floats, out, 0, stream);
}
// As above with the grid capped at max_ctas blocks (0 = no cap), for a reduction that overlaps the backward GEMMs.
int hg_zero_reduce_scatter_capped(void* const* grads, int t, int me, long long shard_floats, void* out, int max_ctas,
                                  void* stream) {
  if (t < 1 || t > kMaxPeers || me < 0 || me >= t || shard_floats <= 0 || (shard_floats & 3)) return -1;
  PeerPtrs pp{};
  for (int r = 0; r < t; ++r) pp.p[r] = grads[r];
  const long long n4 = shard_floats / 4;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int grid = grid_for((n4 + 1) / 2);
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
#define HG_RS(T_) zero_reduce_scatter_kernel<T_><<<grid, kThreads, 0, st>>>(pp, me, shard_floats, n4, (float4*)out)
  switch (t) {
    case 1: HG_RS(1); break;
    case 2: HG_RS(2); break;
    case 3: HG_RS(3); break;
    case 4: HG_RS(4); break;
    case 5: HG_RS(5); break;
    case 6: HG_RS(6); break;
    case 7: HG_RS(7); break;
    default: HG_RS(8); break;
  }
#undef HG_RS
  return int(cudaGetLastError());
}


// bf16 wire: staged[r] = rank r's bf16 staging buffer (t * shard elements, peer-mapped); own = this rank's fp32
// gradient buffer (local).  shard a multiple of 8.  max_ctas > 0 caps the grid (a reduction that runs beside the
// backward GEMMs should not take every SM).  accumulate != 0: out += sum.
// signals[r] = rank r's int[8] signal array (symmetric) and epoch > 0: the kernel does the cross-rank rendezvous
// itself (epoch must increase by one per call on every rank of the group); signals == null or epoch == 0: the
// caller has already ordered the ranks (every rank's staging buffer is complete and visible).
int hg_zero_reduce_scatter_bf16wire(void* const* staged, const void* own, int t, int me, long long shard, void* out,
                                    int accumulate, int max_ctas, void* const* signals, int epoch, void* stream) {
  if (t < 1 || t > kMaxPeers || me < 0 || me >= t || shard <= 0 || (shard & 7) || own == nullptr) return -1;
  PeerPtrs pp{};
  for (int r = 0; r < t; ++r) pp.p[r] = staged[r];
  const hg::Rendezvous rv = hg_host::make_rendezvous(signals, epoch, t, me);
  const long long n8 = shard / 8;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int grid = grid_for(n8);
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
#define HG_RSB(T_, U_)                                                                                              \
  if (accumulate)                                                                                                   \
    zero_reduce_scatter_bf16wire_kernel<T_, true, U_><<<grid, kThreads, 0, st>>>(pp, (const float*)own, me, shard, n8, (float4*)out, rv); \
  else                                                                                                              \
    zero_reduce_scatter_bf16wire_kernel<T_, false, U_><<<grid, kThreads, 0, st>>>(pp, (const float*)own, me, shard, n8, (float4*)out, rv)
  switch (t) {
    case 1: HG_RSB(1, 4); break;
    case 2: HG_RSB(2, 4); break;
    case 3: HG_RSB(3, 2); break;
    case 4: HG_RSB(4, 2); break;
    case 5: HG_RSB(5, 2); break;
    case 6: HG_RSB(6, 1); break;
    case 7: HG_RSB(7, 1); break;
    default: HG_RSB(8, 1); break;
  }
#undef HG_RSB
  return int(cudaGetLastError());
}

// out[0:n] += x[0:n] (fp32, n a multiple of 4, both 16-byte aligned).
int hg_add_inplace_f32(void* out, const void* x, long long n, void* stream) {
  if (n <= 0) return 0;
  if (n & 3) return -1;
  add_inplace_kernel<<<grid_for(n / 4), kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>((float4*)out, (const float4*)x, n / 4);
  return int(cudaGetLastError());
}

// AdamW on n elements (multiple of 8) of fp32 state; bf16 results stored at element offset dst_off of each of the
// t_out buffers in params (peer-mapped parameter buffers, or just the local one).
int hg_zero_adamw_allgather(void* p, const void* g, void* m, void* v, void* const* params, int t_out,
                            long long dst_off, long long n, float lr, float beta1, float beta2, float eps,
                            float weight_decay, int step, const void* gscale, const void* skip, void* stream) {
  if (n <= 0) return 0;
  if (t_out < 1 || t_out > kMaxPeers || (n & 7) || (dst_off & 7)) return -1;
  PeerPtrs pp{};
  for (int r = 0; r < t_out; ++r) pp.p[r] = params[r];
  AdamHyper a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bias1 = 1.f - powf(beta1, float(step));
  a.bias2 = 1.f - powf(beta2, float(step));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  zero_adamw_allgather_kernel<<<grid_for(n / 8), kThreads, 0, st>>>((float*)p, (const float*)g, (float*)m, (float*)v, pp,
                                                                    t_out, dst_off, n / 8, a, (const float*)gscale,
                                                                    (const int*)skip);
  return int(cudaGetLastError());
}

}  // extern "C"
