// RMSNorm / LayerNorm forward and backward with the residual add fused in.
// Memory-bound: every element is read once with 16-byte accesses and kept in registers
// between the statistics pass and the normalisation pass.
// Replaces the flash-attn RMSNorm / DropoutAddLayerNorm extension calls of
// galvatron/core/runtime/transformer/norm.py:6-29.
#include "sm100_common.cuh"

namespace {

constexpr int kThreads = 256;
// per-thread 8-element chunks kept in registers: MAXV = 2 / 4 / 8 covers H <= 4096 / 8192 / 16384

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < kThreads / 32) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const hg_lp2_t* p = reinterpret_cast<const hg_lp2_t*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = hg_lp22ff(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  u.x = hg::pack_bf16(f[0], f[1]);
  u.y = hg::pack_bf16(f[2], f[3]);
  u.z = hg::pack_bf16(f[4], f[5]);
  u.w = hg::pack_bf16(f[6], f[7]);
  return u;
}

// y = norm(x + residual) * w (+ b);  h_out = x + residual (optional);  stats: rstd (and mean for LN).
template <bool RMS, int kMaxVec>
__global__ void __launch_bounds__(kThreads)
norm_fwd_kernel(const hg_lp_t* __restrict__ x, const hg_lp_t* __restrict__ residual,
                const hg_lp_t* __restrict__ w, const hg_lp_t* __restrict__ b,
                hg_lp_t* __restrict__ y, hg_lp_t* __restrict__ h_out, float* __restrict__ rstd_out,
                float* __restrict__ mean_out, int rows, int H, float eps) {
  __shared__ float red[kThreads / 32];
  const int nvec = H >> 3;
  // The next row's loads are issued before this row's reductions, so that a block always has a row in flight
  // across its __syncthreads (with one row per trip the memory system idles while the block reduces).
  uint4 xraw[kMaxVec], rraw[kMaxVec];
  auto fetch = [&](int row) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(row) * H);
    const uint4* rr = residual ? reinterpret_cast<const uint4*>(residual + size_t(row) * H) : nullptr;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = threadIdx.x + i * kThreads;
      if (c < nvec) {
        xraw[i] = xr[c];
        if (rr) rraw[i] = rr[c];
      }
    }
  };
  constexpr bool kPrefetch = kMaxVec <= 4;    // the widest rows keep too much in registers to hold a second row
  if (kPrefetch && int(blockIdx.x) < rows) fetch(blockIdx.x);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    if (!kPrefetch) fetch(row);
    float v[kMaxVec][8];
    float s = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = threadIdx.x + i * kThreads;
      if (c < nvec) {
        unpack8(xraw[i], v[i]);
        if (residual) {
          float r[8];
          unpack8(rraw[i], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += r[j];
          if (h_out) {
            // round the sum to bf16 so that the saved residual stream and the normalised value agree
            uint4 packed = pack8(v[i]);
            reinterpret_cast<uint4*>(h_out + size_t(row) * H)[c] = packed;
            unpack8(packed, v[i]);
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) { s += v[i][j]; s2 += v[i][j] * v[i][j]; }
      }
    }
    if (kPrefetch && row + int(gridDim.x) < rows) fetch(row + gridDim.x);
    float mean = 0.f, var;
    if (RMS) {
      var = block_sum(s2, red) / H;
    } else {
      mean = block_sum(s, red) / H;
      float d2 = 0.f;
#pragma unroll
      for (int i = 0; i < kMaxVec; ++i) {
        const int c = threadIdx.x + i * kThreads;
        if (c < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) { float d = v[i][j] - mean; d2 += d * d; }
        }
      }
      var = block_sum(d2, red) / H;
    }
    const float rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) {
      rstd_out[row] = rstd;
      if (!RMS && mean_out) mean_out[row] = mean;
    }
    uint4* yr = reinterpret_cast<uint4*>(y + size_t(row) * H);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = threadIdx.x + i * kThreads;
      if (c < nvec) {
        float wv[8], o[8];
        unpack8(reinterpret_cast<const uint4*>(w)[c], wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * wv[j];
        if (!RMS && b) {
          float bv[8];
          unpack8(reinterpret_cast<const uint4*>(b)[c], bv);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += bv[j];
        }
        yr[c] = pack8(o);
      }
    }
  }
}

// dx = rstd * (dy*w - xhat*mean(dy*w*xhat) [- mean(dy*w)]) (+ dres);  partial dw/db per CTA (fp32).
template <bool RMS, int kMaxVec>
__global__ void __launch_bounds__(kThreads)
norm_bwd_kernel(const hg_lp_t* __restrict__ dy, const hg_lp_t* __restrict__ h,
                const hg_lp_t* __restrict__ w, const float* __restrict__ rstd_in,
                const float* __restrict__ mean_in, const hg_lp_t* __restrict__ dres,
                hg_lp_t* __restrict__ dx, float* __restrict__ dw_partial, float* __restrict__ db_partial,
                int rows, int H) {
  __shared__ float red[kThreads / 32];
  const int nvec = H >> 3;
  float dw_acc[kMaxVec][8], db_acc[kMaxVec][8];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) { dw_acc[i][j] = 0.f; db_acc[i][j] = 0.f; }
  float wv[kMaxVec][8];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = threadIdx.x + i * kThreads;
    if (c < nvec) unpack8(reinterpret_cast<const uint4*>(w)[c], wv[i]);
  }
  // as in the forward: the next row's dy / h / dres are requested before this row's reductions
  constexpr bool kPrefetch = kMaxVec <= 4;
  uint4 dyraw[kMaxVec], hraw[kMaxVec], drraw[kMaxVec];
  auto fetch = [&](int row) {
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + size_t(row) * H);
    const uint4* hr = reinterpret_cast<const uint4*>(h + size_t(row) * H);
    const uint4* dr = dres ? reinterpret_cast<const uint4*>(dres + size_t(row) * H) : nullptr;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = threadIdx.x + i * kThreads;
      if (c < nvec) {
        dyraw[i] = dyr[c];
        hraw[i] = hr[c];
        if (kPrefetch && dr) drraw[i] = dr[c];
      }
    }
  };
  if (kPrefetch && int(blockIdx.x) < rows) fetch(blockIdx.x);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    if (!kPrefetch) fetch(row);
    const float rstd = rstd_in[row];
    const float mean = RMS ? 0.f : mean_in[row];
    float g[kMaxVec][8], xh[kMaxVec][8];
    uint4 drcur[kMaxVec];   // this row's residual gradient, packed (the prefetch below reuses drraw)
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = threadIdx.x + i * kThreads;
      if (c < nvec) {
        float d[8], hv[8];
        unpack8(dyraw[i], d);
        unpack8(hraw[i], hv);
        if (kPrefetch && dres) drcur[i] = drraw[i];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (hv[j] - mean) * rstd;
          dw_acc[i][j] += d[j] * xh[i][j];
          if (!RMS) db_acc[i][j] += d[j];
          g[i][j] = d[j] * wv[i][j];
          c1 += g[i][j] * xh[i][j];
          c2 += g[i][j];
        }
      }
    }
    if (kPrefetch && row + int(gridDim.x) < rows) fetch(row + gridDim.x);
    c1 = block_sum(c1, red) / H;
    c2 = RMS ? 0.f : block_sum(c2, red) / H;
    uint4* dxr = reinterpret_cast<uint4*>(dx + size_t(row) * H);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = threadIdx.x + i * kThreads;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - xh[i][j] * c1 - c2);
        if (dres) {
          float r[8];
          unpack8(kPrefetch ? drcur[i] : reinterpret_cast<const uint4*>(dres + size_t(row) * H)[c], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        dxr[c] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = threadIdx.x + i * kThreads;
    if (c < nvec) {
      float* dst = dw_partial + size_t(blockIdx.x) * H + c * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) dst[j] = dw_acc[i][j];
      if (!RMS && db_partial) {
        float* dstb = db_partial + size_t(blockIdx.x) * H + c * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) dstb[j] = db_acc[i][j];
      }
    }
  }
}

// out[c] (+)= sum_p partial[p, c]
__global__ void reduce_partials_kernel(const float* __restrict__ partial, float* __restrict__ out, int parts, int H,
                                       int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partial[size_t(p) * H + c];
  out[c] = accumulate ? out[c] + s : s;
}

}  // namespace

extern "C" {

// rms != 0 -> RMSNorm, else LayerNorm.  H must be a multiple of 8 and <= 16384.
int hg_norm_fwd(const void* x, const void* residual, const void* w, const void* b, void* y, void* h_out,
                void* rstd, void* mean, int rows, int H, float eps, int rms, void* stream) {
  if (rows <= 0) return 0;
  if ((H & 7) || H > kThreads * 8 * 8) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  auto X = reinterpret_cast<const hg_lp_t*>(x);
  auto R = reinterpret_cast<const hg_lp_t*>(residual);
  auto W = reinterpret_cast<const hg_lp_t*>(w);
  auto B = reinterpret_cast<const hg_lp_t*>(b);
  auto Y = reinterpret_cast<hg_lp_t*>(y);
  auto Ho = reinterpret_cast<hg_lp_t*>(h_out);
#define HG_FWD(R_, V_) norm_fwd_kernel<R_, V_><<<grid, kThreads, 0, st>>>(X, R, W, B, Y, Ho, (float*)rstd, (float*)mean, rows, H, eps)
  if (rms) { if (H <= 4096) HG_FWD(true, 2); else if (H <= 8192) HG_FWD(true, 4); else HG_FWD(true, 8); }
  else     { if (H <= 4096) HG_FWD(false, 2); else if (H <= 8192) HG_FWD(false, 4); else HG_FWD(false, 8); }
#undef HG_FWD
  return int(cudaGetLastError());
}

// `h` is the tensor that was normalised (x + residual).  `partial` is scratch of parts*H floats
// (and another parts*H for LayerNorm's bias gradient); dw/db are fp32 and are accumulated into when
// `accumulate` != 0.  Returns the number of partial rows used through *parts_used when non-null.
int hg_norm_bwd(const void* dy, const void* h, const void* w, const void* rstd, const void* mean, const void* dres,
                void* dx, void* dw, void* db, void* partial, int parts, int rows, int H, int rms, int accumulate,
                void* stream) {
  if (rows <= 0) return 0;
  if ((H & 7) || H > kThreads * 8 * 8 || parts <= 0) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = rows < parts ? rows : parts;
  float* P = reinterpret_cast<float*>(partial);
  float* PB = P + size_t(parts) * H;
#define HG_BWD(R_, V_)                                                                                              \
  norm_bwd_kernel<R_, V_><<<grid, kThreads, 0, st>>>((const hg_lp_t*)dy, (const hg_lp_t*)h,             \
                                                     (const hg_lp_t*)w, (const float*)rstd,                    \
                                                     (const float*)mean, (const hg_lp_t*)dres,                 \
                                                     (hg_lp_t*)dx, P, (R_) ? nullptr : PB, rows, H)
  if (rms) { if (H <= 4096) HG_BWD(true, 2); else if (H <= 8192) HG_BWD(true, 4); else HG_BWD(true, 8); }
  else     { if (H <= 4096) HG_BWD(false, 2); else if (H <= 8192) HG_BWD(false, 4); else HG_BWD(false, 8); }
#undef HG_BWD
  reduce_partials_kernel<<<(H + 255) / 256, 256, 0, st>>>(P, (float*)dw, grid, H, accumulate);
  if (!rms && db) reduce_partials_kernel<<<(H + 255) / 256, 256, 0, st>>>(PB, (float*)db, grid, H, accumulate);
  return int(cudaGetLastError());
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant of the norm backward (declared and documented in norm_noalloc.h)
// ---------------------------------------------------------------------------------------------------
#include "norm_noalloc.h"

#include <mutex>

namespace {

constexpr int kNoAllocMaxDevices = HG_NORM_NOALLOC_MAX_DEVICES;
constexpr size_t kNoAllocFloats = size_t(2) * HG_NORM_NOALLOC_PARTS * HG_NORM_NOALLOC_MAX_H;

// Per-CTA partial sums: rows [0, PARTS) for the weight gradient, rows [PARTS, 2*PARTS) for LayerNorm's bias
// gradient, each row H floats wide (H <= MAX_H).  One copy per device, shared by every call on that device.
static __device__ __align__(256) float g_norm_bwd_scratch[kNoAllocFloats];

float* g_scratch_addr[kNoAllocMaxDevices] = {};
std::mutex g_scratch_mu;

// Device address of the array on the current device.  In host code the array's name is only a handle for the
// runtime, not a device pointer, so the address is asked for once per device and cached.
int noalloc_scratch(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return -(1000 + int(e));
  if (dev < 0 || dev >= kNoAllocMaxDevices) return HG_NORM_NOALLOC_BAD_DEVICE;
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_norm_bwd_scratch);
    if (e != cudaSuccess || p == nullptr) return -(1000 + int(e));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" int hg_norm_bwd_noalloc(const void* dy, const void* h, const void* w, const void* rstd, const void* mean,
                                   const void* dres, void* dx, void* dw, void* db, int rows, int H, int rms,
                                   int accumulate, void* stream) {
  if (rows <= 0) return 0;
  if ((H & 7) || H <= 0) return -1;
  if (H > HG_NORM_NOALLOC_MAX_H) return HG_NORM_NOALLOC_TOO_WIDE;
  // a null required pointer would be dereferenced on the device: refuse before anything is launched
  if (!dy || !h || !w || !rstd || !dx || !dw || (!rms && !mean)) return HG_NORM_NOALLOC_NULL_ARG;
  float* P = nullptr;
  if (int rc = noalloc_scratch(&P)) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int parts = HG_NORM_NOALLOC_PARTS;
  const int grid = rows < parts ? rows : parts;
  float* PB = P + size_t(parts) * HG_NORM_NOALLOC_MAX_H;
#define HG_BWD_NA(R_, V_)                                                                                           \
  norm_bwd_kernel<R_, V_><<<grid, kThreads, 0, st>>>((const hg_lp_t*)dy, (const hg_lp_t*)h,             \
                                                     (const hg_lp_t*)w, (const float*)rstd,                    \
                                                     (const float*)mean, (const hg_lp_t*)dres,                 \
                                                     (hg_lp_t*)dx, P, (R_) ? nullptr : PB, rows, H)
  if (rms) { if (H <= 4096) HG_BWD_NA(true, 2); else HG_BWD_NA(true, 4); }
  else     { if (H <= 4096) HG_BWD_NA(false, 2); else HG_BWD_NA(false, 4); }
#undef HG_BWD_NA
  reduce_partials_kernel<<<(H + 255) / 256, 256, 0, st>>>(P, (float*)dw, grid, H, accumulate);
  if (!rms && db) reduce_partials_kernel<<<(H + 255) / 256, 256, 0, st>>>(PB, (float*)db, grid, H, accumulate);
  return int(cudaGetLastError());
}
