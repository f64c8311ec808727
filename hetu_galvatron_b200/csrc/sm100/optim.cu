// Optimizer-side kernels working on flat parameter buffers: fused AdamW (fp32 master weights and
// moments, bf16 working copy written in the same pass), squared-L2-norm reduction, and in-place
// scaling by a device-resident coefficient (gradient clipping without a host round trip).
// Replaces apex FusedAdam / multi_tensor_l2norm / multi_tensor_scale as used by
// galvatron/core/runtime/optimizer/utils.py:8-52 and optimizer/clip_grads.py:36-194.
#include "sm100_common.cuh"

namespace {

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias1, bias2;  // bias1 = 1 - beta1^t, bias2 = 1 - beta2^t
};

// grad may be fp32 or bf16; `gscale` (device, optional) multiplies the gradient (clip coefficient,
// 1/accumulation steps, loss-scale inverse).  If *skip (device, optional) is non-zero nothing is updated
// (overflow / rejected step).
template <typename GradT>
__global__ void adamw_kernel(float* __restrict__ p, const GradT* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, hg_lp_t* __restrict__ p_lp, int64_t n, AdamArgs a,
                             const float* __restrict__ gscale, const int* __restrict__ skip) {
  if (skip != nullptr && *skip != 0) return;
  const float gs = gscale ? *gscale : 1.f;
  const float step = a.lr / a.bias1;
  const float inv_b2 = rsqrtf(a.bias2);
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
    float gi;
    if constexpr (sizeof(GradT) == 2) gi = hg_lp2f(g[i]) * gs;
    else gi = float(g[i]) * gs;
    float pi = p[i];
    const float mi = a.beta1 * m[i] + (1.f - a.beta1) * gi;
    const float vi = a.beta2 * v[i] + (1.f - a.beta2) * gi * gi;
    pi -= a.lr * a.weight_decay * pi;  // decoupled weight decay
    pi -= step * mi / (sqrtf(vi) * inv_b2 + a.eps);
    m[i] = mi;
    v[i] = vi;
    p[i] = pi;
    if (p_lp) p_lp[i] = hg_f2lp(pi);
  }
}

__device__ __forceinline__ float adam_one(float& p, float g, float& m, float& v, const AdamArgs& a, float step,
                                          float inv_b2) {
  m = a.beta1 * m + (1.f - a.beta1) * g;
  v = a.beta2 * v + (1.f - a.beta2) * g * g;
  p -= a.lr * a.weight_decay * p;
  p -= step * m / (sqrtf(v) * inv_b2 + a.eps);
  return p;
}

template <typename GradT>
__device__ __forceinline__ float4 load_grad4(const GradT* g, int64_t i4) {
  if constexpr (sizeof(GradT) == 2) {
    const uint2 u = __ldcs(reinterpret_cast<const uint2*>(g) + i4);
    const float2 a = hg_lp22ff(*reinterpret_cast<const hg_lp2_t*>(&u.x));
    const float2 b = hg_lp22ff(*reinterpret_cast<const hg_lp2_t*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
  } else {
    return __ldcs(reinterpret_cast<const float4*>(g) + i4);
  }
}

// Same update on groups of four elements: 16-byte accesses, and the loads of two groups (eight 16-byte loads per
// thread) issued before the first dependent instruction.  n4 = number of whole groups; all pointers 16-byte aligned
// (the low-precision ones 8-byte).
template <typename GradT>
__global__ void __launch_bounds__(256)
adamw_vec_kernel(float* __restrict__ p, const GradT* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                 hg_lp_t* __restrict__ p_lp, int64_t n4, AdamArgs a, const float* __restrict__ gscale,
                 const int* __restrict__ skip) {
  if (skip != nullptr && *skip != 0) return;
  const float gs = gscale ? *gscale : 1.f;
  const float step = a.lr / a.bias1;
  const float inv_b2 = rsqrtf(a.bias2);
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  float4* p4 = reinterpret_cast<float4*>(p);
  float4* m4 = reinterpret_cast<float4*>(m);
  float4* v4 = reinterpret_cast<float4*>(v);
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n4; i += 2 * stride) {
    const int64_t idx[2] = {i, i + stride};
    const bool on[2] = {true, i + stride < n4};
    float4 pv[2], gv[2], mv[2], vv[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (on[h]) {
        pv[h] = p4[idx[h]];
        gv[h] = load_grad4<GradT>(g, idx[h]);
        mv[h] = m4[idx[h]];
        vv[h] = v4[idx[h]];
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (on[h]) {
        const float x0 = adam_one(pv[h].x, gv[h].x * gs, mv[h].x, vv[h].x, a, step, inv_b2);
        const float x1 = adam_one(pv[h].y, gv[h].y * gs, mv[h].y, vv[h].y, a, step, inv_b2);
        const float x2 = adam_one(pv[h].z, gv[h].z * gs, mv[h].z, vv[h].z, a, step, inv_b2);
        const float x3 = adam_one(pv[h].w, gv[h].w * gs, mv[h].w, vv[h].w, a, step, inv_b2);
        p4[idx[h]] = pv[h];
        m4[idx[h]] = mv[h];
        v4[idx[h]] = vv[h];
        if (p_lp) reinterpret_cast<uint2*>(p_lp)[idx[h]] = make_uint2(hg::pack_bf16(x0, x1), hg::pack_bf16(x2, x3));
      }
    }
  }
}

// x as groups of four (fp32) or eight (16-bit) elements, two groups in flight per thread; the caller adds the tail.
template <typename T>
__device__ __forceinline__ float sumsq_group(const T* x, int64_t i) {
  if constexpr (sizeof(T) == 2) {
    const uint4 u = reinterpret_cast<const uint4*>(x)[i];
    const hg_lp2_t* q = reinterpret_cast<const hg_lp2_t*>(&u);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = hg_lp22ff(q[j]);
      s += t.x * t.x + t.y * t.y;
    }
    return s;
  } else {
    const float4 f = reinterpret_cast<const float4*>(x)[i];
    return f.x * f.x + f.y * f.y + f.z * f.z + f.w * f.w;
  }
}

template <typename T>
__global__ void sumsq_partial_kernel(const T* __restrict__ x, int64_t n, float* __restrict__ partial, int vec) {
  float s = 0.f;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  const int64_t first = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  int64_t done = 0;
  if (vec) {
    constexpr int kPer = sizeof(T) == 2 ? 8 : 4;
    const int64_t groups = n / kPer;
    int64_t i = first;
    for (; i + stride < groups; i += 2 * stride) {
      const float a = sumsq_group<T>(x, i), b = sumsq_group<T>(x, i + stride);
      s += a + b;
    }
    if (i < groups) s += sumsq_group<T>(x, i);
    done = groups * kPer;
  }
  for (int64_t i = done + first; i < n; i += stride) {
    float f;
    if constexpr (sizeof(T) == 2) f = hg_lp2f(x[i]);
    else f = float(x[i]);
    s += f * f;
  }
  __shared__ float red[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) partial[blockIdx.x] = s;
  }
}

// out[0] = (accumulate ? out[0] : 0) + scale * sum(partial[0..parts))   -- fixed order, deterministic
__global__ void sumsq_final_kernel(const float* __restrict__ partial, int parts, float* __restrict__ out,
                                   int accumulate, float scale) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < parts; i += blockDim.x) s += partial[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < int(blockDim.x >> 5); ++i) t += red[i];
    out[0] = (accumulate ? out[0] : 0.f) + scale * t;
  }
}

// coef[0] = min(1, max_norm / (sqrt(sumsq[0]) + 1e-6)); norm_out[0] = sqrt(sumsq[0])
__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float max_norm, float* __restrict__ coef,
                                 float* __restrict__ norm_out) {
  const float nrm = sqrtf(sumsq[0]);
  if (norm_out) norm_out[0] = nrm;
  float c = max_norm / (nrm + 1e-6f);
  coef[0] = (max_norm > 0.f && c < 1.f) ? c : 1.f;
}

template <typename T>
__global__ void scale_kernel(T* __restrict__ x, int64_t n, const float* __restrict__ coef, float host_coef, int vec) {
  const float c = (coef ? *coef : 1.f) * host_coef;
  if (c == 1.f) return;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  const int64_t first = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  int64_t done = 0;
  if (vec) {                                 // 16-byte groups, base 16-byte aligned
    constexpr int kPer = sizeof(T) == 2 ? 8 : 4;
    const int64_t groups = n / kPer;
    for (int64_t i = first; i < groups; i += stride) {
      if constexpr (sizeof(T) == 2) {
        uint4 u = reinterpret_cast<uint4*>(x)[i];
        uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 t = hg_lp22ff(*reinterpret_cast<hg_lp2_t*>(&w[j]));
          w[j] = hg::pack_bf16(t.x * c, t.y * c);
        }
        reinterpret_cast<uint4*>(x)[i] = u;
      } else {
        float4 f = reinterpret_cast<float4*>(x)[i];
        f.x *= c; f.y *= c; f.z *= c; f.w *= c;
        reinterpret_cast<float4*>(x)[i] = f;
      }
    }
    done = groups * kPer;
  }
  for (int64_t i = done + first; i < n; i += stride) {
    if constexpr (sizeof(T) == 2) x[i] = hg_f2lp(hg_lp2f(x[i]) * c);
    else x[i] = T(float(x[i]) * c);
  }
}

inline int grid_for(int64_t n) {
  int64_t g = (n + 1023) / 1024;
  return int(g < 1 ? 1 : (g > 148 * 8 ? 148 * 8 : g));
}

}  // namespace

extern "C" {

int hg_adamw(void* p, const void* g, void* m, void* v, void* p_lp, long long n, int grad_is_bf16, float lr,
             float beta1, float beta2, float eps, float weight_decay, int step, const void* gscale, const void* skip,
             void* stream) {
  if (n <= 0) return 0;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bias1 = 1.f - powf(beta1, float(step));
  a.bias2 = 1.f - powf(beta2, float(step));
  cudaStream_t st = (cudaStream_t)stream;
  // whole groups of four through the 16-byte kernel when every pointer allows it; the scalar kernel takes the rest
  const bool aligned = ((uintptr_t(p) | uintptr_t(m) | uintptr_t(v)) & 15) == 0 &&
                       (uintptr_t(g) & (grad_is_bf16 ? 7 : 15)) == 0 && (uintptr_t(p_lp) & 7) == 0;
  const long long n4 = aligned ? n / 4 : 0;
  if (n4 > 0) {
    const int grid = grid_for(n4 * 2);   // two groups per thread and trip
    if (grad_is_bf16)
      adamw_vec_kernel<hg_lp_t><<<grid, 256, 0, st>>>((float*)p, (const hg_lp_t*)g, (float*)m, (float*)v, (hg_lp_t*)p_lp,
                                                      n4, a, (const float*)gscale, (const int*)skip);
    else
      adamw_vec_kernel<float><<<grid, 256, 0, st>>>((float*)p, (const float*)g, (float*)m, (float*)v, (hg_lp_t*)p_lp, n4,
                                                    a, (const float*)gscale, (const int*)skip);
    const long long done = n4 * 4;
    n -= done;
    if (n == 0) return int(cudaGetLastError());
    p = (float*)p + done; m = (float*)m + done; v = (float*)v + done;
    g = grad_is_bf16 ? (const void*)((const hg_lp_t*)g + done) : (const void*)((const float*)g + done);
    if (p_lp) p_lp = (hg_lp_t*)p_lp + done;
  }
  if (grad_is_bf16)
    adamw_kernel<hg_lp_t><<<grid_for(n), 256, 0, st>>>((float*)p, (const hg_lp_t*)g, (float*)m, (float*)v,
                                                             (hg_lp_t*)p_lp, n, a, (const float*)gscale,
                                                             (const int*)skip);
  else
    adamw_kernel<float><<<grid_for(n), 256, 0, st>>>((float*)p, (const float*)g, (float*)m, (float*)v,
                                                     (hg_lp_t*)p_lp, n, a, (const float*)gscale,
                                                     (const int*)skip);
  return int(cudaGetLastError());
}

// out[0] (+)= scale * sum(x^2).  `partial` is scratch of at least 1184 floats.
int hg_sumsq(const void* x, long long n, int is_bf16, void* partial, void* out, int accumulate, float scale,
             void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  const int g = n > 0 ? grid_for(n) : 0;
  const int vec = (uintptr_t(x) & 15) == 0;
  if (g > 0) {
    if (is_bf16) sumsq_partial_kernel<hg_lp_t><<<g, 256, 0, st>>>((const hg_lp_t*)x, n, (float*)partial, vec);
    else sumsq_partial_kernel<float><<<g, 256, 0, st>>>((const float*)x, n, (float*)partial, vec);
  }
  sumsq_final_kernel<<<1, 256, 0, st>>>((const float*)partial, g, (float*)out, accumulate, scale);
  return int(cudaGetLastError());
}

int hg_clip_coef(const void* sumsq, float max_norm, void* coef, void* norm_out, void* stream) {
  clip_coef_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((const float*)sumsq, max_norm, (float*)coef, (float*)norm_out);
  return int(cudaGetLastError());
}

int hg_scale(void* x, long long n, int is_bf16, const void* coef, float host_coef, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int vec = (uintptr_t(x) & 15) == 0;
  if (is_bf16) scale_kernel<hg_lp_t><<<grid_for(n), 256, 0, st>>>((hg_lp_t*)x, n, (const float*)coef, host_coef, vec);
  else scale_kernel<float><<<grid_for(n), 256, 0, st>>>((float*)x, n, (const float*)coef, host_coef, vec);
  return int(cudaGetLastError());
}

}  // extern "C"
