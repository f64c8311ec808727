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

template <typename T>
__global__ void sumsq_partial_kernel(const T* __restrict__ x, int64_t n, float* __restrict__ partial) {
  float s = 0.f;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
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
__global__ void scale_kernel(T* __restrict__ x, int64_t n, const float* __restrict__ coef, float host_coef) {
  const float c = (coef ? *coef : 1.f) * host_coef;
  if (c == 1.f) return;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
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
  if (g > 0) {
    if (is_bf16) sumsq_partial_kernel<hg_lp_t><<<g, 256, 0, st>>>((const hg_lp_t*)x, n, (float*)partial);
    else sumsq_partial_kernel<float><<<g, 256, 0, st>>>((const float*)x, n, (float*)partial);
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
  if (is_bf16) scale_kernel<hg_lp_t><<<grid_for(n), 256, 0, st>>>((hg_lp_t*)x, n, (const float*)coef, host_coef);
  else scale_kernel<float><<<grid_for(n), 256, 0, st>>>((float*)x, n, (const float*)coef, host_coef);
  return int(cudaGetLastError());
}

}  // extern "C"
