// Vocab-parallel cross-entropy, tiled over the local vocabulary shard; fp32 statistics only,
// fp32 logits are never materialised.  Forward produces per-token (max, sum-exp, target logit) of the
// local shard; the caller combines shards (MAX / SUM over the vocab-parallel group) and calls the
// backward, which overwrites the bf16 logits in place with (softmax - onehot) * g.
// Oracle: galvatron/core/runtime/transformer/fused_kernels.py:259-503 and the Triton kernels of
// galvatron/core/runtime/tensor_parallel/triton_cross_entropy.py:21-143.
#include "sm100_common.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const hg_lp2_t* p = reinterpret_cast<const hg_lp2_t*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = hg_lp22ff(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__global__ void __launch_bounds__(kThreads)
xent_stats_kernel(const hg_lp_t* __restrict__ logits, int64_t pitch, const int64_t* __restrict__ targets,
                  int v0, int V, float* __restrict__ out_max, float* __restrict__ out_sum,
                  float* __restrict__ out_pred, int rows) {
  __shared__ float sm[kThreads / 32], ss[kThreads / 32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const hg_lp_t* x = logits + size_t(row) * pitch;
    const int nvec = V >> 3;
    float m = -INFINITY, s = 0.f;
    for (int c = threadIdx.x; c < nvec; c += kThreads) {
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(x)[c], f);
      float cm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) cm = fmaxf(cm, f[j]);
      if (cm > m) { s *= __expf(m - cm); m = cm; }
#pragma unroll
      for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
    }
    for (int k = (nvec << 3) + threadIdx.x; k < V; k += kThreads) {  // ragged tail
      const float f = hg_lp2f(x[k]);
      if (f > m) { s *= __expf(m - f); m = f; }
      s += __expf(f - m);
    }
    // combine (m, s) across the block
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
      const float nm = fmaxf(m, om);
      s = (nm == -INFINITY) ? 0.f : s * __expf(m - nm) + os * __expf(om - nm);
      m = nm;
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) { sm[w] = m; ss[w] = s; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float M = sm[0], S = ss[0];
      for (int i = 1; i < kThreads / 32; ++i) {
        const float nm = fmaxf(M, sm[i]);
        S = (nm == -INFINITY) ? 0.f : S * __expf(M - nm) + ss[i] * __expf(sm[i] - nm);
        M = nm;
      }
      out_max[row] = M;
      out_sum[row] = S;
      const int64_t t = targets[row] - v0;
      out_pred[row] = (t >= 0 && t < V) ? hg_lp2f(x[t]) : 0.f;
    }
  }
}

// logits[row, v] <- (exp(x - gmax[row]) / gsum[row] - [v == target - v0]) * g[row]
__global__ void __launch_bounds__(kThreads)
xent_bwd_kernel(hg_lp_t* __restrict__ logits, int64_t pitch, const int64_t* __restrict__ targets, int v0, int V,
                const float* __restrict__ gmax, const float* __restrict__ gsum, const float* __restrict__ g,
                int rows) {
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    hg_lp_t* x = logits + size_t(row) * pitch;
    const float m = gmax[row], inv = 1.f / gsum[row], gr = g[row];
    const int64_t t = targets[row] - v0;
    const int nvec = V >> 3;
    for (int c = threadIdx.x; c < nvec; c += kThreads) {
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(x)[c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float p = __expf(f[j] - m) * inv;
        if (c * 8 + j == t) p -= 1.f;
        f[j] = p * gr;
      }
      uint4 u;
      u.x = hg::pack_bf16(f[0], f[1]);
      u.y = hg::pack_bf16(f[2], f[3]);
      u.z = hg::pack_bf16(f[4], f[5]);
      u.w = hg::pack_bf16(f[6], f[7]);
      reinterpret_cast<uint4*>(x)[c] = u;
    }
    for (int k = (nvec << 3) + threadIdx.x; k < V; k += kThreads) {
      float p = __expf(hg_lp2f(x[k]) - m) * inv;
      if (k == t) p -= 1.f;
      x[k] = hg_f2lp(p * gr);
    }
  }
}

}  // namespace

extern "C" {

int hg_xent_stats(const void* logits, long long pitch, const void* targets, int v0, int V, void* out_max,
                  void* out_sum, void* out_pred, int rows, void* stream) {
  if (rows <= 0) return 0;
  if (pitch & 7) return -1;
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  xent_stats_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>((const hg_lp_t*)logits, pitch,
                                                                 (const int64_t*)targets, v0, V, (float*)out_max,
                                                                 (float*)out_sum, (float*)out_pred, rows);
  return int(cudaGetLastError());
}

int hg_xent_bwd(void* logits, long long pitch, const void* targets, int v0, int V, const void* gmax, const void* gsum,
                const void* g, int rows, void* stream) {
  if (rows <= 0) return 0;
  if (pitch & 7) return -1;
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  xent_bwd_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>((hg_lp_t*)logits, pitch, (const int64_t*)targets,
                                                               v0, V, (const float*)gmax, (const float*)gsum,
                                                               (const float*)g, rows);
  return int(cudaGetLastError());
}

}  // extern "C"
