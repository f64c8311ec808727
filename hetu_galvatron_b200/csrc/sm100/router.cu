// Top-k router: scores, top-k selection, probabilities and per-expert statistics in one pass, one warp per token.
//
// Modes (logits fp32 [T, E], E <= 256, k <= 8):
//   0  softmax over the k selected logits            (top-k first, then softmax)          probs sum to 1
//   1  softmax over all experts, then top-k          ("pre-softmax")                      probs = selected scores
//   2  sigmoid scores, top-k (optionally on score + bias), normalised by their sum when k > 1
// Outputs: probs [T, k] fp32 (times `scaling`), idx [T, k] int32, scores [T, E] fp32 (full softmax / sigmoid, the
// quantity that load-balancing losses use), counts [E] fp32 += tokens routed to each expert.
// The backward kernel turns (dprobs, dscores) into dlogits with the same one-warp-per-token layout.
#include <cuda_runtime.h>

#include <cstdint>

namespace {

constexpr int kMaxPerLane = 8;  // E <= 256
constexpr int kMaxK = 8;
constexpr int kWarps = 8;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Warp arg-max over (value, index) pairs; ties go to the lower index (what torch.topk does for equal values is
// unspecified; a fixed rule keeps runs reproducible).
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

__global__ void __launch_bounds__(kWarps * 32)
router_fwd_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E, int k, int mode,
                  float scaling, float* __restrict__ probs, int* __restrict__ idx, float* __restrict__ scores,
                  float* __restrict__ counts) {
  const int lane = threadIdx.x & 31;
  const int tok = blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (tok >= T) return;
  const float* row = logits + size_t(tok) * E;
  float l[kMaxPerLane], s[kMaxPerLane], sel[kMaxPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const int e = lane + 32 * j;
    l[j] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, l[j]);
  }
  mx = warp_max(mx);
  float denom = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const int e = lane + 32 * j;
    if (mode == 2) s[j] = e < E ? 1.f / (1.f + __expf(-l[j])) : 0.f;
    else { s[j] = e < E ? __expf(l[j] - mx) : 0.f; denom += s[j]; }
  }
  if (mode != 2) {
    denom = warp_sum(denom);
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) s[j] /= denom;
  }
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const int e = lane + 32 * j;
    if (e < E) scores[size_t(tok) * E + e] = s[j];
    // selection key: raw logits for mode 0 (same order as their softmax), scores otherwise (+ bias for sigmoid)
    sel[j] = e < E ? (mode == 0 ? l[j] : (mode == 2 && bias ? s[j] + bias[e] : s[j])) : -INFINITY;
  }
  float pv[kMaxK];
  int pi[kMaxK];
  float psum = 0.f;
  for (int r = 0; r < k; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (sel[j] > bv || (sel[j] == bv && e < bi)) { bv = sel[j]; bi = e; }
    }
    warp_argmax(bv, bi);
    // value of the winner in the quantity the probability is built from
    float val = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (lane + 32 * j == bi) { val = (mode == 0) ? l[j] : s[j]; sel[j] = -INFINITY; }
    val = __shfl_sync(0xffffffffu, val, bi & 31);
    pv[r] = val;
    pi[r] = bi;
  }
  if (mode == 0) {  // softmax over the selected logits
    const float m0 = pv[0];
    for (int r = 0; r < k; ++r) { pv[r] = __expf(pv[r] - m0); psum += pv[r]; }
    for (int r = 0; r < k; ++r) pv[r] /= psum;
  } else if (mode == 2 && k > 1) {
    for (int r = 0; r < k; ++r) psum += pv[r];
    for (int r = 0; r < k; ++r) pv[r] /= (psum + 1e-20f);
  }
  if (lane < k) {
    // every lane holds all k results; lane r writes entry r
    float outv = 0.f;
    int outi = 0;
    for (int r = 0; r < k; ++r)
      if (r == lane) { outv = pv[r]; outi = pi[r]; }
    probs[size_t(tok) * k + lane] = outv * scaling;
    idx[size_t(tok) * k + lane] = outi;
    if (counts) atomicAdd(counts + outi, 1.f);
  }
}

// dlogits from dprobs [T, k] (gradient of the scaled probabilities) and dscores [T, E] (may be null).
__global__ void __launch_bounds__(kWarps * 32)
router_bwd_kernel(const float* __restrict__ scores, const float* __restrict__ probs, const int* __restrict__ idx,
                  const float* __restrict__ dprobs, const float* __restrict__ dscores, int T, int E, int k, int mode,
                  float scaling, float* __restrict__ dlogits) {
  const int lane = threadIdx.x & 31;
  const int tok = blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (tok >= T) return;
  float s[kMaxPerLane], g[kMaxPerLane];  // g: gradient w.r.t. the score (modes 1, 2) or directly the logit (mode 0)
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const int e = lane + 32 * j;
    s[j] = e < E ? scores[size_t(tok) * E + e] : 0.f;
    g[j] = (e < E && dscores) ? dscores[size_t(tok) * E + e] : 0.f;
  }
  float p[kMaxK], dp[kMaxK];
  int id[kMaxK];
  float dot = 0.f, ssum = 0.f;
  for (int r = 0; r < k; ++r) {
    p[r] = probs[size_t(tok) * k + r] / scaling;
    dp[r] = dprobs[size_t(tok) * k + r] * scaling;
    id[r] = idx[size_t(tok) * k + r];
    dot += p[r] * dp[r];
  }
  float direct[kMaxPerLane];  // gradient that reaches the logit without passing through `scores`
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) direct[j] = 0.f;
  if (mode == 0) {
    // p = softmax(selected logits): dl_j = p_j (dp_j - sum p dp)
    for (int r = 0; r < k; ++r)
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j)
        if (lane + 32 * j == id[r]) direct[j] += p[r] * (dp[r] - dot);
  } else if (mode == 1) {
    for (int r = 0; r < k; ++r)
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j)
        if (lane + 32 * j == id[r]) g[j] += dp[r];
  } else {
    // p_j = s_j / (sum + eps) for k > 1, else s_j:  ds_j = (dp_j - sum p dp) / (sum + eps)
    if (k > 1) {
      for (int r = 0; r < k; ++r)
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j)
          if (lane + 32 * j == id[r]) ssum += s[j];
      ssum = warp_sum(ssum) + 1e-20f;
    }
    for (int r = 0; r < k; ++r)
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j)
        if (lane + 32 * j == id[r]) g[j] += (k > 1) ? (dp[r] - dot) / ssum : dp[r];
  }
  // through the score function
  float sg = 0.f;
  if (mode != 2) {
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) sg += s[j] * g[j];
    sg = warp_sum(sg);
  }
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const int e = lane + 32 * j;
    if (e < E) {
      const float via = (mode == 2) ? g[j] * s[j] * (1.f - s[j]) : s[j] * (g[j] - sg);
      dlogits[size_t(tok) * E + e] = via + direct[j];
    }
  }
}

}  // namespace

extern "C" {

int hg_router_topk_fwd(const void* logits, const void* bias, int T, int E, int k, int mode, float scaling, void* probs,
                       void* idx, void* scores, void* counts, void* stream) {
  if (T <= 0) return 0;
  if (E < 1 || E > 32 * kMaxPerLane || k < 1 || k > kMaxK || k > E || mode < 0 || mode > 2) return -1;
  router_fwd_kernel<<<(T + kWarps - 1) / kWarps, kWarps * 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const float*)logits, (const float*)bias, T, E, k, mode, scaling, (float*)probs, (int*)idx, (float*)scores,
      (float*)counts);
  return int(cudaGetLastError());
}

int hg_router_topk_bwd(const void* scores, const void* probs, const void* idx, const void* dprobs, const void* dscores,
                       int T, int E, int k, int mode, float scaling, void* dlogits, void* stream) {
  if (T <= 0) return 0;
  if (E < 1 || E > 32 * kMaxPerLane || k < 1 || k > kMaxK || mode < 0 || mode > 2) return -1;
  router_bwd_kernel<<<(T + kWarps - 1) / kWarps, kWarps * 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const float*)scores, (const float*)probs, (const int*)idx, (const float*)dprobs, (const float*)dscores, T, E, k,
      mode, scaling, (float*)dlogits);
  return int(cudaGetLastError());
}

}  // extern "C"
