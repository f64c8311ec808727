// Memory-bound element-wise kernels: RoPE (in place on the packed QKV projection), SwiGLU / GeGLU /
// GELU forward and backward, embedding gather and its scatter-add gradient, bf16<->fp32 casts.
// Oracles: galvatron/core/runtime/transformer/rope_utils.py:86-120 (rotate-half form),
// galvatron/core/runtime/transformer/fused_kernels.py:19-48,142-168 (activations),
// galvatron/core/runtime/tensor_parallel/layers.py:120-147 (masked vocab-parallel lookup).
#include "sm100_common.cuh"

namespace {

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

// A grid-stride walk over (row, col) pairs of a [rows, width] index space without a division per step: the
// stride is split into whole rows and a remainder once per thread, then every step is an add and a carry.
// (A 64-bit divide per 16-byte access costs more issue slots than the access leaves room for at HBM speed.)
struct RowColWalk {
  int64_t row;
  int col;
  int64_t d_row;
  int d_col;
  int width;
  __device__ __forceinline__ RowColWalk(int width_) : width(width_) {
    const int64_t first = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    row = first / width;
    col = int(first - row * width);
    d_row = stride / width;
    d_col = int(stride - d_row * width);
  }
  __device__ __forceinline__ void next() {
    row += d_row;
    col += d_col;
    if (col >= width) {
      col -= width;
      ++row;
    }
  }
};

// ---------------------------------------------------------------------------------------------
// RoPE, rotate-half (non-interleaved) form, applied in place to `nheads` heads that sit at
// column offsets head_off[h] (elements) of every token row of a [tokens, row_pitch] buffer.
//   out[i]        = x[i]*cos[i] - x[i+half]*sin[i]
//   out[i+half]   = x[i+half]*cos[i] + x[i]*sin[i]       (sign of sin flipped for the backward)
// Token t has position pos[t] when `pos` is given, else (t / batch) + pos_offset ([S,B] order).
// cos/sin tables are fp32 [max_pos, half].
// ---------------------------------------------------------------------------------------------
__global__ void rope_kernel(hg_lp_t* __restrict__ buf, const int* __restrict__ head_off, int nheads,
                            int row_pitch, int tokens, int batch, const int* __restrict__ pos, int pos_offset,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t, int half, float sign) {
  const int vec_per_head = half >> 3;  // uint4 chunks in one half
  const int per_token = nheads * vec_per_head;
  for (RowColWalk w(per_token); w.row < tokens; w.next()) {
    const int t = int(w.row);
    const int h = w.col / vec_per_head, c = w.col - h * vec_per_head;
    const int p = pos ? pos[t] : (t / batch + pos_offset);
    hg_lp_t* base = buf + size_t(t) * row_pitch + head_off[h] + c * 8;
    float a[8], b[8], cs[8], sn[8];
    unpack8(*reinterpret_cast<const uint4*>(base), a);
    unpack8(*reinterpret_cast<const uint4*>(base + half), b);
    const float4* cp = reinterpret_cast<const float4*>(cos_t + size_t(p) * half + c * 8);
    const float4* sp = reinterpret_cast<const float4*>(sin_t + size_t(p) * half + c * 8);
    *reinterpret_cast<float4*>(cs) = cp[0];
    *reinterpret_cast<float4*>(cs + 4) = cp[1];
    *reinterpret_cast<float4*>(sn) = sp[0];
    *reinterpret_cast<float4*>(sn + 4) = sp[1];
    float oa[8], ob[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = sn[j] * sign;
      oa[j] = a[j] * cs[j] - b[j] * s;
      ob[j] = b[j] * cs[j] + a[j] * s;
    }
    *reinterpret_cast<uint4*>(base) = pack8(oa);
    *reinterpret_cast<uint4*>(base + half) = pack8(ob);
  }
}

// RoPE, interleaved form: channel pairs (2i, 2i+1) rotate by angle i.
//   out[2i]   = x[2i]*cos[i] - x[2i+1]*sin[i]
//   out[2i+1] = x[2i+1]*cos[i] + x[2i]*sin[i]
// One thread takes 8 consecutive channels (4 pairs) of one head of one token.
__global__ void rope_interleaved_kernel(hg_lp_t* __restrict__ buf, const int* __restrict__ head_off, int nheads,
                                        int row_pitch, int tokens, int batch, const int* __restrict__ pos,
                                        int pos_offset, const float* __restrict__ cos_t,
                                        const float* __restrict__ sin_t, int half, float sign) {
  const int vec_per_head = half >> 2;  // uint4 chunks over the 2*half rotated channels
  const int per_token = nheads * vec_per_head;
  for (RowColWalk w(per_token); w.row < tokens; w.next()) {
    const int t = int(w.row);
    const int h = w.col / vec_per_head, c = w.col - h * vec_per_head;
    const int p = pos ? pos[t] : (t / batch + pos_offset);
    hg_lp_t* base = buf + size_t(t) * row_pitch + head_off[h] + c * 8;
    float x[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(base), x);
    const float4 cs = *reinterpret_cast<const float4*>(cos_t + size_t(p) * half + c * 4);
    const float4 sn = *reinterpret_cast<const float4*>(sin_t + size_t(p) * half + c * 4);
    const float cv[4] = {cs.x, cs.y, cs.z, cs.w}, sv[4] = {sn.x * sign, sn.y * sign, sn.z * sign, sn.w * sign};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[2 * j] = x[2 * j] * cv[j] - x[2 * j + 1] * sv[j];
      o[2 * j + 1] = x[2 * j + 1] * cv[j] + x[2 * j] * sv[j];
    }
    *reinterpret_cast<uint4*>(base) = pack8(o);
  }
}

// ---------------------------------------------------------------------------------------------
// Gated activations on y = [y1 | y2] (each F wide, row pitch 2F):  out = act(y1) * y2
//   kind 0: SwiGLU (silu), kind 1: GeGLU (tanh GELU).  Non-gated kind 2: out = gelu_tanh(y) (pitch F).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float silu(float x) { return __fdividef(x, 1.f + __expf(-x)); }
__device__ __forceinline__ float gelu_tanh(float x) {
  return 0.5f * x * (1.f + tanhf(0.79788456f * x * (1.f + 0.044715f * x * x)));
}
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float t = tanhf(0.79788456f * x * (1.f + 0.044715f * x * x));
  return 0.5f * x * ((1.f - t * t) * (0.79788456f + 0.1070322243f * x * x)) + 0.5f * (1.f + t);
}

template <int KIND>
__global__ void glu_fwd_kernel(const hg_lp_t* __restrict__ y, hg_lp_t* __restrict__ out, int64_t rows,
                               int F) {
  for (RowColWalk w(F >> 3); w.row < rows; w.next()) {
    const int64_t r = w.row;
    const int c = w.col;
    float a[8], o[8];
    if (KIND == 2) {
      unpack8(reinterpret_cast<const uint4*>(y + r * F)[c], a);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = gelu_tanh(a[j]);
    } else {
      float b[8];
      unpack8(reinterpret_cast<const uint4*>(y + r * 2 * F)[c], a);
      unpack8(reinterpret_cast<const uint4*>(y + r * 2 * F + F)[c], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (KIND == 0 ? silu(a[j]) : gelu_tanh(a[j])) * b[j];
    }
    reinterpret_cast<uint4*>(out + r * F)[c] = pack8(o);
  }
}

template <int KIND>
__global__ void glu_bwd_kernel(const hg_lp_t* __restrict__ g, const hg_lp_t* __restrict__ y,
                               hg_lp_t* __restrict__ dy, int64_t rows, int F) {
  for (RowColWalk w(F >> 3); w.row < rows; w.next()) {
    const int64_t r = w.row;
    const int c = w.col;
    float gv[8], a[8];
    unpack8(reinterpret_cast<const uint4*>(g + r * F)[c], gv);
    if (KIND == 2) {
      float o[8];
      unpack8(reinterpret_cast<const uint4*>(y + r * F)[c], a);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = gv[j] * gelu_tanh_grad(a[j]);
      reinterpret_cast<uint4*>(dy + r * F)[c] = pack8(o);
    } else {
      float b[8], d1[8], d2[8];
      unpack8(reinterpret_cast<const uint4*>(y + r * 2 * F)[c], a);
      unpack8(reinterpret_cast<const uint4*>(y + r * 2 * F + F)[c], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (KIND == 0) {
          const float s = __fdividef(1.f, 1.f + __expf(-a[j]));
          d1[j] = gv[j] * s * (1.f + a[j] * (1.f - s)) * b[j];
          d2[j] = gv[j] * a[j] * s;
        } else {
          d1[j] = gv[j] * gelu_tanh_grad(a[j]) * b[j];
          d2[j] = gv[j] * gelu_tanh(a[j]);
        }
      }
      reinterpret_cast<uint4*>(dy + r * 2 * F)[c] = pack8(d1);
      reinterpret_cast<uint4*>(dy + r * 2 * F + F)[c] = pack8(d2);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Embedding: out[t,:] = (v0 <= id < v1) ? W[id - v0,:] : 0   (+ pos_emb[t / batch,:] optional)
// Gradient: dW[id - v0,:] += dout[t,:] (fp32 atomics)
// ---------------------------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ ids, const hg_lp_t* __restrict__ W,
                                     const hg_lp_t* __restrict__ pos_emb, hg_lp_t* __restrict__ out,
                                     int tokens, int H, int v0, int v1, int batch, int pos_offset) {
  const int vpr = H >> 3;
  const int64_t total = int64_t(tokens) * vpr;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
    const int t = int(i / vpr), c = int(i % vpr);
    const int64_t id = ids[t];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (id >= v0 && id < v1) v = reinterpret_cast<const uint4*>(W + size_t(id - v0) * H)[c];
    if (pos_emb) {
      float a[8], b[8];
      unpack8(v, a);
      unpack8(reinterpret_cast<const uint4*>(pos_emb + size_t(t / batch + pos_offset) * H)[c], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += b[j];
      v = pack8(a);
    }
    reinterpret_cast<uint4*>(out + size_t(t) * H)[c] = v;
  }
}

__global__ void embedding_bwd_kernel(const int64_t* __restrict__ ids, const hg_lp_t* __restrict__ dout,
                                     float* __restrict__ dW, float* __restrict__ dpos, int tokens, int H, int v0,
                                     int v1, int batch, int pos_offset) {
  const int vpr = H >> 3;
  const int64_t total = int64_t(tokens) * vpr;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
    const int t = int(i / vpr), c = int(i % vpr);
    const int64_t id = ids[t];
    float g[8];
    unpack8(reinterpret_cast<const uint4*>(dout + size_t(t) * H)[c], g);
    if (id >= v0 && id < v1) {
      float* dst = dW + size_t(id - v0) * H + c * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(dst + j, g[j]);
    }
    if (dpos) {
      float* dst = dpos + size_t(t / batch + pos_offset) * H + c * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(dst + j, g[j]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Casts and the bf16 residual add
// ---------------------------------------------------------------------------------------------
__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ in, hg_lp_t* __restrict__ out, int64_t n) {
  const int64_t nv = n >> 3;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < nv; i += int64_t(gridDim.x) * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(in)[2 * i], b = reinterpret_cast<const float4*>(in)[2 * i + 1];
    const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    reinterpret_cast<uint4*>(out)[i] = pack8(f);
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) out[(nv << 3) + threadIdx.x] = hg_f2lp(in[(nv << 3) + threadIdx.x]);
}

__global__ void add_bf16_kernel(const hg_lp_t* __restrict__ a, const hg_lp_t* __restrict__ b,
                                hg_lp_t* __restrict__ out, int64_t n) {
  const int64_t nv = n >> 3;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < nv; i += int64_t(gridDim.x) * blockDim.x) {
    float x[8], y[8];
    unpack8(reinterpret_cast<const uint4*>(a)[i], x);
    unpack8(reinterpret_cast<const uint4*>(b)[i], y);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += y[j];
    reinterpret_cast<uint4*>(out)[i] = pack8(x);
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
    const int64_t k = (nv << 3) + threadIdx.x;
    out[k] = hg_f2lp(hg_lp2f(a[k]) + hg_lp2f(b[k]));
  }
}


// Log-sum-exp merge of two partial attention results over disjoint key sets (ring / context-parallel attention):
//   l = log(exp(lse_acc) + exp(lse_new));  out_acc = exp(lse_acc - l) * out_acc + exp(lse_new - l) * out_new;  lse_acc = l
// out_acc fp32 [S, B*h, d] contiguous, out_new bf16 same shape, lse_new fp32 [B*h, S] contiguous, lse_acc fp32 with
// row pitch `lse_pitch` (a slice of a longer sequence).  LPR = d / 8 lanes share a row; they all read the old lse
// before lane 0 replaces it.
template <int LPR>
__global__ void attn_merge_kernel(float* __restrict__ out_acc, float* __restrict__ lse_acc, long long lse_pitch,
                                  const hg_lp_t* __restrict__ out_new, const float* __restrict__ lse_new, int S,
                                  int BH) {
  const int64_t rows = int64_t(S) * BH;
  const int64_t t = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  const int64_t row = t / LPR;
  const int lane = int(t % LPR);
  const bool live = row < rows;
  float wa = 0.f, wb = 0.f, l = 0.f;
  float* lp = nullptr;
  if (live) {
    const int s = int(row / BH), bh = int(row % BH);
    lp = lse_acc + int64_t(bh) * lse_pitch + s;
    const float la = *lp, ln = lse_new[int64_t(bh) * S + s];
    const float m = fmaxf(la, ln);
    if (m == -INFINITY) {   // neither side has seen a key yet
      l = -INFINITY;
    } else {
      l = m + __logf(__expf(la - m) + __expf(ln - m));
      wa = __expf(la - l);
      wb = __expf(ln - l);
    }
    float4* acc = reinterpret_cast<float4*>(out_acc + (row * LPR + lane) * 8);
    float x[8];
    unpack8(reinterpret_cast<const uint4*>(out_new)[row * LPR + lane], x);
    float4 a0 = acc[0], a1 = acc[1];
    a0.x = wa * a0.x + wb * x[0]; a0.y = wa * a0.y + wb * x[1]; a0.z = wa * a0.z + wb * x[2]; a0.w = wa * a0.w + wb * x[3];
    a1.x = wa * a1.x + wb * x[4]; a1.y = wa * a1.y + wb * x[5]; a1.z = wa * a1.z + wb * x[6]; a1.w = wa * a1.w + wb * x[7];
    acc[0] = a0;
    acc[1] = a1;
  }
  __syncwarp();
  if (live && lane == 0) *lp = l;
}

inline int grid_for(int64_t work, int threads) {
  int64_t g = (work + threads - 1) / threads;
  const int64_t cap = 148 * 16;
  return int(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

extern "C" {

int hg_rope(void* buf, const void* head_off, int nheads, int row_pitch, int tokens, int batch, const void* pos,
            int pos_offset, const void* cos_t, const void* sin_t, int rot_dim, int flags, void* stream) {
  // flags: bit 0 = backward (rotate by the negative angle), bit 1 = interleaved channel pairs
  if (tokens <= 0 || nheads <= 0) return 0;
  const int half = rot_dim / 2;
  if ((half & 7) || (row_pitch & 7)) return -1;
  const float sign = (flags & 1) ? -1.f : 1.f;
  if (flags & 2) {
    const int64_t work = int64_t(tokens) * nheads * (half >> 2);
    rope_interleaved_kernel<<<grid_for(work, 256), 256, 0, (cudaStream_t)stream>>>(
        (hg_lp_t*)buf, (const int*)head_off, nheads, row_pitch, tokens, batch, (const int*)pos, pos_offset,
        (const float*)cos_t, (const float*)sin_t, half, sign);
  } else {
    const int64_t work = int64_t(tokens) * nheads * (half >> 3);
    rope_kernel<<<grid_for(work, 256), 256, 0, (cudaStream_t)stream>>>(
        (hg_lp_t*)buf, (const int*)head_off, nheads, row_pitch, tokens, batch, (const int*)pos, pos_offset,
        (const float*)cos_t, (const float*)sin_t, half, sign);
  }
  return int(cudaGetLastError());
}

int hg_glu_fwd(const void* y, void* out, long long rows, int F, int kind, void* stream) {
  if (rows <= 0) return 0;
  if (F & 7) return -1;
  const int g = grid_for(rows * (F >> 3), 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (kind == 0) glu_fwd_kernel<0><<<g, 256, 0, st>>>((const hg_lp_t*)y, (hg_lp_t*)out, rows, F);
  else if (kind == 1) glu_fwd_kernel<1><<<g, 256, 0, st>>>((const hg_lp_t*)y, (hg_lp_t*)out, rows, F);
  else glu_fwd_kernel<2><<<g, 256, 0, st>>>((const hg_lp_t*)y, (hg_lp_t*)out, rows, F);
  return int(cudaGetLastError());
}

int hg_glu_bwd(const void* g_, const void* y, void* dy, long long rows, int F, int kind, void* stream) {
  if (rows <= 0) return 0;
  if (F & 7) return -1;
  const int g = grid_for(rows * (F >> 3), 256);
  cudaStream_t st = (cudaStream_t)stream;
  auto G = (const hg_lp_t*)g_;
  if (kind == 0) glu_bwd_kernel<0><<<g, 256, 0, st>>>(G, (const hg_lp_t*)y, (hg_lp_t*)dy, rows, F);
  else if (kind == 1) glu_bwd_kernel<1><<<g, 256, 0, st>>>(G, (const hg_lp_t*)y, (hg_lp_t*)dy, rows, F);
  else glu_bwd_kernel<2><<<g, 256, 0, st>>>(G, (const hg_lp_t*)y, (hg_lp_t*)dy, rows, F);
  return int(cudaGetLastError());
}

int hg_embedding_fwd(const void* ids, const void* W, const void* pos_emb, void* out, int tokens, int H, int v0, int v1,
                     int batch, int pos_offset, void* stream) {
  if (tokens <= 0) return 0;
  if (H & 7) return -1;
  embedding_fwd_kernel<<<grid_for(int64_t(tokens) * (H >> 3), 256), 256, 0, (cudaStream_t)stream>>>(
      (const int64_t*)ids, (const hg_lp_t*)W, (const hg_lp_t*)pos_emb, (hg_lp_t*)out, tokens, H, v0,
      v1, batch, pos_offset);
  return int(cudaGetLastError());
}

int hg_embedding_bwd(const void* ids, const void* dout, void* dW, void* dpos, int tokens, int H, int v0, int v1,
                     int batch, int pos_offset, void* stream) {
  if (tokens <= 0) return 0;
  if (H & 7) return -1;
  embedding_bwd_kernel<<<grid_for(int64_t(tokens) * (H >> 3), 256), 256, 0, (cudaStream_t)stream>>>(
      (const int64_t*)ids, (const hg_lp_t*)dout, (float*)dW, (float*)dpos, tokens, H, v0, v1, batch, pos_offset);
  return int(cudaGetLastError());
}

int hg_cast_f32_bf16(const void* in, void* out, long long n, void* stream) {
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_for(n >> 3, 256), 256, 0, (cudaStream_t)stream>>>((const float*)in,
                                                                                    (hg_lp_t*)out, n);
  return int(cudaGetLastError());
}

int hg_add_bf16(const void* a, const void* b, void* out, long long n, void* stream) {
  if (n <= 0) return 0;
  add_bf16_kernel<<<grid_for(n >> 3, 256), 256, 0, (cudaStream_t)stream>>>(
      (const hg_lp_t*)a, (const hg_lp_t*)b, (hg_lp_t*)out, n);
  return int(cudaGetLastError());
}

// See attn_merge_kernel.  d must be 64 or 128; S * BH rows.
int hg_attn_merge(void* out_acc, void* lse_acc, long long lse_pitch, const void* out_new, const void* lse_new, int S,
                  int BH, int d, void* stream) {
  if (S <= 0 || BH <= 0) return 0;
  if (d != 64 && d != 128) return -1;
  const int lpr = d / 8;
  const int64_t threads = int64_t(S) * BH * lpr;
  const int grid = int((threads + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (lpr == 16)
    attn_merge_kernel<16><<<grid, 256, 0, st>>>((float*)out_acc, (float*)lse_acc, lse_pitch, (const hg_lp_t*)out_new,
                                                (const float*)lse_new, S, BH);
  else
    attn_merge_kernel<8><<<grid, 256, 0, st>>>((float*)out_acc, (float*)lse_acc, lse_pitch, (const hg_lp_t*)out_new,
                                               (const float*)lse_new, S, BH);
  return int(cudaGetLastError());
}

}  // extern "C"
