// All-to-all with the layout transform folded in, as peer loads over NVLink.
//
// Every rank publishes its source tensor in a symmetric buffer; the destination rank *pulls* the chunks it needs from
// every peer and writes them at their final position of a plain local tensor.  One launch replaces
// "permute copy -> NCCL all-to-all" (sequence -> heads) or "NCCL all-to-all -> permute copy" (heads -> sequence)
// of Ulysses sequence parallelism, and the variable-size form replaces "permute -> all-to-all-v" of the
// mixture-of-experts token dispatch.
//
//   peer_gather_kernel      fixed-size chunks:  out[r*out_peer_stride + i*out_row_stride + c] =
//                                               src_r[src_off + i*src_stride + c]      r < t, i < rows, c < chunk
//   peer_gather_rows_kernel variable row lists: out[o, :] = sum_k scale[o,k] * src_{peer[o,k]}[row[o,k], :]
//
// Both kernels can carry the cross-rank rendezvous themselves (peer_rendezvous.cuh: signal slots, bounded wait), so a
// whole exchange is a staging copy plus this one launch; without signals the caller orders the ranks with a
// stream-ordered collective.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "peer_rendezvous.cuh"

namespace {

constexpr int kMaxPeers = 8;
constexpr int kThreads = 256;
constexpr int kUnroll = 4;

struct PeerPtrs {
  const void* p[kMaxPeers];
};

inline int grid_for(long long items) {
  long long g = (items + kThreads - 1) / kThreads;
  const long long cap = 148LL * 8;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return int(g);
}

// All quantities in units of 16 bytes (8 bf16).  vec = chunk / 8.
__global__ void __launch_bounds__(kThreads)
peer_gather_kernel(PeerPtrs src, int t, long long rows, int vec, long long src_off, long long src_stride,
                   uint4* __restrict__ out, long long out_peer_stride, long long out_row_stride, int* status,
                   hg::Rendezvous rv) {
  if (!hg::rendezvous(rv)) return;
  if (!HG_BOUNDS_OK(t >= 1 && t <= kMaxPeers && src_off >= 0 && src_stride >= 0 && out_peer_stride >= 0 && out_row_stride >= 0, status))
    return;
  const long long per_peer = rows * vec;
  const long long total = per_peer * t;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (; idx < total; idx += stride * kUnroll) {
    uint4 val[kUnroll];
    long long dst[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long j = idx + u * stride;
      dst[u] = -1;
      if (j < total) {
        const int r = int(j / per_peer);
        const long long rem = j - r * per_peer;
        const long long i = rem / vec;
        const int c = int(rem - i * vec);
        val[u] = __ldcs(reinterpret_cast<const uint4*>(src.p[r]) + src_off + i * src_stride + c);
        dst[u] = r * out_peer_stride + i * out_row_stride + c;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (dst[u] >= 0) out[dst[u]] = val[u];
  }
}

constexpr int kMaxTopK = 8;
long long g_src_rows_limit = 0;   // rows of the peers' source buffers for the debug build's row check (0 = unknown)

__device__ __forceinline__ void fma8(float (&acc)[8], uint4 v, float s) {
  const hg_lp2_t* h = reinterpret_cast<const hg_lp2_t*>(&v);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = hg_lp22ff(h[k]);
    acc[2 * k] += f.x * s;
    acc[2 * k + 1] += f.y * s;
  }
}

// out[o, :] = sum_{k < K} scale[o*K + k] * src_{peer[o*K + k]}[row[o*K + k], :]   (fp32 accumulation; K = 1 and no
// scale is a plain gather).  Entries with peer < 0 contribute nothing (dropped tokens, padding).
template <int K>
__global__ void __launch_bounds__(kThreads)
peer_gather_rows_kernel(PeerPtrs src, const int* __restrict__ peer, const int* __restrict__ row, long long n_out,
                        int vec, long long src_row_stride, uint4* __restrict__ out, const float* __restrict__ scale,
                        int t, long long src_rows, int* status, hg::Rendezvous rv) {
  if (!hg::rendezvous(rv)) return;
  const long long total = n_out * vec;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long j = blockIdx.x * (long long)blockDim.x + threadIdx.x; j < total; j += stride) {
    const long long o = j / vec;
    const int c = int(j - o * vec);
    uint4 val[K];
    float sc[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int pr = peer[o * K + k];
      sc[k] = pr < 0 ? 0.f : (scale ? scale[o * K + k] : 1.f);
      val[k] = make_uint4(0u, 0u, 0u, 0u);
      if (pr >= 0) {
        // the routing table names a peer of the group and a row of its buffer (checked in the debug build)
        const long long rw = row[o * K + k];
        if (!HG_BOUNDS_OK(pr < t && rw >= 0 && (src_rows <= 0 || rw < src_rows), status)) {
          sc[k] = 0.f;
          continue;
        }
        val[k] = __ldcs(reinterpret_cast<const uint4*>(src.p[pr]) + rw * src_row_stride + c);
      }
    }
    if (K == 1 && scale == nullptr) {
      out[j] = val[0];
    } else {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int k = 0; k < K; ++k) fma8(acc, val[k], sc[k]);
      uint4 r;
      hg_lp2_t* h = reinterpret_cast<hg_lp2_t*>(&r);
#pragma unroll
      for (int k = 0; k < 4; ++k) h[k] = hg_ff2lp2(acc[2 * k], acc[2 * k + 1]);
      out[j] = r;
    }
  }
}

}  // namespace

extern "C" {

// Element counts are in bf16 elements and must be multiples of 8; pointers 16-byte aligned.
int hg_peer_gather_bf16_rv(const void* const* src, int t, long long rows, long long chunk, long long src_off,
                           long long src_stride, void* out, long long out_peer_stride, long long out_row_stride,
                           void* const* signals, int me, int epoch, void* stream);
int hg_peer_gather_bf16(const void* const* src, int t, long long rows, long long chunk, long long src_off,
                        long long src_stride, void* out, long long out_peer_stride, long long out_row_stride,
                        void* stream) {
  return hg_peer_gather_bf16_rv(src, t, rows, chunk, src_off, src_stride, out, out_peer_stride, out_row_stride, nullptr,
                                0, 0, stream);
}
// As above with the in-kernel rendezvous: signals[r] = rank r's int[8] signal array, me = this rank's index in the
// group, epoch = the group's call counter (> 0, +1 per exchange on every rank).
int hg_peer_gather_bf16_rv(const void* const* src, int t, long long rows, long long chunk, long long src_off,
                           long long src_stride, void* out, long long out_peer_stride, long long out_row_stride,
                           void* const* signals, int me, int epoch, void* stream) {
  if (t < 1 || t > kMaxPeers || rows < 0 || chunk <= 0) return -1;
  if ((chunk | src_off | src_stride | out_peer_stride | out_row_stride) & 7) return -1;
  const hg::Rendezvous rv = hg_host::make_rendezvous(signals, epoch, t, me);
  if (rows == 0 && rv.epoch == 0) return 0;     // with a rendezvous the peers still wait for this rank's signal
  PeerPtrs pp{};
  for (int r = 0; r < t; ++r) pp.p[r] = src[r];
  const long long total = rows * (chunk / 8) * t;
  peer_gather_kernel<<<grid_for((total + kUnroll - 1) / kUnroll), kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pp, t, rows, int(chunk / 8), src_off / 8, src_stride / 8, reinterpret_cast<uint4*>(out), out_peer_stride / 8,
      out_row_stride / 8, hg_host::status_ptr(), rv);
  return int(cudaGetLastError());
}

// out[o, 0:width] = sum_{k < topk} scale[o*topk+k] * src_{peer[o*topk+k]}[row[o*topk+k], 0:width]; width multiple of 8;
// src rows are src_row_stride elements apart; scale may be null (weights 1); entries with peer < 0 are skipped.
int hg_peer_gather_rows_bf16_rv(const void* const* src, int t, const void* peer, const void* row, long long n_out,
                                int topk, long long width, long long src_row_stride, void* out, const void* scale,
                                void* const* signals, int me, int epoch, void* stream);
int hg_peer_gather_rows_bf16(const void* const* src, int t, const void* peer, const void* row, long long n_out,
                             int topk, long long width, long long src_row_stride, void* out, const void* scale,
                             void* stream) {
  return hg_peer_gather_rows_bf16_rv(src, t, peer, row, n_out, topk, width, src_row_stride, out, scale, nullptr, 0, 0,
                                     stream);
}
// As above with the in-kernel rendezvous (see hg_peer_gather_bf16_rv).
int hg_peer_gather_rows_bf16_rv(const void* const* src, int t, const void* peer, const void* row, long long n_out,
                                int topk, long long width, long long src_row_stride, void* out, const void* scale,
                                void* const* signals, int me, int epoch, void* stream) {
  if (t < 1 || t > kMaxPeers || n_out < 0 || width <= 0 || ((width | src_row_stride) & 7)) return -1;
  if (topk < 1 || topk > kMaxTopK) return -1;
  const hg::Rendezvous rv = hg_host::make_rendezvous(signals, epoch, t, me);
  if (n_out == 0 && rv.epoch == 0) return 0;    // with a rendezvous the peers still wait for this rank's signal
  PeerPtrs pp{};
  for (int r = 0; r < t; ++r) pp.p[r] = src[r];
  const long long total = n_out * (width / 8);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define HG_ROWS(K_)                                                                                               \
  peer_gather_rows_kernel<K_><<<grid_for(total), kThreads, 0, st>>>(                                              \
      pp, reinterpret_cast<const int*>(peer), reinterpret_cast<const int*>(row), n_out, int(width / 8),           \
      src_row_stride / 8, reinterpret_cast<uint4*>(out), reinterpret_cast<const float*>(scale), t, g_src_rows_limit,      \
      hg_host::status_ptr(), rv)
  switch (topk) {
    case 1: HG_ROWS(1); break;
    case 2: HG_ROWS(2); break;
    case 3: HG_ROWS(3); break;
    case 4: HG_ROWS(4); break;
    case 5: HG_ROWS(5); break;
    case 6: HG_ROWS(6); break;
    case 7: HG_ROWS(7); break;
    default: HG_ROWS(8); break;
  }
#undef HG_ROWS
  return int(cudaGetLastError());
}

// Debug build only: tell the row-list gather how many rows the peers' source buffers hold, so that it can check the
// routing table's row indices (0 switches the check off).  Returns the previous value.
long long hg_debug_set_gather_row_limit(long long rows) {
  const long long old = g_src_rows_limit;
  g_src_rows_limit = rows;
  return old;
}

}  // extern "C"
