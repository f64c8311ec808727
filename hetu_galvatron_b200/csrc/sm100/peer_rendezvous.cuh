// Cross-rank rendezvous carried inside a kernel that reads its peers' symmetric buffers.
//
// Every rank of a group calls the same sequence of such kernels; call number `epoch` (1, 2, ...) publishes `epoch` in
// every peer's signal slots (after making this rank's earlier stores visible system-wide) and waits until every peer
// has published at least the same number: from then on the data those peers staged before their call is readable.
// The wait is bounded (10 s: the ranks of a group are only loosely in step, and giving up rejects the whole step);
// when it runs out the status word gets kTimeoutPeerFlag and the caller skips its reads.  No rank ever waits on a
// kernel of its own GPU, and nothing here spins without a limit.
#pragma once
#include "sm100_common.cuh"

namespace hg {

constexpr int kRendezvousMaxPeers = 8;
constexpr uint64_t kRendezvousLimitNs = 10000000000ull;   // 10 s

struct Rendezvous {
  int* peer_slots[kRendezvousMaxPeers];   // peer_slots[r]: rank r's signal array (int[8], symmetric); we write slot `me`
  const int* my_slots;                    // our own array: my_slots[r] >= epoch once rank r's staged data may be read
  int epoch;                              // 0: no rendezvous (the caller ordered the ranks itself)
  int t, me;
  int* status;
};

// Block-collective (contains __syncthreads).  Returns false after a time-out.
__device__ __forceinline__ bool rendezvous(const Rendezvous& rv) {
  __shared__ int ok_s;
  if (rv.epoch == 0) return true;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (blockIdx.x == 0 && int(threadIdx.x) < rv.t && int(threadIdx.x) != rv.me) {
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(rv.peer_slots[threadIdx.x] + rv.me), "r"(rv.epoch) : "memory");
  }
  if (int(threadIdx.x) < rv.t && int(threadIdx.x) != rv.me) {
    const int* flag = rv.my_slots + threadIdx.x;
    const uint64_t t0 = globaltimer_ns();
    int v;
    for (;;) {
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if (v >= rv.epoch) break;
      if (globaltimer_ns() - t0 > kRendezvousLimitNs) {
        set_status(rv.status, kTimeoutPeerFlag);
        ok_s = 0;
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
  return ok_s != 0;
}

}  // namespace hg

namespace hg_host {
// Fill a Rendezvous from the host-side arguments of an entry point (signals == null or epoch <= 0 or t < 2: none).
inline hg::Rendezvous make_rendezvous(void* const* signals, int epoch, int t, int me) {
  hg::Rendezvous rv{};
  rv.t = t;
  rv.me = me;
  rv.epoch = (signals != nullptr && t > 1 && epoch > 0) ? epoch : 0;
  if (rv.epoch) {
    for (int r = 0; r < t && r < hg::kRendezvousMaxPeers; ++r) rv.peer_slots[r] = reinterpret_cast<int*>(signals[r]);
    rv.my_slots = rv.peer_slots[me];
    rv.status = status_ptr();
  }
  return rv;
}
}  // namespace hg_host
