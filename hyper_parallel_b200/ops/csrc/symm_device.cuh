// Device-side primitives of the symmetric-memory layer, shared by the kernels that talk to peer
// GPUs: peer pointer tables, signal pads with monotonically increasing epochs
// (st.release.sys / ld.acquire.sys) and bounded waits that report through a status word.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hpb {

constexpr int kMaxPeers = 16;
constexpr int kFlagsPerSlot = kMaxPeers;

struct PeerTable {
  void* ptr[kMaxPeers];
};

__device__ __forceinline__ uint64_t gtime_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void report(int* status, int code, int detail) {
  if (status && atomicCAS(status, 0, code) == 0) status[1] = detail;
}

// Debug-build index checks (see sm100_common.cuh): record code 7 and skip the access.
#ifndef HPB_BOUNDS_OK
#ifdef HPB_DEBUG_BOUNDS
#define HPB_BOUNDS_OK(cond, status, detail) ((cond) ? true : (::hpb::report((status), 7, static_cast<int>(detail)), false))
#else
#define HPB_BOUNDS_OK(cond, status, detail) (true)
#endif
#endif

// Checks that stay on in every build: indices that come from tensors produced elsewhere (routing
// tables).  A failed check records status code 6 with a detail word and evaluates to false; the
// caller skips the access.
#define HPB_INPUT_OK(cond, status, detail) ((cond) ? true : (::hpb::report((status), 6, static_cast<int>(detail)), false))

// Signal every peer: "rank `rank` reached `epoch` on `slot`".
__device__ __forceinline__ void signal_peers(const PeerTable& pads, int rank, int n, int slot,
                                             uint32_t epoch) {
  for (int p = threadIdx.x; p < n; p += blockDim.x) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(pads.ptr[p]) + slot * kFlagsPerSlot + rank;
    st_release_sys(dst, epoch);
  }
}
// Wait (bounded) until every peer signalled `epoch` on `slot` of MY pad.  Returns false on
// timeout (status recorded).  Called by all threads of a CTA; threads 0..n-1 poll.
__device__ __forceinline__ bool wait_peers(const PeerTable& pads, int rank, int n, int slot,
                                           uint32_t epoch, uint64_t limit_ns, int* status) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (threadIdx.x < n) {
    const uint32_t* src =
        reinterpret_cast<const uint32_t*>(pads.ptr[rank]) + slot * kFlagsPerSlot + threadIdx.x;
    const uint64_t t0 = gtime_ns();
    uint32_t it = 0;
    // epochs only grow; compare with wrap-safe signed difference
    while (static_cast<int32_t>(ld_acquire_sys(src) - epoch) < 0) {
      if ((++it & 0xff) == 0 && gtime_ns() - t0 > limit_ns) {
        report(status, 5 /*kTimeoutPeerFlag*/, (slot << 8) | threadIdx.x);
        s_fail = 1;
        break;
      }
    }
  }
  __syncthreads();
  return s_fail == 0;
}

}  // namespace hpb
