// Symmetric-memory runtime and fused collective kernels over NVLink / NVSwitch peer memory.
//
// Host side: allocate a buffer, export it as a CUDA IPC handle, map the peers' buffers.
// Every rank of a group ends up with a table of N device pointers (its own buffer plus
// N-1 peer mappings) and a table of N signal-pad pointers.
//
// Device side: kernels read peers' memory with plain (non-TMA) global loads -- 16 bytes per
// thread, coalesced -- and synchronise through signal pads: monotonically increasing epoch
// words written with st.release.sys and polled with ld.acquire.sys.  Every poll loop is
// bounded by a wall-clock limit; on expiry the kernel records a status code and returns.
//
//   hpb_symm_barrier     : the signal/wait primitive on its own (also used by the tests of
//                          the timeout path: a flag that nobody sets, a short limit)
//   hpb_p2p_allgather    : parameter all-gather, each rank pulls every peer's shard segments
//                          straight into the final per-parameter full tensors (no copy-out)
//   hpb_fused_rs_adamw   : gradient reduce-scatter + bf16->fp32 cast + scale + AdamW on the
//                          shard, in one pass: each rank sums its slice of all N peers'
//                          gradient buffers in fp32 and updates master / moments / bf16 weights
#include "symm_device.cuh"

#include <string.h>

namespace hpb {

// One parameter of a flat buffer: `n` shard elements that live at `shard_off` in the flat
// shard buffer; rank r's piece of the full tensor lives at `full_off + r * n`.
struct Segment {
  long long full_off;
  long long shard_off;
  long long n;
};

__global__ void symm_barrier_kernel(PeerTable pads, int rank, int n, int slot, uint32_t epoch,
                                    uint64_t limit_ns, int do_signal, int* status) {
  if (do_signal) signal_peers(pads, rank, n, slot, epoch);
  wait_peers(pads, rank, n, slot, epoch, limit_ns, status);
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// ------------------------------------------------------------- all-gather ----
// full[full_off + r*n + j] = peer_r.shard[shard_off + j]   for every segment, rank r, j < n
__global__ void __launch_bounds__(512)
p2p_allgather_kernel(PeerTable shards, PeerTable pads, const Segment* __restrict__ segs,
                     int num_segs, __nv_bfloat16* __restrict__ full, int rank, int n, uint32_t epoch,
                     uint64_t limit_ns, int* status, unsigned int* done_counter) {
  const bool sync = pads.ptr[0] != nullptr && n > 1;
  if (sync) {
    if (blockIdx.x == 0) signal_peers(pads, rank, n, 0, epoch);   // my shard is final
    if (!wait_peers(pads, rank, n, 0, epoch, limit_ns, status)) return;
  }
  for (int s = 0; s < num_segs; ++s) {
    const Segment sg = segs[s];
    const long long nv = sg.n >> 3;  // 16-byte vectors (n and offsets are multiples of 8)
    for (int rr = 0; rr < n; ++rr) {
      const int r = (rank + rr) % n;  // start with my own shard, then spread over the peers
      const uint4* src = reinterpret_cast<const uint4*>(
          reinterpret_cast<const __nv_bfloat16*>(shards.ptr[r]) + sg.shard_off);
      uint4* dst = reinterpret_cast<uint4*>(full + sg.full_off + static_cast<long long>(r) * sg.n);
      const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
      long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
      // four independent 16-byte loads in flight per thread: NVLink latency is ~2 us, so the
      // bytes in flight, not the CTA count, set the achieved bandwidth
      for (; i + 3 * stride < nv; i += 4 * stride) {
        const uint4 v0 = src[i], v1 = src[i + stride], v2 = src[i + 2 * stride], v3 = src[i + 3 * stride];
        dst[i] = v0; dst[i + stride] = v1; dst[i + 2 * stride] = v2; dst[i + 3 * stride] = v3;
      }
      for (; i < nv; i += stride) dst[i] = src[i];
      // tail elements
      if (blockIdx.x == 0)
        for (long long i = (nv << 3) + threadIdx.x; i < sg.n; i += blockDim.x)
          (full + sg.full_off + static_cast<long long>(r) * sg.n)[i] =
              (reinterpret_cast<const __nv_bfloat16*>(shards.ptr[r]) + sg.shard_off)[i];
    }
  }
  if (sync) {
    // "done reading your shard": the last CTA to finish tells the peers and waits for theirs,
    // so that no rank overwrites its shard while somebody still reads it
    __syncthreads();
    __shared__ int s_last;
    if (threadIdx.x == 0) {
      __threadfence();
      s_last = (atomicAdd(done_counter, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (s_last) {
      if (threadIdx.x == 0) *done_counter = 0;
      signal_peers(pads, rank, n, 1, epoch);
      wait_peers(pads, rank, n, 1, epoch, limit_ns, status);
    }
  }
}

// -------------------------------------------------- reduce-scatter + AdamW ----
struct AdamArgs {
  float lr, b1, b2, eps, wd, bc1, bc2, grad_scale;
};

// Launched with 512 threads; the bound of 768 caps the kernel at 80 registers per thread, so
// that a CTA (40 K registers) fits beside a persistent GEMM CTA (192 threads x 96 registers)
// in the 64 K register file of an SM -- otherwise the 8-peer instance would need the whole
// file and could only run in the gaps between GEMM launches.
template <int N>  // N > 0: compile-time peer count (loads fully unrolled); N == 0: runtime `n`
__global__ void __launch_bounds__(768)
fused_rs_adamw_kernel(PeerTable grads, PeerTable pads, const Segment* __restrict__ segs,
                      int num_segs, float* __restrict__ master, float* __restrict__ m,
                      float* __restrict__ v, __nv_bfloat16* __restrict__ param_shard, AdamArgs a,
                      int rank, int n, uint32_t epoch, uint64_t limit_ns, int* status,
                      unsigned int* done_counter) {
  const bool sync = pads.ptr[0] != nullptr && n > 1;
  if (sync) {
    if (blockIdx.x == 0) signal_peers(pads, rank, n, 2, epoch);   // my gradients are complete
    if (!wait_peers(pads, rank, n, 2, epoch, limit_ns, status)) return;
  }
  for (int s = 0; s < num_segs; ++s) {
    const Segment sg = segs[s];
    const long long nv = sg.n >> 3;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nv;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      const long long goff = sg.full_off + static_cast<long long>(rank) * sg.n;
      if constexpr (N > 0) {
        // issue all peer loads first (they are independent), then reduce in fp32
        uint4 buf[N];
#pragma unroll
        for (int rr = 0; rr < N; ++rr) {
          const int r = (rank + rr) % N;
          buf[rr] = reinterpret_cast<const uint4*>(
              reinterpret_cast<const __nv_bfloat16*>(grads.ptr[r]) + goff)[i];
        }
#pragma unroll
        for (int rr = 0; rr < N; ++rr) {
          float f[8];
          unpack8(buf[rr], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] += f[e];
        }
      } else {
        for (int rr = 0; rr < n; ++rr) {
          const int r = (rank + rr) % n;
          float f[8];
          unpack8(reinterpret_cast<const uint4*>(
                      reinterpret_cast<const __nv_bfloat16*>(grads.ptr[r]) + goff)[i], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] += f[e];
        }
      }
      const long long o = sg.shard_off + (i << 3);
      float4 m0 = *reinterpret_cast<float4*>(m + o), m1 = *reinterpret_cast<float4*>(m + o + 4);
      float4 v0 = *reinterpret_cast<float4*>(v + o), v1 = *reinterpret_cast<float4*>(v + o + 4);
      float4 w0 = *reinterpret_cast<float4*>(master + o), w1 = *reinterpret_cast<float4*>(master + o + 4);
      float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
      float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
      float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float g = acc[e] * a.grad_scale;
        mm[e] = a.b1 * mm[e] + (1.f - a.b1) * g;
        vv[e] = a.b2 * vv[e] + (1.f - a.b2) * g * g;
        ww[e] = ww[e] * (1.f - a.lr * a.wd) - a.lr * (mm[e] / a.bc1) / (sqrtf(vv[e] / a.bc2) + a.eps);
      }
      *reinterpret_cast<float4*>(m + o) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(m + o + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
      *reinterpret_cast<float4*>(v + o) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      *reinterpret_cast<float4*>(v + o + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
      *reinterpret_cast<float4*>(master + o) = make_float4(ww[0], ww[1], ww[2], ww[3]);
      *reinterpret_cast<float4*>(master + o + 4) = make_float4(ww[4], ww[5], ww[6], ww[7]);
      uint4 out;
      __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
      for (int e = 0; e < 4; ++e) ob[e] = __floats2bfloat162_rn(ww[2 * e], ww[2 * e + 1]);
      *reinterpret_cast<uint4*>(param_shard + o) = out;
    }
    // tail (n % 8) elements, one CTA
    if (blockIdx.x == 0) {
      for (long long j = (nv << 3) + threadIdx.x; j < sg.n; j += blockDim.x) {
        float g = 0.f;
        for (int r = 0; r < n; ++r)
          g += __bfloat162float((reinterpret_cast<const __nv_bfloat16*>(grads.ptr[r]) + sg.full_off +
                                 static_cast<long long>(rank) * sg.n)[j]);
        g *= a.grad_scale;
        const long long o = sg.shard_off + j;
        const float mi = a.b1 * m[o] + (1.f - a.b1) * g;
        const float vi = a.b2 * v[o] + (1.f - a.b2) * g * g;
        const float wi = master[o] * (1.f - a.lr * a.wd) - a.lr * (mi / a.bc1) / (sqrtf(vi / a.bc2) + a.eps);
        m[o] = mi; v[o] = vi; master[o] = wi;
        param_shard[o] = __float2bfloat16(wi);
      }
    }
  }
  if (sync) {
    __syncthreads();
    __shared__ int s_last;
    if (threadIdx.x == 0) {
      __threadfence();
      s_last = (atomicAdd(done_counter, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (s_last) {
      if (threadIdx.x == 0) *done_counter = 0;
      signal_peers(pads, rank, n, 3, epoch);   // done reading everybody's gradients
      wait_peers(pads, rank, n, 3, epoch, limit_ns, status);
    }
  }
}

// The persistent GEMM needs ~200 KB of shared memory per SM.  A kernel that prefers L1 would
// force every SM it touches to be re-partitioned before a GEMM CTA can land there (the GEMM CTA
// then waits for the communication CTA to finish).  Asking for the maximum shared-memory
// carve-out keeps both kernels co-resident.
template <typename K>
static void prefer_shared(K kernel) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                       cudaSharedmemCarveoutMaxShared);
}

static PeerTable make_table(void* const* ptrs, int n) {
  PeerTable t;
  for (int i = 0; i < kMaxPeers; ++i) t.ptr[i] = (ptrs != nullptr && i < n) ? ptrs[i] : nullptr;
  return t;
}

}  // namespace hpb

using namespace hpb;

// ------------------------------------------------------------ host runtime ----
extern "C" int hpb_symm_alloc(void** out, size_t bytes) {
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaMemset(*out, 0, bytes));
}
extern "C" int hpb_symm_free(void* p) { return static_cast<int>(cudaFree(p)); }
// handle_out: 64 bytes
extern "C" int hpb_symm_export(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return static_cast<int>(e);
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}
extern "C" int hpb_symm_import(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return static_cast<int>(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
}
extern "C" int hpb_symm_unmap(void* p) { return static_cast<int>(cudaIpcCloseMemHandle(p)); }
extern "C" int hpb_symm_handle_bytes() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

// ---------------------------------------------------------------- launchers ----
extern "C" int hpb_symm_barrier(void* const* pads, int rank, int n, int slot, unsigned epoch,
                                unsigned long long limit_ns, int do_signal, int* status,
                                cudaStream_t s) {
  if (n > kMaxPeers) return -2;
  prefer_shared(symm_barrier_kernel);
  symm_barrier_kernel<<<1, 32, 0, s>>>(make_table(pads, n), rank, n, slot, epoch, limit_ns,
                                       do_signal, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int hpb_p2p_allgather(void* const* shard_ptrs, void* const* pads, const void* segs,
                                 int num_segs, void* full, int rank, int n, unsigned epoch,
                                 unsigned long long limit_ns, int* status, unsigned* done_counter,
                                 int num_ctas, cudaStream_t s) {
  if (n > kMaxPeers) return -2;
  prefer_shared(p2p_allgather_kernel);
  p2p_allgather_kernel<<<num_ctas, 512, 0, s>>>(make_table(shard_ptrs, n), make_table(pads, n),
                                                reinterpret_cast<const Segment*>(segs), num_segs,
                                                reinterpret_cast<__nv_bfloat16*>(full), rank, n,
                                                epoch, limit_ns, status, done_counter);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int hpb_fused_rs_adamw(void* const* grad_ptrs, void* const* pads, const void* segs,
                                  int num_segs, float* master, float* m, float* v, void* param_shard,
                                  float lr, float b1, float b2, float eps, float wd, int step,
                                  float grad_scale, int rank, int n, unsigned epoch,
                                  unsigned long long limit_ns, int* status, unsigned* done_counter,
                                  int num_ctas, cudaStream_t s) {
  if (n > kMaxPeers) return -2;
  AdamArgs a{lr, b1, b2, eps, wd, 1.f - powf(b1, (float)step), 1.f - powf(b2, (float)step), grad_scale};
#define HPB_RS(NN)                                                                              \
  prefer_shared(fused_rs_adamw_kernel<NN>);                                                     \
  fused_rs_adamw_kernel<NN><<<num_ctas, 512, 0, s>>>(                                           \
      make_table(grad_ptrs, n), make_table(pads, n), reinterpret_cast<const Segment*>(segs),    \
      num_segs, master, m, v, reinterpret_cast<__nv_bfloat16*>(param_shard), a, rank, n, epoch, \
      limit_ns, status, done_counter)
  switch (n) {
    case 1: HPB_RS(1); break;
    case 2: HPB_RS(2); break;
    case 4: HPB_RS(4); break;
    case 8: HPB_RS(8); break;
    default: HPB_RS(0); break;
  }
#undef HPB_RS
  return static_cast<int>(cudaGetLastError());
}
