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
  long long group;   // index into the AdamTable of the launch (optimizer parameter group)
};

__global__ void symm_barrier_kernel(PeerTable pads, int rank, int n, int slot, uint32_t epoch,
                                    uint64_t limit_ns, int do_signal, int do_wait, int* status) {
  if (do_signal) signal_peers(pads, rank, n, slot, epoch);
  if (do_wait) wait_peers(pads, rank, n, slot, epoch, limit_ns, status);
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
  bool ok = true;
  if (sync) {
    if (blockIdx.x == 0) signal_peers(pads, rank, n, 0, epoch);   // my shard is final
    ok = wait_peers(pads, rank, n, 0, epoch, limit_ns, status);
  }
  // a CTA whose wait ran out copies nothing but still takes part in the last-CTA count below, so
  // that the counter is back at zero for the next launch on this buffer
  for (int s = 0; s < (ok ? num_segs : 0); ++s) {
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
      if (ok) wait_peers(pads, rank, n, 1, epoch, limit_ns, status);
    }
  }
}

// -------------------------------------------------- reduce-scatter + AdamW ----
struct AdamArgs {
  float lr, b1, b2, eps, wd, bc1, bc2, grad_scale;
};
constexpr int kMaxAdamGroups = 4;
// One entry per optimizer parameter group that has a parameter in the flat buffer (Segment::group
// selects the entry): learning rate, weight decay, ... may differ between the matrices and the
// norm weights of one module.
struct AdamTable {
  AdamArgs g[kMaxAdamGroups];
};

// Sum over all ranks of the 8 bf16 gradients at `mc_addr` of a multicast (NVLS) mapping: the
// NVSwitch reads the address on every GPU bound to the multicast object, adds in fp32 and returns
// one rounded bf16 vector, so the data crosses this GPU's NVLink ingress once instead of N-1 times.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}

__device__ __forceinline__ void adam8(const AdamArgs& a, const float (&acc)[8], float* __restrict__ master,
                                      float* __restrict__ m, float* __restrict__ v,
                                      __nv_bfloat16* __restrict__ param_shard, long long o) {
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

// Launched with 512 threads; the bound of 768 caps the kernel at 80 registers per thread, so
// that a CTA (40 K registers) fits beside a persistent GEMM CTA (192 threads x 96 registers)
// in the 64 K register file of an SM -- otherwise the 8-peer instance would need the whole
// file and could only run in the gaps between GEMM launches.
//
// N > 0: compile-time peer count (loads fully unrolled); N == 0: runtime `n`.
// MC: the gradients are read through `mc_grads`, a multicast (NVLS) mapping of all ranks' flat
// gradient buffers, with one multimem.ld_reduce per 16-byte vector instead of N peer loads.
//
// When the update is done the kernel publishes `version` on slot 4 of every peer's signal pad:
// "my parameter shard has reached this version"; the fused all-gather inside the consumer GEMMs
// of the next step waits for it.
template <int N, bool MC>
__global__ void __launch_bounds__(768)
fused_rs_adamw_kernel(PeerTable grads, const __nv_bfloat16* __restrict__ mc_grads, PeerTable pads,
                      const Segment* __restrict__ segs, int num_segs, float* __restrict__ master,
                      float* __restrict__ m, float* __restrict__ v, __nv_bfloat16* __restrict__ param_shard,
                      AdamTable tbl, int rank, int n, uint32_t epoch, uint32_t version, uint64_t limit_ns,
                      int* status, unsigned int* done_counter) {
  const bool sync = pads.ptr[0] != nullptr && n > 1;
  bool ok = true;
  if (sync) {
    if (blockIdx.x == 0) signal_peers(pads, rank, n, 2, epoch);   // my gradients are complete
    ok = wait_peers(pads, rank, n, 2, epoch, limit_ns, status);
  }
  // a CTA whose wait ran out updates nothing but still takes part in the last-CTA count below
  for (int s = 0; s < (ok ? num_segs : 0); ++s) {
    const Segment sg = segs[s];
    const AdamArgs a = tbl.g[sg.group];
    const long long nv = sg.n >> 3;
    const long long goff = sg.full_off + static_cast<long long>(rank) * sg.n;
    if constexpr (MC) {
      // Software pipeline: the kMcDepth reduced vectors of the NEXT trip are requested from the
      // switch before the current ones are consumed, so every thread keeps kMcDepth NVLink round
      // trips (about 3 us each) in flight behind the HBM traffic of the optimizer state.
      constexpr int kMcDepth = 4;
      const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
      const long long nthr = static_cast<long long>(gridDim.x) * blockDim.x;
      uint4 cur[kMcDepth];
#pragma unroll
      for (int u = 0; u < kMcDepth; ++u) {
        const long long i = tid + u * nthr;
        if (i < nv) cur[u] = multimem_ld_reduce_bf16x8(mc_grads + goff + (i << 3));
      }
      for (long long base = tid; base < nv; base += kMcDepth * nthr) {
        uint4 nxt[kMcDepth];
#pragma unroll
        for (int u = 0; u < kMcDepth; ++u) {
          const long long i = base + (kMcDepth + u) * nthr;
          if (i < nv) nxt[u] = multimem_ld_reduce_bf16x8(mc_grads + goff + (i << 3));
        }
#pragma unroll
        for (int u = 0; u < kMcDepth; ++u) {
          const long long i = base + u * nthr;
          if (i < nv) {
            float acc[8];
            unpack8(cur[u], acc);
            adam8(a, acc, master, m, v, param_shard, sg.shard_off + (i << 3));
          }
          cur[u] = nxt[u];
        }
      }
    }
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; !MC && i < nv;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float acc[8];
      if constexpr (MC) {
        // handled above
      } else if constexpr (N > 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
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
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        for (int rr = 0; rr < n; ++rr) {
          const int r = (rank + rr) % n;
          float f[8];
          unpack8(reinterpret_cast<const uint4*>(
                      reinterpret_cast<const __nv_bfloat16*>(grads.ptr[r]) + goff)[i], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] += f[e];
        }
      }
      adam8(a, acc, master, m, v, param_shard, sg.shard_off + (i << 3));
    }
    // tail (n % 8) elements, one CTA
    if (blockIdx.x == 0) {
      for (long long j = (nv << 3) + threadIdx.x; j < sg.n; j += blockDim.x) {
        float g = 0.f;
        for (int r = 0; r < n; ++r)
          g += __bfloat162float((reinterpret_cast<const __nv_bfloat16*>(grads.ptr[r]) + goff)[j]);
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
  {
    __syncthreads();
    __shared__ int s_last;
    if (threadIdx.x == 0) {
      __threadfence();
      s_last = (atomicAdd(done_counter, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (s_last) {
      if (threadIdx.x == 0) {
        *done_counter = 0;
        __threadfence();
      }
      __syncthreads();
      if (sync && ok) {
        signal_peers(pads, rank, n, 3, epoch);     // done reading everybody's gradients
        signal_peers(pads, rank, n, 4, version);   // my parameter shard has reached `version`
        wait_peers(pads, rank, n, 3, epoch, limit_ns, status);
      }
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
                                       do_signal, 1, status);
  return static_cast<int>(cudaGetLastError());
}

// Publish `value` on `slot` of every peer's signal pad without waiting for anybody (stream
// ordered: everything queued before it on `s` is visible to a peer that sees the value).
extern "C" int hpb_symm_signal(void* const* pads, int rank, int n, int slot, unsigned value,
                               cudaStream_t s) {
  if (n > kMaxPeers) return -2;
  prefer_shared(symm_barrier_kernel);
  symm_barrier_kernel<<<1, 32, 0, s>>>(make_table(pads, n), rank, n, slot, value, 0, 1, 0, nullptr);
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

// hyper: num_groups x 5 floats {lr, beta1, beta2, eps, weight_decay}, one row per optimizer
// parameter group referenced by the segments (num_groups <= 4).  mc_grads: multicast (NVLS)
// address of the flat gradient buffers, or null for plain peer loads.  version: the value
// published on slot 4 of the peers' signal pads when this rank's shard has been rewritten.
extern "C" int hpb_fused_rs_adamw(void* const* grad_ptrs, const void* mc_grads, void* const* pads,
                                  const void* segs, int num_segs, float* master, float* m, float* v,
                                  void* param_shard, const float* hyper, int num_groups, int step,
                                  float grad_scale, int rank, int n, unsigned epoch, unsigned version,
                                  unsigned long long limit_ns, int* status, unsigned* done_counter,
                                  int num_ctas, cudaStream_t s) {
  if (n > kMaxPeers || num_groups < 1 || num_groups > kMaxAdamGroups) return -2;
  AdamTable tbl;
  for (int g = 0; g < kMaxAdamGroups; ++g) {
    const float* h = hyper + 5 * (g < num_groups ? g : 0);
    tbl.g[g] = AdamArgs{h[0], h[1], h[2], h[3], h[4], 1.f - powf(h[1], (float)step),
                        1.f - powf(h[2], (float)step), grad_scale};
  }
#define HPB_RS(NN, MCAST)                                                                        \
  prefer_shared(fused_rs_adamw_kernel<NN, MCAST>);                                               \
  fused_rs_adamw_kernel<NN, MCAST><<<num_ctas, 512, 0, s>>>(                                     \
      make_table(grad_ptrs, n), reinterpret_cast<const __nv_bfloat16*>(mc_grads),                \
      make_table(pads, n), reinterpret_cast<const Segment*>(segs), num_segs, master, m, v,       \
      reinterpret_cast<__nv_bfloat16*>(param_shard), tbl, rank, n, epoch, version, limit_ns,     \
      status, done_counter)
  if (mc_grads != nullptr && n > 1) {
    HPB_RS(0, true);
  } else {
    switch (n) {
      case 1: HPB_RS(1, false); break;
      case 2: HPB_RS(2, false); break;
      case 4: HPB_RS(4, false); break;
      case 8: HPB_RS(8, false); break;
      default: HPB_RS(0, false); break;
    }
  }
#undef HPB_RS
  return static_cast<int>(cudaGetLastError());
}
