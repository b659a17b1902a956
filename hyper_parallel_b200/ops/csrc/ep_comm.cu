// Expert-parallel dispatch and combine over NVLink peer memory (pull model, no host round trip).
//
// Every rank stages, in symmetric memory: its token matrix x[T, H]; its (token, expert) pairs
// sorted by expert (`sorted_token[T*k]`, optional `sorted_scale[T*k]`); and the number of pairs
// per expert `counts[E]`.  Experts [r*El, (r+1)*El) live on rank r.
//
//   hpb_ep_dispatch : after a barrier, each rank reads all peers' `counts`, derives the layout of
//       its receive matrix (every local expert's rows start at a multiple of 128, ordered by
//       source rank; padding rows are zeroed) and PULLS each row from its source's staged x over
//       NVLink straight into place.  It also emits the tables of the grouped GEMM
//       (`block_group`, `group_offsets`) on the device, so nothing returns to the host.
//   hpb_ep_combine  : after a barrier ("expert outputs are ready"), each rank pulls, for every
//       token, the k expert-output rows from the owners' output matrices, forms the weighted sum
//       in fp32 and (optionally) keeps the raw rows for the backward of the gate weights.
//
// The backward pass uses the same two kernels: d(expert output) = dispatch of dy scaled by the
// gate weight, dx = combine with unit weights.
//
// All cross-rank waits are bounded and report through the status word; a receive matrix that is
// too small for the routed rows is reported as an error (code 6) and nothing is copied.
#include "symm_device.cuh"

namespace hpb {
namespace ep {

constexpr int kMaxExperts = 512;
constexpr int kMaxLocal = 64;
constexpr int kMaxEp = 8;
constexpr int ROW_BLOCK = 128;

struct DispatchParams {
  int T, k, H, E, n, rank, cap_rows;
  PeerTable x_stage, sorted_token, sorted_scale, counts, pads;
  __nv_bfloat16* recv;   // [cap_rows, H]
  int* block_group;      // [cap_rows / 128]: local expert of the block, -1 = unused
  int* group_offsets;    // [El + 1]
  int* meta;             // [0] padded rows in use
  int* counts_all;       // [n, E] local snapshot of every rank's counts (read by the combine kernel)
  uint32_t epoch;
  uint64_t limit_ns;
  int* status;
};

__device__ __forceinline__ int pad128(int x) { return (x + ROW_BLOCK - 1) / ROW_BLOCK * ROW_BLOCK; }

// Error paths leave "no block in use" / "every expert empty" tables behind, so that the grouped
// GEMMs queued after a failed dispatch skip every block instead of reading uninitialised tables.
__device__ __forceinline__ void write_empty_tables(const DispatchParams& p) {
  for (int b = threadIdx.x; b < p.cap_rows / ROW_BLOCK; b += blockDim.x) p.block_group[b] = -1;
  for (int el = threadIdx.x; el <= p.E / p.n; el += blockDim.x) p.group_offsets[el] = 0;
  if (threadIdx.x == 0) p.meta[0] = 0;
}

__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const DispatchParams p) {
  __shared__ int s_cnt[kMaxEp][kMaxExperts];       // pairs per (source, global expert)
  __shared__ int s_srcpre[kMaxEp][kMaxLocal];      // source-side start of my experts inside its sorted list
  __shared__ int s_start[kMaxLocal + 1];           // padded start row of each local expert
  __shared__ int s_srcoff[kMaxLocal][kMaxEp + 1];  // inside an expert: first row of each source
  const int El = p.E / p.n;
  if (p.n > 1) {
    if (blockIdx.x == 0) signal_peers(p.pads, p.rank, p.n, 0, p.epoch);   // my staging is complete
    if (!wait_peers(p.pads, p.rank, p.n, 0, p.epoch, p.limit_ns, p.status)) {
      if (blockIdx.x == 0) write_empty_tables(p);
      return;
    }
  }
  for (int i = threadIdx.x; i < p.n * p.E; i += blockDim.x) {
    const int s = i / p.E, e = i - s * p.E;
    s_cnt[s][e] = reinterpret_cast<const int*>(p.counts.ptr[s])[e];
  }
  __syncthreads();
  if (threadIdx.x < p.n) {
    // exclusive prefix over the source's experts, kept for my local experts only
    const int s = threadIdx.x;
    int acc = 0;
    for (int e = 0; e < p.E; ++e) {
      const int el = e - p.rank * El;
      if (el >= 0 && el < El) s_srcpre[s][el] = acc;
      acc += s_cnt[s][e];
    }
  }
  if (threadIdx.x == 32) {
    int row = 0;
    for (int el = 0; el < El; ++el) {
      s_start[el] = row;
      int tot = 0;
      for (int s = 0; s < p.n; ++s) {
        s_srcoff[el][s] = tot;
        tot += s_cnt[s][p.rank * El + el];
      }
      s_srcoff[el][p.n] = tot;
      row += pad128(tot);
    }
    s_start[El] = row;
  }
  __syncthreads();
  const int m_pad = s_start[El];
  if (blockIdx.x == 0)
    // the combine kernel of this layer reads the counts from this local snapshot, never from a
    // peer: a rank that runs ahead may already be staging the counts of its next dispatch
    for (int i = threadIdx.x; i < p.n * p.E; i += blockDim.x) p.counts_all[i] = s_cnt[i / p.E][i % p.E];
  if (m_pad > p.cap_rows) {
    // Overflow of the receive matrix is an error (code 6, surfaced by the host's status check).
    if (blockIdx.x == 0) {
      write_empty_tables(p);
      if (threadIdx.x == 0) report(p.status, 6 /*kBadArgument*/, 0x4000 | (m_pad / ROW_BLOCK));
    }
    return;
  }
  if (blockIdx.x == 0) {
    for (int b = threadIdx.x; b < p.cap_rows / ROW_BLOCK; b += blockDim.x) {
      int g = -1;
      const int row = b * ROW_BLOCK;
      if (row < m_pad)
        for (int el = 0; el < El; ++el)
          if (row >= s_start[el] && row < s_start[el + 1]) g = el;
      p.block_group[b] = g;
    }
    for (int el = threadIdx.x; el <= El; el += blockDim.x) p.group_offsets[el] = s_start[el];
    if (threadIdx.x == 0) p.meta[0] = m_pad;
  }
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int vec_per_row = p.H / 8;
  for (int slot = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); slot < m_pad; slot += gridDim.x * warps_per_cta) {
    // local expert of the row (El <= 64: two probes per lane)
    int el = -1;
    for (int c = lane; c < El; c += 32)
      if (slot >= s_start[c] && slot < s_start[c + 1]) el = c;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) el = max(el, __shfl_xor_sync(0xffffffffu, el, o));
    uint4* dst = reinterpret_cast<uint4*>(p.recv + static_cast<long long>(slot) * p.H);
    const int off = slot - s_start[el];
    if (off >= s_srcoff[el][p.n]) {
      for (int c = lane; c < vec_per_row; c += 32) dst[c] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    int s = 0;
    while (off >= s_srcoff[el][s + 1]) ++s;
    const int j = s_srcpre[s][el] + (off - s_srcoff[el][s]);   // index into the source's sorted pair list
    int token = 0;
    float scale = 1.f;
    if (lane == 0) {
      token = reinterpret_cast<const int*>(p.sorted_token.ptr[s])[j];
      if (p.sorted_scale.ptr[0] != nullptr) scale = reinterpret_cast<const float*>(p.sorted_scale.ptr[s])[j];
    }
    token = __shfl_sync(0xffffffffu, token, 0);
    scale = __shfl_sync(0xffffffffu, scale, 0);
    // the pair list comes from the router: a token index outside [0, T) would turn into a wild peer read
    if (!HPB_INPUT_OK(token >= 0 && token < p.T && j >= 0 && j < p.T * p.k && slot < p.cap_rows, p.status,
                      0x100000 | (slot & 0xfffff)))
      continue;
    const uint4* src =
        reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.x_stage.ptr[s]) +
                                       static_cast<long long>(token) * p.H);
    const bool scaled = p.sorted_scale.ptr[0] != nullptr;
    int c = lane;
    // four independent 16-byte loads in flight per lane (NVLink latency)
    for (; c + 96 < vec_per_row; c += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = src[c + 32 * u];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (scaled) {
          __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&v[u]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float2 f = __bfloat1622float2(b2[e]);
            b2[e] = __floats2bfloat162_rn(f.x * scale, f.y * scale);
          }
        }
        dst[c + 32 * u] = v[u];
      }
    }
    for (; c < vec_per_row; c += 32) {
      uint4 v = src[c];
      if (scaled) {
        __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 f = __bfloat1622float2(b2[e]);
          b2[e] = __floats2bfloat162_rn(f.x * scale, f.y * scale);
        }
      }
      dst[c] = v;
    }
  }
}

struct CombineParams {
  int T, k, H, E, n, rank;
  int cap_rows;                    // rows of every rank's expert-output matrix
  PeerTable out, pads;             // expert-output matrices [cap_rows, H] of every rank
  const int* counts_all;           // [n, E] local snapshot written by the dispatch kernel of this layer
  const long long* topk_idx;       // [T, k] global expert of each pair
  const int* sorted_pos;           // [T * k] position of the pair in my sorted-by-expert list
  const float* weights;            // [T, k] or null (unit weights)
  __nv_bfloat16* y;                // [T, H]
  __nv_bfloat16* rows_save;        // [T * k, H] or null
  uint32_t epoch;
  uint64_t limit_ns;
  int* status;
};

__global__ void __launch_bounds__(256)
ep_combine_kernel(const CombineParams p) {
  __shared__ int s_tot[kMaxExperts];        // rows of each global expert over all sources
  __shared__ int s_before[kMaxExperts];     // rows of sources < me inside each expert
  __shared__ int s_dst[kMaxExperts];        // first row of MY pairs of expert e in its owner's matrix
  __shared__ int s_myoff[kMaxExperts];      // start of expert e in my sorted list
  __shared__ const uint4* s_row[8];
  __shared__ float s_w[8];
  const int El = p.E / p.n;
  if (p.n > 1) {
    if (blockIdx.x == 0) signal_peers(p.pads, p.rank, p.n, 1, p.epoch);   // my expert outputs are written
    if (!wait_peers(p.pads, p.rank, p.n, 1, p.epoch, p.limit_ns, p.status)) return;
  }
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
    int tot = 0, before = 0;
    for (int s = 0; s < p.n; ++s) {
      const int c = p.counts_all[s * p.E + e];
      if (s < p.rank) before += c;
      tot += c;
    }
    s_tot[e] = tot;
    s_before[e] = before;
  }
  __syncthreads();
  if (threadIdx.x < p.n) {
    const int r = threadIdx.x;
    int row = 0;
    for (int el = 0; el < El; ++el) {
      const int e = r * El + el;
      s_dst[e] = row + s_before[e];
      row += pad128(s_tot[e]);
    }
  }
  if (threadIdx.x == 32) {
    int acc = 0;
    const int* mine = p.counts_all + p.rank * p.E;
    for (int e = 0; e < p.E; ++e) {
      s_myoff[e] = acc;
      acc += mine[e];
    }
  }
  __syncthreads();
  const int vec_per_row = p.H / 8;
  for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
    if (threadIdx.x < p.k) {
      const int pair = t * p.k + threadIdx.x;
      const int e = static_cast<int>(p.topk_idx[pair]);
      // expert ids come from the router: anything outside [0, E) must not index the tables
      const bool e_ok = HPB_INPUT_OK(e >= 0 && e < p.E, p.status, 0x200000 | (pair & 0xfffff));
      const int slot = e_ok ? s_dst[e] + (p.sorted_pos[pair] - s_myoff[e]) : -1;
      if (e_ok && HPB_INPUT_OK(slot >= 0 && slot < p.cap_rows, p.status, 0x300000 | (pair & 0xfffff))) {
        s_row[threadIdx.x] = reinterpret_cast<const uint4*>(
            reinterpret_cast<const __nv_bfloat16*>(p.out.ptr[e / El]) + static_cast<long long>(slot) * p.H);
        s_w[threadIdx.x] = p.weights ? p.weights[pair] : 1.f;
      } else {        // bad routing entry: reported through the status word, the row counts as zeros
        s_row[threadIdx.x] = nullptr;
        s_w[threadIdx.x] = 0.f;
      }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < vec_per_row; c += blockDim.x) {
      uint4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < p.k) v[j] = s_row[j] != nullptr ? s_row[j][c] : make_uint4(0u, 0u, 0u, 0u);
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j < p.k) {
          if (p.rows_save)
            reinterpret_cast<uint4*>(p.rows_save + (static_cast<long long>(t) * p.k + j) * p.H)[c] = v[j];
          const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&v[j]);
          const float w = s_w[j];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(b2[e]);
            acc[2 * e] += w * f.x;
            acc[2 * e + 1] += w * f.y;
          }
        }
      }
      uint4 o;
      __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) ob[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
      reinterpret_cast<uint4*>(p.y + static_cast<long long>(t) * p.H)[c] = o;
    }
    __syncthreads();
  }
}

static PeerTable table(void* const* ptrs, int n) {
  PeerTable t;
  for (int i = 0; i < kMaxPeers; ++i) t.ptr[i] = (ptrs != nullptr && i < n) ? ptrs[i] : nullptr;
  return t;
}

}  // namespace ep
}  // namespace hpb

using namespace hpb;

// x_stage / sorted_token / sorted_scale / counts / pads: arrays of n device pointers (symmetric
// memory; sorted_scale may be null).  recv [cap_rows, H], block_group [cap_rows / 128],
// group_offsets [E / n + 1], meta [1] and counts_all [n, E] are local outputs.
extern "C" int hpb_ep_dispatch(void* const* x_stage, void* const* sorted_token, void* const* sorted_scale,
                               void* const* counts, void* const* pads, void* recv, int* block_group,
                               int* group_offsets, int* meta, int* counts_all, int T, int k, int H, int E, int n,
                               int rank,
                               int cap_rows, unsigned epoch, unsigned long long limit_ns, int* status, int num_ctas,
                               cudaStream_t stream) {
  if (n < 1 || n > ep::kMaxEp || E > ep::kMaxExperts || E % n || E / n > ep::kMaxLocal || (H % 8) ||
      (cap_rows % ep::ROW_BLOCK) || k < 1 || k > 8)
    return -2;
  ep::DispatchParams p;
  p.T = T; p.k = k; p.H = H; p.E = E; p.n = n; p.rank = rank; p.cap_rows = cap_rows;
  p.x_stage = ep::table(x_stage, n);
  p.sorted_token = ep::table(sorted_token, n);
  p.sorted_scale = ep::table(sorted_scale, n);
  p.counts = ep::table(counts, n);
  p.pads = ep::table(pads, n);
  p.recv = reinterpret_cast<__nv_bfloat16*>(recv);
  p.block_group = block_group; p.group_offsets = group_offsets; p.meta = meta;
  p.counts_all = counts_all;
  p.epoch = epoch; p.limit_ns = limit_ns; p.status = status;
  cudaFuncSetAttribute(ep::ep_dispatch_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                       cudaSharedmemCarveoutMaxShared);
  ep::ep_dispatch_kernel<<<num_ctas, 256, 0, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

// out / pads: arrays of n device pointers (symmetric memory); counts_all [n, E] is the local
// snapshot that the dispatch kernel of the same layer wrote.  topk_idx [T, k] int64,
// sorted_pos [T*k] int32, weights [T, k] fp32 or null; y [T, H]; rows_save [T*k, H] or null.
extern "C" int hpb_ep_combine(void* const* out, const int* counts_all, void* const* pads, const void* topk_idx,
                              const int* sorted_pos, const float* weights, void* y, void* rows_save, int T, int k,
                              int H, int E, int n, int rank, int cap_rows, unsigned epoch, unsigned long long limit_ns,
                              int* status, int num_ctas, cudaStream_t stream) {
  if (n < 1 || n > ep::kMaxEp || E > ep::kMaxExperts || E % n || (H % 8) || k < 1 || k > 8) return -2;
  ep::CombineParams p;
  p.T = T; p.k = k; p.H = H; p.E = E; p.n = n; p.rank = rank; p.cap_rows = cap_rows;
  p.out = ep::table(out, n);
  p.counts_all = counts_all;
  p.pads = ep::table(pads, n);
  p.topk_idx = reinterpret_cast<const long long*>(topk_idx);
  p.sorted_pos = sorted_pos;
  p.weights = weights;
  p.y = reinterpret_cast<__nv_bfloat16*>(y);
  p.rows_save = reinterpret_cast<__nv_bfloat16*>(rows_save);
  p.epoch = epoch; p.limit_ns = limit_ns; p.status = status;
  cudaFuncSetAttribute(ep::ep_combine_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                       cudaSharedmemCarveoutMaxShared);
  ep::ep_combine_kernel<<<num_ctas, 256, 0, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}
