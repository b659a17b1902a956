// Token embedding for sm_100a: the row gather of the forward pass and a deterministic dense
// weight gradient for the backward pass (bf16 rows, fp32 accumulation).
//
// Backward.  dW[v, :] = sum over the tokens t with idx[t] == v of dY[t, :], every row of dW written
// exactly once (rows that no token names are written as zeros, so the caller passes uninitialised
// memory).  No sort over the tokens and no floating-point atomics:
//
//   1. count   cnt[v] += 1 per token (integer atomics: the result does not depend on the order)
//   2. scan    off[v] = exclusive prefix sum of cnt over the vocabulary (one CTA)
//   3. fill    bucket[off[v] + k] = t, k handed out by an integer atomic (order inside a bucket varies)
//   4. sum     one CTA per vocabulary row: the bucket is rank-sorted by token index in shared memory
//              (token indices are distinct, buckets are short), then the rows are added in that
//              order -- the same order, hence the same bits, on every run.  Buckets longer than
//              kMaxSorted tokens are added in bucket order (still correct, order not fixed).
//
// Indices outside [0, V) contribute nothing (forward: a zero row) and record kBadArgument in the
// status word.
#include "sm100_common.cuh"

namespace hpb {
namespace emb {

constexpr int kMaxSorted = 1024;

__global__ void embed_fwd_kernel(const int64_t* __restrict__ idx, const uint4* __restrict__ w, uint4* __restrict__ out,
                                 int64_t T, int V, int vec_per_row, int* status) {
  const int64_t total = T * vec_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / vec_per_row;
    const int c = static_cast<int>(i - t * vec_per_row);
    const int64_t v = idx[t];
    if (v < 0 || v >= V) {
      if (c == 0) report_error(status, kBadArgument, static_cast<int>(t));
      out[i] = make_uint4(0, 0, 0, 0);
    } else {
      out[i] = w[v * vec_per_row + c];
    }
  }
}

__global__ void embed_count_kernel(const int64_t* __restrict__ idx, int* __restrict__ cnt, int64_t T, int V,
                                   int* status) {
  for (int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; t < T;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t v = idx[t];
    if (v < 0 || v >= V)
      report_error(status, kBadArgument, static_cast<int>(t));
    else
      atomicAdd(&cnt[v], 1);
  }
}

// off[v] = sum of cnt[0..v); cursor[v] = 0.  One CTA of 1024 threads, each scanning a contiguous chunk.
__global__ void __launch_bounds__(1024) embed_scan_kernel(const int* __restrict__ cnt, int* __restrict__ off,
                                                          int* __restrict__ cursor, int V) {
  __shared__ int part[1024];
  const int chunk = (V + 1023) / 1024;
  const int lo = min(static_cast<int>(threadIdx.x) * chunk, V), hi = min(lo + chunk, V);
  int s = 0;
  for (int v = lo; v < hi; ++v) s += cnt[v];
  part[threadIdx.x] = s;
  __syncthreads();
  // inclusive Hillis-Steele scan of the 1024 partial sums
  for (int d = 1; d < 1024; d <<= 1) {
    const int add = threadIdx.x >= d ? part[threadIdx.x - d] : 0;
    __syncthreads();
    part[threadIdx.x] += add;
    __syncthreads();
  }
  int run = part[threadIdx.x] - s;
  for (int v = lo; v < hi; ++v) {
    off[v] = run;
    run += cnt[v];
    cursor[v] = 0;
  }
}

__global__ void embed_fill_kernel(const int64_t* __restrict__ idx, const int* __restrict__ off, int* __restrict__ cursor,
                                  int* __restrict__ bucket, int64_t T, int V) {
  for (int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; t < T;
       t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t v = idx[t];
    if (v < 0 || v >= V) continue;
    bucket[off[v] + atomicAdd(&cursor[v], 1)] = static_cast<int>(t);
  }
}

// One CTA per vocabulary row (grid-stride); thread c owns the 16-byte vector c, c + blockDim.x, ... of the row.
__global__ void __launch_bounds__(256) embed_sum_kernel(const uint4* __restrict__ dy, const int* __restrict__ cnt,
                                                        const int* __restrict__ off, const int* __restrict__ bucket,
                                                        uint4* __restrict__ dw, int V, int vec_per_row) {
  __shared__ int raw[kMaxSorted];
  __shared__ int sorted[kMaxSorted];
  for (int v = blockIdx.x; v < V; v += gridDim.x) {
    const int n = cnt[v];
    uint4* dst = dw + static_cast<int64_t>(v) * vec_per_row;
    if (n == 0) {
      for (int c = threadIdx.x; c < vec_per_row; c += blockDim.x) dst[c] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const int* b = bucket + off[v];
    const int* order = b;
    if (n <= kMaxSorted) {
      __syncthreads();                       // the previous row's readers are done with the arrays
      for (int i = threadIdx.x; i < n; i += blockDim.x) raw[i] = b[i];
      __syncthreads();
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int t = raw[i];
        int rank = 0;
        for (int j = 0; j < n; ++j) rank += raw[j] < t;
        sorted[rank] = t;
      }
      __syncthreads();
      order = sorted;
    }
    for (int c = threadIdx.x; c < vec_per_row; c += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int i = 0; i < n; ++i) {
        const uint4 x = dy[static_cast<int64_t>(order[i]) * vec_per_row + c];
        const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(xb[e]);
          acc[2 * e] += f.x;
          acc[2 * e + 1] += f.y;
        }
      }
      uint4 o;
      __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) ob[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
      dst[c] = o;
    }
  }
}

}  // namespace emb
}  // namespace hpb

using namespace hpb;

// out[T, H] = w[idx[T], :]; bf16, H % 8 == 0, 16-byte aligned pointers.
extern "C" int hpb_embedding_fwd(const int64_t* idx, const void* w, void* out, int64_t T, int V, int H, int* status,
                                 int num_sms, cudaStream_t s) {
  if (H <= 0 || H % 8 || V <= 0) return -2;
  if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15) return -2;
  if (T == 0) return 0;
  const int64_t total = T * (H / 8);
  const int64_t want = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(num_sms > 0 ? num_sms : 148) * 16;
  emb::embed_fwd_kernel<<<static_cast<unsigned>(want < cap ? want : cap), 256, 0, s>>>(
      idx, reinterpret_cast<const uint4*>(w), reinterpret_cast<uint4*>(out), T, V, H / 8, status);
  return static_cast<int>(cudaGetLastError());
}

// Number of int32 words of scratch that hpb_embedding_bwd needs.
extern "C" int64_t hpb_embedding_bwd_scratch_words(int64_t T, int V) { return 3ll * V + T; }

// dw[V, H] = scatter-add of dy[T, H] by idx (every row written); scratch: hpb_embedding_bwd_scratch_words ints.
extern "C" int hpb_embedding_bwd(const int64_t* idx, const void* dy, void* dw, int* scratch, int64_t T, int V, int H,
                                 int* status, int num_sms, cudaStream_t s) {
  if (H <= 0 || H % 8 || V <= 0 || T < 0 || T > 0x7fffffff) return -2;
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dw)) & 15) return -2;
  int* cnt = scratch;
  int* off = scratch + V;
  int* cursor = scratch + 2ll * V;
  int* bucket = scratch + 3ll * V;
  cudaError_t e = cudaMemsetAsync(cnt, 0, sizeof(int) * static_cast<size_t>(V), s);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int sms = num_sms > 0 ? num_sms : 148;
  if (T > 0) {
    const int64_t want = (T + 255) / 256;
    emb::embed_count_kernel<<<static_cast<unsigned>(want < sms * 8 ? want : sms * 8), 256, 0, s>>>(idx, cnt, T, V,
                                                                                                 status);
  }
  emb::embed_scan_kernel<<<1, 1024, 0, s>>>(cnt, off, cursor, V);
  if (T > 0) {
    const int64_t want = (T + 255) / 256;
    emb::embed_fill_kernel<<<static_cast<unsigned>(want < sms * 8 ? want : sms * 8), 256, 0, s>>>(idx, off, cursor,
                                                                                                bucket, T, V);
  }
  const int rows = V < sms * 32 ? V : sms * 32;
  emb::embed_sum_kernel<<<rows, 256, 0, s>>>(reinterpret_cast<const uint4*>(dy), cnt, off, bucket,
                                             reinterpret_cast<uint4*>(dw), V, H / 8);
  return static_cast<int>(cudaGetLastError());
}
