// MoE router for sigmoid gating with group-limited top-k selection (DeepSeek-V3 style).
//
// One warp per token.  logits[T, E] (fp32) -> scores = sigmoid(logits); selection score =
// scores + bias (aux-loss-free balancing bias); experts are split into n_group contiguous
// groups, a group's score is the sum of its two best selection scores, the topk_group best
// groups survive; the top_k best surviving experts are selected; the gate weight of a selected
// expert is its UN-biased score, normalised over the selection and multiplied by `scale`.
// Also counts tokens per expert (atomicAdd) for the dispatch that follows.
//
// Each lane owns VPL = E / 32 consecutive experts; all reductions are warp shuffles.
#include <cuda_runtime.h>
#include <stdint.h>

namespace hpb {

constexpr float kNegInf = -3.0e38f;

template <int VPL>
__global__ void __launch_bounds__(256)
moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                 int64_t* __restrict__ topk_idx, float* __restrict__ topk_w,
                 int* __restrict__ expert_counts, int T, int E, int top_k, int n_group,
                 int topk_group, float scale) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T) return;
  const float* row = logits + static_cast<int64_t>(warp) * E;
  float s[VPL], sel[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int e = lane * VPL + i;
    s[i] = 1.f / (1.f + __expf(-row[e]));
    sel[i] = s[i] + bias[e];
  }
  if (n_group > 1) {
    // group score = sum of the two best selection scores of the group
    const int experts_per_group = E / n_group;
    const int lanes_per_group = experts_per_group / VPL;      // >= 1 (checked on the host)
    float b1 = kNegInf, b2 = kNegInf;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      if (sel[i] > b1) { b2 = b1; b1 = sel[i]; } else if (sel[i] > b2) { b2 = sel[i]; }
    }
    for (int o = 1; o < lanes_per_group; o <<= 1) {
      const float o1 = __shfl_xor_sync(0xffffffffu, b1, o), o2 = __shfl_xor_sync(0xffffffffu, b2, o);
      // merge two sorted pairs
      const float n1 = fmaxf(b1, o1);
      const float n2 = fmaxf(fminf(b1, o1), fmaxf(b2, o2));
      b1 = n1; b2 = n2;
    }
    const float gscore = b1 + (experts_per_group > 1 ? b2 : 0.f);
    const int my_group = lane / lanes_per_group;
    // rank of my group among all groups (ties broken by lower index, like torch.topk on CPU order)
    int rank = 0;
    for (int g = 0; g < n_group; ++g) {
      const float og = __shfl_sync(0xffffffffu, gscore, g * lanes_per_group);
      if (og > gscore || (og == gscore && g < my_group)) ++rank;
    }
    if (rank >= topk_group) {
#pragma unroll
      for (int i = 0; i < VPL; ++i) sel[i] = kNegInf;
    }
  }
  // iterative arg-max: top_k rounds
  float wsum = 0.f;
  float my_w = 0.f;      // lane j keeps the j-th selection
  int my_e = 0;
  for (int r = 0; r < top_k; ++r) {
    float best = kNegInf;
    int bi = 0;
#pragma unroll
    for (int i = 0; i < VPL; ++i)
      if (sel[i] > best) { best = sel[i]; bi = i; }
    int be = lane * VPL + bi;
    float bs = s[bi];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      const float os = __shfl_xor_sync(0xffffffffu, bs, o);
      if (ov > best || (ov == best && oe < be)) { best = ov; be = oe; bs = os; }
    }
    if (be / VPL == lane) {
#pragma unroll
      for (int i = 0; i < VPL; ++i)
        if (i == be % VPL) sel[i] = kNegInf;
    }
    wsum += bs;
    if (lane == r) { my_w = bs; my_e = be; }
  }
  if (lane < top_k) {
    topk_idx[static_cast<int64_t>(warp) * top_k + lane] = my_e;
    topk_w[static_cast<int64_t>(warp) * top_k + lane] = my_w / (wsum + 1e-20f) * scale;
    if (expert_counts) atomicAdd(expert_counts + my_e, 1);
  }
}

}  // namespace hpb

extern "C" int hpb_moe_route(const float* logits, const float* bias, int64_t* topk_idx, float* topk_w,
                             int* expert_counts, int T, int E, int top_k, int n_group, int topk_group,
                             float scale, cudaStream_t s) {
  using namespace hpb;
  if (T == 0) return 0;
  if (E % 32 || E > 512 || top_k > 32 || top_k < 1 || n_group < 1 || E % n_group) return -2;
  const int vpl = E / 32;
  if (n_group > 1) {
    const int epg = E / n_group;
    if (epg % vpl || (32 % (epg / vpl))) return -2;       // a group must be a power-of-two run of lanes
    int lpg = epg / vpl;
    if (lpg & (lpg - 1)) return -2;
    if (topk_group < 1 || topk_group > n_group) return -2;
  }
  const int threads = 256, warps_per_block = threads / 32;
  const int grid = (T + warps_per_block - 1) / warps_per_block;
#define HPB_ROUTE(V)                                                                          \
  moe_route_kernel<V><<<grid, threads, 0, s>>>(logits, bias, topk_idx, topk_w, expert_counts, T, E, \
                                               top_k, n_group, topk_group, scale)
  switch (vpl) {
    case 1: HPB_ROUTE(1); break;
    case 2: HPB_ROUTE(2); break;
    case 4: HPB_ROUTE(4); break;
    case 8: HPB_ROUTE(8); break;
    case 16: HPB_ROUTE(16); break;
    default: return -2;
  }
#undef HPB_ROUTE
  return static_cast<int>(cudaGetLastError());
}
