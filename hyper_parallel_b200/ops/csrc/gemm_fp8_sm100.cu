// FP8 (e4m3) GEMM with DeepSeek-V3 style block scaling on tcgen05 (sm_100a), plus the quantisers.
//
//   C[M,N] (bf16) = sum_kb  sa[kb, m] * sb[n/128, kb] * ( Aq[m, kb*128:(kb+1)*128] . Bq[n, kb*128:...] )
//
//   activations : e4m3, one fp32 scale per 1x128 tile   -> sa stored [K/128, M] (K-block major, so the
//                                                          epilogue threads of a tile read consecutive floats)
//   weights     : e4m3, one fp32 scale per 128x128 tile -> sb stored [N/128, K/128]
//
// The scales change every 128 elements of K, so a tile cannot be accumulated in tensor memory over
// the whole K loop.  Two-level accumulation: for every 128-wide K block the MMA warp issues four
// tcgen05.mma.kind::f8f6f4 (K = 32 each) into one of four 128x128 fp32 TMEM buffers; the epilogue
// warps read that partial product, multiply by the block's scales and add it to the running sum they
// keep in registers (128 fp32 per thread).  MMA of block kb+1..kb+3 overlaps the promotion of block kb.
// Persistent, TMA-fed (6 stages of 16 KB + 16 KB), bounded waits as everywhere in this library.
#include "sm100_common.cuh"

#include <cuda_fp8.h>

namespace hpb {
namespace f8 {

constexpr int BM = 128, BN = 128, BK = 128;       // BK in elements = bytes
constexpr int UMMA_K = 32;
constexpr int STAGES = 6;
constexpr int A_TILE = BM * BK, B_TILE = BN * BK, STAGE_BYTES = A_TILE + B_TILE;
constexpr int THREADS = 320;      // producer, MMA, 2 x 4 promotion warps (each group owns 64 columns)
constexpr int NBUF = 4;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

struct Params {
  int M, N, K;
  const float* sa;      // [K/128, M]
  const float* sb;      // [N/128, K/128]
  __nv_bfloat16* C;
  long long ldc;
  int* status;
  // grouped (expert) mode: rows of A / C are grouped by expert, every group padded to a multiple of
  // 128; block_group[m_blk] names the expert of each 128-row block (-1: unused block, skipped);
  // B stacks the experts' [b_group_rows, K] weights along its rows, sb their [b_group_rows/128, K/128]
  // scale tiles.  block_group == nullptr: plain GEMM.
  const int* block_group;
  int b_group_rows;
  int num_groups;
};

// Expert of the row block (0 for a plain GEMM) and the number of K blocks the tile runs (0: skip).
__device__ __forceinline__ int tile_group(const Params& p, int m_blk, int num_k, int& k_blocks) {
  int g = p.block_group != nullptr ? p.block_group[m_blk] : 0;
  if (!HPB_BOUNDS_OK(g < p.num_groups, p.status, 0x600000 | m_blk)) g = -1;      // debug build: skip the block
  k_blocks = g < 0 ? 0 : num_k;
  return g < 0 ? 0 : g;
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* part_full = empty_bar + STAGES;     // [NBUF]
  uint64_t* part_empty = part_full + NBUF;      // [NBUF]
  uint64_t* drain_bar = part_empty + NBUF;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_k = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < NBUF; ++b) {
      mbar_init(&part_full[b], 1);
      mbar_init(&part_empty[b], 8);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m0 = (t % num_m) * BM;
        int kbs;
        const int n0 = tile_group(p, t % num_m, num_k, kbs) * p.b_group_rows + (t / num_m) * BN;
        for (int kb = 0; kb < kbs; ++kb) {
          ok = mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kTimeoutEmptyBarrier, blockIdx.x);
          if (!ok) break;
          uint8_t* sa = smem + stage * STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * BK, m0);
          tma_load_2d(sa + A_TILE, &tmap_b, &full_bar[stage], kb * BK, n0);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(0, 0, 0, 0, BM, BN);      // e4m3 x e4m3 -> fp32
      int stage = 0;
      uint32_t phase = 0;
      long it = 0;                                                      // k blocks issued so far
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int kbs;
        tile_group(p, t % num_m, num_k, kbs);
        for (int kb = 0; kb < kbs; ++kb, ++it) {
          const int pb = static_cast<int>(it % NBUF);
          const uint32_t pphase = static_cast<uint32_t>((it / NBUF) & 1);
          ok = mbar_wait_bounded(&part_empty[pb], pphase ^ 1, abort_flag, p.status, kTimeoutTmemEmpty, blockIdx.x);
          if (!ok) break;
          ok = mbar_wait_bounded(&full_bar[stage], phase, abort_flag, p.status, kTimeoutFullBarrier, blockIdx.x);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES), sb = sa + A_TILE;
          const uint32_t tmem_d = tmem_base + pb * BN;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            umma_f8f6f4(tmem_d, make_smem_desc_sw128(sa + kk * UMMA_K, 0, 1024),
                        make_smem_desc_sw128(sb + kk * UMMA_K, 0, 1024), idesc, kk > 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          umma_commit(&part_full[pb]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        umma_commit(drain_bar);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 100000000ull) {}
      }
    }
  } else {
    // promotion: every 128-deep partial product is scaled by (activation scale of the row) x
    // (weight scale of the block) and added to the fp32 accumulator in registers.  Two groups of
    // four warps split the 128 columns, so two warps share each scheduler and hide each other's
    // tensor-memory load latency; the scales of the next block are fetched one block ahead.
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int HN = BN / 2;
    const int kblocks = (p.K + BK - 1) / BK;
    long it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const int m0 = (t % num_m) * BM, n_blk = t / num_m, n0 = n_blk * BN + half * HN;
      int kbs;
      const int grp = tile_group(p, t % num_m, num_k, kbs);
      if (kbs == 0) continue;                 // unused row block: no products, output rows left alone
      const int row = m0 + q * 32 + lane;
      const int srow = row < p.M ? row : p.M - 1;
      float2 acc[HN / 2];
#pragma unroll
      for (int j = 0; j < HN / 2; ++j) acc[j] = make_float2(0.f, 0.f);
      const float* sa_row = p.sa + srow;
      const float* sb_row = p.sb + (static_cast<long long>(grp) * (p.b_group_rows / BN) + n_blk) * kblocks;
      // scales are fetched four blocks ahead (an L2 round trip is longer than one block) and
      // multiplied only when they are used, so that the loads never stall the promotion
      constexpr int PF = 4;
      float sa_v[PF], sb_v[PF];
#pragma unroll
      for (int u = 0; u < PF; ++u) {
        const int kq = u < num_k ? u : num_k - 1;
        sa_v[u] = sa_row[static_cast<long long>(kq) * p.M];
        sb_v[u] = sb_row[kq];
      }
      for (int kb0 = 0; kb0 < num_k && ok; kb0 += PF) {
#pragma unroll
        for (int u = 0; u < PF; ++u) {
          const int kb = kb0 + u;
          if (kb >= num_k) break;
          const int pb = static_cast<int>(it % NBUF);
          const uint32_t pphase = static_cast<uint32_t>((it / NBUF) & 1);
          ++it;
          const float scale = sa_v[u] * sb_v[u];
          {
            const int kq = kb + PF < num_k ? kb + PF : num_k - 1;
            sa_v[u] = sa_row[static_cast<long long>(kq) * p.M];
            sb_v[u] = sb_row[kq];
          }
          ok = mbar_wait_bounded(&part_full[pb], pphase, abort_flag, p.status, kTimeoutTmemFull, blockIdx.x);
          if (!ok) break;
          tc_fence_after();
          const uint32_t taddr = tmem_base + pb * BN + half * HN + (static_cast<uint32_t>(q * 32) << 16);
          uint32_t r[HN];
          tmem_ld_32x32b_x32(taddr, *reinterpret_cast<uint32_t(*)[32]>(r));
          tmem_ld_32x32b_x32(taddr + 32, *reinterpret_cast<uint32_t(*)[32]>(r + 32));
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&part_empty[pb]);      // the values are in registers
          const float2 s2 = make_float2(scale, scale);
#pragma unroll
          for (int j = 0; j < HN / 2; ++j) {
            unsigned long long d;
            const float2 x = make_float2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            asm("fma.rn.f32x2 %0, %1, %2, %3;"
                : "=l"(d)
                : "l"(*reinterpret_cast<const unsigned long long*>(&x)),
                  "l"(*reinterpret_cast<const unsigned long long*>(&s2)),
                  "l"(*reinterpret_cast<const unsigned long long*>(&acc[j])));
            acc[j] = *reinterpret_cast<float2*>(&d);
          }
        }
      }
      if (!ok) break;
      if (row < p.M) {
        __nv_bfloat16* dst = p.C + static_cast<long long>(row) * p.ldc + n0;
        if (n0 + HN <= p.N && (p.ldc & 7) == 0) {
#pragma unroll
          for (int j = 0; j < HN / 8; ++j) {
            uint4 v;
            __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) vb[e] = __floats2bfloat162_rn(acc[4 * j + e].x, acc[4 * j + e].y);
            reinterpret_cast<uint4*>(dst)[j] = v;
          }
        } else {
#pragma unroll
          for (int j = 0; j < HN / 2; ++j) {         // static indices keep `acc` in registers
            if (n0 + 2 * j < p.N) dst[2 * j] = __float2bfloat16(acc[j].x);
            if (n0 + 2 * j + 1 < p.N) dst[2 * j + 1] = __float2bfloat16(acc[j].y);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ quantisers --
constexpr float kE4M3Max = 448.f;

// x[M, K] bf16 -> q[M, K] e4m3, scales[K/128, M]; one warp per (row, 128-column block)
__global__ void quant_act_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                       float* __restrict__ scales, int M, int K) {
  const int kblocks = K / 128;
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(M) * kblocks) return;
  const int row = static_cast<int>(w / kblocks), kb = static_cast<int>(w % kblocks);
  const __nv_bfloat16* src = x + static_cast<long long>(row) * K + kb * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(pb[0]), b = __bfloat1622float2(pb[1]);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = fmaxf(amax, 1e-10f) / kE4M3Max;
  const float inv = 1.f / scale;
  if (lane == 0) scales[static_cast<long long>(kb) * M + row] = scale;
  uint32_t out = 0;
  const float v[4] = {a.x * inv, a.y * inv, b.x * inv, b.y * inv};
#pragma unroll
  for (int e = 0; e < 4; ++e)
    out |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(v[e], __NV_SATFINITE, __NV_E4M3)) << (8 * e);
  *reinterpret_cast<uint32_t*>(q + static_cast<long long>(row) * K + kb * 128 + lane * 4) = out;
}

// w[N, K] bf16 -> q[N, K] e4m3, scales[N/128, K/128]; one CTA (256 threads) per 128x128 block
__global__ void __launch_bounds__(256)
quant_weight_128x128_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q,
                            float* __restrict__ scales, int N, int K) {
  __shared__ float red[8];
  __shared__ float s_scale;
  const int kblocks = K / 128;
  const int nb = blockIdx.x / kblocks, kb = blockIdx.x % kblocks;
  // thread t handles row (t / 2) and its half (64 columns)
  const int r = threadIdx.x >> 1, half = threadIdx.x & 1;
  const int row = nb * 128 + r;
  float vals[64];
  float amax = 0.f;
  if (row < N) {
    const uint4* src = reinterpret_cast<const uint4*>(w + static_cast<long long>(row) * K + kb * 128 + half * 64);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 u = src[i];
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(pb[e]);
        vals[i * 8 + 2 * e] = f.x;
        vals[i * 8 + 2 * e + 1] = f.y;
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.f;
    for (int i = 0; i < 8; ++i) m = fmaxf(m, red[i]);
    s_scale = fmaxf(m, 1e-10f) / kE4M3Max;
    scales[static_cast<long long>(nb) * kblocks + kb] = s_scale;
  }
  __syncthreads();
  if (row < N) {
    const float inv = 1.f / s_scale;
    uint32_t* dst = reinterpret_cast<uint32_t*>(q + static_cast<long long>(row) * K + kb * 128 + half * 64);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      uint32_t out = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        out |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(vals[4 * i + e] * inv, __NV_SATFINITE, __NV_E4M3)) << (8 * e);
      dst[i] = out;
    }
  }
}

}  // namespace f8

int make_tmap_2d(CUtensorMap* map, const void* ptr, CUtensorMapDataType dtype, int elem_bytes, uint64_t inner,
                 uint64_t outer, uint64_t ld, uint32_t box_inner, uint32_t box_outer);

}  // namespace hpb

using namespace hpb;
using namespace hpb::f8;

// Aq [M, K] e4m3 with sa [K/128, M]; Bq [N, K] e4m3 with sb [N/128, K/128]; C bf16 [M, N].
extern "C" int hpb_gemm_fp8_blockscale(const void* Aq, const float* sa, const void* Bq, const float* sb, void* C,
                                       long long ldc, int M, int N, int K, int* status, int num_sms,
                                       cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 128) || (reinterpret_cast<uintptr_t>(Aq) & 15) || (reinterpret_cast<uintptr_t>(Bq) & 15)) return -2;
  cudaFree(nullptr);
  CUtensorMap ta, tb;
  int r = make_tmap_2d(&ta, Aq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, M, K, BK, BM);
  if (r) return r;
  r = make_tmap_2d(&tb, Bq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, N, K, BK, BN);
  if (r) return r;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  Params p{M, N, K, sa, sb, reinterpret_cast<__nv_bfloat16*>(C), ldc, status, nullptr, 0, 1};
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  gemm_fp8_kernel<<<tiles < num_sms ? tiles : num_sms, THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

// Grouped (expert) form: Aq [M, K] with sa [K/128, M], rows grouped by expert in 128-row blocks
// (block_group [M/128], -1 = unused block); Bq [E * N, K] with sb [E * N/128, K/128]; C [M, N] bf16
// with C rows of expert e = A rows of e times W_e^T.  N must be a multiple of 128, M of 128.
extern "C" int hpb_gemm_fp8_blockscale_grouped(const void* Aq, const float* sa, const void* Bq, const float* sb,
                                               void* C, long long ldc, int M, int N, int K, int num_experts,
                                               const int* block_group, int* status, int num_sms,
                                               cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || num_experts <= 0) return 0;
  if ((K % 128) || (N % 128) || (M % 128) || block_group == nullptr || (reinterpret_cast<uintptr_t>(Aq) & 15) ||
      (reinterpret_cast<uintptr_t>(Bq) & 15))
    return -2;
  cudaFree(nullptr);
  CUtensorMap ta, tb;
  int r = make_tmap_2d(&ta, Aq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, M, K, BK, BM);
  if (r) return r;
  r = make_tmap_2d(&tb, Bq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, static_cast<uint64_t>(num_experts) * N, K, BK, BN);
  if (r) return r;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  Params p{M, N, K, sa, sb, reinterpret_cast<__nv_bfloat16*>(C), ldc, status, block_group, N, num_experts};
  const int tiles = (M / BM) * (N / BN);
  gemm_fp8_kernel<<<tiles < num_sms ? tiles : num_sms, THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int hpb_quant_act_1x128(const void* x, void* q, float* scales, int M, int K, cudaStream_t s) {
  if (K % 128 || M <= 0) return K % 128 ? -2 : 0;
  const long long warps = static_cast<long long>(M) * (K / 128);
  const int threads = 256;
  quant_act_1x128_kernel<<<static_cast<unsigned>((warps * 32 + threads - 1) / threads), threads, 0, s>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<uint8_t*>(q), scales, M, K);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int hpb_quant_weight_128x128(const void* w, void* q, float* scales, int N, int K, cudaStream_t s) {
  if (K % 128 || N <= 0) return K % 128 ? -2 : 0;
  const int blocks = ((N + 127) / 128) * (K / 128);
  quant_weight_128x128_kernel<<<blocks, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(w),
                                                     reinterpret_cast<uint8_t*>(q), scales, N, K);
  return static_cast<int>(cudaGetLastError());
}
