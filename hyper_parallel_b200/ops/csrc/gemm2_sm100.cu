// bf16 GEMM with CTA pairs (tcgen05 cta_group::2): one 256x256 output tile per pair of SMs.
//
// Same contract as gemm_sm100.cu (C[M,N] (+)= opA * opB^T, K-major or MN-major operands), but two
// CTAs of a 2-CTA cluster cooperate on a tile: each loads its own 128 rows of A and its own 128
// rows (columns of C) of B, the leader CTA issues one UMMA of shape 256x256x16 that reads both
// CTAs' shared memory and writes both CTAs' tensor memory.  Per SM and per K step this moves
// 16 KB + 16 KB instead of 16 KB + 32 KB through shared memory, which is what limits the 1-CTA
// 128x256 kernel, and leaves room for a 6-stage ring.
//
// Synchronisation:
//   full[s]   (leader only) : armed by the leader's producer with the bytes of BOTH CTAs; both
//                             CTAs' TMA loads complete on it (cta_group::2 loads signal the
//                             leader's barrier at the same shared-memory offset)
//   empty[s]  (both CTAs)   : tcgen05.commit multicast from the leader's MMA thread
//   tmem_full[b] (both)     : tcgen05.commit multicast when a tile's accumulation is done
//   tmem_empty[b] (leader)  : 8 arrivals, 4 epilogue warps of each CTA (the peer arrives remotely)
// Operand loads are plain per-CTA TMA copies.  Every wait is bounded (see sm100_common.cuh).
#include "gemm2_pair.cuh"

namespace hpb {
namespace g2 {

template <bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM>
__global__ void __launch_bounds__(THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;       // [2]
  uint64_t* drain_bar = tmem_empty + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();          // 0 = leader
  const bool leader = cta == 0;
  const int num_m = (p.M + TILE_M - 1) / TILE_M, num_n = (p.N + TILE_N - 1) / TILE_N;
  const int num_tiles = num_m * num_n;
  const int num_k = (p.K + BLOCK_K - 1) / BLOCK_K;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 8);      // 4 epilogue warps x 2 CTAs
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc2(tmem_base_slot, TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();                          // both CTAs' barriers and TMEM are ready
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // -------------------------------------------------------- TMA producer (both CTAs) --
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        int m_blk, n_blk;
        tile_coords(t, num_m, num_n, m_blk, n_blk);
        const int m0 = m_blk * TILE_M + cta * CTA_M;       // my rows of A
        const int n0 = n_blk * TILE_N + cta * CTA_NB;      // my rows of B
        for (int kb = 0; kb < num_k; ++kb) {
          ok = mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kTimeoutEmptyBarrier,
                                 blockIdx.x);
          if (!ok) break;
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const uint32_t bar = mapa(smem_u32(&full_bar[stage]), 0);      // the leader's barrier
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
          const int k0 = kb * BLOCK_K;
          if constexpr (!A_MN) {
            tma_load_2d_pair(sa, &tmap_a, bar, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < CTA_M / 64; ++j) tma_load_2d_pair(sa + j * ATOM_BYTES, &tmap_a, bar, m0 + 64 * j, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(sb, &tmap_b, bar, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < CTA_NB / 64; ++j) tma_load_2d_pair(sb + j * ATOM_BYTES, &tmap_b, bar, n0 + 64 * j, k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader) --
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc(1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0, TILE_M, TILE_N);
      int stage = 0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++local_tile) {
        const int buf = local_tile & 1;
        const uint32_t buf_phase = (local_tile >> 1) & 1;
        ok = mbar_wait_bounded(&tmem_empty[buf], buf_phase ^ 1, abort_flag, p.status, kTimeoutTmemEmpty,
                               blockIdx.x);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * TILE_N;
        for (int kb = 0; kb < num_k; ++kb) {
          ok = mbar_wait_bounded(&full_bar[stage], phase, abort_flag, p.status, kTimeoutFullBarrier, blockIdx.x);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BLOCK_K / UMMA_K; ++kk) {
            uint64_t adesc, bdesc;
            if constexpr (!A_MN) adesc = make_smem_desc_sw128(sa + kk * UMMA_K * 2, 0, 1024);
            else adesc = make_smem_desc_sw128(sa + kk * UMMA_K * 128, ATOM_BYTES, 1024);
            if constexpr (!B_MN) bdesc = make_smem_desc_sw128(sb + kk * UMMA_K * 2, 0, 1024);
            else bdesc = make_smem_desc_sw128(sb + kk * UMMA_K * 128, ATOM_BYTES, 1024);
            umma2_f16(tmem_d, adesc, bdesc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma2_commit_both(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma2_commit_both(&tmem_full[buf]);
      }
      if (!ok) {
        umma2_commit_both(drain_bar);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 100000000ull) {}
      }
    }
  } else {
    // --------------------------------------------------------------- epilogue (both) --
    const int q = warp & 3;
    int local_tile = 0;
    bool ok = true;
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++local_tile) {
      int m_blk, n_blk;
      tile_coords(t, num_m, num_n, m_blk, n_blk);
      const int buf = local_tile & 1;
      const uint32_t buf_phase = (local_tile >> 1) & 1;
      ok = mbar_wait_bounded(&tmem_full[buf], buf_phase, abort_flag, p.status, kTimeoutTmemFull, blockIdx.x);
      if (!ok) break;
      tc_fence_after();
      const int row = m_blk * TILE_M + cta * CTA_M + q * 32 + lane;
      const int col0 = n_blk * TILE_N;
      const uint32_t taddr = tmem_base + buf * TILE_N + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < TILE_N / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = col0 + c * 32;
        if (row < p.M && col < p.N) {
          if constexpr (OUT_F32) {
            float* dst = reinterpret_cast<float*>(p.C) + static_cast<int64_t>(row) * p.ldc + col;
            if (col + 32 <= p.N && (p.ldc & 3) == 0) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                       __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                float4* d4 = reinterpret_cast<float4*>(dst) + j;
                if constexpr (ACCUM) {
                  float4 o = *d4;
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                *d4 = v;
              }
            } else {
              for (int j = 0; j < 32 && col + j < p.N; ++j) {
                float v = __uint_as_float(r[j]);
                if constexpr (ACCUM) v += dst[j];
                dst[j] = v;
              }
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<int64_t>(row) * p.ldc + col;
            if (col + 32 <= p.N && (p.ldc & 7) == 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4* d4 = reinterpret_cast<uint4*>(dst) + j;
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * j + e]);
                if constexpr (ACCUM) {
                  uint4 o = *d4;
                  const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    float2 of = __bfloat1622float2(ob[e]);
                    f[2 * e] += of.x;
                    f[2 * e + 1] += of.y;
                  }
                }
                uint4 v;
                __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
                for (int e = 0; e < 4; ++e) vb[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
                *d4 = v;
              }
            } else {
              for (int j = 0; j < 32 && col + j < p.N; ++j) {
                float v = __uint_as_float(r[j]);
                if constexpr (ACCUM) v += __bfloat162float(dst[j]);
                dst[j] = __float2bfloat16(v);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (leader) mbar_arrive(&tmem_empty[buf]);
        else remote_arrive(mapa(smem_u32(&tmem_empty[buf]), 0));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();      // the leader's MMAs read the peer's shared memory: nobody leaves early
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, int num_sms, cudaStream_t stream) {
  auto kern = gemm2_bf16_kernel<A_MN, B_MN, OUT_F32, ACCUM>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int num_tiles = ((p.M + TILE_M - 1) / TILE_M) * ((p.N + TILE_N - 1) / TILE_N);
  int clusters = num_sms / 2;
  if (num_tiles < clusters) clusters = num_tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kern, ta, tb, p));
}


}  // namespace g2

int make_tmap_2d(CUtensorMap* map, const void* ptr, CUtensorMapDataType dtype, int elem_bytes, uint64_t inner,
                 uint64_t outer, uint64_t ld, uint32_t box_inner, uint32_t box_outer);

}  // namespace hpb

// Same arguments as hpb_gemm_bf16; uses CTA pairs.
extern "C" int hpb_gemm2_bf16(const void* A, int a_mn, int64_t lda, const void* B, int b_mn, int64_t ldb, void* C,
                              int64_t ldc, int out_f32, int accumulate, int M, int N, int K, int* status,
                              int num_sms, cudaStream_t stream) {
  using namespace hpb;
  using namespace hpb::g2;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -2;
  cudaFree(nullptr);
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, BLOCK_K, CTA_M);
  else r = make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, 64, BLOCK_K);
  if (r) return r;
  if (!b_mn) r = make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BLOCK_K, CTA_NB);
  else r = make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, 64, BLOCK_K);
  if (r) return r;
  Params p{M, N, K, C, ldc, status};
  const int key = (a_mn ? 8 : 0) | (b_mn ? 4 : 0) | (out_f32 ? 2 : 0) | (accumulate ? 1 : 0);
  switch (key) {
#define HPB_CASE(k, a, b, o, c) \
  case k:                       \
    return g2::launch<a, b, o, c>(ta, tb, p, num_sms, stream);
    HPB_CASE(0, false, false, false, false)
    HPB_CASE(1, false, false, false, true)
    HPB_CASE(2, false, false, true, false)
    HPB_CASE(3, false, false, true, true)
    HPB_CASE(4, false, true, false, false)
    HPB_CASE(5, false, true, false, true)
    HPB_CASE(6, false, true, true, false)
    HPB_CASE(7, false, true, true, true)
    HPB_CASE(8, true, false, false, false)
    HPB_CASE(9, true, false, false, true)
    HPB_CASE(10, true, false, true, false)
    HPB_CASE(11, true, false, true, true)
    HPB_CASE(12, true, true, false, false)
    HPB_CASE(13, true, true, false, true)
    HPB_CASE(14, true, true, true, false)
    HPB_CASE(15, true, true, true, true)
#undef HPB_CASE
  }
  return -3;
}

