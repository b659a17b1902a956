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
#include "sm100_common.cuh"

#include <stdlib.h>

namespace hpb {
namespace g2 {

constexpr int TILE_M = 256;            // per CTA pair
constexpr int TILE_N = 256;
constexpr int CTA_M = 128;             // rows of A / C per CTA
constexpr int CTA_NB = 128;            // rows of B loaded per CTA
constexpr int BLOCK_K = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int A_BYTES = CTA_M * BLOCK_K * 2;    // 16 KB
constexpr int B_BYTES = CTA_NB * BLOCK_K * 2;   // 16 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // 32 KB
constexpr int ATOM_BYTES = 64 * BLOCK_K * 2;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 8;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

struct Params {
  int M, N, K;
  void* C;
  int64_t ldc;
  int* status;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void remote_arrive(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tiled load into THIS CTA's shared memory; completion bytes go to the barrier at
// `bar_cluster_addr` (the leader's barrier).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at this shared-memory offset in BOTH CTAs once the MMAs issued so far retire
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(static_cast<uint16_t>(3))
      : "memory");
}

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& m_blk, int& n_blk) {
  const int per_group = GROUP_M * num_n;
  const int group = t / per_group;
  const int first_m = group * GROUP_M;
  const int gsz = min(num_m - first_m, GROUP_M);
  const int r = t - group * per_group;
  m_blk = first_m + r % gsz;
  n_blk = r / gsz;
}

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


// ====================================================================================
// HSDP weight all-gather fused into the GEMM that consumes the weight.
//
//   forward : C[M, N]  = A[M, K] * W[N, K]^T        (W is the K-major B operand)
//   dgrad   : C[M, Kin] = A[M, Nout] * W[Nout, Kin]  (W is the MN-major B operand; the
//                                                    contraction runs over W's rows)
//
// W is sharded over `n` ranks along its rows (rank r owns rows [r*Ns, (r+1)*Ns), one
// contiguous chunk of `shard_elems` elements in r's symmetric memory).  Four extra warps per
// CTA ("communication warps") claim 16 KB chunks of W from a device-side work queue -- own
// shard first, then rank+1, rank+2, ... -- and copy them with 16-byte loads (peer loads over
// NVLink for remote chunks) into a LOCAL staging matrix; a per-panel counter (panel = 128 rows
// of W) grows with every finished chunk.  The TMA producer of a tile waits (bounded) until the
// panels it is about to load are complete, then loads from local memory with ordinary per-CTA
// TMA.  Tiles (forward) or K blocks (dgrad) are visited in arrival order, so the math on the
// rows that are already here hides the transfer of the rest.  No TMA load touches peer memory.
//
// The work queue makes the CTAs independent of each other's residency: a chunk is copied by
// whichever resident CTA claims it, so the kernel does not need every CTA of the grid (or the
// whole GPU) to be co-resident.  The only cross-GPU wait is for the peers' "shard version"
// flag, which a rank publishes when its optimizer step has rewritten its shard; nothing waits
// for a peer's kernel of the same step.
struct GatherParams {
  const void* shard[16];      // every rank's shard of this weight (bf16)
  const uint32_t* my_pad;     // this rank's signal pad (null: single rank / versions not used)
  uint4* staging;             // local full weight [rows, row_elems], contiguous
  unsigned* panel_cnt;        // [num_panels] chunk counters, grow by the panel's chunk count per launch
  unsigned* done_total;       // chunks copied so far over all launches (grows by num_chunks per launch)
  int num_panels;
  unsigned* claim;            // work-queue head; zero between launches (the last claimer resets it)
  long long shard_elems;      // elements per rank
  long long total_vecs;       // n * shard_elems / 8
  long long panel_vecs;       // 128 * row_elems / 8 (a multiple of chunk_vecs)
  int chunk_vecs;             // 16-byte vectors per work-queue item: 1024 or 2048
  int group_m;                // m blocks per raster group (forward: how fast the sweep over W is)
  int n, rank;
  int first_unit;             // forward: first n block of the rotation; dgrad: first k block
  int first_chunk;            // first chunk of the copy order (the chunk that holds my first element)
  unsigned seq;               // number of gathers of this weight so far, this one included
  unsigned version;           // peers' shards must have reached this version
  int version_slot;           // signal-pad slot of the version flags
  unsigned long long limit_ns;
};

constexpr int kCommThreads = 128;
constexpr int kMaxChunkVecs = 2048;            // 32 KB: 16 independent 16-byte loads per thread in flight
constexpr int THREADS_G = THREADS + kCommThreads;

__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_relaxed_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
// the staging rows were written with generic-proxy stores; TMA reads through the async proxy
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ unsigned panel_chunks(const GatherParams& g, int panel) {
  const long long left = g.total_vecs - static_cast<long long>(panel) * g.panel_vecs;
  const long long v = left < g.panel_vecs ? left : g.panel_vecs;
  return v <= 0 ? 0u : static_cast<unsigned>((v + g.chunk_vecs - 1) / g.chunk_vecs);
}

// Bounded wait until panel `panel` of the staging matrix is complete.
__device__ __forceinline__ bool wait_panel(const GatherParams& g, int panel, volatile int* abort_flag, int* status) {
  const unsigned target = g.seq * panel_chunks(g, panel);
  const unsigned* p = g.panel_cnt + panel;
  if (static_cast<int>(ld_acquire_gpu_u32(p) - target) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  unsigned it = 0;
  while (static_cast<int>(ld_acquire_gpu_u32(p) - target) < 0) {
    if ((++it & 0x3f) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > g.limit_ns) {
        *abort_flag = 1;
        report_error(status, kTimeoutPeerFlag, 0x2000 | panel);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void tile_coords_g(int t, int num_m, int num_n, int group_m, int& m_blk, int& n_blk) {
  const int per_group = group_m * num_n;
  const int group = t / per_group;
  const int first_m = group * group_m;
  const int gsz = min(num_m - first_m, group_m);
  const int r = t - group * per_group;
  m_blk = first_m + r % gsz;
  n_blk = r / gsz;
}

template <bool B_MN>
__global__ void __launch_bounds__(THREADS_G, 1)
gemm2_agw_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const Params p, const GatherParams g) {
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
  volatile int* s_chunk = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();
  const bool leader = cta == 0;
  const int num_m = (p.M + TILE_M - 1) / TILE_M, num_n = (p.N + TILE_N - 1) / TILE_N;
  const int num_tiles = num_m * num_n;
  const int num_k = (p.K + BLOCK_K - 1) / BLOCK_K;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  // forward: n blocks rotate so that the tiles of my own rows of W come first; dgrad: K blocks do
  const int n_rot = B_MN ? 0 : g.first_unit;
  const int k_rot = B_MN ? g.first_unit : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 8);
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
  cluster_sync();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // -------------------------------------------------------- TMA producer (both CTAs) --
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int have_panel = -1;
      int ahead = 0;
      // Readiness checks are kept off the producer's critical path.  (1) `done_total` says when the
      // WHOLE weight has arrived: its value is fetched with a relaxed load one tile ahead (the load
      // is in flight while the tile's TMA copies are issued) and, once it has reached the target,
      // one acquire fence + one proxy fence make every later check unnecessary.  (2) Until then a
      // forward tile waits for its own panel, and a dgrad tile, which sweeps all panels, checks
      // them eight at a time (eight loads in one round trip instead of one round trip each).
      bool all_ready = false;
      const unsigned total_target = g.seq * static_cast<unsigned>((g.total_vecs + g.chunk_vecs - 1) / g.chunk_vecs);
      unsigned seen_total = ld_relaxed_gpu_u32(g.done_total);
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        int m_blk, n_blk;
        tile_coords_g(t, num_m, num_n, g.group_m, m_blk, n_blk);
        n_blk += n_rot;
        if (n_blk >= num_n) n_blk -= num_n;
        const int m0 = m_blk * TILE_M + cta * CTA_M;
        const int n0 = n_blk * TILE_N + cta * CTA_NB;
        if (!all_ready) {
          if (static_cast<int>(seen_total - total_target) >= 0) {
            fence_acq_rel_gpu();
            fence_proxy_async_all();
            all_ready = true;
          } else {
            seen_total = ld_relaxed_gpu_u32(g.done_total);      // consumed at the next tile
          }
        }
        if constexpr (!B_MN) {
          // my 128 rows of W are exactly one panel
          if (!all_ready && n0 < p.N) {
            ok = wait_panel(g, n0 >> 7, abort_flag, p.status);
            if (!ok) break;
            fence_proxy_async_all();
          }
        }
        for (int kb = 0; kb < num_k; ++kb) {
          int kr = kb + k_rot;
          if (kr >= num_k) kr -= num_k;
          const int k0 = kr * BLOCK_K;
          if constexpr (B_MN) {
            const int panel = k0 >> 7;
            if (!all_ready && panel != have_panel) {
              have_panel = panel;
              if (ahead == 0) {
                for (int j = 0; j < 8 && ok; ++j) {
                  int pj = panel + j;
                  if (pj >= g.num_panels) pj -= g.num_panels;
                  ok = wait_panel(g, pj, abort_flag, p.status);
                }
                if (!ok) break;
                fence_proxy_async_all();
                ahead = 8;
              }
              --ahead;
            }
          }
          ok = mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kTimeoutEmptyBarrier,
                                 blockIdx.x);
          if (!ok) break;
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const uint32_t bar = mapa(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
          tma_load_2d_pair(sa, &tmap_a, bar, k0, m0);
          if constexpr (!B_MN) {
            tma_load_2d_pair(sb, &tmap_b, bar, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < CTA_NB / 64; ++j) tma_load_2d_pair(sb + j * ATOM_BYTES, &tmap_b, bar, n0 + 64 * j, k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (B_MN && ok) all_ready = true;       // a dgrad tile has swept (and checked) every panel
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader) --
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc(1, 1, 0, B_MN ? 1 : 0, TILE_M, TILE_N);
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
            const uint64_t adesc = make_smem_desc_sw128(sa + kk * UMMA_K * 2, 0, 1024);
            uint64_t bdesc;
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
  } else if (warp < 6) {
    // --------------------------------------------------------------- epilogue (both) --
    const int q = warp & 3;
    int local_tile = 0;
    bool ok = true;
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++local_tile) {
      int m_blk, n_blk;
      tile_coords_g(t, num_m, num_n, g.group_m, m_blk, n_blk);
      n_blk += n_rot;
      if (n_blk >= num_n) n_blk -= num_n;
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
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<int64_t>(row) * p.ldc + col;
          if (col + 32 <= p.N && (p.ldc & 7) == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v;
              __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
              for (int e = 0; e < 4; ++e)
                vb[e] = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * e]), __uint_as_float(r[8 * j + 2 * e + 1]));
              reinterpret_cast<uint4*>(dst)[j] = v;
            }
          } else {
            for (int j = 0; j < 32 && col + j < p.N; ++j) dst[j] = __float2bfloat16(__uint_as_float(r[j]));
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
  } else {
    // ------------------------------------------- communication warps: gather the weight --
    const int ct = threadIdx.x - 6 * 32;                  // 0 .. kCommThreads-1
    const int cv = g.chunk_vecs;
    const unsigned num_chunks = static_cast<unsigned>((g.total_vecs + cv - 1) / cv);
    unsigned verified = 1u << g.rank;                     // peers whose shard version has been seen
    for (;;) {
      if (ct == 0) {
        const unsigned idx = atomicAdd(g.claim, 1u);
        int c = -1;
        if (idx < num_chunks) {
          unsigned cc = idx + static_cast<unsigned>(g.first_chunk);
          if (cc >= num_chunks) cc -= num_chunks;
          c = static_cast<int>(cc);
          if (g.my_pad != nullptr) {
            const long long e0 = static_cast<long long>(cc) * cv * 8;
            const long long e1 = min(e0 + static_cast<long long>(cv) * 8, g.total_vecs * 8) - 1;
            const int o0 = static_cast<int>(e0 / g.shard_elems), o1 = static_cast<int>(e1 / g.shard_elems);
            for (int o = o0; o <= o1 && c >= 0; ++o) {
              if (verified & (1u << o)) continue;
              const unsigned* flag = g.my_pad + g.version_slot * 16 + o;   // 16 flags per signal-pad slot
              const uint64_t t0 = globaltimer_ns();
              unsigned it = 0;
              while (static_cast<int>(ld_acquire_sys_u32(flag) - g.version) < 0) {
                if ((++it & 0x3f) == 0 && (*abort_flag || globaltimer_ns() - t0 > g.limit_ns)) {
                  if (!*abort_flag) report_error(p.status, kTimeoutPeerFlag, 0x3000 | o);
                  *abort_flag = 1;
                  c = -2;
                  break;
                }
              }
              if (c >= 0) verified |= 1u << o;
            }
          }
        } else if (idx == num_chunks + gridDim.x - 1) {
          *g.claim = 0u;      // every CTA has made its one failing claim: the queue is idle again
        }
        *s_chunk = c;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const int c = *s_chunk;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (c < 0) break;
      const long long v0 = static_cast<long long>(c) * cv;
      const long long e0 = v0 * 8;
      const int o0 = static_cast<int>(e0 / g.shard_elems);
      const long long bnd = static_cast<long long>(o0 + 1) * g.shard_elems;
      const long long v_end = min(v0 + cv, g.total_vecs);
      uint4 buf[kMaxChunkVecs / kCommThreads];
#pragma unroll
      for (int u = 0; u < kMaxChunkVecs / kCommThreads; ++u) {
        const long long v = v0 + ct + u * kCommThreads;
        if (v < v_end) {
          const long long e = v * 8;
          const int o = o0 + (e >= bnd ? 1 : 0);
          buf[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(g.shard[o]) +
                                                   (e - static_cast<long long>(o) * g.shard_elems));
        }
      }
#pragma unroll
      for (int u = 0; u < kMaxChunkVecs / kCommThreads; ++u) {
        const long long v = v0 + ct + u * kCommThreads;
        if (v < v_end) g.staging[v] = buf[u];
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ct == 0) {
        __threadfence();
        atomicAdd(g.panel_cnt + static_cast<int>(v0 / g.panel_vecs), 1u);
        atomicAdd(g.done_total, 1u);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

template <bool B_MN>
static int launch_agw(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, const GatherParams& g,
                      int num_sms, cudaStream_t stream) {
  auto kern = gemm2_agw_kernel<B_MN>;
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
  if (clusters < 1) clusters = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(THREADS_G, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kern, ta, tb, p, g));
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


// HSDP weight all-gather fused into the consumer GEMM (see gemm2_agw_kernel).
//   w_mn = 0 : C[M, N] = A[M, K] * W^T,  W = [N, K]   (forward)
//   w_mn = 1 : C[M, N] = A[M, K] * W,    W = [K, N]   (dgrad; W rows are the contraction)
// shard_ptrs: n device pointers, rank r's shard of W (w_rows / n rows of w_cols elements each);
// staging: local [w_rows, w_cols] bf16 that receives the gathered weight (it holds all of W when
// the kernel returns); counters: ceil(w_rows / 128) + 2 words (per-panel chunk counters, the
// total, the work-queue head), zeroed once at allocation and owned by this weight; seq: 1, 2, ...
// per launch on this weight.
// my_pad / version_slot / version: the peers' "shard version" flags to wait for (my_pad may be
// null: no wait).  Returns -6 when the shape does not meet the kernel's granularity rules
// (w_cols % 64, shard_elems % 8, shard_elems >= 16384); the caller then gathers separately.
extern "C" int hpb_gemm2_agw(const void* A, int64_t lda, void* const* shard_ptrs, void* staging, int w_mn,
                             int64_t w_rows, int64_t w_cols, void* C, int64_t ldc, int M, int n, int rank,
                             unsigned* counters, unsigned seq, const void* my_pad,
                             int version_slot, unsigned version, unsigned long long limit_ns, int* status,
                             int num_sms, cudaStream_t stream) {
  using namespace hpb;
  using namespace hpb::g2;
  if (M <= 0 || w_rows <= 0 || w_cols <= 0 || n < 1 || n > 16 || rank < 0 || rank >= n) return -2;
  if ((lda % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(staging) & 15)) return -2;
  if ((w_rows % n) || (w_cols % 64)) return -6;
  const long long shard_elems = (w_rows / n) * w_cols;
  if ((shard_elems % 8) || shard_elems < 8 * kMaxChunkVecs || w_rows * w_cols / 8 / 1024 > 0x7fffffffLL) return -6;
  const int N = w_mn ? static_cast<int>(w_cols) : static_cast<int>(w_rows);
  const int K = w_mn ? static_cast<int>(w_rows) : static_cast<int>(w_cols);
  cudaFree(nullptr);
  CUtensorMap ta, tb;
  int r = make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, BLOCK_K, CTA_M);
  if (r) return r;
  if (!w_mn) r = make_tmap_2d(&tb, staging, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, w_cols, BLOCK_K, CTA_NB);
  else r = make_tmap_2d(&tb, staging, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, w_cols, 64, BLOCK_K);
  if (r) return r;
  Params p{M, N, K, C, ldc, status};
  GatherParams g;
  for (int i = 0; i < 16; ++i) g.shard[i] = i < n ? shard_ptrs[i] : nullptr;
  g.my_pad = n > 1 ? reinterpret_cast<const uint32_t*>(my_pad) : nullptr;
  g.staging = reinterpret_cast<uint4*>(staging);
  g.num_panels = static_cast<int>((w_rows + 127) / 128);
  g.panel_cnt = counters;
  g.done_total = counters + g.num_panels;
  g.claim = counters + g.num_panels + 1;
  g.shard_elems = shard_elems;
  g.total_vecs = w_rows * w_cols / 8;
  g.panel_vecs = 128 * w_cols / 8;
  g.n = n;
  g.rank = rank;
  const long long my_row0 = static_cast<long long>(rank) * (w_rows / n);
  if (!w_mn) {
    const int num_n = (N + TILE_N - 1) / TILE_N;
    g.first_unit = static_cast<int>(((my_row0 + TILE_N - 1) / TILE_N) % num_n);
  } else {
    const int num_k = (K + BLOCK_K - 1) / BLOCK_K;
    g.first_unit = static_cast<int>(((my_row0 + BLOCK_K - 1) / BLOCK_K) % num_k);
  }
  g.chunk_vecs = (w_cols % 128 == 0) ? 2048 : 1024;       // a chunk never straddles two panels
  g.first_chunk = static_cast<int>(static_cast<long long>(rank) * shard_elems / 8 / g.chunk_vecs);
  // Forward: a raster group of `group_m` row blocks sweeps all of W once, so the gather has
  // group_m / num_m of the kernel's duration to deliver it: 16 row blocks instead of the 8 of the
  // plain kernel (measured: a full-height group loses more to L2 misses on A than it gains).
  {
    const int num_m = (M + TILE_M - 1) / TILE_M;
    int gm = 2 * GROUP_M;
    if (gm > num_m) gm = num_m;
    g.group_m = w_mn ? GROUP_M : gm;
    if (const char* e = getenv("HPB_AGW_GROUP_M")) {       // tuning override
      const int v = atoi(e);
      if (v > 0) g.group_m = v;
    }
  }
  g.seq = seq;
  g.version = version;
  g.version_slot = version_slot;
  g.limit_ns = limit_ns;
  return w_mn ? g2::launch_agw<true>(ta, tb, p, g, num_sms, stream)
              : g2::launch_agw<false>(ta, tb, p, g, num_sms, stream);
}
