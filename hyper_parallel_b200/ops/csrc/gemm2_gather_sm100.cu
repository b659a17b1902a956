// HSDP weight all-gather carried by the tcgen05 GEMM kernels (CTA pairs, see gemm2_sm100.cu).
//
// A weight W [rows, cols] is sharded over `n` ranks along its rows (rank r owns rows
// [r*Ns, (r+1)*Ns), one contiguous chunk of `shard_elems` elements in r's symmetric memory).
// Gathering it means copying every rank's chunk into a LOCAL staging matrix.  That copy is never
// a kernel of its own: four extra warps per CTA ("communication warps") of the GEMM kernels do it
// while the tensor cores work, pulling remote chunks with 16-byte peer loads over NVLink.  The
// weight is cut into work items of 16 or 32 KB that the CTAs claim from a device-side queue (own
// shard first, then rank+1, rank+2, ...); per-panel counters (panel = 128 rows of W) and a total
// grow with every finished item.
//
// A GEMM launch can carry two gathers:
//   own  : the GEMM CONSUMES the weight as its B operand,
//             forward : C[M, N]   = A[M, K] * W[N, K]^T        (W K-major)
//             dgrad   : C[M, Kin] = A[M, Nout] * W[Nout, Kin]  (W MN-major; its rows are contracted)
//          Its communication warps first finish whatever part of W is still missing; the TMA
//          producer of a tile waits (bounded) for the panels it is about to load -- tiles (forward)
//          or K blocks (dgrad) are visited in arrival order -- and loads them from local memory
//          with ordinary per-CTA TMA.  No TMA load touches peer memory.
//   ride : a weight that a LATER GEMM will consume.  The communication warps work on it for as
//          long as this CTA still has tiles to compute, then stop; the next GEMM continues where
//          they left off (the queue head lives in global memory), and the consumer finishes the
//          rest.  In a steady training loop every weight has therefore arrived before its
//          consumer starts, and no GEMM is stretched by a transfer.
//
// The queue makes the CTAs independent of each other's residency: an item is copied by whichever
// resident CTA claims it, so the kernel does not need every CTA of the grid (or the whole GPU) to
// be co-resident.  The only cross-GPU wait is for the peers' "shard version" flag, which a rank
// publishes when its optimizer step has rewritten its shard; nothing waits for a peer's kernel of
// the same step.  All waits are bounded and report through the status word.
#include "gemm2_pair.cuh"

#include <stdlib.h>
#include <string.h>

namespace hpb {
namespace g2 {

struct GatherParams {
  const void* shard[16];      // every rank's shard of this weight (bf16)
  const uint32_t* my_pad;     // this rank's signal pad (null: versions not used)
  uint4* staging;             // local full weight [rows, row_elems], contiguous
  unsigned* panel_cnt;        // [num_panels] item counters, grow by the panel's item count per round
  unsigned* done_total;       // items copied so far over all rounds (grows by num_items per round)
  unsigned* claim;            // work-queue head of the current round; zero between rounds
  long long shard_elems;      // elements per rank
  long long total_vecs;       // n * shard_elems / 8; zero: no gather
  long long panel_vecs;       // 128 * row_elems / 8 (a multiple of chunk_vecs)
  int num_panels;
  int chunk_vecs;             // 16-byte vectors per work item: 1024 or 2048
  int n, rank;
  int first_unit;             // own, forward: first n block of the rotation; own, dgrad: first k block
  int first_chunk;            // first item of the copy order (the one that holds my first element)
  unsigned seq;               // gather round of this weight: 1, 2, ...
  unsigned version;           // peers' shards must have reached this version
  int version_slot;           // signal-pad slot of the version flags
  unsigned long long limit_ns;
};

constexpr int kCommThreads = 128;
constexpr int kMaxChunkVecs = 2048;            // 32 KB: 16 independent 16-byte loads per thread in flight
constexpr int THREADS_G = THREADS + kCommThreads;
constexpr int GROUP_M_OWN = 16;                // forward raster group while consuming a gathered weight

__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_relaxed_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
// the staging rows were written with generic-proxy stores; TMA reads through the async proxy
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ unsigned num_items(const GatherParams& g) {
  return static_cast<unsigned>((g.total_vecs + g.chunk_vecs - 1) / g.chunk_vecs);
}
__device__ __forceinline__ unsigned panel_items(const GatherParams& g, int panel) {
  const long long left = g.total_vecs - static_cast<long long>(panel) * g.panel_vecs;
  const long long v = left < g.panel_vecs ? left : g.panel_vecs;
  return v <= 0 ? 0u : static_cast<unsigned>((v + g.chunk_vecs - 1) / g.chunk_vecs);
}

// Bounded wait until panel `panel` of the staging matrix is complete.
__device__ __forceinline__ bool wait_panel(const GatherParams& g, int panel, volatile int* abort_flag, int* status) {
  const unsigned target = g.seq * panel_items(g, panel);
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

// The communication warps' loop over one gather.  RIDE = false: this kernel consumes the weight;
// items are claimed with atomicAdd until the queue is empty, every CTA makes exactly one failing
// claim and the last of those resets the head for the next round.  RIDE = true: a later kernel
// consumes it; items are claimed with compare-and-swap (the head never passes the end, so the
// consumer's reset rule still holds) and the loop ends as soon as this CTA's math is done.
// Returns false after a bounded wait expired.
template <bool RIDE>
__device__ __forceinline__ bool gather_loop(const GatherParams& g, int ct, volatile int* abort_flag,
                                            volatile int* math_done, volatile int* s_chunk, int* status) {
  const int cv = g.chunk_vecs;
  const unsigned items = num_items(g);
  unsigned verified = 1u << g.rank;                     // peers whose shard version has been seen
  for (;;) {
    if (ct == 0) {
      int c = -1;
      unsigned idx = items;
      if constexpr (RIDE) {
        if (!*math_done && !*abort_flag) {
          unsigned old = ld_relaxed_gpu_u32(g.claim);
          while (old < items) {
            const unsigned prev = atomicCAS(g.claim, old, old + 1u);
            if (prev == old) {
              idx = old;
              break;
            }
            old = prev;
          }
        }
      } else {
        idx = atomicAdd(g.claim, 1u);
        if (idx == items + gridDim.x - 1) *g.claim = 0u;   // every CTA has made its one failing claim
      }
      if (idx < items) {
        unsigned cc = idx + static_cast<unsigned>(g.first_chunk);
        if (cc >= items) cc -= items;
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
                if (!*abort_flag) report_error(status, kTimeoutPeerFlag, 0x3000 | o);
                *abort_flag = 1;
                c = -2;
                break;
              }
            }
            if (c >= 0) verified |= 1u << o;
          }
        }
      }
      *s_chunk = c;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const int c = *s_chunk;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (c < 0) return c == -1;
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
        if (!HPB_BOUNDS_OK(o >= 0 && o < g.n && e - static_cast<long long>(o) * g.shard_elems + 8 <= g.shard_elems,
                           status, 0x500000 | o)) {
          buf[u] = make_uint4(0u, 0u, 0u, 0u);
          continue;
        }
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

// OWN: the B operand is the staging matrix of `own` (its panels are waited for).  `ride` is
// worked on by the communication warps after `own` is complete, while this CTA has tiles left.
template <bool A_MN, bool B_MN, bool ACCUM, bool OWN>
__global__ void __launch_bounds__(THREADS_G, 1)
gemm2_gather_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const Params p, const GatherParams own, const GatherParams ride, const int group_m) {
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
  volatile int* math_done = abort_flag + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();
  const bool leader = cta == 0;
  const int num_m = (p.M + TILE_M - 1) / TILE_M, num_n = (p.N + TILE_N - 1) / TILE_N;
  const int num_tiles = num_m * num_n;
  const int num_k = (p.K + BLOCK_K - 1) / BLOCK_K;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  // own, forward: n blocks rotate so that the tiles of my own rows of W come first; own, dgrad: K blocks do
  const int n_rot = (OWN && !B_MN) ? own.first_unit : 0;
  const int k_rot = (OWN && B_MN) ? own.first_unit : 0;

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
    *math_done = 0;
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
      bool all_ready = !OWN;
      unsigned total_target = 0, seen_total = 0;
      if constexpr (OWN) {
        total_target = own.seq * num_items(own);
        seen_total = ld_relaxed_gpu_u32(own.done_total);
      }
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        int m_blk, n_blk;
        tile_coords_g(t, num_m, num_n, group_m, m_blk, n_blk);
        n_blk += n_rot;
        if (n_blk >= num_n) n_blk -= num_n;
        const int m0 = m_blk * TILE_M + cta * CTA_M;
        const int n0 = n_blk * TILE_N + cta * CTA_NB;
        if constexpr (OWN) {
          if (!all_ready) {
            if (static_cast<int>(seen_total - total_target) >= 0) {
              fence_acq_rel_gpu();
              fence_proxy_async_all();
              all_ready = true;
            } else {
              seen_total = ld_relaxed_gpu_u32(own.done_total);      // consumed at the next tile
            }
          }
          if constexpr (!B_MN) {
            // my 128 rows of W are exactly one panel
            if (!all_ready && n0 < p.N) {
              ok = wait_panel(own, n0 >> 7, abort_flag, p.status);
              if (!ok) break;
              fence_proxy_async_all();
            }
          }
        }
        for (int kb = 0; kb < num_k; ++kb) {
          int kr = kb + k_rot;
          if (kr >= num_k) kr -= num_k;
          const int k0 = kr * BLOCK_K;
          if constexpr (OWN && B_MN) {
            const int panel = k0 >> 7;
            if (!all_ready && panel != have_panel) {
              have_panel = panel;
              if (ahead == 0) {
                for (int j = 0; j < 8 && ok; ++j) {
                  int pj = panel + j;
                  if (pj >= own.num_panels) pj -= own.num_panels;
                  ok = wait_panel(own, pj, abort_flag, p.status);
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
        if (OWN && B_MN && ok) all_ready = true;       // a dgrad tile has swept (and checked) every panel
      }
      *math_done = 1;       // the last loads are issued: a riding gather stops claiming work
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
  } else if (warp < 6) {
    // --------------------------------------------------------------- epilogue (both) --
    const int q = warp & 3;
    int local_tile = 0;
    bool ok = true;
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++local_tile) {
      int m_blk, n_blk;
      tile_coords_g(t, num_m, num_n, group_m, m_blk, n_blk);
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
              uint4* d4 = reinterpret_cast<uint4*>(dst) + j;
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * j + e]);
              if constexpr (ACCUM) {
                const uint4 o = *d4;
                const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 of = __bfloat1622float2(ob[e]);
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (leader) mbar_arrive(&tmem_empty[buf]);
        else remote_arrive(mapa(smem_u32(&tmem_empty[buf]), 0));
      }
    }
  } else {
    // ------------------------------------------- communication warps: gather the weights --
    const int ct = threadIdx.x - 6 * 32;                  // 0 .. kCommThreads-1
    bool ok = true;
    if constexpr (OWN) ok = gather_loop<false>(own, ct, abort_flag, math_done, s_chunk, p.status);
    if (ok && ride.total_vecs > 0) gather_loop<true>(ride, ct, abort_flag, math_done, s_chunk, p.status);
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN, bool ACCUM, bool OWN>
static int launch_gather(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, const GatherParams& own,
                         const GatherParams& ride, int group_m, int num_sms, cudaStream_t stream) {
  auto kern = gemm2_gather_kernel<A_MN, B_MN, ACCUM, OWN>;
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
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kern, ta, tb, p, own, ride, group_m));
}

}  // namespace g2

int make_tmap_2d(CUtensorMap* map, const void* ptr, CUtensorMapDataType dtype, int elem_bytes, uint64_t inner,
                 uint64_t outer, uint64_t ld, uint32_t box_inner, uint32_t box_outer);

}  // namespace hpb

// One weight to gather (see the header comment).  counters: ceil(rows / 128) + 2 words (per-panel
// item counters, the total, the work-queue head), zeroed once and owned by this weight; seq: the
// gather round, 1, 2, ... -- every launch that works on the same round passes the same value;
// my_pad / version_slot / version: the peers' "shard version" flags to wait for (my_pad may be
// null: no wait).
extern "C" struct HpbGather {
  void* const* shard_ptrs;
  void* staging;
  int64_t rows, cols;
  int n, rank;
  unsigned* counters;
  unsigned seq;
  const void* my_pad;
  int version_slot;
  unsigned version;
};

// 0 when the kernel can gather a weight of this shape over n ranks, else -6 (the caller gathers it
// another way): cols % 64, rows % n, shard a whole number of vectors and at least one work item.
extern "C" int hpb_gather_shape_ok(int64_t rows, int64_t cols, int n) {
  if (rows <= 0 || cols <= 0 || n < 1 || n > 16) return -2;
  if ((rows % n) || (cols % 64)) return -6;
  const long long shard_elems = (rows / n) * cols;
  if ((shard_elems % 8) || shard_elems < 8 * hpb::g2::kMaxChunkVecs || rows * cols / 8 / 1024 > 0x7fffffffLL) return -6;
  return 0;
}

static int fill_gather(hpb::g2::GatherParams& g, const HpbGather* s, unsigned long long limit_ns) {
  using namespace hpb::g2;
  memset(&g, 0, sizeof(g));
  if (s == nullptr || s->staging == nullptr) return 0;
  const int rc = hpb_gather_shape_ok(s->rows, s->cols, s->n);
  if (rc) return rc;
  if (s->rank < 0 || s->rank >= s->n || (reinterpret_cast<uintptr_t>(s->staging) & 15)) return -2;
  for (int i = 0; i < 16; ++i) g.shard[i] = i < s->n ? s->shard_ptrs[i] : nullptr;
  g.my_pad = s->n > 1 ? reinterpret_cast<const uint32_t*>(s->my_pad) : nullptr;
  g.staging = reinterpret_cast<uint4*>(s->staging);
  g.num_panels = static_cast<int>((s->rows + 127) / 128);
  g.panel_cnt = s->counters;
  g.done_total = s->counters + g.num_panels;
  g.claim = s->counters + g.num_panels + 1;
  g.shard_elems = (s->rows / s->n) * s->cols;
  g.total_vecs = s->rows * s->cols / 8;
  g.panel_vecs = 128 * s->cols / 8;
  g.chunk_vecs = (s->cols % 128 == 0) ? 2048 : 1024;       // an item never straddles two panels
  g.n = s->n;
  g.rank = s->rank;
  g.first_chunk = static_cast<int>(static_cast<long long>(s->rank) * g.shard_elems / 8 / g.chunk_vecs);
  g.seq = s->seq;
  g.version = s->version;
  g.version_slot = s->version_slot;
  g.limit_ns = limit_ns;
  return 0;
}

// C[M, N] (+)= opA * opB^T (bf16 out) on the CTA-pair kernel, with up to two weight gathers aboard.
//   own  != null : B is the weight being gathered (its staging matrix); own_w_mn = 0: C = A * W^T
//                  with W [N, K] (forward), own_w_mn = 1: C = A * W with W [K, N] (dgrad).  B, b_mn,
//                  ldb, N and K are taken from `own`; the staging matrix holds all of W afterwards.
//   ride != null : a weight for a later GEMM; copied while this GEMM has tiles left (possibly only
//                  in part -- the queue head stays in `counters`).
// Supported operand orders: (a_mn, b_mn) = (0,0), (0,1), (1,1); accumulate only for (1,1).
extern "C" int hpb_gemm2_gather(const void* A, int a_mn, int64_t lda, const void* B, int b_mn, int64_t ldb, void* C,
                                int64_t ldc, int accumulate, int M, int N, int K, const HpbGather* own,
                                int own_w_mn, const HpbGather* ride, unsigned long long limit_ns, int* status,
                                int num_sms, cudaStream_t stream) {
  using namespace hpb;
  using namespace hpb::g2;
  GatherParams go, gr;
  int r = fill_gather(go, own, limit_ns);
  if (r) return r;
  r = fill_gather(gr, ride, limit_ns);
  if (r) return r;
  const bool has_own = go.total_vecs > 0;
  if (has_own) {
    if (a_mn || accumulate) return -3;
    B = own->staging;
    b_mn = own_w_mn;
    ldb = own->cols;
    N = static_cast<int>(own_w_mn ? own->cols : own->rows);
    K = static_cast<int>(own_w_mn ? own->rows : own->cols);
  }
  if (M <= 0 || N <= 0 || K <= 0) return -2;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -2;
  int group_m = GROUP_M;
  if (has_own) {
    const long long my_row0 = static_cast<long long>(own->rank) * (own->rows / own->n);
    if (!own_w_mn) {
      // A raster group of `group_m` row blocks sweeps all of W once, so the gather has
      // group_m / num_m of the kernel's duration to deliver it: 16 row blocks instead of the 8 of
      // the plain kernel (a full-height group loses more to L2 misses on A than it gains).
      const int num_n = (N + TILE_N - 1) / TILE_N;
      go.first_unit = static_cast<int>(((my_row0 + TILE_N - 1) / TILE_N) % num_n);
      group_m = GROUP_M_OWN;
    } else {
      const int num_k = (K + BLOCK_K - 1) / BLOCK_K;
      go.first_unit = static_cast<int>(((my_row0 + BLOCK_K - 1) / BLOCK_K) % num_k);
    }
  }
  cudaFree(nullptr);
  CUtensorMap ta, tb;
  if (!a_mn) r = make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, BLOCK_K, CTA_M);
  else r = make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, 64, BLOCK_K);
  if (r) return r;
  if (!b_mn) r = make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BLOCK_K, CTA_NB);
  else r = make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, 64, BLOCK_K);
  if (r) return r;
  Params p{M, N, K, C, ldc, status};
  const int key = (a_mn ? 8 : 0) | (b_mn ? 4 : 0) | (accumulate ? 2 : 0) | (has_own ? 1 : 0);
  switch (key) {
    case 0: return g2::launch_gather<false, false, false, false>(ta, tb, p, go, gr, group_m, num_sms, stream);
    case 1: return g2::launch_gather<false, false, false, true>(ta, tb, p, go, gr, group_m, num_sms, stream);
    case 4: return g2::launch_gather<false, true, false, false>(ta, tb, p, go, gr, group_m, num_sms, stream);
    case 5: return g2::launch_gather<false, true, false, true>(ta, tb, p, go, gr, group_m, num_sms, stream);
    case 12: return g2::launch_gather<true, true, false, false>(ta, tb, p, go, gr, group_m, num_sms, stream);
    case 14: return g2::launch_gather<true, true, true, false>(ta, tb, p, go, gr, group_m, num_sms, stream);
  }
  return -3;
}

// The fused gather + GEMM on its own (one weight, consumed by this launch); see hpb_gemm2_gather.
extern "C" int hpb_gemm2_agw(const void* A, int64_t lda, void* const* shard_ptrs, void* staging, int w_mn,
                             int64_t w_rows, int64_t w_cols, void* C, int64_t ldc, int M, int n, int rank,
                             unsigned* counters, unsigned seq, const void* my_pad, int version_slot,
                             unsigned version, unsigned long long limit_ns, int* status, int num_sms,
                             cudaStream_t stream) {
  HpbGather own{shard_ptrs, staging, w_rows, w_cols, n, rank, counters, seq, my_pad, version_slot, version};
  return hpb_gemm2_gather(A, 0, lda, nullptr, 0, 0, C, ldc, 0, M, 0, 0, &own, w_mn, nullptr, limit_ns, status,
                          num_sms, stream);
}
