// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sm_100a).
//
//   hpb_ag_gemm : C[n*Ms, N] = gather_r(A_r[Ms, K]) * B[N, K]^T         ("all-gather -> GEMM")
//   hpb_gemm_rs : out[Ms, N]  = sum_r (A_r[n*Ms, K] * B_r[N, K]^T)[my rows]   ("GEMM -> reduce-scatter")
//
// Both are ONE persistent tcgen05 kernel per rank (128x256x64 tiles, TMA-fed, TMEM accumulators,
// same pipeline as gemm_sm100.cu) with two extra "communication" warps per CTA.
//
// all-gather -> GEMM.  Every rank's activation shard sits in symmetric memory.  The communication
// warps of all CTAs copy the panels (own shard first, then peer r+1, r+2, ...) with 16-byte loads
// from the peers' memory into a LOCAL staging matrix and bump a per-panel counter; the TMA producer
// waits (bounded) for a panel's counter before it loads tiles of that panel from local memory.  A
// remote panel therefore crosses NVLink exactly once and its transfer overlaps the math of the panels
// that are already there.  No TMA load touches peer memory and none uses cluster multicast.
//
// GEMM -> reduce-scatter.  Output tiles are produced destination by destination (peers first, own
// rows last); the epilogue stores a tile whose rows belong to rank r straight into r's receive slot
// `recv[src = me]` in symmetric memory (peer stores), and the CTA that completes the last tile of a
// destination publishes a flag there.  The tiles of a rank's own rows come last: their epilogue
// waits (bounded) for the flags of all sources, adds the received partial slabs to the fp32
// accumulator and writes the bf16 output shard.
//
// Cross-rank ordering uses signal pads with monotonically increasing epochs (st.release.sys /
// ld.acquire.sys); every wait is bounded and reports through the status word.
#include "sm100_common.cuh"

namespace hpb {
namespace gc {

constexpr int BLOCK_M = 128, BLOCK_N = 256, BLOCK_K = 64, UMMA_K = 16, STAGES = 4;
constexpr int A_TILE = BLOCK_M * BLOCK_K * 2, B_TILE = BLOCK_N * BLOCK_K * 2, STAGE_BYTES = A_TILE + B_TILE;
constexpr int THREADS = 256;            // producer, MMA, 4 epilogue warps, 2 communication warps
constexpr int COMM_THREADS = 64;
constexpr int TMEM_COLS = 512;
constexpr int XPOSE_BYTES = 32 * 128;    // per epilogue warp: 32 rows x 64 bf16, for 128-byte peer stores
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + 4 * XPOSE_BYTES;
constexpr int kMaxPeers = 8;
constexpr int kSlots = 16;              // flags per signal slot

struct Peers {
  void* ptr[kMaxPeers];
};

struct AgParams {
  int Ms, N, K, n, rank;        // rows per shard, output columns, contraction, ranks, my rank
  Peers shards;                 // every rank's A shard [Ms, K] (bf16, symmetric memory)
  Peers pads;                   // every rank's signal pad
  void* staging;                // local [n*Ms, K] bf16
  unsigned* panel_count;        // local [n] counters (zero before launch)
  void* C;
  long long ldc;
  unsigned epoch;
  unsigned long long limit_ns;
  int* status;
};

struct RsParams {
  int Ms, N, K, n, rank;        // output rows per rank, columns, contraction, ranks, my rank
  Peers recv;                   // every rank's receive area [n][Ms, N] bf16 (symmetric memory)
  Peers pads;
  unsigned* dest_count;         // local [n] tile counters (zero before launch)
  void* out;                    // local [Ms, N] bf16
  unsigned epoch;
  unsigned long long limit_ns;
  int* status;
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}
// spin (bounded) until *p reaches `target`; acquire at system scope
__device__ __forceinline__ bool wait_flag_sys(const unsigned* p, unsigned target, unsigned long long limit_ns,
                                              volatile int* abort_flag, int* status, int detail) {
  const uint64_t t0 = globaltimer_ns();
  unsigned it = 0;
  while (static_cast<int>(ld_acquire_sys(p) - target) < 0) {
    if ((++it & 0x3f) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        report_error(status, kTimeoutPeerFlag, detail);
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ bool wait_count_gpu(const unsigned* p, unsigned target, unsigned long long limit_ns,
                                               volatile int* abort_flag, int* status, int detail) {
  const uint64_t t0 = globaltimer_ns();
  unsigned it = 0;
  while (ld_acquire_gpu(p) < target) {
    if ((++it & 0x3f) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        report_error(status, kTimeoutPeerFlag, 0x1000 | detail);
        return false;
      }
    }
  }
  return true;
}

struct Smem {
  uint8_t* base;
  uint64_t *full_bar, *empty_bar, *tmem_full, *tmem_empty, *drain_bar;
  uint32_t* tmem_slot;
  volatile int* abort_flag;
};
__device__ __forceinline__ Smem carve(uint8_t* raw) {
  Smem s;
  s.base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~static_cast<uintptr_t>(1023));
  s.full_bar = reinterpret_cast<uint64_t*>(s.base + STAGES * STAGE_BYTES);
  s.empty_bar = s.full_bar + STAGES;
  s.tmem_full = s.empty_bar + STAGES;
  s.tmem_empty = s.tmem_full + 2;
  s.drain_bar = s.tmem_empty + 2;
  s.tmem_slot = reinterpret_cast<uint32_t*>(s.drain_bar + 1);
  s.abort_flag = reinterpret_cast<volatile int*>(s.tmem_slot + 1);
  return s;
}
__device__ __forceinline__ void init_pipeline(const Smem& s, int warp) {
  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&s.full_bar[i], 1);
      mbar_init(&s.empty_bar[i], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s.tmem_full[b], 1);
      mbar_init(&s.tmem_empty[b], 4);
    }
    mbar_init(s.drain_bar, 1);
    *s.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(s.tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
}

// One K loop of UMMAs for the tile whose operands arrive through the smem ring.
__device__ __forceinline__ bool mma_tile(const Smem& s, uint32_t tmem_d, int num_k, int& stage, uint32_t& phase,
                                         int* status) {
  constexpr uint32_t idesc = make_idesc(1, 1, 0, 0, BLOCK_M, BLOCK_N);
  for (int kb = 0; kb < num_k; ++kb) {
    if (!mbar_wait_bounded(&s.full_bar[stage], phase, s.abort_flag, status, kTimeoutFullBarrier, blockIdx.x))
      return false;
    tc_fence_after();
    const uint32_t sa = smem_u32(s.base + stage * STAGE_BYTES), sb = sa + A_TILE;
#pragma unroll
    for (int kk = 0; kk < BLOCK_K / UMMA_K; ++kk)
      umma_f16(tmem_d, make_smem_desc_sw128(sa + kk * UMMA_K * 2, 0, 1024),
               make_smem_desc_sw128(sb + kk * UMMA_K * 2, 0, 1024), idesc, (kb > 0 || kk > 0) ? 1u : 0u);
    umma_commit(&s.empty_bar[stage]);
    if (++stage == STAGES) { stage = 0; phase ^= 1; }
  }
  return true;
}

// Store 32 fp32 accumulators of one row as bf16 (vector path needs 16-byte alignment).
__device__ __forceinline__ void store_row32(__nv_bfloat16* dst, const uint32_t (&r)[32], int valid, bool vec_ok) {
  if (valid >= 32 && vec_ok) {
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
    for (int j = 0; j < 32 && j < valid; ++j) dst[j] = __float2bfloat16(__uint_as_float(r[j]));
  }
}

// ------------------------------------------------------------ all-gather -> GEMM --
__global__ void __launch_bounds__(THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const AgParams p) {
  extern __shared__ uint8_t smem_raw[];
  const Smem s = carve(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  init_pipeline(s, warp);
  const uint32_t tmem_base = *s.tmem_slot;
  const int mb_per_panel = (p.Ms + BLOCK_M - 1) / BLOCK_M;
  const int num_n = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int tiles_per_panel = mb_per_panel * num_n;
  const int num_tiles = p.n * tiles_per_panel;
  const int num_k = (p.K + BLOCK_K - 1) / BLOCK_K;
  // tile t -> (panel order index, m block inside the panel, n block); panels are visited in
  // arrival order: own shard, then rank+1, rank+2, ...
  auto decode = [&](int t, int& panel, int& m0, int& n0) {
    const int pi = t / tiles_per_panel, r = t - pi * tiles_per_panel;
    panel = (p.rank + pi) % p.n;
    m0 = panel * p.Ms + (r % mb_per_panel) * BLOCK_M;
    n0 = (r / mb_per_panel) * BLOCK_N;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int have_panel = -1;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int panel, m0, n0;
        decode(t, panel, m0, n0);
        if (panel != have_panel) {
          ok = wait_count_gpu(p.panel_count + panel, gridDim.x, p.limit_ns, s.abort_flag, p.status, panel);
          if (!ok) break;
          fence_proxy_async_global();         // the staging rows were written with generic stores
          have_panel = panel;
        }
        for (int kb = 0; kb < num_k; ++kb) {
          ok = mbar_wait_bounded(&s.empty_bar[stage], phase ^ 1, s.abort_flag, p.status, kTimeoutEmptyBarrier,
                                 blockIdx.x);
          if (!ok) break;
          uint8_t* sa = s.base + stage * STAGE_BYTES;
          mbar_arrive_expect_tx(&s.full_bar[stage], STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, &s.full_bar[stage], kb * BLOCK_K, m0);
          tma_load_2d(sa + A_TILE, &tmap_b, &s.full_bar[stage], kb * BLOCK_K, n0);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0, local_tile = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local_tile) {
        const int buf = local_tile & 1;
        ok = mbar_wait_bounded(&s.tmem_empty[buf], ((local_tile >> 1) & 1) ^ 1, s.abort_flag, p.status,
                               kTimeoutTmemEmpty, blockIdx.x);
        if (!ok) break;
        tc_fence_after();
        ok = mma_tile(s, tmem_base + buf * BLOCK_N, num_k, stage, phase, p.status);
        if (ok) umma_commit(&s.tmem_full[buf]);
      }
      if (!ok) {
        umma_commit(s.drain_bar);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(s.drain_bar, 0) && globaltimer_ns() - t0 < 100000000ull) {}
      }
    }
  } else if (warp < 6) {
    const int q = warp & 3;
    int local_tile = 0;
    bool ok = true;
    const bool vec_ok = (p.ldc & 7) == 0;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local_tile) {
      int panel, m0, n0;
      decode(t, panel, m0, n0);
      const int buf = local_tile & 1;
      ok = mbar_wait_bounded(&s.tmem_full[buf], (local_tile >> 1) & 1, s.abort_flag, p.status, kTimeoutTmemFull,
                             blockIdx.x);
      if (!ok) break;
      tc_fence_after();
      const int row_in_panel = m0 - panel * p.Ms + q * 32 + lane;
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + buf * BLOCK_N + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BLOCK_N / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (row_in_panel < p.Ms && col < p.N)
          store_row32(reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col, r,
                      p.N - col, vec_ok);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.tmem_empty[buf]);
    }
  } else {
    // ------------------------------------------------ communication warps: pull the panels --
    const int ct = threadIdx.x - 6 * 32;                       // 0..63
    const long long panel_vecs = static_cast<long long>(p.Ms) * p.K / 8;     // 16-byte vectors per panel
    const long long per_cta = (panel_vecs + gridDim.x - 1) / gridDim.x;
    const long long v0 = blockIdx.x * per_cta, v1 = min(v0 + per_cta, panel_vecs);
    if (blockIdx.x == 0 && ct < p.n)                           // "my shard of this call is in place"
      st_release_sys(reinterpret_cast<unsigned*>(p.pads.ptr[ct]) + 0 * kSlots + p.rank, p.epoch);
    bool ok = true;
    for (int pi = 0; pi < p.n && ok; ++pi) {
      const int r = (p.rank + pi) % p.n;
      if (r != p.rank) {
        if (ct == 0)
          ok = wait_flag_sys(reinterpret_cast<const unsigned*>(p.pads.ptr[p.rank]) + 0 * kSlots + r, p.epoch,
                             p.limit_ns, s.abort_flag, p.status, r);
        ok = __shfl_sync(0xffffffffu, ok, 0) && !*s.abort_flag;
        asm volatile("bar.sync 1, 64;" ::: "memory");
        if (*s.abort_flag) ok = false;
      }
      if (ok) {
        const uint4* src = reinterpret_cast<const uint4*>(p.shards.ptr[r]);
        uint4* dst = reinterpret_cast<uint4*>(p.staging) + static_cast<long long>(r) * panel_vecs;
        long long i = v0 + ct;
        for (; i + 3 * COMM_THREADS < v1; i += 4 * COMM_THREADS) {
          const uint4 a0 = src[i], a1 = src[i + COMM_THREADS], a2 = src[i + 2 * COMM_THREADS],
                      a3 = src[i + 3 * COMM_THREADS];
          dst[i] = a0; dst[i + COMM_THREADS] = a1; dst[i + 2 * COMM_THREADS] = a2; dst[i + 3 * COMM_THREADS] = a3;
        }
        for (; i < v1; i += COMM_THREADS) dst[i] = src[i];
        __threadfence();
      }
      asm volatile("bar.sync 1, 64;" ::: "memory");
      if (ct == 0) atomicAdd(p.panel_count + r, 1u);             // even after a failure: nobody spins on us
    }
    // No "done reading" signal is needed: callers alternate between two shard buffers, and a rank can
    // only start call i+2 (which overwrites the buffer of call i) after its call i+1 saw every peer's
    // "in place" signal of call i+1, which a peer sends after its call i has completed.
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// --------------------------------------------------------- GEMM -> reduce-scatter --
__global__ void __launch_bounds__(THREADS, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const RsParams p) {
  extern __shared__ uint8_t smem_raw[];
  const Smem s = carve(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  init_pipeline(s, warp);
  const uint32_t tmem_base = *s.tmem_slot;
  const int mb_per_dest = (p.Ms + BLOCK_M - 1) / BLOCK_M;
  const int num_n = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int tiles_per_dest = mb_per_dest * num_n;
  const int num_tiles = p.n * tiles_per_dest;
  const int num_k = (p.K + BLOCK_K - 1) / BLOCK_K;
  // destinations in the order rank+1, rank+2, ..., rank (own rows last)
  auto decode = [&](int t, int& dest, int& m_local, int& n0) {
    const int di = t / tiles_per_dest, r = t - di * tiles_per_dest;
    dest = (p.rank + 1 + di) % p.n;
    m_local = (r % mb_per_dest) * BLOCK_M;
    n0 = (r / mb_per_dest) * BLOCK_N;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int dest, m_local, n0;
        decode(t, dest, m_local, n0);
        const int m0 = dest * p.Ms + m_local;
        for (int kb = 0; kb < num_k; ++kb) {
          ok = mbar_wait_bounded(&s.empty_bar[stage], phase ^ 1, s.abort_flag, p.status, kTimeoutEmptyBarrier,
                                 blockIdx.x);
          if (!ok) break;
          uint8_t* sa = s.base + stage * STAGE_BYTES;
          mbar_arrive_expect_tx(&s.full_bar[stage], STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, &s.full_bar[stage], kb * BLOCK_K, m0);
          tma_load_2d(sa + A_TILE, &tmap_b, &s.full_bar[stage], kb * BLOCK_K, n0);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0, local_tile = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local_tile) {
        const int buf = local_tile & 1;
        ok = mbar_wait_bounded(&s.tmem_empty[buf], ((local_tile >> 1) & 1) ^ 1, s.abort_flag, p.status,
                               kTimeoutTmemEmpty, blockIdx.x);
        if (!ok) break;
        tc_fence_after();
        ok = mma_tile(s, tmem_base + buf * BLOCK_N, num_k, stage, phase, p.status);
        if (ok) umma_commit(&s.tmem_full[buf]);
      }
      if (!ok) {
        umma_commit(s.drain_bar);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(s.drain_bar, 0) && globaltimer_ns() - t0 < 100000000ull) {}
      }
    }
  } else if (warp < 6) {
    // ---------------------------------------------------------------- epilogue --
    // Tiles for a peer: bf16 rows are transposed through a per-warp shared-memory tile so that
    // every store instruction writes four full 128-byte lines of the peer's receive slab (row-
    // owned 16-byte stores would cross NVLink as partial sectors).  One system fence and one
    // counter update per (warp, destination), not per tile.  Tiles of this rank's own rows come
    // last: by then the peers' partial slabs have arrived, and the epilogue adds them to the
    // accumulator and writes the final output -- there is no separate reduction pass.
    const int q = warp & 3;
    int local_tile = 0;
    bool ok = true;
    uint8_t* xp = s.base + STAGES * STAGE_BYTES + 256 + q * XPOSE_BYTES;
    int cur_dest = -1;
    unsigned cur_cnt = 0;
    bool have_peers = false;
    auto publish = [&]() {
      if (cur_dest >= 0 && cur_dest != p.rank && cur_cnt > 0) {
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          const unsigned done = atomicAdd(p.dest_count + cur_dest, cur_cnt) + cur_cnt;
          if (done == static_cast<unsigned>(tiles_per_dest) * 4u) {
            __threadfence_system();
            st_release_sys(reinterpret_cast<unsigned*>(p.pads.ptr[cur_dest]) + 2 * kSlots + p.rank, p.epoch);
          }
        }
      }
      cur_cnt = 0;
    };
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local_tile) {
      int dest, m_local, n0;
      decode(t, dest, m_local, n0);
      if (dest != cur_dest) {
        publish();
        cur_dest = dest;
      }
      const int buf = local_tile & 1;
      ok = mbar_wait_bounded(&s.tmem_full[buf], (local_tile >> 1) & 1, s.abort_flag, p.status, kTimeoutTmemFull,
                             blockIdx.x);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + buf * BLOCK_N + (static_cast<uint32_t>(q * 32) << 16);
      const int row0 = m_local + q * 32;                       // first row of this warp inside the slab
      if (dest != p.rank) {
        __nv_bfloat16* slab = reinterpret_cast<__nv_bfloat16*>(p.recv.ptr[dest]) +
                              static_cast<long long>(p.rank) * p.Ms * p.N;
#pragma unroll 1
        for (int c = 0; c < BLOCK_N / 64; ++c) {
          uint32_t r[64];
          tmem_ld_32x32b_x32(taddr + c * 64, *reinterpret_cast<uint32_t(*)[32]>(r));
          tmem_ld_32x32b_x32(taddr + c * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(r + 32));
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 v;
            __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              vb[e] = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * e]), __uint_as_float(r[8 * j + 2 * e + 1]));
            *reinterpret_cast<uint4*>(xp + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
          }
          __syncwarp();
          const int col = n0 + c * 64 + (lane & 7) * 8;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = i * 4 + (lane >> 3);
            const uint4 v = *reinterpret_cast<const uint4*>(xp + rr * 128 + (((lane & 7) ^ (rr & 7)) << 4));
            if (row0 + rr < p.Ms && col < p.N)
              *reinterpret_cast<uint4*>(slab + static_cast<long long>(row0 + rr) * p.N + col) = v;
          }
          __syncwarp();
        }
      } else {
        if (!have_peers) {
          // all partial slabs for my rows must have landed (flags raised by the peers' epilogues)
          bool got = true;
          if (lane < p.n && lane != p.rank)
            got = wait_flag_sys(reinterpret_cast<const unsigned*>(p.pads.ptr[p.rank]) + 2 * kSlots + lane, p.epoch,
                                p.limit_ns, s.abort_flag, p.status, 0x200 | lane);
          ok = __all_sync(0xffffffffu, got);
          if (!ok) break;
          have_peers = true;
        }
        const int row = row0 + lane;
        const long long slab_elems = static_cast<long long>(p.Ms) * p.N;
        const __nv_bfloat16* mine = reinterpret_cast<const __nv_bfloat16*>(p.recv.ptr[p.rank]);
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out);
#pragma unroll 1
        for (int c = 0; c < BLOCK_N / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c * 32, r);
          tmem_ld_wait();
          const int col = n0 + c * 32;
          if (row < p.Ms && col < p.N) {
            const long long off = static_cast<long long>(row) * p.N + col;
            const int nv = min(4, (p.N - col) / 8);
            for (int j = 0; j < nv; ++j) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * j + e]);
              for (int src = 0; src < p.n; ++src) {
                if (src == p.rank) continue;
                const uint4 v = *reinterpret_cast<const uint4*>(mine + src * slab_elems + off + 8 * j);
                const __nv_bfloat162* vb = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 x = __bfloat1622float2(vb[e]);
                  f[2 * e] += x.x;
                  f[2 * e + 1] += x.y;
                }
              }
              uint4 o;
              __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int e = 0; e < 4; ++e) ob[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
              *reinterpret_cast<uint4*>(out + off + 8 * j) = o;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.tmem_empty[buf]);
      ++cur_cnt;
    }
    if (ok) publish();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace gc

int make_tmap_2d(CUtensorMap* map, const void* ptr, CUtensorMapDataType dtype, int elem_bytes, uint64_t inner,
                 uint64_t outer, uint64_t ld, uint32_t box_inner, uint32_t box_outer);

}  // namespace hpb

using namespace hpb;
using namespace hpb::gc;

static int set_smem(const void* kern) {
  static bool done[2][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const int which = kern == reinterpret_cast<const void*>(ag_gemm_kernel) ? 0 : 1;
  if (dev >= 0 && dev < 64 && done[which][dev]) return 0;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev >= 0 && dev < 64) done[which][dev] = true;
  return 0;
}

// shards / pads: arrays of n device pointers.  staging [n*Ms, K] and panel_count [n] (zeroed by the
// caller on the same stream) are local.  B is this rank's weight [N, K]; C is [n*Ms, N] (ldc elements).
extern "C" int hpb_ag_gemm(void* const* shards, void* const* pads, void* staging, unsigned* panel_count,
                           const void* B, void* C, long long ldc, int Ms, int N, int K, int n, int rank,
                           unsigned epoch, unsigned long long limit_ns, int* status, int num_sms,
                           cudaStream_t stream) {
  if (n < 1 || n > kMaxPeers || Ms <= 0 || N <= 0 || K <= 0) return -2;
  if ((K % 8) || (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(staging) & 15) ||
      (static_cast<long long>(Ms) * K) % 8)
    return -2;
  cudaFree(nullptr);
  CUtensorMap ta, tb;
  int r = make_tmap_2d(&ta, staging, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, static_cast<uint64_t>(n) * Ms, K,
                       BLOCK_K, BLOCK_M);
  if (r) return r;
  r = make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, K, BLOCK_K, BLOCK_N);
  if (r) return r;
  AgParams p{};
  p.Ms = Ms; p.N = N; p.K = K; p.n = n; p.rank = rank;
  for (int i = 0; i < kMaxPeers; ++i) {
    p.shards.ptr[i] = i < n ? shards[i] : nullptr;
    p.pads.ptr[i] = i < n ? pads[i] : nullptr;
  }
  p.staging = staging; p.panel_count = panel_count; p.C = C; p.ldc = ldc; p.epoch = epoch;
  p.limit_ns = limit_ns; p.status = status;
  if ((r = set_smem(reinterpret_cast<const void*>(ag_gemm_kernel)))) return r;
  // every CTA contributes to every panel's counter, so all CTAs must be launched (and co-resident)
  ag_gemm_kernel<<<num_sms, THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

// A is this rank's [n*Ms, K] activation (columns of the contraction it owns), B its weight slice
// [N, K]; recv: every rank's receive area [n][Ms, N]; out: local [Ms, N]; dest_count [n] zeroed.
extern "C" int hpb_gemm_rs(const void* A, const void* B, void* const* recv, void* const* pads,
                           unsigned* dest_count, void* out, int Ms, int N, int K, int n, int rank,
                           unsigned epoch, unsigned long long limit_ns, int* status, int num_sms,
                           cudaStream_t stream) {
  if (n < 1 || n > kMaxPeers || Ms <= 0 || N <= 0 || K <= 0) return -2;
  if ((K % 8) || (N % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -2;
  cudaFree(nullptr);
  CUtensorMap ta, tb;
  int r = make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, static_cast<uint64_t>(n) * Ms, K, BLOCK_K,
                       BLOCK_M);
  if (r) return r;
  r = make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, K, BLOCK_K, BLOCK_N);
  if (r) return r;
  RsParams p{};
  p.Ms = Ms; p.N = N; p.K = K; p.n = n; p.rank = rank;
  for (int i = 0; i < kMaxPeers; ++i) {
    p.recv.ptr[i] = i < n ? recv[i] : nullptr;
    p.pads.ptr[i] = i < n ? pads[i] : nullptr;
  }
  p.dest_count = dest_count; p.out = out; p.epoch = epoch; p.limit_ns = limit_ns; p.status = status;
  if ((r = set_smem(reinterpret_cast<const void*>(gemm_rs_kernel)))) return r;
  const int tiles = n * ((Ms + BLOCK_M - 1) / BLOCK_M) * ((N + BLOCK_N - 1) / BLOCK_N);
  gemm_rs_kernel<<<tiles < num_sms ? tiles : num_sms, THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}
