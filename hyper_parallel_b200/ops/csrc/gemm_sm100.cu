// bf16 GEMM for sm_100a on the 5th-generation tensor cores.
//
//   C[M,N] (+)= sum_k opA[m,k] * opB[n,k]        fp32 accumulation in TMEM
//
// Each operand is either "K-major" (stored [rows, K], K contiguous) or
// "MN-major" (stored [K, rows], rows contiguous), which covers the three GEMMs
// of a linear layer without any transpose copy:
//   forward  y  = x  W^T : A = x  (K-major),  B = W  (K-major)
//   dgrad    dx = dy W   : A = dy (K-major),  B = W  (MN-major)
//   wgrad    dW = dy^T x : A = dy (MN-major), B = x  (MN-major)
//
// Structure: persistent kernel, one CTA per SM, 128x256 output tile, K step 64
// (one 128-byte swizzle atom of bf16), 4-stage TMA->smem ring.  Warp roles:
//   warp 0    : TMA producer (one elected lane)
//   warp 1    : TMEM allocator + tcgen05.mma issuer (one lane)
//   warps 2-5 : epilogue, tcgen05.ld TMEM -> registers -> global
// The 512 TMEM columns hold two 128x256 fp32 accumulators, so the epilogue of
// tile i overlaps the main loop of tile i+1.
//
// All waits are bounded (see sm100_common.cuh); on expiry the kernel records a
// code in `status`, drains, frees TMEM and returns.
#include "sm100_common.cuh"

#include <mutex>
#include <unordered_map>

namespace hpb {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_N = 256;
constexpr int BLOCK_K = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_TILE_BYTES = BLOCK_M * BLOCK_K * 2;  // 16 KB
constexpr int B_TILE_BYTES = BLOCK_N * BLOCK_K * 2;  // 32 KB
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int ATOM_BYTES = 64 * BLOCK_K * 2;  // one 64-wide MN atom: 8 KB
constexpr int GEMM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 8;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;

// mode 0: plain GEMM.
// mode 1: grouped-M.  Rows of A (and C) are grouped by expert, every group padded to a multiple
//         of BLOCK_M; block_group[m_blk] names the expert of each 128-row block; operand B holds
//         all experts stacked along its row axis, b_group_rows rows per expert.
// mode 2: grouped-K (expert weight gradients).  One [M, N] output per expert, stacked in C; the
//         contraction runs over the expert's rows [group_offsets[e], group_offsets[e+1]) of the
//         two MN-major operands (offsets are multiples of BLOCK_K; padding rows are zero).
struct GemmParams {
  int M, N, K;
  void* C;
  int64_t ldc;
  int* status;
  int mode;
  const int* block_group;
  const int* group_offsets;
  int num_groups;
  int b_group_rows;
};

struct TileInfo {
  int m0, n0;        // tile origin in C (mode 2: inside the expert's [M, N] block)
  int group;         // expert (0 for mode 0)
  int k_row0;        // first contraction row (mode 2), else 0
  int num_k;         // number of BLOCK_K steps
};

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& m_blk, int& n_blk) {
  const int per_group = GROUP_M * num_n;
  const int group = t / per_group;
  const int first_m = group * GROUP_M;
  const int gsz = min(num_m - first_m, GROUP_M);
  const int r = t - group * per_group;
  m_blk = first_m + r % gsz;
  n_blk = r / gsz;
}

__device__ __forceinline__ int total_tiles(const GemmParams& p) {
  const int num_m = (p.M + BLOCK_M - 1) / BLOCK_M, num_n = (p.N + BLOCK_N - 1) / BLOCK_N;
  return (p.mode == 2 ? p.num_groups : 1) * num_m * num_n;
}

__device__ __forceinline__ TileInfo tile_info(int t, const GemmParams& p) {
  const int num_m = (p.M + BLOCK_M - 1) / BLOCK_M, num_n = (p.N + BLOCK_N - 1) / BLOCK_N;
  TileInfo ti;
  int m_blk, n_blk;
  if (p.mode == 2) {
    const int per = num_m * num_n;
    ti.group = t / per;
    tile_coords(t - ti.group * per, num_m, num_n, m_blk, n_blk);
    // offsets come from a device-side table: clamp them to the operands' row count (p.K in this
    // mode) so that a corrupt table can never turn into an unbounded K loop
    const int r0 = min(max(p.group_offsets[ti.group], 0), p.K);
    const int r1 = min(max(p.group_offsets[ti.group + 1], r0), p.K);
    ti.k_row0 = r0;
    ti.num_k = (r1 - r0 + BLOCK_K - 1) / BLOCK_K;
  } else {
    tile_coords(t, num_m, num_n, m_blk, n_blk);
    ti.group = p.mode == 1 ? p.block_group[m_blk] : 0;
    if (!HPB_BOUNDS_OK(ti.group < p.num_groups, p.status, 0x400000 | m_blk)) ti.group = -1;   // debug build: skip
    ti.k_row0 = 0;
    // a negative group marks an unused row block of an over-allocated (capacity-sized) operand:
    // no loads, no products, and the epilogue leaves the output rows alone
    ti.num_k = ti.group < 0 ? 0 : (p.K + BLOCK_K - 1) / BLOCK_K;
  }
  ti.m0 = m_blk * BLOCK_M;
  ti.n0 = n_blk * BLOCK_N;
  return ti;
}

template <bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;  // [2]
  uint64_t* tmem_empty = tmem_full + 2;      // [2]
  uint64_t* drain_bar = tmem_empty + 2;      // [1]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = total_tiles(p);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);  // one arrive per epilogue warp
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer --
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const TileInfo ti = tile_info(t, p);
        const int m0 = ti.m0, n0 = ti.n0;
        const int num_k = ti.num_k;
        // row offset of this tile's expert inside the stacked B operand (mode 1)
        const int b_row_off = p.mode == 1 ? ti.group * p.b_group_rows : 0;
        for (int kb = 0; kb < num_k; ++kb) {
          ok = mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, p.status,
                                 kTimeoutEmptyBarrier, blockIdx.x);
          if (!ok) break;
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_TILE_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
          const int k0 = ti.k_row0 + kb * BLOCK_K;
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tmap_a, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BLOCK_M / 64; ++j)
              tma_load_2d(sa + j * ATOM_BYTES, &tmap_a, &full_bar[stage], m0 + 64 * j, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], k0, b_row_off + n0);
          } else {
#pragma unroll
            for (int j = 0; j < BLOCK_N / 64; ++j)
              tma_load_2d(sb + j * ATOM_BYTES, &tmap_b, &full_bar[stage], n0 + 64 * j, b_row_off + k0);
          }
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Drain: wait (bounded, ignoring the abort flag) for the copies this
        // thread issued and nobody consumed, so none lands after the CTA exits.
        int n_back = issued < STAGES ? static_cast<int>(issued) : STAGES;
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < n_back; ++i) {
          if (--s < 0) { s = STAGES - 1; ph ^= 1; }
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&full_bar[s], ph) && globaltimer_ns() - t0 < 100000000ull) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0, BLOCK_M, BLOCK_N);
      int stage = 0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local_tile) {
        const int buf = local_tile & 1;
        const uint32_t buf_phase = (local_tile >> 1) & 1;
        ok = mbar_wait_bounded(&tmem_empty[buf], buf_phase ^ 1, abort_flag, p.status,
                               kTimeoutTmemEmpty, blockIdx.x);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BLOCK_N;
        const int num_k = tile_info(t, p).num_k;
        for (int kb = 0; kb < num_k; ++kb) {
          ok = mbar_wait_bounded(&full_bar[stage], phase, abort_flag, p.status,
                                 kTimeoutFullBarrier, blockIdx.x);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_TILE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BLOCK_K / UMMA_K; ++kk) {
            uint64_t adesc, bdesc;
            if constexpr (!A_MN)
              adesc = make_smem_desc_sw128(sa + kk * UMMA_K * 2, 0, 1024);
            else
              adesc = make_smem_desc_sw128(sa + kk * UMMA_K * 128, ATOM_BYTES, 1024);
            if constexpr (!B_MN)
              bdesc = make_smem_desc_sw128(sb + kk * UMMA_K * 2, 0, 1024);
            else
              bdesc = make_smem_desc_sw128(sb + kk * UMMA_K * 128, ATOM_BYTES, 1024);
            umma_f16(tmem_d, adesc, bdesc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees this smem stage when the MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[buf]);
      }
      if (!ok) {
        umma_commit(drain_bar);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 100000000ull) {}
      }
    }
  } else {
    // --------------------------------------------------------- epilogue --
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int local_tile = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local_tile) {
      const TileInfo ti = tile_info(t, p);
      const int buf = local_tile & 1;
      const uint32_t buf_phase = (local_tile >> 1) & 1;
      ok = mbar_wait_bounded(&tmem_full[buf], buf_phase, abort_flag, p.status, kTimeoutTmemFull,
                             blockIdx.x);
      if (!ok) break;
      tc_fence_after();
      const int row_local = ti.m0 + q * 32 + lane;           // row inside the [M, N] problem
      const int64_t row = (p.mode == 2 ? static_cast<int64_t>(ti.group) * p.M : 0) + row_local;
      const int col0 = ti.n0;
      const bool empty_k = ti.num_k == 0;                    // expert without tokens: the tile is zero
      const uint32_t taddr = tmem_base + buf * BLOCK_N + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BLOCK_N / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (empty_k) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        const int col = col0 + c * 32;
        if (row_local < p.M && col < p.N && ti.group >= 0) {
          if constexpr (OUT_F32) {
            float* dst = reinterpret_cast<float*>(p.C) + row * p.ldc + col;
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
            __nv_bfloat16* dst =
                reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col;
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
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows,
// row stride `ld` elements; box = box_inner x box_outer, 128-byte swizzle.
int make_tmap_2d(CUtensorMap* map, const void* ptr, CUtensorMapDataType dtype, int elem_bytes,
                 uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                 uint32_t box_outer) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * elem_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dtype, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

template <bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int num_sms,
                  cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN, OUT_F32, ACCUM>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int num_tiles = ((p.M + BLOCK_M - 1) / BLOCK_M) * ((p.N + BLOCK_N - 1) / BLOCK_N) *
                        (p.mode == 2 ? p.num_groups : 1);
  const int grid = num_tiles < num_sms ? num_tiles : num_sms;
  kern<<<grid, GEMM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace hpb

// C = opA * opB^T.  a_mn / b_mn select the storage order of each operand (see
// the header comment).  lda / ldb / ldc are row strides in elements.  Returns 0
// on success, a CUDA / driver error code otherwise (negative: bad argument).
extern "C" int hpb_gemm_bf16(const void* A, int a_mn, int64_t lda, const void* B, int b_mn,
                             int64_t ldb, void* C, int64_t ldc, int out_f32, int accumulate, int M,
                             int N, int K, int* status, int num_sms, cudaStream_t stream) {
  using namespace hpb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15))
    return -2;  // TMA needs 16-byte aligned bases and row strides
  // cuTensorMapEncodeTiled needs a current context on the calling thread; a fresh
  // thread (e.g. an autograd worker) may not have one bound yet.
  cudaFree(nullptr);
  CUtensorMap ta, tb;
  int r;
  if (!a_mn)
    r = make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, BLOCK_K, BLOCK_M);
  else
    r = make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, 64, BLOCK_K);
  if (r) return r;
  if (!b_mn)
    r = make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BLOCK_K, BLOCK_N);
  else
    r = make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, 64, BLOCK_K);
  if (r) return r;
  GemmParams p{M, N, K, C, ldc, status, 0, nullptr, nullptr, 1, 0};
  const int key = (a_mn ? 8 : 0) | (b_mn ? 4 : 0) | (out_f32 ? 2 : 0) | (accumulate ? 1 : 0);
  switch (key) {
#define HPB_CASE(k, a, b, o, c) \
  case k:                       \
    return launch<a, b, o, c>(ta, tb, p, num_sms, stream);
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


// Grouped GEMMs of an expert layer (see GemmParams).
//   mode 1: C[Mtot, N] = A[Mtot, K] * B_e^T, expert of each 128-row block from block_group;
//           B stacked [E * b_group_rows, ...] (K-major: [E*N, K]; MN-major: [E*K, N]).
//   mode 2: C[e] [M, N] (+)= A[rows_e, M]^T * B[rows_e, N] for every expert e (both MN-major);
//           lda/ldb are the row strides of the [rows_total, M] / [rows_total, N] operands.
extern "C" int hpb_gemm_bf16_grouped(const void* A, int a_mn, int64_t lda, int64_t a_rows,
                                     const void* B, int b_mn, int64_t ldb, int64_t b_rows, void* C,
                                     int64_t ldc, int out_f32, int accumulate, int M, int N, int K,
                                     int mode, const int* block_group, const int* group_offsets,
                                     int num_groups, int b_group_rows, int* status, int num_sms,
                                     cudaStream_t stream) {
  using namespace hpb;
  if (M <= 0 || N <= 0 || num_groups <= 0) return 0;
  if (mode != 1 && mode != 2) return -4;
  if (mode == 2 && !(a_mn && b_mn)) return -5;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15))
    return -2;
  cudaFree(nullptr);
  CUtensorMap ta, tb;
  int r;
  // tensor maps cover the whole stacked operands; a_rows / b_rows are their outer extents
  if (!a_mn)
    r = make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, a_rows, lda, BLOCK_K, BLOCK_M);
  else
    r = make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, a_rows, lda, 64, BLOCK_K);
  if (r) return r;
  if (!b_mn)
    r = make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, b_rows, ldb, BLOCK_K, BLOCK_N);
  else
    r = make_tmap_2d(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, b_rows, ldb, 64, BLOCK_K);
  if (r) return r;
  // mode 2 contracts over operand rows: K carries their total count (the bound of every expert's range)
  GemmParams p{M, N, mode == 2 ? static_cast<int>(a_rows < b_rows ? a_rows : b_rows) : K, C, ldc, status, mode,
               block_group, group_offsets, num_groups, b_group_rows};
  const int key = (a_mn ? 8 : 0) | (b_mn ? 4 : 0) | (out_f32 ? 2 : 0) | (accumulate ? 1 : 0);
  switch (key) {
#define HPB_CASE(k, a, b, o, c) \
  case k:                       \
    return launch<a, b, o, c>(ta, tb, p, num_sms, stream);
    HPB_CASE(0, false, false, false, false)
    HPB_CASE(1, false, false, false, true)
    HPB_CASE(2, false, false, true, false)
    HPB_CASE(3, false, false, true, true)
    HPB_CASE(4, false, true, false, false)
    HPB_CASE(5, false, true, false, true)
    HPB_CASE(6, false, true, true, false)
    HPB_CASE(7, false, true, true, true)
    HPB_CASE(12, true, true, false, false)
    HPB_CASE(13, true, true, false, true)
    HPB_CASE(14, true, true, true, false)
    HPB_CASE(15, true, true, true, true)
#undef HPB_CASE
  }
  return -3;
}
