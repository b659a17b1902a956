// Flash attention for sm_100a (head dimension 128, bf16, optional causal mask, grouped-query
// heads): S = Q K^T and O += P V run on tcgen05 with the score tile and the output accumulator
// in tensor memory; the online softmax runs on CUDA cores between the two.
//
// Forward kernel.  One CTA owns 256 query rows of one (batch, head) as two 128-row tiles that
// ping-pong: while the softmax warps of tile 0 turn S0 into P0, the tensor core computes
// S1 / O1 and vice versa.
//
//   warp 0      TMA producer: Q0, Q1 once; then K_0, V_0, K_1, V_1, ... through a 3-stage ring
//   warp 1      MMA issuer (one elected thread): S_t = Q_t K_j^T, O_t += P_t V_j
//   warps 2-5   softmax of tile 0: thread = row; reads S from TMEM, writes bf16 P into
//   warps 6-9   softmax of tile 1      swizzled shared memory (A operand of the PV product)
//
// TMEM (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each.
// The row maximum is only raised when it grows by more than 2^8 (P stays bounded by 256 and
// the accumulator in TMEM is rescaled rarely); the result is exact after the final 1/l.
//
// All tiles are [128 rows x 128 bf16] stored as two 64-column halves of 16 KB with the 128-byte
// swizzle, rows contiguous by 128 B -- the layout serves as K-major operand (Q, K, P) and as
// MN-major operand (V) alike.
//
// Every wait is bounded; on expiry a status code is recorded and all roles unwind.
#include "attention_common.cuh"

namespace hpb {
namespace fa {

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int HD = 128;
constexpr int TILE_BYTES = 128 * 128 * 2;  // 32 KB
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int FWD_THREADS = 320;
// P either goes through shared memory (3-stage K/V ring + two P tiles) or stays in tensor memory
// on top of the scores it was computed from (5-stage ring); both variants use 7 tiles of 32 KB.
template <bool P_TMEM>
struct FwdCfg {
  static constexpr int KV_STAGES = P_TMEM ? 5 : 3;
};
constexpr int FWD_SMEM = 7 * TILE_BYTES + 1024 + 256;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct FwdParams {
  int B, S, Hq, Hkv;
  float scale_log2;  // softmax scale * log2(e)
  int causal;
  __nv_bfloat16* O;  // [B, S, Hq, 128] contiguous
  float* lse;        // [B, Hq, S] natural-log sum-exp
  int* status;
};

// Number of key tiles that query tile `qt` (tile index) attends to.
__device__ __forceinline__ int kv_tiles_for(int qt, int S, int causal) {
  const int total = (S + BN - 1) / BN;
  if (qt * BM >= S) return 0;
  return causal ? min(total, qt + 1) : total;
}

template <bool P_TMEM>
__global__ void __launch_bounds__(FWD_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  constexpr int KV_STAGES = FwdCfg<P_TMEM>::KV_STAGES;
  uint8_t* sQ = smem;                                  // 2 tiles
  uint8_t* sKV = smem + 2 * TILE_BYTES;                // KV_STAGES tiles
  uint8_t* sP = sKV + 3 * TILE_BYTES;                  // 2 tiles (shared-memory P variant only)
  uint64_t* q_full = reinterpret_cast<uint64_t*>(smem + 7 * TILE_BYTES);
  uint64_t* kv_full = q_full + 1;           // [KV_STAGES]
  uint64_t* kv_empty = kv_full + KV_STAGES; // [KV_STAGES]
  uint64_t* s_full = kv_empty + KV_STAGES;  // [2]
  uint64_t* p_full = s_full + 2;            // [2]
  uint64_t* pv_done = p_full + 2;           // [2]
  uint64_t* drain_bar = pv_done + 2;        // [1]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // heavy (late) query blocks first: they have the most key tiles under a causal mask
  const int num_pairs = (p.S + 2 * BM - 1) / (2 * BM);
  const int hb = static_cast<int>(blockIdx.x) % (p.Hq * p.B);
  const int pair = num_pairs - 1 - static_cast<int>(blockIdx.x) / (p.Hq * p.B);
  const int head = hb % p.Hq;
  const int batch = hb / p.Hq;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int n0 = kv_tiles_for(2 * pair, p.S, p.causal);
  const int n1 = kv_tiles_for(2 * pair + 1, p.S, p.causal);
  const int n_kv = max(n0, n1);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 4);   // one arrive per softmax warp
      mbar_init(&pv_done[t], 1);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, 2 * TILE_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          tma_load_3d(sQ + t * TILE_BYTES + h * HALF_BYTES, &tmap_q, q_full, head * HD + h * 64,
                      (2 * pair + t) * BM, batch);
      int issued = 0;
      bool ok = true;
      for (int idx = 0; idx < 2 * n_kv && ok; ++idx) {
        const int stage = idx % KV_STAGES;
        const uint32_t phase = (idx / KV_STAGES) & 1;
        ok = mbar_wait_bounded(&kv_empty[stage], phase ^ 1, abort_flag, p.status, kTimeoutEmptyBarrier,
                               blockIdx.x);
        if (!ok) break;
        const int j = idx >> 1;
        const CUtensorMap* tm = (idx & 1) ? &tmap_v : &tmap_k;
        uint8_t* dst = sKV + stage * TILE_BYTES;
        mbar_arrive_expect_tx(&kv_full[stage], TILE_BYTES);
#pragma unroll
        for (int h = 0; h < 2; ++h)
          tma_load_3d(dst + h * HALF_BYTES, tm, &kv_full[stage], kv_head * HD + h * 64, j * BN, batch);
        ++issued;
      }
      if (!ok) {
        // wait (bounded) for the copies already issued, so that none lands after the CTA exits
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(q_full, 0) && globaltimer_ns() - t0 < 100000000ull) {}
        for (int b = 1; b <= min(issued, KV_STAGES); ++b) {
          const int idx = issued - b;
          const uint64_t t1 = globaltimer_ns();
          while (!mbar_try_wait(&kv_full[idx % KV_STAGES], (idx / KV_STAGES) & 1) &&
                 globaltimer_ns() - t1 < 100000000ull) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t idesc_s = make_idesc(1, 1, 0, 0, BM, BN);   // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_o = make_idesc(1, 1, 0, 1, BM, HD);   // P (K-major) x V (MN-major)
      const uint32_t q_addr = smem_u32(sQ), kv_addr = smem_u32(sKV), p_addr = smem_u32(sP);
      const int nt[2] = {n0, n1};
      bool ok = true;
      auto wait_kv = [&](int idx) {
        return mbar_wait_bounded(&kv_full[idx % KV_STAGES], (idx / KV_STAGES) & 1, abort_flag, p.status,
                                 kTimeoutFullBarrier, blockIdx.x);
      };
      const uint64_t q_desc = make_smem_desc_sw128(q_addr, 0, 1024);
      const uint64_t k_desc = make_smem_desc_sw128(kv_addr, 0, 1024);            // K tile, K-major
      const uint64_t v_desc = make_smem_desc_sw128(kv_addr, HALF_BYTES, 1024);   // V tile, MN-major
      const uint64_t p_desc = make_smem_desc_sw128(p_addr, 0, 1024);
      auto issue_s = [&](int t, int idx) {
        const uint64_t qa = desc_at(q_desc, t * TILE_BYTES);
        const uint64_t ka = desc_at(k_desc, (idx % KV_STAGES) * TILE_BYTES);
        const uint32_t d = tmem_base + t * BN;
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(d, desc_at(qa, kb * HALF_BYTES + kk * 32), desc_at(ka, kb * HALF_BYTES + kk * 32), idesc_s,
                     (kb | kk) ? 1u : 0u);
        umma_commit(&s_full[t]);
      };
      auto issue_pv = [&](int t, int idx, bool accumulate) {
        // P: kv index is the contraction (64-wide halves, +32 B per 16); V: 16 kv rows = 2048 B,
        // the two 64-wide halves of the head dimension are HALF_BYTES apart (leading offset)
        const uint64_t va = desc_at(v_desc, (idx % KV_STAGES) * TILE_BYTES);
        const uint32_t d = tmem_base + 2 * BN + t * HD;
        if constexpr (P_TMEM) {
          // P (bf16 pairs) occupies the first 64 columns of the score tile: 16 kv = 8 columns per step
          const uint32_t pt = tmem_base + t * BN;
          umma_f16_ts(d, pt, va, idesc_o, accumulate ? 1u : 0u);
#pragma unroll
          for (int k8 = 1; k8 < 8; ++k8) umma_f16_ts(d, pt + k8 * 8, desc_at(va, k8 * 2048), idesc_o, 1u);
        } else {
          const uint64_t pa = desc_at(p_desc, t * TILE_BYTES);
          umma_f16(d, pa, va, idesc_o, accumulate ? 1u : 0u);
#pragma unroll
          for (int k8 = 1; k8 < 8; ++k8)
            umma_f16(d, desc_at(pa, (k8 >> 2) * HALF_BYTES + (k8 & 3) * 32), desc_at(va, k8 * 2048), idesc_o, 1u);
        }
        umma_commit(&pv_done[t]);
      };
      ok = mbar_wait_bounded(q_full, 0, abort_flag, p.status, kTimeoutFullBarrier, blockIdx.x);
      if (ok) ok = wait_kv(0);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < 2; ++t)
          if (nt[t] > 0) issue_s(t, 0);
        umma_commit(&kv_empty[0]);                           // K_0 is free once both S_t(K_0) retire
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        ok = wait_kv(2 * j + 1);                      // V_j
        if (ok && j + 1 < n_kv) ok = wait_kv(2 * j + 2);  // K_{j+1}
        if (!ok) break;
        tc_fence_after();
        for (int t = 0; t < 2 && ok; ++t) {
          if (j < nt[t]) {
            ok = mbar_wait_bounded(&p_full[t], j & 1, abort_flag, p.status, kTimeoutTmemFull, blockIdx.x);
            if (!ok) break;
            tc_fence_after();
            issue_pv(t, 2 * j + 1, j > 0);
          }
          if (j + 1 < nt[t]) issue_s(t, 2 * j + 2);
        }
        if (!ok) break;
        umma_commit(&kv_empty[(2 * j + 1) % KV_STAGES]);                      // V_j
        if (j + 1 < n_kv) umma_commit(&kv_empty[(2 * j + 2) % KV_STAGES]);    // K_{j+1}: both S_t issued above
      }
      if (!ok) {
        umma_commit(drain_bar);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 100000000ull) {}
      }
    }
  } else {
    // ------------------------------------------------------------- softmax --
    const int t = (warp - 2) >> 2;            // query tile of this warpgroup
    const int quarter = warp & 3;             // TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;      // row inside the tile
    const int n_t = t == 0 ? n0 : n1;
    const int q_row = (2 * pair + t) * BM + row;   // sequence position of this thread's query
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + t * BN + lane_off;
    const uint32_t o_addr = tmem_base + 2 * BN + t * HD + lane_off;
    uint8_t* p_row = sP + t * TILE_BYTES + row * 128;
    const int sw = row & 7;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_t && ok; ++j) {
      ok = mbar_wait_bounded(&s_full[t], j & 1, abort_flag, p.status, kTimeoutTmemFull, blockIdx.x);
      if (!ok) break;
      tc_fence_after();
      const int k0 = j * BN;
      // columns [0, limit) of this tile are visible to this row
      int limit = p.S - k0;
      if (p.causal) limit = min(limit, q_row - k0 + 1);
      const bool masked = limit < BN;
      // the whole score row of this thread (128 fp32) in one batch of loads
      uint32_t sr[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + c * 32, sr + c * 32);
      tmem_ld_wait();
      if (masked) {
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (i >= limit) sr[i] = 0xff800000u;   // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 128; i += 4) {
        mx0 = max3(mx0, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
        mx1 = max3(mx1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
      }
      const float m_new = fmaxf(m, fmaxf(mx0, mx1) * p.scale_log2);
      float alpha = 1.f;
      bool need = false;
      if (j == 0) {
        m = m_new;
      } else if (m_new > m + kRescaleThreshold) {
        need = true;
        alpha = fast_exp2(m - m_new);
        m = m_new;
        l *= alpha;
      }
      if (j > 0) {
        // Shared-memory P: the previous P V product must have retired before its P tile is
        // overwritten.  Tensor-memory P lies under the scores just produced, which the tensor
        // core wrote after that product, so only a rescale of the accumulator has to wait.
        const bool any_need = __any_sync(0xffffffffu, need);
        if (!P_TMEM || any_need) {
          ok = mbar_wait_bounded(&pv_done[t], (j - 1) & 1, abort_flag, p.status, kTimeoutTmemEmpty, blockIdx.x);
          if (!ok) break;
          tc_fence_after();
        }
        if (any_need) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(o_addr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32b_x32(o_addr + c * 32, r);
          }
          tmem_st_wait();
        }
      }
      // P = 2^(s * scale - m) (masked scores are -inf -> 0), row sum, bf16 into the swizzled A tile
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
      const float2 nm2 = make_float2(-m, -m);
      float2 l2 = make_float2(0.f, 0.f);
      if constexpr (P_TMEM) {
        // pack in place: sr[i] <- bf16 pair (2i, 2i+1); two stores of 32 columns put the row back
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          float2 x = fma2(make_float2(__uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1])), sc2, nm2);
          x.x = fast_exp2(x.x);
          x.y = fast_exp2(x.y);
          l2 = add2(l2, x);
          const __nv_bfloat162 b2 = __floats2bfloat162_rn(x.x, x.y);
          sr[i] = *reinterpret_cast<const uint32_t*>(&b2);
        }
        tmem_st_32x32b_x32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(sr));
        tmem_st_32x32b_x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(sr + 32));
        tmem_st_wait();
      } else {
#pragma unroll
        for (int c8 = 0; c8 < 16; ++c8) {     // 16 chunks of 8 columns = one 16-byte store each
          uint4 v;
          __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = c8 * 8 + 2 * e;
            float2 x = fma2(make_float2(__uint_as_float(sr[i]), __uint_as_float(sr[i + 1])), sc2, nm2);
            x.x = fast_exp2(x.x);
            x.y = fast_exp2(x.y);
            l2 = add2(l2, x);
            vb[e] = __floats2bfloat162_rn(x.x, x.y);
          }
          uint8_t* blk = p_row + (c8 >> 3) * HALF_BYTES;
          *reinterpret_cast<uint4*>(blk + (((c8 & 7) ^ sw) << 4)) = v;
        }
      }
      l += l2.x + l2.y;
      if constexpr (!P_TMEM) fence_proxy_async();   // generic-proxy writes of P -> visible to the tensor core
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
    }
    if (ok && n_t > 0) {
      ok = mbar_wait_bounded(&pv_done[t], (n_t - 1) & 1, abort_flag, p.status, kTimeoutTmemEmpty, blockIdx.x);
      if (ok) {
        tc_fence_after();
        const float inv = 1.f / l;
        const bool live = q_row < p.S;
        __nv_bfloat16* dst = p.O + ((static_cast<int64_t>(batch) * p.S + q_row) * p.Hq + head) * HD;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(o_addr + c * 32, r);
          tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 v;
              __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
              for (int e = 0; e < 4; ++e)
                vb[e] = __floats2bfloat162_rn(__uint_as_float(r[8 * q4 + 2 * e]) * inv,
                                              __uint_as_float(r[8 * q4 + 2 * e + 1]) * inv);
              reinterpret_cast<uint4*>(dst + c * 32)[q4] = v;
            }
          }
        }
        if (live)
          p.lse[(static_cast<int64_t>(batch) * p.Hq + head) * p.S + q_row] =
              (m + log2f(l)) * 0.6931471805599453f;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}


// ============================================================ backward ========
// One CTA owns one 128-row key/value tile of one (batch, kv head) and walks over the query heads
// of its group and their 64-row query tiles.  Everything is computed transposed, so that the
// softmax threads (thread = key row) write the A operands of the following products as plain
// 128-byte rows:
//
//   S^T  = K Q^T            [kv 128 x q 64]   tensor memory (double buffered)
//   dP^T = V dO^T           [kv 128 x q 64]   tensor memory (double buffered)
//   P^T  = exp2(S^T * c - lse)                                 -> bf16 pairs, back into tensor memory over
//                                                                 the dP^T columns the thread has read
//   dS^T = P^T o (dP^T - D)                                    -> bf16, shared memory
//   dV  += P^T dO           [kv 128 x d 128]  tensor memory, accumulated over the whole walk
//   dK  += dS^T Q           [kv 128 x d 128]  tensor memory, accumulated over the whole walk
//   dQ^T = K^T dS^T         [d 128 x q 64]    tensor memory (in the S^T buffer just consumed),
//                                             added to the fp32 dQ in global memory with
//                                             coalesced reductions (lane = head element)
//
//   warp 0       TMA producer: K, V once; (Q_i, dO_i) through a 3-stage ring
//   warp 1       MMA issuer
//   warps 2-9    softmax / dS: two groups of four warps, each owning 32 of the 64 query columns;
//                they also write dV / dK at the end
//   warps 10-13  dQ read-out: fp32 tiles staged in a buffer of their own and added to global
//                memory by TMA reduces, so the read-out never holds back the softmax warps
constexpr int BQ = 64;                        // query rows per step
constexpr int QDO_STAGES = 3;
constexpr int QTILE_BYTES = BQ * HD * 2;      // 16 KB
constexpr int PT_BYTES = BN * BQ * 2;         // 16 KB
constexpr int BWD_THREADS = 448;
constexpr int STAGE_TILE = BQ * 32 * 4;       // 8 KB: [64 query rows x 32 head elements] fp32
constexpr int BWD_SMEM = 2 * TILE_BYTES + QDO_STAGES * 2 * QTILE_BYTES + 2 * PT_BYTES + 4 * STAGE_TILE +
                         2 * 2 * BQ * 4 + 1024 + 256;

struct BwdParams {
  int B, S, Hq, Hkv;
  float scale, scale_log2;
  int causal;
  int head_group;      // (batch, kv head) pairs scheduled together
  const float* lse;    // [B, Hq, S]
  const float* delta;  // [B, Hq, S]  rowsum(dO o O)
  float* dQ;           // [B, S, Hq, 128] fp32, zero-initialised
  __nv_bfloat16* dK;   // [B, S, Hkv, 128], token stride dkv_row_stride elements
  __nv_bfloat16* dV;   // likewise
  long long dkv_row_stride;
  int* status;
};

__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                 const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                 const __grid_constant__ CUtensorMap tmap_dq, const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE_BYTES;
  uint8_t* sQdO = sV + TILE_BYTES;                            // per stage: Q (16 KB) | dO (16 KB)
  uint8_t* sDS = sQdO + QDO_STAGES * 2 * QTILE_BYTES;         // dS^T, two buffers of 16 KB
  uint8_t* sStage = sDS + 2 * PT_BYTES;                       // dQ staging: one 8 KB tile per dQ warp
  float* sStat = reinterpret_cast<float*>(sStage + 4 * STAGE_TILE);  // [2][2][64]: lse*log2e, delta
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(sStat + 2 * 2 * BQ);
  uint64_t* qdo_full = kv_full + 1;              // [QDO_STAGES]
  uint64_t* qdo_empty = qdo_full + QDO_STAGES;   // [QDO_STAGES]
  uint64_t* st_full = qdo_empty + QDO_STAGES;    // [2]  S^T and dP^T of a step are complete
  uint64_t* ds_full = st_full + 2;               // [2]  P^T / dS^T written (4 warp arrivals)
  uint64_t* pt_free = ds_full + 2;               // [2]  products reading dS^T buffer b retired
  uint64_t* dq_full = pt_free + 2;               // [2]
  uint64_t* dq_drained = dq_full + 2;            // [2]  (4 warp arrivals)
  uint64_t* stat_full = dq_drained + 2;          // [2]  lse / delta of a step staged (4 warp arrivals)
  uint64_t* acc_full = stat_full + 2;            // [1]
  uint64_t* drain_bar = acc_full + 1;            // [1]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // (batch, kv head) pairs are processed in groups of `head_group`: the CTAs that run at the same
  // time then add into a few MB of the fp32 dQ (and re-read the same Q / dO), which stays in L2;
  // inside a group the key tiles go in ascending order (causal: low tiles have the longest walk)
  int hb, jt;
  {
    const int n_tiles = (p.S + BN - 1) / BN;
    const int pairs = p.Hkv * p.B;
    const int hg = max(1, min(p.head_group, pairs));
    const int g0 = static_cast<int>(blockIdx.x) / (hg * n_tiles) * hg;
    const int gsz = min(hg, pairs - g0);
    const int r = static_cast<int>(blockIdx.x) - g0 * n_tiles;
    jt = r / gsz;
    hb = g0 + r % gsz;
  }
  const int kv_head = hb % p.Hkv;
  const int batch = hb / p.Hkv;
  const int group = p.Hq / p.Hkv;
  const int k0 = jt * BN;
  const int nq = (p.S + BQ - 1) / BQ;
  const int i_start = p.causal ? (k0 / BQ) : 0;       // first query tile that sees this key tile
  const int per_head = nq - i_start;
  const int n_it = per_head * group;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < QDO_STAGES; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&st_full[b], 1);
      mbar_init(&ds_full[b], 8);
      mbar_init(&pt_free[b], 1);     // committed by the MMA issuer behind the last reader of dS^T
      mbar_init(&dq_full[b], 1);
      mbar_init(&dq_drained[b], 4);
      mbar_init(&stat_full[b], 4);
    }
    mbar_init(acc_full, 1);
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_do);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_dq);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  // tensor-memory columns
  constexpr uint32_t COL_ST = 0;      // 2 x 64   (S^T, later dQ^T)
  constexpr uint32_t COL_DPT = 128;   // 2 x 64
  constexpr uint32_t COL_DV = 256;    // 128
  constexpr uint32_t COL_DK = 384;    // 128

  if (warp == 0) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 2 * TILE_BYTES);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        tma_load_3d(sK + h * HALF_BYTES, &tmap_k, kv_full, kv_head * HD + h * 64, k0, batch);
        tma_load_3d(sV + h * HALF_BYTES, &tmap_v, kv_full, kv_head * HD + h * 64, k0, batch);
      }
      int issued = 0;
      bool ok = true;
      for (int it = 0; it < n_it && ok; ++it) {
        const int stage = it % QDO_STAGES;
        const uint32_t phase = (it / QDO_STAGES) & 1;
        ok = mbar_wait_bounded(&qdo_empty[stage], phase ^ 1, abort_flag, p.status, kTimeoutEmptyBarrier,
                               blockIdx.x);
        if (!ok) break;
        const int head = kv_head * group + it / per_head;
        const int q0 = (i_start + it % per_head) * BQ;
        uint8_t* dq = sQdO + stage * 2 * QTILE_BYTES;
        mbar_arrive_expect_tx(&qdo_full[stage], 2 * QTILE_BYTES);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          tma_load_3d(dq + h * (QTILE_BYTES / 2), &tmap_q, &qdo_full[stage], head * HD + h * 64, q0, batch);
          tma_load_3d(dq + QTILE_BYTES + h * (QTILE_BYTES / 2), &tmap_do, &qdo_full[stage], head * HD + h * 64,
                      q0, batch);
        }
        ++issued;
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(kv_full, 0) && globaltimer_ns() - t0 < 100000000ull) {}
        for (int b = 1; b <= min(issued, QDO_STAGES); ++b) {
          const int it = issued - b;
          const uint64_t t1 = globaltimer_ns();
          while (!mbar_try_wait(&qdo_full[it % QDO_STAGES], (it / QDO_STAGES) & 1) &&
                 globaltimer_ns() - t1 < 100000000ull) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_st = make_idesc(1, 1, 0, 0, BN, BQ);    // K (K-major) x Q (K-major)
      constexpr uint32_t idesc_acc = make_idesc(1, 1, 0, 1, BN, HD);   // P^T (K-major) x dO (MN-major)
      constexpr uint32_t idesc_dq = make_idesc(1, 1, 1, 1, HD, BQ);    // K^T (MN-major) x dS^T (MN-major)
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), qdo_addr = smem_u32(sQdO),
                     ds_addr = smem_u32(sDS);
      bool ok = true;
      const uint64_t k_desc = make_smem_desc_sw128(k_addr, 0, 1024);              // K as K-major A
      const uint64_t v_desc = make_smem_desc_sw128(v_addr, 0, 1024);              // V as K-major A
      const uint64_t kt_desc = make_smem_desc_sw128(k_addr, HALF_BYTES, 1024);    // K^T as MN-major A
      const uint64_t qk_desc = make_smem_desc_sw128(qdo_addr, 0, 1024);           // Q / dO as K-major B
      const uint64_t qm_desc = make_smem_desc_sw128(qdo_addr, QTILE_BYTES / 2, 1024);   // Q / dO as MN-major B
      const uint64_t dsk_desc = make_smem_desc_sw128(ds_addr, 0, 1024);           // dS^T as K-major A
      const uint64_t dsm_desc = make_smem_desc_sw128(ds_addr, PT_BYTES, 1024);    // dS^T as MN-major B
      // S^T(it) and dP^T(it) into buffer it & 1 (st_full follows the S^T product, issued last)
      auto issue_dpt = [&](int it) {
        const int b = it & 1;
        const uint64_t doa = desc_at(qk_desc, (it % QDO_STAGES) * 2 * QTILE_BYTES + QTILE_BYTES);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(tmem_base + COL_DPT + b * BQ, desc_at(v_desc, kb * HALF_BYTES + kk * 32),
                     desc_at(doa, kb * (QTILE_BYTES / 2) + kk * 32), idesc_st, (kb | kk) ? 1u : 0u);
      };
      auto issue_st = [&](int it) {
        const int b = it & 1;
        const uint64_t qa = desc_at(qk_desc, (it % QDO_STAGES) * 2 * QTILE_BYTES);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(tmem_base + COL_ST + b * BQ, desc_at(k_desc, kb * HALF_BYTES + kk * 32),
                     desc_at(qa, kb * (QTILE_BYTES / 2) + kk * 32), idesc_st, (kb | kk) ? 1u : 0u);
        umma_commit(&st_full[b]);
      };
      auto wait_qdo = [&](int it) {
        return mbar_wait_bounded(&qdo_full[it % QDO_STAGES], (it / QDO_STAGES) & 1, abort_flag, p.status,
                                 kTimeoutFullBarrier, blockIdx.x);
      };
      ok = mbar_wait_bounded(kv_full, 0, abort_flag, p.status, kTimeoutFullBarrier, blockIdx.x);
      for (int it = 0; it < 2 && it < n_it && ok; ++it) {
        ok = wait_qdo(it);
        if (ok) {
          tc_fence_after();
          issue_dpt(it);
          issue_st(it);
        }
      }
      // Per step, once the softmax warps have written P^T / dS^T: dQ^T first (its read-out and
      // the reduce that follows are the longest dependency of the walk), then dV / dK, then the
      // scores of step it + 2 -- dP^T right away, S^T once the dQ^T tile that shares its buffer
      // has been read out.
      for (int it = 0; it < n_it && ok; ++it) {
        const int b = it & 1;
        const uint32_t par = (it >> 1) & 1;
        ok = mbar_wait_bounded(&ds_full[b], par, abort_flag, p.status, kTimeoutTmemFull, blockIdx.x);
        if (!ok) break;
        tc_fence_after();
        const uint64_t qa = desc_at(qm_desc, (it % QDO_STAGES) * 2 * QTILE_BYTES);
        const uint64_t doa = desc_at(qa, QTILE_BYTES);
        const uint64_t dsa = desc_at(dsk_desc, b * PT_BYTES);
        const uint64_t dsm = desc_at(dsm_desc, b * PT_BYTES);
        const uint32_t first = it ? 1u : 0u;
        // dQ^T = K^T dS^T  (contraction over the 128 key rows: 8 steps of 16) into the S^T buffer
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_f16(tmem_base + COL_ST + b * BQ, desc_at(kt_desc, kk * 2048), desc_at(dsm, kk * 2048), idesc_dq,
                   kk ? 1u : 0u);
        umma_commit(&dq_full[b]);
        // dV += P^T dO ; dK += dS^T Q   (contraction over the 64 query rows: 4 steps of 16).  P^T lies
        // in the dP^T buffer of the step: query rows 0..31 in columns 0..15, 32..63 in columns 32..47
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_f16_ts(tmem_base + COL_DV, tmem_base + COL_DPT + b * BQ + (kk >> 1) * 32 + (kk & 1) * 8,
                      desc_at(doa, kk * 2048), idesc_acc, kk ? 1u : first);
        umma_f16(tmem_base + COL_DK, dsa, qa, idesc_acc, first);
#pragma unroll
        for (int kk = 1; kk < 4; ++kk)
          umma_f16(tmem_base + COL_DK, desc_at(dsa, kk * 32), desc_at(qa, kk * 2048), idesc_acc, 1u);
        umma_commit(&qdo_empty[it % QDO_STAGES]);
        umma_commit(&pt_free[b]);      // every reader of dS^T of this step has been issued
        if (it + 2 < n_it) {
          ok = wait_qdo(it + 2);
          if (!ok) break;
          tc_fence_after();
          issue_dpt(it + 2);
          ok = mbar_wait_bounded(&dq_drained[b], par, abort_flag, p.status, kTimeoutTmemEmpty, blockIdx.x);
          if (!ok) break;
          tc_fence_after();
          issue_st(it + 2);
        }
      }
      if (ok) umma_commit(acc_full);
      if (!ok) {
        umma_commit(drain_bar);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 100000000ull) {}
      }
    }
  } else {
    const int wg = (warp - 2) >> 2;           // 0, 1: softmax / dS of query columns [32 wg, 32 wg + 32); 2: dQ
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;      // TMEM lane handled by this thread
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    bool ok = true;
    if (wg < 2) {
      // ------------------------------------------------------ softmax / dS --
      const int tid = threadIdx.x - 64;       // 0..255 over both softmax groups; 0..127 stage the statistics
      const int kv_row = k0 + row;
      const bool row_live = kv_row < p.S;
      const int sw = row & 7;
      auto load_stat = [&](int it) -> float {
        // threads 0..63 fetch lse (scaled to log2), 64..127 fetch delta, of step `it`
        if (it >= n_it || tid >= 128) return 0.f;
        const int head = kv_head * group + it / per_head;
        const int q = (i_start + it % per_head) * BQ + (tid & 63);
        if (q >= p.S) return tid < 64 ? INFINITY : 0.f;
        const int64_t off = (static_cast<int64_t>(batch) * p.Hq + head) * p.S + q;
        return tid < 64 ? p.lse[off] : p.delta[off];     // raw: scaled when staged, a step later
      };
      float stat_next = load_stat(0);
      for (int it = 0; it < n_it && ok; ++it) {
        const int b = it & 1;
        const uint32_t par = (it >> 1) & 1;
        float* stat = sStat + b * 2 * BQ;
        // dS^T buffer b is free again (the products of step it - 2 that read it have retired); this
        // also means that all eight softmax warps have finished step it - 2, so the statistics
        // buffer b can be rewritten
        ok = mbar_wait_bounded(&pt_free[b], par ^ 1, abort_flag, p.status, kTimeoutTmemEmpty, blockIdx.x);
        if (!ok) break;
        if (tid < 128) stat[tid] = tid < 64 ? stat_next * 1.4426950408889634f : stat_next;
        stat_next = load_stat(it + 1);
        __syncwarp();
        if (lane == 0 && wg == 0) mbar_arrive(&stat_full[b]);
        ok = mbar_wait_bounded(&stat_full[b], par, abort_flag, p.status, kTimeoutFullBarrier, blockIdx.x);
        if (ok) ok = mbar_wait_bounded(&st_full[b], par, abort_flag, p.status, kTimeoutTmemFull, blockIdx.x);
        if (!ok) break;
        tc_fence_after();
        const int q0 = (i_start + it % per_head) * BQ;
        // visible iff key <= query:  column c >= kv_row - q0
        const int cmin = p.causal ? kv_row - q0 : 0;
        // warp-uniform: does any row of this warp hide any column of this step?
        const bool masked = (k0 + quarter * 32 + 32 > p.S) || (p.causal && k0 + quarter * 32 + 31 - q0 > 0);
        uint8_t* ds_row = sDS + b * PT_BYTES + row * 128;
        {
          const int c = wg;                    // this group's 32 query columns
          uint32_t rs[32], rp[32];
          tmem_ld_32x32b_x32(tmem_base + COL_ST + b * BQ + c * 32 + lane_off, rs);
          tmem_ld_32x32b_x32(tmem_base + COL_DPT + b * BQ + c * 32 + lane_off, rp);
          tmem_ld_wait();
          uint32_t pk[16], dk[16];
          const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
#pragma unroll
          for (int i2 = 0; i2 < 16; ++i2) {
            const float2 ls = *reinterpret_cast<const float2*>(stat + c * 32 + 2 * i2);
            const float2 dl = *reinterpret_cast<const float2*>(stat + BQ + c * 32 + 2 * i2);
            float2 e = fma2(make_float2(__uint_as_float(rs[2 * i2]), __uint_as_float(rs[2 * i2 + 1])), sc2,
                            make_float2(-ls.x, -ls.y));
            e.x = fast_exp2(e.x);
            e.y = fast_exp2(e.y);
            if (masked) {
              const int col = c * 32 + 2 * i2;
              if (!row_live || col < cmin) e.x = 0.f;
              if (!row_live || col + 1 < cmin) e.y = 0.f;
            }
            const float2 d = mul2(e, add2(make_float2(__uint_as_float(rp[2 * i2]), __uint_as_float(rp[2 * i2 + 1])),
                                          make_float2(-dl.x, -dl.y)));
            const __nv_bfloat162 eb = __floats2bfloat162_rn(e.x, e.y), db = __floats2bfloat162_rn(d.x, d.y);
            pk[i2] = *reinterpret_cast<const uint32_t*>(&eb);
            dk[i2] = *reinterpret_cast<const uint32_t*>(&db);
          }
          // P^T over the first 16 of the 32 dP^T columns just read (this thread's own)
          tmem_st_32x32b_x16(tmem_base + COL_DPT + b * BQ + c * 32 + lane_off, pk);
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int chunk = c * 4 + q4;
            *reinterpret_cast<uint4*>(ds_row + ((chunk ^ sw) << 4)) =
                make_uint4(dk[4 * q4], dk[4 * q4 + 1], dk[4 * q4 + 2], dk[4 * q4 + 3]);
          }
          tmem_st_wait();
        }
        fence_proxy_async();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ds_full[b]);
      }
    } else {
      // ------------------------------------------------------ dQ reduction --
      // dQ^T (lane = head element, column = query row) is transposed through this warp's staging
      // tile as a dense fp32 [64 query rows x 32 head elements] tile of 8 KB, which one TMA
      // reduce adds to the fp32 dQ in global memory.
      uint8_t* tile = sStage + quarter * STAGE_TILE;
      float* stage = reinterpret_cast<float*>(tile) + lane;
      for (int it = 0; it < n_it && ok; ++it) {
        const int b = it & 1;
        const uint32_t par = (it >> 1) & 1;
        ok = mbar_wait_bounded(&dq_full[b], par, abort_flag, p.status, kTimeoutTmemFull, blockIdx.x);
        if (!ok) break;
        tc_fence_after();
        const int head = kv_head * group + it / per_head;
        const int q0 = (i_start + it % per_head) * BQ;
        uint32_t r[64];
        tmem_ld32(tmem_base + COL_ST + b * BQ + lane_off, r);
        tmem_ld32(tmem_base + COL_ST + b * BQ + 32 + lane_off, r + 32);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&dq_drained[b]);                 // the S^T buffer may be overwritten
          tma_store_wait_read<0>();                    // the tile of the step before has left the staging memory
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 64; ++i) stage[i * 32] = __uint_as_float(r[i]) * p.scale;
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          tma_reduce_add_3d(&tmap_dq, tile, head * HD + quarter * 32, q0, batch);
          tma_store_commit();
        }
      }
      if (lane == 0) tma_store_wait<0>();
    }
    // ------------------------------------------------- dV / dK write-out --
    if (ok && n_it > 0 && wg < 2) {
      ok = mbar_wait_bounded(acc_full, 0, abort_flag, p.status, kTimeoutTmemFull, blockIdx.x);
      if (ok) {
        tc_fence_after();
        const int kv_row = k0 + row;
        const float mul = wg == 0 ? 1.f : p.scale;
        __nv_bfloat16* dst = (wg == 0 ? p.dV : p.dK) +
                             (static_cast<int64_t>(batch) * p.S + kv_row) * p.dkv_row_stride + kv_head * HD;
        const uint32_t src = tmem_base + (wg == 0 ? COL_DV : COL_DK) + lane_off;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(src + c * 32, r);
          tmem_ld_wait();
          if (kv_row < p.S) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 v;
              __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
              for (int e = 0; e < 4; ++e)
                vb[e] = __floats2bfloat162_rn(__uint_as_float(r[8 * q4 + 2 * e]) * mul,
                                              __uint_as_float(r[8 * q4 + 2 * e + 1]) * mul);
              reinterpret_cast<uint4*>(dst + c * 32)[q4] = v;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace fa
}  // namespace hpb

// ------------------------------------------------------------------ host ----

using namespace hpb;

// Backward schedule: (batch, kv head) pairs per group; <= 0 = all pairs in one group (key-tile major).
static int g_bwd_head_group = 8;
extern "C" void hpb_flash_attn_set_head_group(int pairs) { g_bwd_head_group = pairs; }

// Forward variant: 1 = P stays in tensor memory (default), 0 = P goes through shared memory.
static int g_fwd_p_in_tmem = 1;
extern "C" void hpb_flash_attn_set_variant(int p_in_tmem) { g_fwd_p_in_tmem = p_in_tmem; }

// q [B, S, Hq, 128], k / v [B, S, Hkv, 128] bf16: the head dimension contiguous, head stride 128,
// row (token) and batch strides given in elements (so views into a packed qkv tensor work).
// O [B, S, Hq, 128] contiguous bf16, lse [B, Hq, S] fp32.
extern "C" int hpb_flash_attn_fwd(const void* q, long long q_batch_stride, long long q_row_stride, const void* k,
                                  long long k_batch_stride, long long k_row_stride, const void* v,
                                  long long v_batch_stride, long long v_row_stride, void* O, float* lse, int B,
                                  int S, int Hq, int Hkv, float softmax_scale, int causal, int* status,
                                  cudaStream_t stream) {
  if (B <= 0 || S <= 0) return 0;
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv) return -2;
  if ((q_row_stride | k_row_stride | v_row_stride | q_batch_stride | k_batch_stride | v_batch_stride) & 7) return -2;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(O)) & 15)
    return -2;
  cudaFree(nullptr);
  CUtensorMap tq, tk, tv;
  int r = make_tmap_bsd(&tq, q, B, S, Hq * fa::HD, q_batch_stride, q_row_stride);
  if (r) return r;
  r = make_tmap_bsd(&tk, k, B, S, Hkv * fa::HD, k_batch_stride, k_row_stride);
  if (r) return r;
  r = make_tmap_bsd(&tv, v, B, S, Hkv * fa::HD, v_batch_stride, v_row_stride);
  if (r) return r;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fa::flash_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         fa::FWD_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(fa::flash_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               fa::FWD_SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  fa::FwdParams p;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.causal = causal;
  p.O = reinterpret_cast<__nv_bfloat16*>(O);
  p.lse = lse;
  p.status = status;
  dim3 grid(((S + 2 * fa::BM - 1) / (2 * fa::BM)) * Hq * B);
  if (g_fwd_p_in_tmem)
    fa::flash_fwd_kernel<true><<<grid, fa::FWD_THREADS, fa::FWD_SMEM, stream>>>(tq, tk, tv, p);
  else
    fa::flash_fwd_kernel<false><<<grid, fa::FWD_THREADS, fa::FWD_SMEM, stream>>>(tq, tk, tv, p);
  return static_cast<int>(cudaGetLastError());
}

// Backward.  dO [B, S, Hq, 128] (strided like q), O / lse from the forward.  Outputs: dQ
// [B, S, Hq, 128] bf16, dK / dV [B, S, Hkv, 128] bf16 with token strides dq_row_stride / dkv_row_stride
// elements (so that they may be the three column ranges of one packed gradient).  Workspace: dq_acc fp32
// [B, S, Hq, 128] and delta fp32 [B, Hq, S]; dq_acc is cleared here.
extern "C" int hpb_flash_attn_bwd(const void* q, long long q_batch_stride, long long q_row_stride, const void* k,
                                  long long k_batch_stride, long long k_row_stride, const void* v,
                                  long long v_batch_stride, long long v_row_stride, const void* O, const float* lse,
                                  const void* dO, long long do_batch_stride, long long do_row_stride, void* dQ,
                                  void* dK, void* dV, long long dq_row_stride, long long dkv_row_stride,
                                  float* dq_acc, float* delta, int B, int S, int Hq, int Hkv, float softmax_scale,
                                  int causal, int* status, cudaStream_t stream) {
  if (B <= 0 || S <= 0) return 0;
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv) return -2;
  if ((q_row_stride | k_row_stride | v_row_stride | do_row_stride | q_batch_stride | k_batch_stride |
       v_batch_stride | do_batch_stride) & 7)
    return -2;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(dO) | reinterpret_cast<uintptr_t>(dQ) | reinterpret_cast<uintptr_t>(dK) |
       reinterpret_cast<uintptr_t>(dV) | reinterpret_cast<uintptr_t>(O) | reinterpret_cast<uintptr_t>(dq_acc)) & 15)
    return -2;
  if ((dq_row_stride | dkv_row_stride) & 7) return -2;
  cudaFree(nullptr);
  CUtensorMap tq, tdo, tk, tv;
  int r = make_tmap_bsd(&tq, q, B, S, Hq * fa::HD, q_batch_stride, q_row_stride, fa::BQ);
  if (r) return r;
  r = make_tmap_bsd(&tdo, dO, B, S, Hq * fa::HD, do_batch_stride, do_row_stride, fa::BQ);
  if (r) return r;
  r = make_tmap_bsd(&tk, k, B, S, Hkv * fa::HD, k_batch_stride, k_row_stride);
  if (r) return r;
  r = make_tmap_bsd(&tv, v, B, S, Hkv * fa::HD, v_batch_stride, v_row_stride);
  if (r) return r;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fa::flash_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         fa::BWD_SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  const int64_t nq = static_cast<int64_t>(B) * S * Hq * fa::HD;
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, nq * sizeof(float), stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  {
    const int64_t warps = static_cast<int64_t>(B) * S * Hq;
    const int threads = 256;
    const int64_t blocks = (warps * 32 + threads - 1) / threads;
    fa::attn_delta_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(dO), do_batch_stride, do_row_stride,
        reinterpret_cast<const __nv_bfloat16*>(O), delta, B, S, Hq);
  }
  fa::BwdParams p;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.causal = causal;
  p.head_group = g_bwd_head_group > 0 ? g_bwd_head_group : (1 << 30);
  p.lse = lse;
  p.delta = delta;
  p.dQ = dq_acc;
  p.dK = reinterpret_cast<__nv_bfloat16*>(dK);
  p.dV = reinterpret_cast<__nv_bfloat16*>(dV);
  p.dkv_row_stride = dkv_row_stride;
  p.status = status;
  dim3 grid(((S + fa::BN - 1) / fa::BN) * Hkv * B);
  CUtensorMap tdq;
  {
    EncodeTiledFn enc = fa_encode_fn();
    if (enc == nullptr) return -1;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(Hq) * fa::HD, static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(B)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(Hq) * fa::HD * 4, static_cast<cuuint64_t>(S) * Hq * fa::HD * 4};
    cuuint32_t box[3] = {32, fa::BQ, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult cr = enc(&tdq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, dq_acc, dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return static_cast<int>(cr);
  }
  fa::flash_bwd_kernel<<<grid, fa::BWD_THREADS, fa::BWD_SMEM, stream>>>(tq, tdo, tk, tv, tdq, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  {
    const int cols = Hq * fa::HD;
    const int64_t rows = static_cast<int64_t>(B) * S;
    dim3 cgrid((cols / 8 + 255) / 256, static_cast<unsigned>(rows < 4096 ? rows : 4096));
    fa::f32_to_bf16_rows_kernel<<<cgrid, 256, 0, stream>>>(dq_acc, reinterpret_cast<__nv_bfloat16*>(dQ), rows, cols,
                                                          dq_row_stride);
  }
  return static_cast<int>(cudaGetLastError());
}
