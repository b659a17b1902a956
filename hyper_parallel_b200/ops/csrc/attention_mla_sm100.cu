// Multi-head latent attention in the training (expanded) form of DeepSeek-V3 for sm_100a: every
// head has a 192-wide query / key (128 "nope" columns + 64 rotary columns) and a 128-wide value;
// the rotary key columns are one vector per token shared by all heads.  bf16, causal or full.
//
// The operands are read where the projections left them, without any concatenation:
//   q   [B, S, H, 192]   nope | rope per head (rope already applied)
//   kv  [B, S, H, 256]   k_nope | v per head (the output of the kv up-projection)
//   kr  [B, S, 64]       rotary key, shared by the heads
//   O   [B, S, H, 128]
//
// Forward kernel: the design of the 128-wide kernel (two 128-row query tiles per CTA that
// ping-pong between the tensor core and the softmax warps; scores, probabilities and output
// accumulators in tensor memory), with the operand staging re-planned for the wider contraction:
// all tiles are cut into 16 KB units of [128 rows x 64 columns] (K-major operands: Q, K) or
// [64 key rows x 128 columns] (the MN-major operand V); the two query tiles hold 6 units and the
// remaining shared memory is ONE ring of 8 units through which K_0 (3 units), V_0 (2 units), K_1,
// V_1, ... stream, each unit with its own full / empty barrier, so that a unit is refilled as
// soon as the last product that reads it has retired.
//
//   warp 0      TMA producer      warp 1      MMA issuer      warps 2-5 / 6-9   softmax of tile 0 / 1
//
// TMEM (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each; P (bf16 pairs) overwrites the
// first 64 columns of its score tile and is the A operand of the P V product from there.
//
// Backward kernel: see below.  Every wait is bounded; on expiry a status code is recorded and all
// roles unwind.
#include "attention_common.cuh"

namespace hpb {
namespace mla {

using namespace hpb::fa;

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int DQK = 192;
constexpr int DV = 128;
constexpr int DKV = 256;                    // k_nope | v per head in the packed kv tensor
constexpr int DR = 64;
constexpr int UNIT_BYTES = 128 * 64 * 2;    // 16 KB
constexpr int QK_UNITS = DQK / 64;          // 3
constexpr int V_UNITS = 2;
constexpr int KV_UNITS = QK_UNITS + V_UNITS;
constexpr int RING = 8;
constexpr int Q_BYTES = 2 * QK_UNITS * UNIT_BYTES;
constexpr int FWD_THREADS = 320;
constexpr int FWD_SMEM = Q_BYTES + RING * UNIT_BYTES + 1024 + 256;
constexpr float kRescaleThreshold = 8.0f;   // log2 units

struct FwdParams {
  int B, S, H;
  float scale_log2;   // softmax scale * log2(e)
  int causal;
  __nv_bfloat16* O;   // [B, S, H, 128] contiguous
  float* lse;         // [B, H, S] natural-log sum-exp
  int* status;
};

__device__ __forceinline__ int kv_tiles_for(int qt, int S, int causal) {
  const int total = (S + BN - 1) / BN;
  if (qt * BM >= S) return 0;
  return causal ? min(total, qt + 1) : total;
}

__global__ void __launch_bounds__(FWD_THREADS, 1)
mla_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
               const __grid_constant__ CUtensorMap tmap_kv64, const __grid_constant__ CUtensorMap tmap_kr,
               const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;                         // 2 tiles x 3 units
  uint8_t* sRing = smem + Q_BYTES;            // RING units
  uint64_t* q_full = reinterpret_cast<uint64_t*>(sRing + RING * UNIT_BYTES);
  uint64_t* u_full = q_full + 1;              // [RING]
  uint64_t* u_empty = u_full + RING;          // [RING]
  uint64_t* s_full = u_empty + RING;          // [2]
  uint64_t* p_full = s_full + 2;              // [2]
  uint64_t* pv_done = p_full + 2;             // [2]
  uint64_t* drain_bar = pv_done + 2;          // [1]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // heavy (late) query blocks first: they have the most key tiles under a causal mask
  const int num_pairs = (p.S + 2 * BM - 1) / (2 * BM);
  const int hb = static_cast<int>(blockIdx.x) % (p.H * p.B);
  const int pair = num_pairs - 1 - static_cast<int>(blockIdx.x) / (p.H * p.B);
  const int head = hb % p.H;
  const int batch = hb / p.H;
  const int n0 = kv_tiles_for(2 * pair, p.S, p.causal);
  const int n1 = kv_tiles_for(2 * pair + 1, p.S, p.causal);
  const int n_kv = max(n0, n1);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < RING; ++s) {
      mbar_init(&u_full[s], 1);
      mbar_init(&u_empty[s], 1);
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
    tma_prefetch_desc(&tmap_kv);
    tma_prefetch_desc(&tmap_kv64);
    tma_prefetch_desc(&tmap_kr);
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
      mbar_arrive_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int h = 0; h < QK_UNITS; ++h)
          tma_load_3d(sQ + (t * QK_UNITS + h) * UNIT_BYTES, &tmap_q, q_full, head * DQK + h * 64,
                      (2 * pair + t) * BM, batch);
      int u = 0;        // units issued so far; unit u lives in ring slot u % RING
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        for (int h = 0; h < KV_UNITS && ok; ++h, ++u) {
          const int slot = u % RING;
          ok = mbar_wait_bounded(&u_empty[slot], ((u / RING) & 1) ^ 1, abort_flag, p.status, kTimeoutEmptyBarrier,
                                 blockIdx.x);
          if (!ok) break;
          uint8_t* dst = sRing + slot * UNIT_BYTES;
          mbar_arrive_expect_tx(&u_full[slot], UNIT_BYTES);
          if (h < 2) {                      // K_j, nope columns [64 h, 64 h + 64)
            tma_load_3d(dst, &tmap_kv, &u_full[slot], head * DKV + h * 64, j * BN, batch);
          } else if (h == 2) {              // K_j, rotary columns (shared by the heads)
            tma_load_3d(dst, &tmap_kr, &u_full[slot], 0, j * BN, batch);
          } else {                          // V_j, key rows [64 (h - 3), +64): two boxes of 64 x 64
            const int r0 = j * BN + (h - 3) * 64;
            tma_load_3d(dst, &tmap_kv64, &u_full[slot], head * DKV + DV, r0, batch);
            tma_load_3d(dst + UNIT_BYTES / 2, &tmap_kv64, &u_full[slot], head * DKV + DV + 64, r0, batch);
          }
        }
      }
      if (!ok) {
        // wait (bounded) for the copies already issued, so that none lands after the CTA exits
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(q_full, 0) && globaltimer_ns() - t0 < 100000000ull) {}
        for (int b = 1; b <= min(u, RING); ++b) {
          const int idx = u - b;
          const uint64_t t1 = globaltimer_ns();
          while (!mbar_try_wait(&u_full[idx % RING], (idx / RING) & 1) && globaltimer_ns() - t1 < 100000000ull) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t idesc_s = make_idesc(1, 1, 0, 0, BM, BN);   // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_o = make_idesc(1, 1, 0, 1, BM, DV);   // P (tensor memory) x V (MN-major)
      const int nt[2] = {n0, n1};
      bool ok = true;
      const uint64_t q_desc = make_smem_desc_sw128(smem_u32(sQ), 0, 1024);
      const uint64_t k_desc = make_smem_desc_sw128(smem_u32(sRing), 0, 1024);                  // K unit, K-major
      const uint64_t v_desc = make_smem_desc_sw128(smem_u32(sRing), UNIT_BYTES / 2, 1024);     // V unit, MN-major
      auto wait_units = [&](int first, int count) {
        bool good = true;
        for (int u = first; u < first + count && good; ++u)
          good = mbar_wait_bounded(&u_full[u % RING], (u / RING) & 1, abort_flag, p.status, kTimeoutFullBarrier,
                                   blockIdx.x);
        return good;
      };
      auto free_units = [&](int first, int count) {
        for (int u = first; u < first + count; ++u) umma_commit(&u_empty[u % RING]);
      };
      // S_t = Q_t K_j^T: 3 units of 64 columns, 4 steps of 16 columns (32 bytes) each
      auto issue_s = [&](int t, int j) {
        const uint32_t d = tmem_base + t * BN;
#pragma unroll
        for (int kb = 0; kb < QK_UNITS; ++kb) {
          const uint64_t qa = desc_at(q_desc, (t * QK_UNITS + kb) * UNIT_BYTES);
          const uint64_t ka = desc_at(k_desc, ((j * KV_UNITS + kb) % RING) * UNIT_BYTES);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(d, desc_at(qa, kk * 32), desc_at(ka, kk * 32), idesc_s, (kb | kk) ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      };
      // O_t (+)= P_t V_j: P (bf16 pairs) occupies the first 64 columns of the score tile, 16 key
      // rows = 8 columns per step; V unit = 64 key rows, 16 rows = 2048 bytes per step
      auto issue_pv = [&](int t, int j, bool accumulate) {
        const uint32_t d = tmem_base + 2 * BN + t * DV;
        const uint32_t pt = tmem_base + t * BN;
#pragma unroll
        for (int k8 = 0; k8 < 8; ++k8) {
          const uint64_t va = desc_at(v_desc, ((j * KV_UNITS + QK_UNITS + (k8 >> 2)) % RING) * UNIT_BYTES +
                                                  (k8 & 3) * 2048);
          umma_f16_ts(d, pt + k8 * 8, va, idesc_o, (accumulate || k8) ? 1u : 0u);
        }
        umma_commit(&pv_done[t]);
      };
      ok = mbar_wait_bounded(q_full, 0, abort_flag, p.status, kTimeoutFullBarrier, blockIdx.x);
      if (ok) ok = wait_units(0, QK_UNITS);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < 2; ++t)
          if (nt[t] > 0) issue_s(t, 0);
        free_units(0, QK_UNITS);                             // K_0 is free once both S_t(K_0) retire
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        ok = wait_units(j * KV_UNITS + QK_UNITS, V_UNITS);   // V_j
        if (!ok) break;
        tc_fence_after();
        bool k_next = false;
        for (int t = 0; t < 2 && ok; ++t) {
          if (j < nt[t]) {
            ok = mbar_wait_bounded(&p_full[t], j & 1, abort_flag, p.status, kTimeoutTmemFull, blockIdx.x);
            if (!ok) break;
            tc_fence_after();
            issue_pv(t, j, j > 0);
          }
          if (j + 1 < nt[t]) {
            if (!k_next) {
              ok = wait_units((j + 1) * KV_UNITS, QK_UNITS);   // K_{j+1}
              if (!ok) break;
              tc_fence_after();
              k_next = true;
            }
            issue_s(t, j + 1);
          }
        }
        if (!ok) break;
        free_units(j * KV_UNITS + QK_UNITS, V_UNITS);                       // V_j
        if (j + 1 < n_kv) free_units((j + 1) * KV_UNITS, QK_UNITS);         // K_{j+1}: both S_t issued above
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
    const uint32_t o_addr = tmem_base + 2 * BN + t * DV + lane_off;
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
        // the maximum is only raised when it grows by more than 2^8: P stays bounded by 256 and
        // the accumulator is rescaled rarely; the result is exact after the final 1 / l
        need = true;
        alpha = fast_exp2(m - m_new);
        m = m_new;
        l *= alpha;
      }
      if (j > 0) {
        // P lies under the scores just produced, which the tensor core wrote after the previous
        // P V product: only a rescale of the accumulator has to wait for that product
        const bool any_need = __any_sync(0xffffffffu, need);
        if (any_need) {
          ok = mbar_wait_bounded(&pv_done[t], (j - 1) & 1, abort_flag, p.status, kTimeoutTmemEmpty, blockIdx.x);
          if (!ok) break;
          tc_fence_after();
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
      // P = 2^(s * scale - m) (masked scores are -inf -> 0), row sum, bf16 pairs packed in place
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
      const float2 nm2 = make_float2(-m, -m);
      float2 l2 = make_float2(0.f, 0.f);
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
      l += l2.x + l2.y;
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
        __nv_bfloat16* dst = p.O + ((static_cast<int64_t>(batch) * p.S + q_row) * p.H + head) * DV;
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
          p.lse[(static_cast<int64_t>(batch) * p.H + head) * p.S + q_row] = (m + log2f(l)) * 0.6931471805599453f;
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


}  // namespace mla
}  // namespace hpb

using namespace hpb;

// q [B, S, H, 192] (nope | rope), kv [B, S, H, 256] (k_nope | v), kr [B, S, 64] bf16: innermost dimension
// contiguous, row (token) and batch strides in elements.  O [B, S, H, 128] contiguous bf16, lse [B, H, S].
extern "C" int hpb_mla_attn_fwd(const void* q, long long q_batch_stride, long long q_row_stride, const void* kv,
                                long long kv_batch_stride, long long kv_row_stride, const void* kr,
                                long long kr_batch_stride, long long kr_row_stride, void* O, float* lse, int B, int S,
                                int H, float softmax_scale, int causal, int* status, cudaStream_t stream) {
  if (B <= 0 || S <= 0) return 0;
  if (H <= 0) return -2;
  if ((q_row_stride | kv_row_stride | kr_row_stride | q_batch_stride | kv_batch_stride | kr_batch_stride) & 7)
    return -2;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kv) | reinterpret_cast<uintptr_t>(kr) |
       reinterpret_cast<uintptr_t>(O)) & 15)
    return -2;
  cudaFree(nullptr);
  CUtensorMap tq, tkv, tkv64, tkr;
  int r = make_tmap_bsd(&tq, q, B, S, H * mla::DQK, q_batch_stride, q_row_stride);
  if (r) return r;
  r = make_tmap_bsd(&tkv, kv, B, S, H * mla::DKV, kv_batch_stride, kv_row_stride);
  if (r) return r;
  r = make_tmap_bsd(&tkv64, kv, B, S, H * mla::DKV, kv_batch_stride, kv_row_stride, 64);
  if (r) return r;
  r = make_tmap_bsd(&tkr, kr, B, S, mla::DR, kr_batch_stride, kr_row_stride);
  if (r) return r;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(mla::mla_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         mla::FWD_SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  mla::FwdParams p;
  p.B = B; p.S = S; p.H = H;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.causal = causal;
  p.O = reinterpret_cast<__nv_bfloat16*>(O);
  p.lse = lse;
  p.status = status;
  dim3 grid(((S + 2 * mla::BM - 1) / (2 * mla::BM)) * H * B);
  mla::mla_fwd_kernel<<<grid, mla::FWD_THREADS, mla::FWD_SMEM, stream>>>(tq, tkv, tkv64, tkr, p);
  return static_cast<int>(cudaGetLastError());
}
