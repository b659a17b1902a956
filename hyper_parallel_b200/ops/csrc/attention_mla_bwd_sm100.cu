// Backward of multi-head latent attention (192-wide query / key, 128-wide value, rotary key
// columns shared by the heads) for sm_100a.  Operand layout as in attention_mla_sm100.cu.
//
// One CTA owns one 128-row key/value tile of one (batch, head) and walks over the 64-row query
// tiles that see it.  Everything is computed transposed, so that the softmax threads (thread =
// key row) write the A operands of the following products as plain 128-byte rows:
//
//   S^T  = K Q^T            [kv 128 x q 64]   contraction 192
//   dP^T = V dO^T           [kv 128 x q 64]   contraction 128
//   P^T  = exp2(S^T c - lse)                                  -> bf16 pairs, tensor memory
//   dS^T = P^T o (dP^T - D)                                   -> bf16, shared memory
//   dV  += P^T dO           [kv 128 x 128]    accumulated over the whole walk
//   dK  += dS^T Q           [kv 128 x 192]    accumulated over the whole walk
//   dQ^T = K^T dS^T         [d 192 x q 64]    as two products of 128 rows: head elements 0..127 into
//                                             a buffer of their own, 64..191 (of which rows 64..127 =
//                                             elements 128..191 are read out) into the S^T buffer
//                                             between two score tiles
//
// Tensor memory (512 columns): S^T 64 | dP^T 64 | dQ^T 64 | dV 128 | dK 192.  The two accumulators
// leave room for three 64-column buffers only, so nothing is double buffered; instead every buffer
// is handed back as early as possible and the products of neighbouring steps interleave:
//
//   * the softmax warps release S^T as soon as their scores are in registers, so S^T of step
//     i + 2 is formed while step i + 1 is still being exponentiated;
//   * P^T (bf16 pairs) goes back into tensor memory, over the dP^T columns that the same thread has
//     just read, and is the A operand of the dV product from there; only dS^T goes through shared
//     memory (it is also a B operand), double buffered and handed back by the tensor core;
//   * per step the tensor core runs dV(i), dP^T(i + 1) (the softmax of step i + 1 waits for it;
//     in-order execution keeps it behind the read of P^T), dK(i), the upper dQ^T(i) into the S^T
//     buffer (the scores of step i + 1 are in registers by then), the lower dQ^T(i) while that
//     tile is read out, and then S^T(i + 2).
//
//   warp 0       TMA producer: K, V once; Q_i and dO_i through two 2-slot rings
//   warp 1       MMA issuer
//   warps 2-9    softmax / dS: two groups of four warps, each owning 32 of the 64 query columns;
//                they also write dV / dK at the end
//   warps 10-13  dQ read-out: fp32 tiles staged in a buffer of their own (32 KB) and added to the
//                fp32 dQ in global memory by TMA reduces, so the read-out never holds back the
//                softmax warps
//
// dK of the rotary columns is written per head; the caller sums it over the heads.
// Every wait is bounded; on expiry a status code is recorded and all roles unwind.
#include "attention_common.cuh"

namespace hpb {
namespace mla {

using namespace hpb::fa;

constexpr int BN = 128;
constexpr int BQ = 64;
constexpr int DQK = 192;
constexpr int DV = 128;
constexpr int DKV = 256;
constexpr int DR = 64;
constexpr int UNIT_BYTES = 128 * 64 * 2;        // 16 KB: [128 key rows x 64 columns]
constexpr int QSUB_BYTES = BQ * 64 * 2;         // 8 KB:  [64 query rows x 64 columns]
constexpr int Q_BYTES = 3 * QSUB_BYTES;         // 24 KB
constexpr int DO_BYTES = 2 * QSUB_BYTES;        // 16 KB
constexpr int RING = 2;
constexpr int PT_BYTES = BN * BQ * 2;           // 16 KB
constexpr int BWD_THREADS = 448;
constexpr int STAGE_TILE = BQ * 32 * 4;          // 8 KB: [64 query rows x 32 head elements] fp32
constexpr int BWD_SMEM = 3 * UNIT_BYTES + 2 * UNIT_BYTES + RING * (Q_BYTES + DO_BYTES) + 2 * PT_BYTES +
                         4 * STAGE_TILE + 2 * 2 * BQ * 4 + 1024 + 256;
static_assert(BWD_SMEM <= 227 * 1024, "shared memory budget");

struct BwdParams {
  int B, S, H;
  float scale, scale_log2;
  int causal;
  int head_group;        // (batch, head) pairs scheduled together
  int probe;             // timing probes (results are wrong): 1 = no dQ staging / reduce, 2 = no exponentials,
                         // 4 / 8 / 16 = the dQ^T / dK, dV / S^T, dP^T products are not issued
  const float* lse;      // [B, H, S]
  const float* delta;    // [B, H, S]  rowsum(dO o O)
  __nv_bfloat16* dKV;    // [B, S, H, 256]: dK nope | dV
  __nv_bfloat16* dKR;    // [B, S, H, 64]: dK of the rotary columns, per head
  int* status;
  long long* prof;       // optional [16]: cycles that one softmax thread of CTA 0 spent per phase, summed over its walk
};

__global__ void __launch_bounds__(BWD_THREADS, 1)
mla_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
               const __grid_constant__ CUtensorMap tmap_kv, const __grid_constant__ CUtensorMap tmap_kr,
               const __grid_constant__ CUtensorMap tmap_dq, const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;                                         // 3 units: nope 0..63, nope 64..127, rope
  uint8_t* sV = sK + 3 * UNIT_BYTES;                          // 2 units: columns 0..63, 64..127
  uint8_t* sQ = sV + 2 * UNIT_BYTES;                          // ring of Q tiles (3 x 8 KB each)
  uint8_t* sDO = sQ + RING * Q_BYTES;                         // ring of dO tiles (2 x 8 KB each)
  uint8_t* sDS = sDO + RING * DO_BYTES;                       // dS^T, two buffers of 16 KB
  uint8_t* sStage = sDS + 2 * PT_BYTES;                       // dQ staging: one 8 KB tile per dQ warp
  float* sStat = reinterpret_cast<float*>(sStage + 4 * STAGE_TILE);  // [2][2][64]: lse * log2e, delta
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(sStat + 2 * 2 * BQ);
  uint64_t* q_full = kv_full + 1;                // [2]
  uint64_t* q_empty = q_full + RING;             // [2]
  uint64_t* do_full = q_empty + RING;            // [2]
  uint64_t* do_empty = do_full + RING;           // [2]
  uint64_t* st_full = do_empty + RING;           // [1]  S^T of a step complete
  uint64_t* st_consumed = st_full + 1;           // [1]  S^T of a step is in registers (8 warp arrivals)
  uint64_t* dpt_full = st_consumed + 1;          // [1]  dP^T of a step complete
  uint64_t* ds_full = dpt_full + 1;              // [2]  P^T / dS^T written, dP^T read (8 warp arrivals)
  uint64_t* pt_free = ds_full + 2;               // [2]  every product reading dS^T buffer b has retired
  uint64_t* dq_lo_full = pt_free + 2;            // [1]
  uint64_t* dq_hi_full = dq_lo_full + 1;         // [1]
  uint64_t* dq_lo_drained = dq_hi_full + 1;      // [1]  (4 warp arrivals)
  uint64_t* dq_hi_drained = dq_lo_drained + 1;   // [1]  (2 warp arrivals)
  uint64_t* stat_full = dq_hi_drained + 1;       // [2]  lse / delta of a step staged (4 warp arrivals)
  uint64_t* acc_full = stat_full + 2;            // [1]
  uint64_t* drain_bar = acc_full + 1;            // [1]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // (batch, head) pairs are processed in groups of `head_group`: the CTAs that run at the same time
  // then add into a few MB of the fp32 dQ (and re-read the same Q / dO), which stays in L2; inside
  // a group the key tiles go in ascending order (causal: low tiles have the longest walk)
  int hb, jt;
  {
    const int n_tiles = (p.S + BN - 1) / BN;
    const int pairs = p.H * p.B;
    const int hg = max(1, min(p.head_group, pairs));
    const int g0 = static_cast<int>(blockIdx.x) / (hg * n_tiles) * hg;
    const int gsz = min(hg, pairs - g0);
    const int r = static_cast<int>(blockIdx.x) - g0 * n_tiles;
    jt = r / gsz;
    hb = g0 + r % gsz;
  }
  const int head = hb % p.H;
  const int batch = hb / p.H;
  const int k0 = jt * BN;
  const int nq = (p.S + BQ - 1) / BQ;
  const int i_start = p.causal ? (k0 / BQ) : 0;       // first query tile that sees this key tile
  const int n_it = nq - i_start;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < RING; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
      mbar_init(&do_full[s], 1);
      mbar_init(&do_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&ds_full[b], 8);
      mbar_init(&pt_free[b], 1);
      mbar_init(&stat_full[b], 4);
    }
    mbar_init(st_full, 1);
    mbar_init(st_consumed, 8);
    mbar_init(dpt_full, 1);
    mbar_init(dq_lo_full, 1);
    mbar_init(dq_hi_full, 1);
    mbar_init(dq_lo_drained, 4);
    mbar_init(dq_hi_drained, 2);
    mbar_init(acc_full, 1);
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_do);
    tma_prefetch_desc(&tmap_kv);
    tma_prefetch_desc(&tmap_kr);
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
  constexpr uint32_t COL_ST = 0;      // 64
  constexpr uint32_t COL_DPT = 64;    // 64
  constexpr uint32_t COL_DQ = 128;    // 64
  constexpr uint32_t COL_DV = 192;    // 128
  constexpr uint32_t COL_DK = 320;    // 192

  if (warp == 0) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 5 * UNIT_BYTES);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        tma_load_3d(sK + h * UNIT_BYTES, &tmap_kv, kv_full, head * DKV + h * 64, k0, batch);
        tma_load_3d(sV + h * UNIT_BYTES, &tmap_kv, kv_full, head * DKV + DV + h * 64, k0, batch);
      }
      tma_load_3d(sK + 2 * UNIT_BYTES, &tmap_kr, kv_full, 0, k0, batch);
      int q_issued = 0, do_issued = 0;
      bool ok = true;
      for (int it = 0; it < n_it && ok; ++it) {
        const int slot = it % RING;
        const uint32_t phase = (it / RING) & 1;
        const int q0 = (i_start + it) * BQ;
        ok = mbar_wait_bounded(&q_empty[slot], phase ^ 1, abort_flag, p.status, kTimeoutEmptyBarrier, blockIdx.x);
        if (!ok) break;
        mbar_arrive_expect_tx(&q_full[slot], Q_BYTES);
#pragma unroll
        for (int h = 0; h < 3; ++h)
          tma_load_3d(sQ + slot * Q_BYTES + h * QSUB_BYTES, &tmap_q, &q_full[slot], head * DQK + h * 64, q0, batch);
        ++q_issued;
        ok = mbar_wait_bounded(&do_empty[slot], phase ^ 1, abort_flag, p.status, kTimeoutEmptyBarrier, blockIdx.x);
        if (!ok) break;
        mbar_arrive_expect_tx(&do_full[slot], DO_BYTES);
#pragma unroll
        for (int h = 0; h < 2; ++h)
          tma_load_3d(sDO + slot * DO_BYTES + h * QSUB_BYTES, &tmap_do, &do_full[slot], head * DV + h * 64, q0, batch);
        ++do_issued;
      }
      if (!ok) {
        // wait (bounded) for the copies already issued, so that none lands after the CTA exits
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(kv_full, 0) && globaltimer_ns() - t0 < 100000000ull) {}
        for (int b = 1; b <= min(q_issued, RING); ++b) {
          const int it = q_issued - b;
          const uint64_t t1 = globaltimer_ns();
          while (!mbar_try_wait(&q_full[it % RING], (it / RING) & 1) && globaltimer_ns() - t1 < 100000000ull) {}
        }
        for (int b = 1; b <= min(do_issued, RING); ++b) {
          const int it = do_issued - b;
          const uint64_t t1 = globaltimer_ns();
          while (!mbar_try_wait(&do_full[it % RING], (it / RING) & 1) && globaltimer_ns() - t1 < 100000000ull) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_st = make_idesc(1, 1, 0, 0, BN, BQ);    // K / V (K-major) x Q / dO (K-major)
      constexpr uint32_t idesc_dv = make_idesc(1, 1, 0, 1, BN, DV);    // P^T (K-major) x dO (MN-major)
      constexpr uint32_t idesc_dk = make_idesc(1, 1, 0, 1, BN, DQK);   // dS^T (K-major) x Q (MN-major)
      constexpr uint32_t idesc_dq = make_idesc(1, 1, 1, 1, 128, BQ);   // K^T (MN-major) x dS^T (MN-major)
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), q_addr = smem_u32(sQ), do_addr = smem_u32(sDO),
                     ds_addr = smem_u32(sDS);
      bool ok = true;
      const uint64_t k_desc = make_smem_desc_sw128(k_addr, 0, 1024);               // K as K-major A
      const uint64_t v_desc = make_smem_desc_sw128(v_addr, 0, 1024);               // V as K-major A
      const uint64_t kt_desc = make_smem_desc_sw128(k_addr, UNIT_BYTES, 1024);     // K^T as MN-major A
      const uint64_t qk_desc = make_smem_desc_sw128(q_addr, 0, 1024);              // Q as K-major B
      const uint64_t qm_desc = make_smem_desc_sw128(q_addr, QSUB_BYTES, 1024);     // Q as MN-major B
      const uint64_t dok_desc = make_smem_desc_sw128(do_addr, 0, 1024);            // dO as K-major B
      const uint64_t dom_desc = make_smem_desc_sw128(do_addr, QSUB_BYTES, 1024);   // dO as MN-major B
      const uint64_t dsk_desc = make_smem_desc_sw128(ds_addr, 0, 1024);            // dS^T as K-major A
      const uint64_t dsm_desc = make_smem_desc_sw128(ds_addr, PT_BYTES, 1024);     // dS^T as MN-major B
      auto wait_on = [&](uint64_t* bar, uint32_t parity, int code) {
        return mbar_wait_bounded(bar, parity, abort_flag, p.status, code, blockIdx.x);
      };
      auto q_ready = [&](int it) { return wait_on(&q_full[it % RING], (it / RING) & 1, kTimeoutFullBarrier); };
      auto do_ready = [&](int it) { return wait_on(&do_full[it % RING], (it / RING) & 1, kTimeoutFullBarrier); };
      // S^T(it) = K Q^T: 3 units of 64 columns, 4 steps of 16 columns (32 bytes) each
      auto issue_st = [&](int it) {
        const uint64_t qa = desc_at(qk_desc, (it % RING) * Q_BYTES);
        if (!(p.probe & 16))
#pragma unroll
        for (int kb = 0; kb < 3; ++kb)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(tmem_base + COL_ST, desc_at(k_desc, kb * UNIT_BYTES + kk * 32),
                     desc_at(qa, kb * QSUB_BYTES + kk * 32), idesc_st, (kb | kk) ? 1u : 0u);
        umma_commit(st_full);
      };
      // dP^T(it) = V dO^T
      auto issue_dpt = [&](int it) {
        const uint64_t doa = desc_at(dok_desc, (it % RING) * DO_BYTES);
        if (!(p.probe & 16))
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(tmem_base + COL_DPT, desc_at(v_desc, kb * UNIT_BYTES + kk * 32),
                     desc_at(doa, kb * QSUB_BYTES + kk * 32), idesc_st, (kb | kk) ? 1u : 0u);
        umma_commit(dpt_full);
      };
      ok = wait_on(kv_full, 0, kTimeoutFullBarrier);
      if (ok) ok = q_ready(0);
      if (ok) {
        tc_fence_after();
        issue_st(0);
        ok = do_ready(0);
      }
      if (ok) {
        tc_fence_after();
        issue_dpt(0);
      }
      if (ok && n_it > 1) {
        ok = wait_on(st_consumed, 0, kTimeoutTmemEmpty);
        if (ok) ok = q_ready(1);
        if (ok) {
          tc_fence_after();
          issue_st(1);
        }
      }
      const bool prof = p.prof != nullptr && blockIdx.x == 0;
      long long acc[5] = {0, 0, 0, 0, 0};
      long long tp = prof ? clock64() : 0;
      auto tick = [&](int i) {
        if (prof) {
          const long long t = clock64();
          acc[i] += t - tp;
          tp = t;
        }
      };
      for (int it = 0; it < n_it && ok; ++it) {
        const int b = it & 1;
        ok = wait_on(&ds_full[b], (it >> 1) & 1, kTimeoutTmemFull);
        if (!ok) break;
        tick(0);
        tc_fence_after();
        const uint64_t qa = desc_at(qm_desc, (it % RING) * Q_BYTES);
        const uint64_t doa = desc_at(dom_desc, (it % RING) * DO_BYTES);
        const uint64_t dsa = desc_at(dsk_desc, b * PT_BYTES);
        const uint64_t dsm = desc_at(dsm_desc, b * PT_BYTES);
        const uint32_t first = it ? 1u : 0u;
        // dV += P^T dO (contraction over the 64 query rows: 4 steps of 16).  P^T lies in the dP^T
        // buffer: query rows 0..31 in columns 0..15, 32..63 in columns 32..47 (8 columns per step)
        if (!(p.probe & 8))
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_f16_ts(tmem_base + COL_DV, tmem_base + COL_DPT + (kk >> 1) * 32 + (kk & 1) * 8, desc_at(doa, kk * 2048),
                      idesc_dv, kk ? 1u : first);
        umma_commit(&do_empty[it % RING]);
        // dP^T of the next step: its softmax is waiting for nothing else (executes behind dV, which
        // reads the buffer it overwrites)
        if (it + 1 < n_it) {
          ok = do_ready(it + 1);
          if (!ok) break;
          tc_fence_after();
          issue_dpt(it + 1);
        }
        // dK += dS^T Q; frees the Q slot, so that the load of step it + 2 starts early
        if (!(p.probe & 8))
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_f16(tmem_base + COL_DK, desc_at(dsa, kk * 32), desc_at(qa, kk * 2048), idesc_dk, kk ? 1u : first);
        umma_commit(&q_empty[it % RING]);
        tick(1);
        // dQ^T = K^T dS^T (contraction over the 128 key rows: 8 steps of 16).  Head elements 64..191
        // (units 1, 2 of K) go into the S^T buffer, free once the scores of step it + 1 are in
        // registers (the three products above have kept the tensor core busy meanwhile)
        if (it + 1 < n_it) {
          ok = wait_on(st_consumed, (it + 1) & 1, kTimeoutTmemEmpty);
          if (!ok) break;
          tc_fence_after();
        }
        tick(2);
        if (!(p.probe & 4))
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_f16(tmem_base + COL_ST, desc_at(kt_desc, UNIT_BYTES + kk * 2048), desc_at(dsm, kk * 2048), idesc_dq,
                   kk ? 1u : 0u);
        umma_commit(dq_hi_full);
        // head elements 0..127 (units 0, 1 of K) go into the dQ^T buffer, free once the tile of the
        // step before was read; this product runs while the upper tile is read out
        if (it > 0) {
          ok = wait_on(dq_lo_drained, (it - 1) & 1, kTimeoutTmemEmpty);
          if (!ok) break;
          tc_fence_after();
        }
        if (!(p.probe & 4))
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_f16(tmem_base + COL_DQ, desc_at(kt_desc, kk * 2048), desc_at(dsm, kk * 2048), idesc_dq, kk ? 1u : 0u);
        umma_commit(dq_lo_full);
        umma_commit(&pt_free[b]);     // every reader of dS^T of this step has been issued
        tick(3);
        // The upper tile must have left the S^T buffer before anything else is written there: S^T of
        // step it + 2, or -- in the last two steps, where no score tile follows -- the upper tile of
        // the next step (this wait also keeps the phase of dq_hi_full at most one ahead of its readers)
        if (it + 1 < n_it) {
          ok = wait_on(dq_hi_drained, it & 1, kTimeoutTmemEmpty);
          if (!ok) break;
          if (it + 2 < n_it) {
            ok = q_ready(it + 2);
            if (!ok) break;
            tc_fence_after();
            issue_st(it + 2);
          }
        }
        tick(4);
      }
      if (prof)
        for (int i = 0; i < 5; ++i) p.prof[10 + i] = acc[i];
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
      const int c = wg;                       // this group's 32 query columns
      auto load_stat = [&](int it) -> float {
        // threads 0..63 fetch lse (scaled to log2), 64..127 fetch delta, of step `it`
        if (it >= n_it || tid >= 128) return 0.f;
        const int q = (i_start + it) * BQ + (tid & 63);
        if (q >= p.S) return tid < 64 ? INFINITY : 0.f;
        const int64_t off = (static_cast<int64_t>(batch) * p.H + head) * p.S + q;
        return tid < 64 ? p.lse[off] : p.delta[off];     // raw: scaled when staged, a step later
      };
      float stat_next = load_stat(0);
      const bool prof = p.prof != nullptr && blockIdx.x == 0 && threadIdx.x == 64;
      long long acc[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
      long long tp = prof ? clock64() : 0;
      auto tick = [&](int i) {
        if (prof) {
          const long long t = clock64();
          acc[i] += t - tp;
          tp = t;
        }
      };
      for (int it = 0; it < n_it && ok; ++it) {
        const int b = it & 1;
        const uint32_t par = (it >> 1) & 1;
        float* stat = sStat + b * 2 * BQ;
        // dS^T buffer b is free again (the products of step it - 2 that read it have retired); this
        // also means that all eight softmax warps have finished step it - 2, so the statistics
        // buffer b can be rewritten
        ok = mbar_wait_bounded(&pt_free[b], par ^ 1, abort_flag, p.status, kTimeoutTmemEmpty, blockIdx.x);
        if (!ok) break;
        tick(0);
        if (tid < 128) stat[tid] = tid < 64 ? stat_next * 1.4426950408889634f : stat_next;
        stat_next = load_stat(it + 1);
        __syncwarp();
        if (lane == 0 && wg == 0) mbar_arrive(&stat_full[b]);
        ok = mbar_wait_bounded(&stat_full[b], par, abort_flag, p.status, kTimeoutFullBarrier, blockIdx.x);
        tick(1);
        if (ok) ok = mbar_wait_bounded(st_full, it & 1, abort_flag, p.status, kTimeoutTmemFull, blockIdx.x);
        if (!ok) break;
        tick(2);
        tc_fence_after();
        uint32_t rs[32];
        tmem_ld_32x32b_x32(tmem_base + COL_ST + c * 32 + lane_off, rs);
        tmem_ld_wait();
        // the scores are in registers: the tensor core may form S^T of the next step but one
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(st_consumed);
        tick(3);
        const int q0 = (i_start + it) * BQ;
        // visible iff key <= query:  column c >= kv_row - q0
        const int cmin = p.causal ? kv_row - q0 : 0;
        // warp-uniform: does any row of this warp hide any column of this step?
        const bool masked = (k0 + quarter * 32 + 32 > p.S) || (p.causal && k0 + quarter * 32 + 31 - q0 > 0);
        uint8_t* ds_row = sDS + b * PT_BYTES + row * 128;
        float2 ev[16];
        uint32_t pk[16];
        {
          const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
#pragma unroll
          for (int i2 = 0; i2 < 16; ++i2) {
            const float2 ls = *reinterpret_cast<const float2*>(stat + c * 32 + 2 * i2);
            float2 e = fma2(make_float2(__uint_as_float(rs[2 * i2]), __uint_as_float(rs[2 * i2 + 1])), sc2,
                            make_float2(-ls.x, -ls.y));
            if (!(p.probe & 2)) {
              e.x = fast_exp2(e.x);
              e.y = fast_exp2(e.y);
            }
            if (masked) {
              const int col = c * 32 + 2 * i2;
              if (!row_live || col < cmin) e.x = 0.f;
              if (!row_live || col + 1 < cmin) e.y = 0.f;
            }
            ev[i2] = e;
            const __nv_bfloat162 eb = __floats2bfloat162_rn(e.x, e.y);
            pk[i2] = *reinterpret_cast<const uint32_t*>(&eb);
          }
        }
        tick(4);
        ok = mbar_wait_bounded(dpt_full, it & 1, abort_flag, p.status, kTimeoutTmemFull, blockIdx.x);
        if (!ok) break;
        tick(5);
        tc_fence_after();
        {
          uint32_t rp[32], dk[16];
          tmem_ld_32x32b_x32(tmem_base + COL_DPT + c * 32 + lane_off, rp);
          tmem_ld_wait();
          // P^T over the first 16 of the 32 columns just read (this thread's own)
          tmem_st_32x32b_x16(tmem_base + COL_DPT + c * 32 + lane_off, pk);
          tick(6);
#pragma unroll
          for (int i2 = 0; i2 < 16; ++i2) {
            const float2 dl = *reinterpret_cast<const float2*>(stat + BQ + c * 32 + 2 * i2);
            const float2 d = mul2(ev[i2], add2(make_float2(__uint_as_float(rp[2 * i2]), __uint_as_float(rp[2 * i2 + 1])),
                                               make_float2(-dl.x, -dl.y)));
            const __nv_bfloat162 db = __floats2bfloat162_rn(d.x, d.y);
            dk[i2] = *reinterpret_cast<const uint32_t*>(&db);
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int chunk = c * 4 + q4;
            *reinterpret_cast<uint4*>(ds_row + ((chunk ^ sw) << 4)) =
                make_uint4(dk[4 * q4], dk[4 * q4 + 1], dk[4 * q4 + 2], dk[4 * q4 + 3]);
          }
        }
        tick(7);
        tmem_st_wait();
        fence_proxy_async();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ds_full[b]);
        tick(8);
      }
      if (prof) {
        for (int i = 0; i < 9; ++i) p.prof[i] = acc[i];
        p.prof[9] = n_it;
      }
    } else {
      // ------------------------------------------------------ dQ reduction --
      // dQ^T (lane = head element, column = query row) is transposed through this warp's staging
      // tile as a dense fp32 [64 query rows x 32 head elements] tile, which one TMA reduce adds to
      // the fp32 dQ in global memory.  Warps 2 and 3 own lanes 64..127, where the upper product
      // leaves the head elements 128..191: they pass a second tile per step through the same
      // staging memory.
      const bool has_hi = quarter >= 2;
      const bool staged = !(p.probe & 1);
      uint8_t* tile = sStage + quarter * STAGE_TILE;
      float* stage = reinterpret_cast<float*>(tile) + lane;
      for (int it = 0; it < n_it && ok; ++it) {
        const int q0 = (i_start + it) * BQ;
        uint32_t r[64];
        if (has_hi) {
          // the upper tile first: the next score tile waits for its buffer
          ok = mbar_wait_bounded(dq_hi_full, it & 1, abort_flag, p.status, kTimeoutTmemFull, blockIdx.x);
          if (!ok) break;
          tc_fence_after();
          tmem_ld32(tmem_base + COL_ST + lane_off, r);
          tmem_ld32(tmem_base + COL_ST + 32 + lane_off, r + 32);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(dq_hi_drained);                // S^T of the step after next may overwrite the buffer
            tma_store_wait_read<0>();                  // the tile of the step before has left the staging memory
          }
          __syncwarp();
          if (staged) {
#pragma unroll
            for (int i = 0; i < 64; ++i) stage[i * 32] = __uint_as_float(r[i]) * p.scale;
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              tma_reduce_add_3d(&tmap_dq, tile, head * DQK + 128 + (quarter - 2) * 32, q0, batch);
              tma_store_commit();
            }
          }
        }
        ok = mbar_wait_bounded(dq_lo_full, it & 1, abort_flag, p.status, kTimeoutTmemFull, blockIdx.x);
        if (!ok) break;
        tc_fence_after();
        tmem_ld32(tmem_base + COL_DQ + lane_off, r);
        tmem_ld32(tmem_base + COL_DQ + 32 + lane_off, r + 32);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(dq_lo_drained);                  // the lower product of the next step may overwrite the buffer
          tma_store_wait_read<0>();
        }
        __syncwarp();
        if (staged) {
#pragma unroll
          for (int i = 0; i < 64; ++i) stage[i * 32] = __uint_as_float(r[i]) * p.scale;
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            tma_reduce_add_3d(&tmap_dq, tile, head * DQK + quarter * 32, q0, batch);
            tma_store_commit();
          }
        }
      }
      if (lane == 0) tma_store_wait<0>();
    }
    // ------------------------------------------------- dV / dK write-out --
    // group 0: dV (128 columns) and the rotary 64 columns of dK; group 1: the 128 nope columns of dK
    if (ok && n_it > 0 && wg < 2) {
      ok = mbar_wait_bounded(acc_full, 0, abort_flag, p.status, kTimeoutTmemFull, blockIdx.x);
      if (ok) {
        tc_fence_after();
        const int kv_row = k0 + row;
        const float mul = wg == 0 ? 1.f : p.scale;
        const int64_t tok = static_cast<int64_t>(batch) * p.S + kv_row;
        __nv_bfloat16* dst = p.dKV + (tok * p.H + head) * DKV + (wg == 0 ? DV : 0);
        const uint32_t src = tmem_base + (wg == 0 ? COL_DV : COL_DK) + lane_off;
        auto put32 = [&](uint32_t taddr, __nv_bfloat16* out, float f) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr, r);
          tmem_ld_wait();
          if (kv_row < p.S) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 v;
              __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
              for (int e = 0; e < 4; ++e)
                vb[e] = __floats2bfloat162_rn(__uint_as_float(r[8 * q4 + 2 * e]) * f,
                                              __uint_as_float(r[8 * q4 + 2 * e + 1]) * f);
              reinterpret_cast<uint4*>(out)[q4] = v;
            }
          }
        };
#pragma unroll 1
        for (int c = 0; c < 4; ++c) put32(src + c * 32, dst + c * 32, mul);
        if (wg == 0) {
          __nv_bfloat16* dr = p.dKR + (tok * p.H + head) * DR;
#pragma unroll 1
          for (int c = 0; c < 2; ++c) put32(tmem_base + COL_DK + 128 + c * 32 + lane_off, dr + c * 32, p.scale);
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

// out[t, c] = sum over heads of in[t, h, c] (64 columns, fp32 accumulation); one warp per token
__global__ void mla_sum_heads_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                     int64_t tokens, int H) {
  const int64_t w = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= tokens) return;
  const __nv_bfloat162* src = reinterpret_cast<const __nv_bfloat162*>(in + w * H * DR) + lane;
  float2 acc = make_float2(0.f, 0.f);
  for (int h = 0; h < H; ++h) {
    const float2 x = __bfloat1622float2(src[h * (DR / 2)]);
    acc.x += x.x;
    acc.y += x.y;
  }
  reinterpret_cast<__nv_bfloat162*>(out + w * DR)[lane] = __floats2bfloat162_rn(acc.x, acc.y);
}

}  // namespace mla
}  // namespace hpb

using namespace hpb;

// Backward schedule: (batch, head) pairs per group; <= 0 = all pairs in one group (key-tile major).
static int g_mla_bwd_head_group = 16;
extern "C" void hpb_mla_attn_set_head_group(int pairs) { g_mla_bwd_head_group = pairs; }
// Timing probes for the benchmarks (the gradients are wrong while one is set): see BwdParams::probe.
static long long* g_mla_bwd_prof = nullptr;
// Device buffer of 16 int64 that receives the phase timings of one softmax thread (nullptr = off).
extern "C" void hpb_mla_attn_set_prof(long long* buf) { g_mla_bwd_prof = buf; }
static int g_mla_bwd_probe = 0;
extern "C" void hpb_mla_attn_set_probe(int mask) { g_mla_bwd_probe = mask; }

// Backward.  q [B, S, H, 192], kv [B, S, H, 256] (k_nope | v), kr [B, S, 64], O / dO [B, S, H, 128] bf16
// with the innermost dimension contiguous and row (token) / batch strides in elements; lse from the
// forward.  Outputs (contiguous bf16): dQ [B, S, H, 192], dKV [B, S, H, 256] (dK nope | dV), dKR
// [B, S, 64] (summed over the heads).  Workspace: dq_acc fp32 [B, S, H, 192] (cleared here), delta
// fp32 [B, H, S], dkr_heads bf16 [B, S, H, 64].
extern "C" int hpb_mla_attn_bwd(const void* q, long long q_batch_stride, long long q_row_stride, const void* kv,
                                long long kv_batch_stride, long long kv_row_stride, const void* kr,
                                long long kr_batch_stride, long long kr_row_stride, const void* O, const float* lse,
                                const void* dO, long long do_batch_stride, long long do_row_stride, void* dQ,
                                void* dKV, void* dKR, float* dq_acc, float* delta, void* dkr_heads, int B, int S,
                                int H, float softmax_scale, int causal, int* status, cudaStream_t stream) {
  if (B <= 0 || S <= 0) return 0;
  if (H <= 0) return -2;
  if ((q_row_stride | kv_row_stride | kr_row_stride | do_row_stride | q_batch_stride | kv_batch_stride |
       kr_batch_stride | do_batch_stride) & 7)
    return -2;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kv) | reinterpret_cast<uintptr_t>(kr) |
       reinterpret_cast<uintptr_t>(dO) | reinterpret_cast<uintptr_t>(dQ) | reinterpret_cast<uintptr_t>(dKV) |
       reinterpret_cast<uintptr_t>(dKR) | reinterpret_cast<uintptr_t>(O) | reinterpret_cast<uintptr_t>(dq_acc) |
       reinterpret_cast<uintptr_t>(dkr_heads)) & 15)
    return -2;
  cudaFree(nullptr);
  CUtensorMap tq, tdo, tkv, tkr, tdq;
  int r = make_tmap_bsd(&tq, q, B, S, H * mla::DQK, q_batch_stride, q_row_stride, mla::BQ);
  if (r) return r;
  r = make_tmap_bsd(&tdo, dO, B, S, H * mla::DV, do_batch_stride, do_row_stride, mla::BQ);
  if (r) return r;
  r = make_tmap_bsd(&tkv, kv, B, S, H * mla::DKV, kv_batch_stride, kv_row_stride);
  if (r) return r;
  r = make_tmap_bsd(&tkr, kr, B, S, mla::DR, kr_batch_stride, kr_row_stride);
  if (r) return r;
  {
    EncodeTiledFn enc = fa_encode_fn();
    if (enc == nullptr) return -1;
    const cuuint64_t cols = static_cast<cuuint64_t>(H) * mla::DQK;
    cuuint64_t dims[3] = {cols, static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(B)};
    cuuint64_t strides[2] = {cols * 4, static_cast<cuuint64_t>(S) * cols * 4};
    cuuint32_t box[3] = {32, mla::BQ, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult cr = enc(&tdq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, dq_acc, dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return static_cast<int>(cr);
  }
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(mla::mla_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         mla::BWD_SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  const int64_t nq = static_cast<int64_t>(B) * S * H * mla::DQK;
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, nq * sizeof(float), stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  {
    const int64_t warps = static_cast<int64_t>(B) * S * H;
    const int threads = 256;
    const int64_t blocks = (warps * 32 + threads - 1) / threads;
    fa::attn_delta_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(dO), do_batch_stride, do_row_stride,
        reinterpret_cast<const __nv_bfloat16*>(O), delta, B, S, H);
  }
  mla::BwdParams p;
  p.B = B; p.S = S; p.H = H;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.causal = causal;
  p.head_group = g_mla_bwd_head_group > 0 ? g_mla_bwd_head_group : (1 << 30);
  p.probe = g_mla_bwd_probe;
  p.prof = g_mla_bwd_prof;
  p.lse = lse;
  p.delta = delta;
  p.dKV = reinterpret_cast<__nv_bfloat16*>(dKV);
  p.dKR = reinterpret_cast<__nv_bfloat16*>(dkr_heads);
  p.status = status;
  dim3 grid(((S + mla::BN - 1) / mla::BN) * H * B);
  mla::mla_bwd_kernel<<<grid, mla::BWD_THREADS, mla::BWD_SMEM, stream>>>(tq, tdo, tkv, tkr, tdq, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  {
    const int cols = H * mla::DQK;
    const int64_t rows = static_cast<int64_t>(B) * S;
    dim3 cgrid((cols / 8 + 255) / 256, static_cast<unsigned>(rows < 4096 ? rows : 4096));
    fa::f32_to_bf16_rows_kernel<<<cgrid, 256, 0, stream>>>(dq_acc, reinterpret_cast<__nv_bfloat16*>(dQ), rows, cols,
                                                          cols);
    const int64_t tokens = rows;
    mla::mla_sum_heads_kernel<<<static_cast<unsigned>((tokens * 32 + 255) / 256), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(dkr_heads), reinterpret_cast<__nv_bfloat16*>(dKR), tokens, H);
  }
  return static_cast<int>(cudaGetLastError());
}
