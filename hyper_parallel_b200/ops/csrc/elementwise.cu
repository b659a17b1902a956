// Memory-bound kernels of the transformer step (sm_100a): RMSNorm fwd/bwd (with
// optional fused residual add), SwiGLU fwd/bwd, RoPE fwd/bwd, fused softmax
// cross-entropy fwd+bwd, and the fused AdamW update with fp32 master weights.
// All of them stream their operands exactly once with 16-byte accesses; the
// roofline for each is bytes / HBM bandwidth.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "hpb_noalloc.h"

namespace hpb {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; `red` is >= 32 floats of shared memory.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  return warp_max(t);
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const bf162* p = reinterpret_cast<const bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  bf162* p = reinterpret_cast<bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// ------------------------------------------------------------- RMSNorm ----
constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXV = 4;  // up to 256*8*4 = 8192 columns cached in registers

// y = (x [+ res]) * rstd * w ; optionally writes h = x + res ; rstd per row (fp32).
template <bool HAS_RES, int NV>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res,
                   const bf16* __restrict__ w, bf16* __restrict__ y, bf16* __restrict__ h_out,
                   float* __restrict__ rstd_out, int H, float eps) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const int nvec = H >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  const uint4* rr = HAS_RES ? reinterpret_cast<const uint4*>(res + row * H) : nullptr;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  float v[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      unpack8(xr[c], v[i]);
      if constexpr (HAS_RES) {
        float r[8];
        unpack8(rr[c], r);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] += r[e];
        // the normalised value must be computed from the bf16-rounded sum that is stored
        uint4 hu = pack8(v[i]);
        reinterpret_cast<uint4*>(h_out + row * H)[c] = hu;
        unpack8(hu, v[i]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      float wv[8], o[8];
      unpack8(wr[c], wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = v[i][e] * rstd * wv[e];
      reinterpret_cast<uint4*>(y + row * H)[c] = pack8(o);
    }
  }
}

// dx = rstd * (dy*w) - x * rstd^3/H * sum(dy*w*x)  [+ dres_in] ; per-CTA partial dw (fp32).
template <bool HAS_DRES, int NV>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                   const bf16* __restrict__ w, const float* __restrict__ rstd,
                   const bf16* __restrict__ dres_in, bf16* __restrict__ dx,
                   float* __restrict__ dw_partial, int T, int H) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  float wv[NV][8], dwacc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) unpack8(wr[c], wv[i]);
#pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[i][e] = 0.f;
  }
  for (int64_t row = blockIdx.x; row < T; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + row * H);
    const float rs = rstd[row];
    float xv[NV][8], gv[NV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
        unpack8(xr[c], xv[i]);
        unpack8(gr[c], gv[i]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          dwacc[i][e] += gv[i][e] * xv[i][e] * rs;
          gv[i][e] *= wv[i][e];
          dot += gv[i][e] * xv[i][e];
        }
      }
    }
    dot = block_sum(dot, red);
    const float coef = dot * rs * rs * rs / H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = gv[i][e] * rs - xv[i][e] * coef;
        if constexpr (HAS_DRES) {
          float r[8];
          unpack8(reinterpret_cast<const uint4*>(dres_in + row * H)[c], r);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += r[e];
        }
        reinterpret_cast<uint4*>(dx + row * H)[c] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      float4* dst = reinterpret_cast<float4*>(dw_partial + static_cast<int64_t>(blockIdx.x) * H + c * 8);
      dst[0] = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      dst[1] = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
    }
  }
}

// dw[c] = sum_p partial[p, c]  (fp32 in, bf16 or fp32 out, optional accumulate)
template <bool OUT_F32>
__global__ void colsum_kernel(const float* __restrict__ partial, void* __restrict__ out, int P,
                              int H, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += partial[static_cast<int64_t>(p) * H + c];
  if constexpr (OUT_F32) {
    float* o = reinterpret_cast<float*>(out);
    o[c] = accumulate ? o[c] + s : s;
  } else {
    bf16* o = reinterpret_cast<bf16*>(out);
    o[c] = __float2bfloat16(accumulate ? __bfloat162float(o[c]) + s : s);
  }
}

// -------------------------------------------------------------- SwiGLU ----
// gu is [T, 2F] with gate in columns [0,F) and up in [F,2F);  out[T,F] = silu(gate)*up
// Rows are walked by CTA pairs of (row, column chunk) without any division; every thread keeps two
// independent 16-byte gate/up pairs in flight.
__device__ __forceinline__ float fast_sigmoid(float g) { return __fdividef(1.f, 1.f + __expf(-g)); }

__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int64_t T, int F) {
  const int fv = F >> 3;
  for (int64_t t = blockIdx.y; t < T; t += gridDim.y) {
    const uint4* row = reinterpret_cast<const uint4*>(gu + t * 2 * F);
    uint4* orow = reinterpret_cast<uint4*>(out + t * F);
    for (int c = blockIdx.x * 512 + threadIdx.x; c < fv; c += gridDim.x * 512) {
      const int c2 = c + 256;
      const bool two = c2 < fv;
      const uint4 g0 = row[c], u0 = row[fv + c];
      uint4 g1 = g0, u1 = u0;
      if (two) {
        g1 = row[c2];
        u1 = row[fv + c2];
      }
      float g[8], u[8], o[8];
      unpack8(g0, g);
      unpack8(u0, u);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = g[e] * fast_sigmoid(g[e]) * u[e];
      orow[c] = pack8(o);
      if (two) {
        unpack8(g1, g);
        unpack8(u1, u);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = g[e] * fast_sigmoid(g[e]) * u[e];
        orow[c2] = pack8(o);
      }
    }
  }
}
// dgu[T,2F]: dgate = dout*up*(sig + g*sig*(1-sig)), dup = dout*silu(g)
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const bf16* __restrict__ gu, const bf16* __restrict__ dout, bf16* __restrict__ dgu, int64_t T,
                  int F) {
  const int fv = F >> 3;
  for (int64_t t = blockIdx.y; t < T; t += gridDim.y) {
    const uint4* row = reinterpret_cast<const uint4*>(gu + t * 2 * F);
    const uint4* drow = reinterpret_cast<const uint4*>(dout + t * F);
    uint4* orow = reinterpret_cast<uint4*>(dgu + t * 2 * F);
    for (int c = blockIdx.x * 512 + threadIdx.x; c < fv; c += gridDim.x * 512) {
      const int c2 = c + 256;
      const bool two = c2 < fv;
      const uint4 g0 = row[c], u0 = row[fv + c], d0 = drow[c];
      uint4 g1 = g0, u1 = u0, d1 = d0;
      if (two) {
        g1 = row[c2];
        u1 = row[fv + c2];
        d1 = drow[c2];
      }
      float g[8], u[8], d[8], dg[8], du[8];
      unpack8(g0, g);
      unpack8(u0, u);
      unpack8(d0, d);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float sg = fast_sigmoid(g[e]);
        dg[e] = d[e] * u[e] * sg * (1.f + g[e] * (1.f - sg));
        du[e] = d[e] * g[e] * sg;
      }
      orow[c] = pack8(dg);
      orow[fv + c] = pack8(du);
      if (two) {
        unpack8(g1, g);
        unpack8(u1, u);
        unpack8(d1, d);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float sg = fast_sigmoid(g[e]);
          dg[e] = d[e] * u[e] * sg * (1.f + g[e] * (1.f - sg));
          du[e] = d[e] * g[e] * sg;
        }
        orow[c2] = pack8(dg);
        orow[fv + c2] = pack8(du);
      }
    }
  }
}

// ---------------------------------------------------------------- RoPE ----
// In-place rotation of x[T, NH, D] (row stride `ld` elements between tokens) by the
// position pos[t] (or t % S when pos == nullptr); pairs are (i, i + D/2)
// ("rotate-half" convention).  sign = +1 forward, -1 backward (inverse rotation).
__global__ void rope_kernel(bf16* __restrict__ x, const int* __restrict__ pos, int64_t T, int S,
                            int NH, int D, int64_t ld, float theta_log2, float sign) {
  const int half = D >> 1;
  const int64_t total = T * NH * half;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(i % half);
    const int64_t th = i / half;
    const int h = static_cast<int>(th % NH);
    const int64_t t = th / NH;
    const float p = pos ? static_cast<float>(pos[t]) : static_cast<float>(t % S);
    const float inv_freq = exp2f(-theta_log2 * (2.f * j) / D);
    float sn, cs;
    sincosf(p * inv_freq, &sn, &cs);
    sn *= sign;
    bf16* base = x + t * ld + static_cast<int64_t>(h) * D;
    const float a = __bfloat162float(base[j]), b = __bfloat162float(base[j + half]);
    base[j] = __float2bfloat16(a * cs - b * sn);
    base[j + half] = __float2bfloat16(b * cs + a * sn);
  }
}

// Table-driven, vectorised variant: cs_table[S, D/2] holds (cos, sin) of position * inv_freq, so
// the kernel is pure streaming: 16-byte loads of both halves, 8 rotations per thread.
__global__ void rope_table_init_kernel(float2* __restrict__ table, int S, int half, int D, float theta_log2) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= S * half) return;
  const int j = i % half, pos = i / half;
  const float inv_freq = exp2f(-theta_log2 * (2.f * j) / D);
  float sn, cs;
  sincosf(pos * inv_freq, &sn, &cs);
  table[i] = make_float2(cs, sn);
}

__global__ void rope_vec_kernel(bf16* __restrict__ x, const float2* __restrict__ table,
                                const int* __restrict__ pos, int64_t T, int S, int NH, int D, int64_t ld,
                                int64_t head_stride, float sign) {
  const int half = D >> 1, hv = half >> 3;
  const int64_t total = T * NH * hv;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % hv);
    const int64_t th = i / hv;
    const int h = static_cast<int>(th % NH);
    const int64_t t = th / NH;
    const int p = pos ? pos[t] : static_cast<int>(t % S);
    bf16* base = x + t * ld + h * head_stride + c * 8;
    const float4* tb = reinterpret_cast<const float4*>(table + static_cast<int64_t>(p) * half + c * 8);
    float a[8], b[8], oa[8], ob[8];
    unpack8(*reinterpret_cast<const uint4*>(base), a);
    unpack8(*reinterpret_cast<const uint4*>(base + half), b);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float4 cs2 = tb[e];              // (cos0, sin0, cos1, sin1)
      const float s0 = cs2.y * sign, s1 = cs2.w * sign;
      oa[2 * e] = a[2 * e] * cs2.x - b[2 * e] * s0;
      ob[2 * e] = b[2 * e] * cs2.x + a[2 * e] * s0;
      oa[2 * e + 1] = a[2 * e + 1] * cs2.z - b[2 * e + 1] * s1;
      ob[2 * e + 1] = b[2 * e + 1] * cs2.z + a[2 * e + 1] * s1;
    }
    *reinterpret_cast<uint4*>(base) = pack8(oa);
    *reinterpret_cast<uint4*>(base + half) = pack8(ob);
  }
}

// ------------------------------------------------------- cross entropy ----
// One CTA per token row.  Reads logits[row, :V] (bf16), writes loss[row] (fp32) and
// overwrites the row IN PLACE with d(loss_sum * grad_scale)/dlogits =
// (softmax - onehot) * grad_scale.  Rows with target < 0 get zero loss and gradient.
constexpr int CE_THREADS = 1024;
__global__ void __launch_bounds__(CE_THREADS)
cross_entropy_fwd_bwd_kernel(bf16* __restrict__ logits, const int64_t* __restrict__ target,
                             float* __restrict__ loss, int V, int64_t ld, float grad_scale) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  bf16* lr = logits + row * ld;
  const int64_t tgt = target[row];
  const int nvec = V >> 3;
  uint4* lv = reinterpret_cast<uint4*>(lr);
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < nvec; c += CE_THREADS) {
    float f[8];
    unpack8(lv[c], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) mx = fmaxf(mx, f[e]);
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += CE_THREADS) mx = fmaxf(mx, __bfloat162float(lr[c]));
  mx = block_max(mx, red);
  float se = 0.f;
  for (int c = threadIdx.x; c < nvec; c += CE_THREADS) {
    float f[8];
    unpack8(lv[c], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) se += __expf(f[e] - mx);
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += CE_THREADS) se += __expf(__bfloat162float(lr[c]) - mx);
  se = block_sum(se, red);
  const float lse = mx + __logf(se);
  const bool valid = tgt >= 0 && tgt < V;
  if (threadIdx.x == 0) loss[row] = valid ? lse - __bfloat162float(lr[tgt]) : 0.f;
  __syncthreads();
  const float gs = valid ? grad_scale : 0.f;
  for (int c = threadIdx.x; c < nvec; c += CE_THREADS) {
    float f[8];
    unpack8(lv[c], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float pr = __expf(f[e] - lse);
      if (c * 8 + e == tgt) pr -= 1.f;
      f[e] = pr * gs;
    }
    lv[c] = pack8(f);
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += CE_THREADS) {
    float pr = __expf(__bfloat162float(lr[c]) - lse);
    if (c == tgt) pr -= 1.f;
    lr[c] = __float2bfloat16(pr * gs);
  }
}

// ---------------------------------------------------------------- AdamW ----
// Flat fused update with fp32 master weights (decoupled weight decay):
//   g = grad * grad_scale ; m = b1 m + (1-b1) g ; v = b2 v + (1-b2) g^2
//   master = master * (1 - lr*wd) - lr * (m / bc1) / (sqrt(v / bc2) + eps)
//   param_bf16 = bf16(master)
template <typename GradT>
__global__ void adamw_kernel(const GradT* __restrict__ grad, float* __restrict__ master,
                             float* __restrict__ m, float* __restrict__ v,
                             bf16* __restrict__ param, int64_t n, float lr, float b1, float b2,
                             float eps, float wd, float bc1, float bc2, float grad_scale) {
  const int64_t nv = n >> 2;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nv;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float g[4];
    if constexpr (sizeof(GradT) == 2) {
      uint2 u = reinterpret_cast<const uint2*>(grad)[i];
      const bf162* p = reinterpret_cast<const bf162*>(&u);
      float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]);
      g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
    } else {
      float4 u = reinterpret_cast<const float4*>(grad)[i];
      g[0] = u.x; g[1] = u.y; g[2] = u.z; g[3] = u.w;
    }
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float4 ww = reinterpret_cast<float4*>(master)[i];
    float* mp = &mm.x; float* vp = &vv.x; float* wp = &ww.x;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float ge = g[e] * grad_scale;
      mp[e] = b1 * mp[e] + (1.f - b1) * ge;
      vp[e] = b2 * vp[e] + (1.f - b2) * ge * ge;
      const float upd = (mp[e] / bc1) / (sqrtf(vp[e] / bc2) + eps);
      wp[e] = wp[e] * (1.f - lr * wd) - lr * upd;
    }
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    reinterpret_cast<float4*>(master)[i] = ww;
    if (param) {
      uint2 o;
      bf162* op = reinterpret_cast<bf162*>(&o);
      op[0] = __floats2bfloat162_rn(wp[0], wp[1]);
      op[1] = __floats2bfloat162_rn(wp[2], wp[3]);
      reinterpret_cast<uint2*>(param)[i] = o;
    }
  }
  // tail (n % 4 elements)
  const int64_t tail0 = nv << 2;
  const int64_t i = tail0 + blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i < n) {
    float ge;
    if constexpr (sizeof(GradT) == 2) ge = __bfloat162float(reinterpret_cast<const bf16*>(grad)[i]);
    else ge = reinterpret_cast<const float*>(grad)[i];
    ge *= grad_scale;
    const float mi = b1 * m[i] + (1.f - b1) * ge;
    const float vi = b2 * v[i] + (1.f - b2) * ge * ge;
    const float wi = master[i] * (1.f - lr * wd) - lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    m[i] = mi; v[i] = vi; master[i] = wi;
    if (param) param[i] = __float2bfloat16(wi);
  }
}

static inline int grid_for(int64_t work, int threads, int num_sms) {
  int64_t g = (work + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(num_sms) * 8;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace hpb

using namespace hpb;

extern "C" int hpb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out,
                               float* rstd, int64_t T, int H, float eps, cudaStream_t s) {
  if (H % 8 || H > NORM_THREADS * 8 * NORM_MAXV) return -2;
  if (T == 0) return 0;
  const int nv = (H / 8 + NORM_THREADS - 1) / NORM_THREADS;
#define HPB_FWD(NVV)                                                                              \
  if (res)                                                                                        \
    rmsnorm_fwd_kernel<true, NVV><<<static_cast<unsigned>(T), NORM_THREADS, 0, s>>>(              \
        (const bf16*)x, (const bf16*)res, (const bf16*)w, (bf16*)y, (bf16*)h_out, rstd, H, eps);  \
  else                                                                                            \
    rmsnorm_fwd_kernel<false, NVV><<<static_cast<unsigned>(T), NORM_THREADS, 0, s>>>(             \
        (const bf16*)x, nullptr, (const bf16*)w, (bf16*)y, nullptr, rstd, H, eps);
  if (nv == 1) { HPB_FWD(1) } else if (nv == 2) { HPB_FWD(2) } else if (nv == 3) { HPB_FWD(3) } else { HPB_FWD(4) }
#undef HPB_FWD
  return static_cast<int>(cudaGetLastError());
}

// dw_partial: fp32 scratch of [num_partials, H]; dw written as bf16 (dw_f32=0) or fp32.
extern "C" int hpb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                               const void* dres_in, void* dx, float* dw_partial, int num_partials,
                               void* dw, int dw_f32, int dw_accumulate, int64_t T, int H,
                               cudaStream_t s) {
  if (H % 8 || H > NORM_THREADS * 8 * NORM_MAXV) return -2;
  if (T == 0) return 0;
  int P = num_partials < T ? num_partials : static_cast<int>(T);
  const int nv = (H / 8 + NORM_THREADS - 1) / NORM_THREADS;
#define HPB_BWD(NVV)                                                                            \
  if (dres_in)                                                                                  \
    rmsnorm_bwd_kernel<true, NVV><<<P, NORM_THREADS, 0, s>>>(                                   \
        (const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, (const bf16*)dres_in, (bf16*)dx, \
        dw_partial, (int)T, H);                                                                 \
  else                                                                                          \
    rmsnorm_bwd_kernel<false, NVV><<<P, NORM_THREADS, 0, s>>>(                                  \
        (const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, nullptr, (bf16*)dx, dw_partial,  \
        (int)T, H);
  if (nv == 1) { HPB_BWD(1) } else if (nv == 2) { HPB_BWD(2) } else if (nv == 3) { HPB_BWD(3) } else { HPB_BWD(4) }
#undef HPB_BWD
  if (dw_f32)
    colsum_kernel<true><<<(H + 255) / 256, 256, 0, s>>>(dw_partial, dw, P, H, dw_accumulate);
  else
    colsum_kernel<false><<<(H + 255) / 256, 256, 0, s>>>(dw_partial, dw, P, H, dw_accumulate);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int hpb_swiglu_fwd(const void* gu, void* out, int64_t T, int F, int num_sms,
                              cudaStream_t s) {
  if (F % 8) return -2;
  if (T == 0) return 0;
  {
    const int gx = (F / 8 + 511) / 512;
    int64_t gy = (static_cast<int64_t>(num_sms) * 8 + gx - 1) / gx;
    if (gy > T) gy = T;
    if (gy > 65535) gy = 65535;
    swiglu_fwd_kernel<<<dim3(gx, static_cast<unsigned>(gy)), 256, 0, s>>>((const bf16*)gu, (bf16*)out, T, F);
  }
  return static_cast<int>(cudaGetLastError());
}
extern "C" int hpb_swiglu_bwd(const void* gu, const void* dout, void* dgu, int64_t T, int F,
                              int num_sms, cudaStream_t s) {
  if (F % 8) return -2;
  if (T == 0) return 0;
  {
    const int gx = (F / 8 + 511) / 512;
    int64_t gy = (static_cast<int64_t>(num_sms) * 8 + gx - 1) / gx;
    if (gy > T) gy = T;
    if (gy > 65535) gy = 65535;
    swiglu_bwd_kernel<<<dim3(gx, static_cast<unsigned>(gy)), 256, 0, s>>>((const bf16*)gu, (const bf16*)dout,
                                                                       (bf16*)dgu, T, F);
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int hpb_rope(void* x, const int* pos, int64_t T, int S, int NH, int D, int64_t ld,
                        float theta, int backward, int num_sms, cudaStream_t s) {
  if (D % 2) return -2;
  if (T == 0) return 0;
  rope_kernel<<<grid_for(T * NH * (D / 2), 256, num_sms), 256, 0, s>>>(
      (bf16*)x, pos, T, S, NH, D, ld, log2f(theta), backward ? -1.f : 1.f);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int hpb_cross_entropy(void* logits, const int64_t* target, float* loss, int64_t T, int V,
                                 int64_t ld, float grad_scale, cudaStream_t s) {
  if (ld % 8 || (reinterpret_cast<uintptr_t>(logits) & 15)) return -2;
  if (T == 0) return 0;
  cross_entropy_fwd_bwd_kernel<<<static_cast<unsigned>(T), CE_THREADS, 0, s>>>(
      (bf16*)logits, target, loss, V, ld, grad_scale);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int hpb_adamw(const void* grad, int grad_f32, float* master, float* m, float* v,
                         void* param, int64_t n, float lr, float b1, float b2, float eps, float wd,
                         int step, float grad_scale, int num_sms, cudaStream_t s) {
  if (n == 0) return 0;
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  const int g = grid_for((n + 3) / 4, 256, num_sms);
  if (grad_f32)
    adamw_kernel<float><<<g, 256, 0, s>>>((const float*)grad, master, m, v, (bf16*)param, n, lr, b1,
                                          b2, eps, wd, bc1, bc2, grad_scale);
  else
    adamw_kernel<bf16><<<g, 256, 0, s>>>((const bf16*)grad, master, m, v, (bf16*)param, n, lr, b1,
                                         b2, eps, wd, bc1, bc2, grad_scale);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------
// RMSNorm backward for callers that must not allocate device memory.
//
// hpb_rmsnorm_bwd() needs a [num_partials, H] fp32 scratch area for the per-CTA partial
// weight gradients and expects the caller to provide it.  Some callers cannot: a host
// program that has handed all device memory to its own pool (an inference / RL server in
// steady state, where a fresh cudaMalloc would fail or stall every stream), or one that
// runs under a "no allocation after start-up" rule.  For them this variant keeps the
// scratch in a fixed array that is part of the library image.  It performs the same two
// launches as hpb_rmsnorm_bwd() and calls no cudaMalloc / cudaFree / allocating routine.
//
// Limits and sharing:
//  * H <= kNoAllocMaxH (8192) and H % 8 == 0; at most kNoAllocMaxPartials (128) partial
//    rows are used.  The array is 128 * 8192 * 4 B = 4 MiB and every GPU that loads the
//    library holds it until the process exits.  Larger H is rejected with
//    HPB_NOALLOC_E_TOO_LARGE (see hpb_noalloc_strerror()).
//  * Every call on a device uses the SAME array, which keeps whatever the previous call
//    left there.  Nothing has to start at zero: each call overwrites rows [0, P) x [0, H)
//    before it reads them.  Two calls that overlap on the GPU (different streams, no
//    ordering between them) race on the array; order them or use hpb_rmsnorm_bwd().
//  * The first call on each device looks up the device address of the array
//    (cudaGetSymbolAddress, with that device current) and caches it.  Make that first call
//    before any stream capture begins.
namespace hpb {
constexpr int kNoAllocMaxPartials = 128;
constexpr int kNoAllocMaxH = 8192;
static __device__ __align__(256) float g_noalloc_rmsnorm_scratch[kNoAllocMaxPartials * kNoAllocMaxH];
constexpr int kNoAllocMaxDevices = 64;
static float* g_noalloc_scratch_addr[kNoAllocMaxDevices] = {};
}  // namespace hpb

extern "C" const char* hpb_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case HPB_NOALLOC_E_TOO_LARGE:
      return "hpb_rmsnorm_bwd_noalloc: H exceeds the built-in scratch (max H = 8192); "
             "use hpb_rmsnorm_bwd with caller-provided scratch";
    case HPB_NOALLOC_E_BAD_SHAPE: return "hpb_rmsnorm_bwd_noalloc: H must be a positive multiple of 8 and T >= 0";
    case HPB_NOALLOC_E_DEVICE: return "hpb_rmsnorm_bwd_noalloc: cannot query the current device or device index >= 64";
    case HPB_NOALLOC_E_SYMBOL: return "hpb_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed for the scratch array";
    default: return "hpb_rmsnorm_bwd_noalloc: CUDA launch error (positive codes are cudaError_t values)";
  }
}

extern "C" int hpb_noalloc_max_h() { return hpb::kNoAllocMaxH; }

extern "C" int hpb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                       const void* dres_in, void* dx, void* dw, int dw_f32,
                                       int dw_accumulate, int64_t T, int H, cudaStream_t s) {
  if (H <= 0 || H % 8 || T < 0) return HPB_NOALLOC_E_BAD_SHAPE;
  if (H > kNoAllocMaxH) return HPB_NOALLOC_E_TOO_LARGE;
  if (T == 0) return 0;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices)
    return HPB_NOALLOC_E_DEVICE;
  float* scratch = g_noalloc_scratch_addr[dev];
  if (scratch == nullptr) {
    // Host code must not pass the array's name to a kernel: on the host that name is only a
    // stand-in.  Ask the runtime for the device address (once per device, that device current).
    void* addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_noalloc_rmsnorm_scratch) != cudaSuccess || addr == nullptr)
      return HPB_NOALLOC_E_SYMBOL;
    scratch = static_cast<float*>(addr);
    g_noalloc_scratch_addr[dev] = scratch;
  }
  // the existing launcher does the work; it only launches kernels
  return hpb_rmsnorm_bwd(dy, x, w, rstd, dres_in, dx, scratch, kNoAllocMaxPartials, dw, dw_f32,
                         dw_accumulate, T, H, s);
}

// cos/sin table for positions [0, S): table is float2[S * D/2]
extern "C" int hpb_rope_table(float* table, int S, int D, float theta, cudaStream_t s) {
  const int n = S * (D / 2);
  if (n <= 0) return 0;
  rope_table_init_kernel<<<(n + 255) / 256, 256, 0, s>>>(reinterpret_cast<float2*>(table), S, D / 2, D,
                                                         log2f(theta));
  return static_cast<int>(cudaGetLastError());
}

// In-place RoPE using a precomputed table; needs D % 16 == 0, ld % 8 == 0, head_stride % 8 == 0 (elements
// between the rotated D columns of consecutive heads; D when the heads are packed) and 16-byte aligned x.
extern "C" int hpb_rope_vec_strided(void* x, const float* table, const int* pos, int64_t T, int S, int NH, int D,
                                    int64_t ld, int64_t head_stride, int backward, int num_sms, cudaStream_t s) {
  if (D % 16 || ld % 8 || head_stride % 8 || (reinterpret_cast<uintptr_t>(x) & 15)) return -2;
  if (T == 0) return 0;
  rope_vec_kernel<<<grid_for(T * NH * (D / 16), 256, num_sms), 256, 0, s>>>(
      (bf16*)x, reinterpret_cast<const float2*>(table), pos, T, S, NH, D, ld, head_stride, backward ? -1.f : 1.f);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int hpb_rope_vec(void* x, const float* table, const int* pos, int64_t T, int S, int NH, int D,
                            int64_t ld, int backward, int num_sms, cudaStream_t s) {
  return hpb_rope_vec_strided(x, table, pos, T, S, NH, D, ld, D, backward, num_sms, s);
}
