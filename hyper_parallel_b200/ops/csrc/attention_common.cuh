// Device helpers shared by the attention kernels (head dimension 128, and the 192 / 128 multi-head
// latent attention variant): tensor-memory stores, descriptor arithmetic, packed fp32 pair
// arithmetic, the tensor-memory-operand MMA, and the host-side tensor-map encoder.
#pragma once
#include "sm100_common.cuh"

#include <mutex>

namespace hpb {
namespace fa {

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// Descriptor of the same operand `bytes` further into shared memory (the start-address field
// holds address >> 4 and cannot overflow inside the 228 KB window).
__device__ __forceinline__ uint64_t desc_at(uint64_t desc, uint32_t bytes) {
  // one 32-bit add: the address field sits in the low word and cannot carry out of it
  const uint32_t lo = static_cast<uint32_t>(desc) + (bytes >> 4);
  return (desc & 0xffffffff00000000ull) | lo;
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  tmem_ld_32x32b_x32(taddr, *reinterpret_cast<uint32_t(*)[32]>(r));
}
// packed pair arithmetic of sm_100: one instruction for two fp32 lanes
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
        "l"(*reinterpret_cast<unsigned long long*>(&c)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  unsigned long long d;
  asm("mul.rn.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// D[tmem] (+)= A[tmem] * B[smem desc]: the A operand (row = lane, two bf16 per 32-bit column)
// is read from tensor memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// fp32 tile in shared memory (dense rows) added to global memory by the TMA unit
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* m, const void* smem_src, int x, int y, int z) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
          reinterpret_cast<uint64_t>(m)),
      "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// delta[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]; one warp per (b, s, h) row of 128.
static __global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dO, int64_t do_batch_stride,
                                  int64_t do_row_stride, const __nv_bfloat16* __restrict__ O,
                                  float* __restrict__ delta, int B, int S, int H) {
  const int64_t w = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<int64_t>(B) * S * H) return;
  const int h = static_cast<int>(w % H);
  const int64_t bs = w / H;
  const int s = static_cast<int>(bs % S);
  const int b = static_cast<int>(bs / S);
  const uint2 a = *reinterpret_cast<const uint2*>(dO + b * do_batch_stride + s * do_row_stride + h * 128 + lane * 4);
  const uint2 o = *reinterpret_cast<const uint2*>(O + ((static_cast<int64_t>(b) * S + s) * H + h) * 128 + lane * 4);
  const __nv_bfloat162* ab = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&o);
  float acc = 0.f;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const float2 x = __bfloat1622float2(ab[e]), y = __bfloat1622float2(ob[e]);
    acc += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) delta[(static_cast<int64_t>(b) * H + h) * S + s] = acc;
}

// dst[row, 0:cols] (token stride dst_stride) = bf16(src[row, 0:cols]); cols a multiple of 8.
static __global__ void f32_to_bf16_rows_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                        int64_t rows, int cols, int64_t dst_stride) {
  const int vec_per_row = cols >> 3;
  for (int64_t row = blockIdx.y; row < rows; row += gridDim.y) {
    const float4* s4 = reinterpret_cast<const float4*>(src + row * cols);
    uint4* d4 = reinterpret_cast<uint4*>(dst + row * dst_stride);
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < vec_per_row; c += gridDim.x * blockDim.x) {
      const float4 a = s4[2 * c], b = s4[2 * c + 1];
      uint4 v;
      __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
      vb[0] = __floats2bfloat162_rn(a.x, a.y);
      vb[1] = __floats2bfloat162_rn(a.z, a.w);
      vb[2] = __floats2bfloat162_rn(b.x, b.y);
      vb[3] = __floats2bfloat162_rn(b.z, b.w);
      d4[c] = v;
    }
  }
}

}  // namespace fa

// ------------------------------------------------------------------ host ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn fa_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// [B, S, cols] bf16 view with element strides (batch_stride, row_stride, 1); box = 64 x box_rows x 1.
inline int make_tmap_bsd(CUtensorMap* map, const void* ptr, int B, int S, int cols, int64_t batch_stride,
                         int64_t row_stride, uint32_t box_rows = 128) {
  EncodeTiledFn enc = fa_encode_fn();
  if (enc == nullptr) return -1;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(B)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(row_stride) * 2, static_cast<cuuint64_t>(batch_stride) * 2};
  cuuint32_t box[3] = {64, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

}  // namespace hpb
