// Per-tensor FP8 quantisation producers (the second low-precision recipe of this library, next to
// MXFP8): bf16 [R, C] -> e4m3 or e5m2 codes scaled by ONE factor for the whole tensor, in the two
// K-major copies a training step needs -
//   * q_row [R, C]   (contraction along C), and / or
//   * q_col [C, R]   the transposed copy (contraction along R) for the weight-gradient GEMM -
// plus the tensor's absolute maximum accumulated into a device word (atomic max on the float's bits),
// from which the host-side recipe derives the NEXT step's factor (delayed scaling): no reduction has
// to finish before the cast, so the pass reads the input once.
//
// Same recipe as the reference's HSTU FP8 path - per-tensor e4m3 activations and weights with a
// calibrated factor, e5m2 gradients with a delayed factor refreshed on a cadence
// (generative_recommenders/ops/triton/triton_fp8.py, generative_recommenders/ops/triton/bwd_fp8.py) -
// and as the FP8 phase that the FLUX forward switches to
// (flux1/primus/patches/flux_fprop_switch.py:36-279).
#include <cuda_fp8.h>

#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int TILE = 128;
constexpr int PITCH = TILE + 2;

B200_DEVICE int tile_off(int r) { return r * PITCH + (r >> 4) * 4; }

template <int E5M2>
B200_DEVICE uint32_t pack4(float a, float b, float c, float d) {
  constexpr __nv_fp8_interpretation_t kind = E5M2 ? __NV_E5M2 : __NV_E4M3;
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, kind);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, kind);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

// grid (C / 128, R / 128), 256 threads; same tile walk as the MXFP8 producer.
template <int E5M2>
__global__ void __launch_bounds__(256, 4)
quant_fp8_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int R, int C, const float* __restrict__ scale,
                 uint8_t* __restrict__ q_row, uint8_t* __restrict__ q_col, unsigned int* __restrict__ amax_bits) {
  __shared__ __align__(16) __nv_bfloat16 tile[TILE * PITCH + 32];
  __shared__ float red[8];
  const int c0 = blockIdx.x * TILE, r0 = blockIdx.y * TILE;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sub_row = lane >> 4, chunk = lane & 15;
  const float s = scale != nullptr ? *scale : 1.f;
  float amax = 0.f;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 16 + warp * 2 + sub_row;
    const uint4 v = *reinterpret_cast<const uint4*>(x + (long long)(r0 + r) * ldx + c0 + chunk * 8);
    const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
    const float f[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
    if (q_row != nullptr)
      *reinterpret_cast<uint2*>(q_row + (long long)(r0 + r) * C + c0 + chunk * 8) =
          make_uint2(pack4<E5M2>(f[0] * s, f[1] * s, f[2] * s, f[3] * s), pack4<E5M2>(f[4] * s, f[5] * s, f[6] * s, f[7] * s));
    if (q_col != nullptr) {
      uint32_t* t = reinterpret_cast<uint32_t*>(tile + tile_off(r) + chunk * 8);
      t[0] = v.x; t[1] = v.y; t[2] = v.z; t[3] = v.w;
    }
  }
  amax = warp_max(amax);
  if (lane == 0) red[warp] = amax;
  __syncthreads();
  if (tid == 0 && amax_bits != nullptr) {
    float m = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
    atomicMax(amax_bits, __float_as_uint(m));     // non-negative floats order like their bit patterns
  }
  if (q_col == nullptr) return;
  const int sub = lane & 7;
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int c = pass * 32 + warp * 4 + (lane >> 3);
    float f[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) f[i] = __bfloat162float(tile[tile_off(sub * 16 + i) + c]) * s;
    *reinterpret_cast<uint4*>(q_col + (long long)(c0 + c) * R + r0 + sub * 16) =
        make_uint4(pack4<E5M2>(f[0], f[1], f[2], f[3]), pack4<E5M2>(f[4], f[5], f[6], f[7]),
                   pack4<E5M2>(f[8], f[9], f[10], f[11]), pack4<E5M2>(f[12], f[13], f[14], f[15]));
  }
}

// Row-wise copy only, any number of rows (jagged token buffers): a thread converts 8 elements.
template <int E5M2>
__global__ void __launch_bounds__(256)
quant_fp8_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, long long R, int C, const float* __restrict__ scale,
                      uint8_t* __restrict__ q, long long ldq, unsigned int* __restrict__ amax_bits) {
  __shared__ float red[8];
  const float s = scale != nullptr ? *scale : 1.f;
  const int vpr = C / 8;
  const long long total = R * vpr;
  float amax = 0.f;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const long long r = i / vpr;
    const int v = (int)(i - r * vpr);
    const uint4 u = *reinterpret_cast<const uint4*>(x + r * ldx + v * 8);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    const float f[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
    *reinterpret_cast<uint2*>(q + r * ldq + v * 8) =
        make_uint2(pack4<E5M2>(f[0] * s, f[1] * s, f[2] * s, f[3] * s), pack4<E5M2>(f[4] * s, f[5] * s, f[6] * s, f[7] * s));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0 && amax_bits != nullptr) {
    float m = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
    atomicMax(amax_bits, __float_as_uint(m));
  }
}

}  // namespace

// x: bf16 [R, C] with row pitch ldx (elements), any R, C a multiple of 8; q: [R, C] codes with row pitch ldq (bytes,
// a multiple of 8).  scale / amax_bits as in b200_quant_fp8.
B200_API int b200_quant_fp8_rows(const void* x, long long ldx, long long R, int C, const float* scale, int e5m2, void* q,
                                 long long ldq, void* amax_bits, void* stream) {
  if (R <= 0) return 0;
  if (C % 8 != 0 || ldx % 8 != 0 || ldq % 8 != 0 || ((uintptr_t)x & 15) != 0 || ((uintptr_t)q & 7) != 0)
    return b200::fail(722, "quant_fp8_rows: C=%d and the pitches must be multiples of 8, the buffers aligned", C);
  long long g = (R * (C / 8) + 255) / 256;
  const long long cap = (long long)b200::sm_count() * 8;
  const int grid = (int)(g < cap ? g : cap);
  if (e5m2)
    quant_fp8_rows_kernel<1><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, R, C, scale, (uint8_t*)q, ldq,
                                                                    (unsigned int*)amax_bits);
  else
    quant_fp8_rows_kernel<0><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, R, C, scale, (uint8_t*)q, ldq,
                                                                    (unsigned int*)amax_bits);
  b200::count_launch();
  return b200::check_launch("quant_fp8_rows");
}

// x: bf16 [R, C] (row pitch ldx elements; R, C multiples of 128).  scale: one device float multiplied
// into every element before the cast (null = 1).  q_row [R, C] / q_col [C, R]: outputs, either may be
// null.  amax_bits: device word that receives max(|x|) as float bits through an atomic max (may be null).
B200_API int b200_quant_fp8(const void* x, long long ldx, int R, int C, const float* scale, int e5m2, void* q_row,
                            void* q_col, void* amax_bits, void* stream) {
  if (R % 128 != 0 || C % 128 != 0) return b200::fail(720, "quant_fp8: R=%d and C=%d must be multiples of 128", R, C);
  if (ldx % 8 != 0 || ((uintptr_t)x & 15) != 0) return b200::fail(721, "quant_fp8: input must be 16-byte aligned");
  dim3 grid(C / 128, R / 128);
  if (e5m2)
    quant_fp8_kernel<1><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, R, C, scale, (uint8_t*)q_row,
                                                               (uint8_t*)q_col, (unsigned int*)amax_bits);
  else
    quant_fp8_kernel<0><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, R, C, scale, (uint8_t*)q_row,
                                                               (uint8_t*)q_col, (unsigned int*)amax_bits);
  b200::count_launch();
  return b200::check_launch("quant_fp8");
}
