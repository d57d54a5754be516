// MXFP8 quantisation producers: bf16 [R, C] -> e4m3 codes + one UE8M0 scale per 32 elements
// along the contraction axis, in the layouts the block-scaled tcgen05 GEMM consumes directly.
//
// One pass over the input produces (either or both of)
//   * the row-wise copy     q_row [R, C]   scaled along C  (operand whose contraction axis is C)
//   * the column-wise copy  q_col [C, R]   scaled along R, written transposed, so that it is
//                                          again a K-major operand (contraction axis R)
// Scales are written pre-arranged for tcgen05.cp: the operand's rows are cut into tiles of
// `tile_rows` (the GEMM's M or N tile), each tile into atoms of 128 rows, and for every atom and
// every group of 4 scale columns (= 128 contraction elements) 512 bytes are stored as
//   byte[(r % 32) * 16 + (r / 32) * 4 + k],   r = row in atom, k = scale column in group,
// indexed [tile][k_group][atom].  The GEMM's TMA producer then moves whole atoms with plain bulk
// copies and the MMA warp forwards them to TMEM unchanged.
//
// Scale rule: e = ceil(log2(amax / 448)) clamped to [-127, 127], stored biased (e + 127); codes
// are round-to-nearest-even e4m3 of x * 2^-e with saturation.  amax == 0 gives scale 2^-127, codes 0.
//
// Reference counterparts: Transformer Engine's MXFP8/MXFP4 block-scaling recipes selected by
// small_llm_pretraining/primus/conf/llama3.1_8B-pretrain-fp4.yaml:108-112, the one-pass cast + amax
// kernels of generative_recommenders/ops/triton/bwd_fp8.py (_quantize_amax*), and the LN store of
// generative_recommenders/ops/hip/ln_store_mx6.cu (codes + E8M0 per 32).
#include <cuda_fp8.h>

#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int TILE = 128;
constexpr int PITCH = TILE + 2;  // bf16 elements per shared-memory row (odd word count: no bank conflicts on columns)

B200_DEVICE uint32_t e8m0_from_amax(float amax) {
  // smallest power of two s with amax / s <= 448
  if (!(amax > 0.f)) return 0u;
  const float t = __fdiv_rn(amax, 448.0f);
  const uint32_t bits = __float_as_uint(t);
  int e = (int)((bits >> 23) & 0xff) - 127;
  if (bits & 0x7fffffu) e += 1;
  e = max(-127, min(127, e));
  return (uint32_t)(e + 127);
}
B200_DEVICE float scale_inv_from_e8m0(uint32_t b) {
  // 2^-(b - 127)
  return __uint_as_float((uint32_t)(254 - (int)b) << 23);
}
B200_DEVICE uint32_t pack4_e4m3(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}
// byte offset of scale (row r of the operand, scale column kc) in the atom layout
B200_DEVICE long long sf_offset(long long r, int kc, int tile_rows, int atoms_per_tile, long long k_groups) {
  const long long tile = r / tile_rows;
  const int rr = (int)(r - tile * tile_rows);
  const int atom = rr >> 7, ra = rr & 127;
  return ((tile * k_groups + (kc >> 2)) * atoms_per_tile + atom) * 512 + (ra & 31) * 16 + (ra >> 5) * 4 + (kc & 3);
}

// grid: (C / 128, R / 128); 256 threads
__global__ void __launch_bounds__(256, 3)
quant_mxfp8_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int R, int C, uint8_t* __restrict__ q_row,
                   uint8_t* __restrict__ sf_row, int row_tile, uint8_t* __restrict__ q_col,
                   uint8_t* __restrict__ sf_col, int col_tile) {
  __shared__ __nv_bfloat16 tile[TILE * PITCH];
  const int c0 = blockIdx.x * TILE, r0 = blockIdx.y * TILE;
  const int tid = threadIdx.x;
  // ---- load the 128 x 128 tile (each thread: one row half = 64 contiguous elements) ----
  {
    const int r = tid >> 1, h = tid & 1;
    const __nv_bfloat16* src = x + (long long)(r0 + r) * ldx + c0 + h * 64;
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = reinterpret_cast<const uint4*>(src)[i];
    // row-wise quantisation straight from registers: two blocks of 32
    if (q_row != nullptr) {
      uint8_t* dst = q_row + (long long)(r0 + r) * C + c0 + h * 64;
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        float f[32];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 u = v[blk * 4 + i];
          const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
          f[8 * i + 0] = a.x; f[8 * i + 1] = a.y; f[8 * i + 2] = b.x; f[8 * i + 3] = b.y;
          f[8 * i + 4] = c.x; f[8 * i + 5] = c.y; f[8 * i + 6] = d.x; f[8 * i + 7] = d.y;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(f[i]));
        const uint32_t e = e8m0_from_amax(amax);
        const float inv = scale_inv_from_e8m0(e);
        uint4 o[2];
        uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
        for (int i = 0; i < 8; ++i) ow[i] = pack4_e4m3(f[4 * i] * inv, f[4 * i + 1] * inv, f[4 * i + 2] * inv, f[4 * i + 3] * inv);
        reinterpret_cast<uint4*>(dst + blk * 32)[0] = o[0];
        reinterpret_cast<uint4*>(dst + blk * 32)[1] = o[1];
        const int kc = (c0 >> 5) + h * 2 + blk;
        sf_row[sf_offset(r0 + r, kc, row_tile, (row_tile + 127) >> 7, C >> 7)] = (uint8_t)e;
      }
    }
    if (q_col != nullptr) {
      uint32_t* trow = reinterpret_cast<uint32_t*>(tile + r * PITCH + h * 64);
#pragma unroll
      for (int i = 0; i < 8; ++i) { trow[4 * i] = v[i].x; trow[4 * i + 1] = v[i].y; trow[4 * i + 2] = v[i].z; trow[4 * i + 3] = v[i].w; }
    }
  }
  if (q_col == nullptr) return;
  __syncthreads();
  // ---- column-wise: thread = (column c, half h of the rows); two blocks of 32 rows ----
  {
    const int c = tid & 127, h = tid >> 7;
    uint8_t* dst = q_col + (long long)(c0 + c) * R + r0 + h * 64;
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      float f[32];
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        f[i] = __bfloat162float(tile[(h * 64 + blk * 32 + i) * PITCH + c]);
        amax = fmaxf(amax, fabsf(f[i]));
      }
      const uint32_t e = e8m0_from_amax(amax);
      const float inv = scale_inv_from_e8m0(e);
      uint4 o[2];
      uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
      for (int i = 0; i < 8; ++i) ow[i] = pack4_e4m3(f[4 * i] * inv, f[4 * i + 1] * inv, f[4 * i + 2] * inv, f[4 * i + 3] * inv);
      reinterpret_cast<uint4*>(dst + blk * 32)[0] = o[0];
      reinterpret_cast<uint4*>(dst + blk * 32)[1] = o[1];
      const int kc = (r0 >> 5) + h * 2 + blk;
      sf_col[sf_offset(c0 + c, kc, col_tile, (col_tile + 127) >> 7, R >> 7)] = (uint8_t)e;
    }
  }
}

}  // namespace

// Bytes of the scale buffer of an operand with `rows` rows and `k` contraction elements whose rows
// are tiled by `tile_rows` in the GEMM.
B200_API long long b200_mxfp8_sf_bytes(long long rows, long long k, int tile_rows) {
  const long long tiles = (rows + tile_rows - 1) / tile_rows;
  const long long atoms = (tile_rows + 127) / 128;
  return tiles * (k / 128) * atoms * 512;
}

// x: bf16 [R, C] with row pitch ldx (elements); R and C multiples of 128.
// q_row / sf_row (row-wise copy, rows tiled by row_tile) and q_col / sf_col (column-wise copy stored
// transposed as [C, R], rows tiled by col_tile) may each be null.  Scale buffers must be zero-filled
// by the caller when tile_rows is not a multiple of 128 (padding rows of the last atom are not written).
B200_API int b200_quant_mxfp8(const void* x, long long ldx, int R, int C, void* q_row, void* sf_row, int row_tile,
                              void* q_col, void* sf_col, int col_tile, void* stream) {
  if (R % 128 != 0 || C % 128 != 0) return b200::fail(700, "quant_mxfp8: R=%d and C=%d must be multiples of 128", R, C);
  if (ldx % 8 != 0 || ((uintptr_t)x & 15) != 0) return b200::fail(701, "quant_mxfp8: input must be 16-byte aligned");
  if ((q_row && (row_tile % 32 != 0 || row_tile <= 0)) || (q_col && (col_tile % 32 != 0 || col_tile <= 0)))
    return b200::fail(702, "quant_mxfp8: tile rows must be positive multiples of 32");
  dim3 grid(C / 128, R / 128);
  quant_mxfp8_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, R, C, (uint8_t*)q_row,
                                                            (uint8_t*)sf_row, row_tile, (uint8_t*)q_col,
                                                            (uint8_t*)sf_col, col_tile);
  b200::count_launch();
  return b200::check_launch("quant_mxfp8");
}
