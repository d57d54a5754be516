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

// shared-memory tile: row r starts at r * PITCH + (r >> 4) * 4 bf16 elements.  The odd word pitch
// spreads a column over the banks and the per-16-row skew separates the eight lanes that walk one
// column in the column pass.
B200_DEVICE int tile_off(int r) { return r * PITCH + (r >> 4) * 4; }

B200_DEVICE uint2 quant8(const float (&f)[8], float inv) {
  return make_uint2(pack4_e4m3(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv),
                    pack4_e4m3(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv));
}

// grid: (ceil(C / 128), R / 128); 256 threads.  R is a multiple of 128, C a multiple of 32: in the last column tile
// the columns past C read as zero and nothing is stored for them (their scale bytes are written as 0).
//   row pass:    a warp instruction covers 2 rows x 256 bytes of input (lane = 8 elements); a block of
//                32 elements is 4 lanes, so amax is two shuffles; codes leave as 2 x 128 contiguous bytes.
//   column pass: 8 lanes walk one column (16 rows each, amax of a 32-block = one shuffle) and write the
//                column's 128 codes as one contiguous 128-byte piece of the transposed copy.
//   scales:      staged in shared memory and written as one 32-bit word per operand row.
//
// MODE selects what the tile is made of (the values are rounded to bf16 first, so the codes equal
// those of quantising the stand-alone kernel's bf16 output):
//   0  x[r, c]
//   1  SwiGLU forward   a[r, c]   = silu(gu[r, c]) * gu[r, F + c],          x = gu [R, 2F], C = F
//   2  SwiGLU backward  dgu[r, c] = da * up * silu'(gate)  for c <  F
//                                 = da * silu(gate)        for c >= F,      x = gu [R, 2F], aux = da [R, F], C = 2F
template <int MODE>
B200_DEVICE uint4 produce8(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ aux,
                           long long ldaux, int F, long long row, int col) {
  if constexpr (MODE == 0) {
    return *reinterpret_cast<const uint4*>(x + row * ldx + col);
  } else {
    const int cc = (MODE == 2 && col >= F) ? col - F : col;
    const uint4 ug = *reinterpret_cast<const uint4*>(x + row * ldx + cc);
    const uint4 uu = *reinterpret_cast<const uint4*>(x + row * ldx + F + cc);
    const float2 g0 = unpack_bf16x2(ug.x), g1 = unpack_bf16x2(ug.y), g2 = unpack_bf16x2(ug.z), g3 = unpack_bf16x2(ug.w);
    const float2 u0 = unpack_bf16x2(uu.x), u1 = unpack_bf16x2(uu.y), u2 = unpack_bf16x2(uu.z), u3 = unpack_bf16x2(uu.w);
    const float g[8] = {g0.x, g0.y, g1.x, g1.y, g2.x, g2.y, g3.x, g3.y};
    const float u[8] = {u0.x, u0.y, u1.x, u1.y, u2.x, u2.y, u3.x, u3.y};
    float o[8];
    if constexpr (MODE == 1) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    } else {
      const uint4 ud = *reinterpret_cast<const uint4*>(aux + row * ldaux + cc);
      const float2 d0 = unpack_bf16x2(ud.x), d1 = unpack_bf16x2(ud.y), d2 = unpack_bf16x2(ud.z), d3 = unpack_bf16x2(ud.w);
      const float d[8] = {d0.x, d0.y, d1.x, d1.y, d2.x, d2.y, d3.x, d3.y};
      const bool up_part = col >= F;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float sg = 1.f / (1.f + __expf(-g[j]));
        o[j] = up_part ? d[j] * (g[j] * sg) : d[j] * u[j] * sg * (1.f + g[j] * (1.f - sg));
      }
    }
    return make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]), pack_bf16x2(o[6], o[7]));
  }
}

template <int MODE>
__global__ void __launch_bounds__(256, 4)
quant_mxfp8_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int R, int C, uint8_t* __restrict__ q_row,
                   uint8_t* __restrict__ sf_row, int row_tile, uint8_t* __restrict__ q_col,
                   uint8_t* __restrict__ sf_col, int col_tile, const __nv_bfloat16* __restrict__ aux, long long ldaux,
                   int F) {
  __shared__ __align__(16) __nv_bfloat16 tile[TILE * PITCH + 32];
  __shared__ __align__(4) uint8_t sfs[2][TILE][4];     // [row pass | column pass][operand row][scale column]
  const int c0 = blockIdx.x * TILE, r0 = blockIdx.y * TILE;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sub_row = lane >> 4, chunk = lane & 15;
  const bool col_live = c0 + chunk * 8 < C;
  uint4 v[8];
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 16 + warp * 2 + sub_row;
    v[it] = col_live ? produce8<MODE>(x, ldx, aux, ldaux, F, (long long)(r0 + r), c0 + chunk * 8) : make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 16 + warp * 2 + sub_row;
    if (q_row != nullptr) {
      const float2 a = unpack_bf16x2(v[it].x), b = unpack_bf16x2(v[it].y), c = unpack_bf16x2(v[it].z), d = unpack_bf16x2(v[it].w);
      const float f[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const uint32_t e = e8m0_from_amax(amax);
      if (col_live)
        *reinterpret_cast<uint2*>(q_row + (long long)(r0 + r) * C + c0 + chunk * 8) = quant8(f, scale_inv_from_e8m0(e));
      if ((chunk & 3) == 0) sfs[0][r][chunk >> 2] = (uint8_t)e;
    }
    if (q_col != nullptr) {
      uint32_t* t = reinterpret_cast<uint32_t*>(tile + tile_off(r) + chunk * 8);
      t[0] = v[it].x; t[1] = v[it].y; t[2] = v[it].z; t[3] = v[it].w;
    }
  }
  __syncthreads();
  if (q_row != nullptr && tid < TILE) {
    const long long o = sf_offset(r0 + tid, c0 >> 5, row_tile, (row_tile + 127) >> 7, (C + 127) >> 7);
    *reinterpret_cast<uint32_t*>(sf_row + o) = *reinterpret_cast<const uint32_t*>(&sfs[0][tid][0]);
  }
  if (q_col == nullptr) return;
  const int sub = lane & 7;                      // rows sub * 16 .. + 15 of the column
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int c = pass * 32 + warp * 4 + (lane >> 3);
    float f[16];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      f[i] = __bfloat162float(tile[tile_off(sub * 16 + i) + c]);
      amax = fmaxf(amax, fabsf(f[i]));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const uint32_t e = e8m0_from_amax(amax);
    const float inv = scale_inv_from_e8m0(e);
    const float lo[8] = {f[0], f[1], f[2], f[3], f[4], f[5], f[6], f[7]};
    const float hi[8] = {f[8], f[9], f[10], f[11], f[12], f[13], f[14], f[15]};
    const uint2 q0 = quant8(lo, inv), q1 = quant8(hi, inv);
    if (c0 + c < C)
      *reinterpret_cast<uint4*>(q_col + (long long)(c0 + c) * R + r0 + sub * 16) = make_uint4(q0.x, q0.y, q1.x, q1.y);
    if ((sub & 1) == 0) sfs[1][c][sub >> 1] = (uint8_t)e;
  }
  __syncthreads();
  if (tid < TILE && c0 + tid < C) {
    const long long o = sf_offset(c0 + tid, r0 >> 5, col_tile, (col_tile + 127) >> 7, R >> 7);
    *reinterpret_cast<uint32_t*>(sf_col + o) = *reinterpret_cast<const uint32_t*>(&sfs[1][tid][0]);
  }
}


template <int MODE>
int launch_quant(const void* x, long long ldx, const void* aux, long long ldaux, int R, int C, void* q_row, void* sf_row,
                 int row_tile, void* q_col, void* sf_col, int col_tile, int F, cudaStream_t stream, const char* what) {
  dim3 grid((C + TILE - 1) / TILE, R / TILE);
  quant_mxfp8_kernel<MODE><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, R, C, (uint8_t*)q_row, (uint8_t*)sf_row,
                                                     row_tile, (uint8_t*)q_col, (uint8_t*)sf_col, col_tile,
                                                     (const __nv_bfloat16*)aux, ldaux, F);
  b200::count_launch();
  return b200::check_launch(what);
}

}  // namespace

// Bytes of the scale buffer of an operand with `rows` rows and `k` contraction elements whose rows
// are tiled by `tile_rows` in the GEMM.
B200_API long long b200_mxfp8_sf_bytes(long long rows, long long k, int tile_rows) {
  const long long tiles = (rows + tile_rows - 1) / tile_rows;
  const long long atoms = (tile_rows + 127) / 128;
  return tiles * ((k + 127) / 128) * atoms * 512;
}

// x: bf16 [R, C] with row pitch ldx (elements); R a multiple of 128, C a multiple of 32.
// q_row / sf_row (row-wise copy, rows tiled by row_tile) and q_col / sf_col (column-wise copy stored
// transposed as [C, R], rows tiled by col_tile) may each be null.  Scale buffers must be zero-filled
// by the caller when tile_rows or the operand's row count is not a multiple of 128 (padding rows of
// the last atom are not written).
B200_API int b200_quant_mxfp8(const void* x, long long ldx, int R, int C, void* q_row, void* sf_row, int row_tile,
                              void* q_col, void* sf_col, int col_tile, void* stream) {
  if (R % 128 != 0 || C % 32 != 0 || R <= 0 || C <= 0)
    return b200::fail(700, "quant_mxfp8: R=%d must be a multiple of 128 and C=%d of 32", R, C);
  if (ldx % 8 != 0 || ((uintptr_t)x & 15) != 0) return b200::fail(701, "quant_mxfp8: input must be 16-byte aligned");
  if ((q_row && (row_tile % 16 != 0 || row_tile <= 0)) || (q_col && (col_tile % 16 != 0 || col_tile <= 0)))
    return b200::fail(702, "quant_mxfp8: tile rows must be positive multiples of 16");
  return launch_quant<0>(x, ldx, nullptr, 0, R, C, q_row, sf_row, row_tile, q_col, sf_col, col_tile, 0, (cudaStream_t)stream,
                         "quant_mxfp8");
}

// Quantised SwiGLU: the codes / scales of a = silu(gate) * up without writing a.
//   gu: bf16 [R, 2F] (gate columns first), pitch ldgu.  Outputs as b200_quant_mxfp8 for the matrix a [R, F].
B200_API int b200_quant_swiglu_mxfp8(const void* gu, long long ldgu, int R, int F, void* q_row, void* sf_row, int row_tile,
                                     void* q_col, void* sf_col, int col_tile, void* stream) {
  if (R % 128 != 0 || F % 32 != 0 || R <= 0 || F <= 0)
    return b200::fail(710, "quant_swiglu: R=%d must be a multiple of 128 and F=%d of 32", R, F);
  if (ldgu % 8 != 0 || ((uintptr_t)gu & 15) != 0) return b200::fail(711, "quant_swiglu: input must be 16-byte aligned");
  return launch_quant<1>(gu, ldgu, nullptr, 0, R, F, q_row, sf_row, row_tile, q_col, sf_col, col_tile, F, (cudaStream_t)stream,
                         "quant_swiglu_mxfp8");
}

// Quantised SwiGLU backward: the codes / scales of dgu [R, 2F] (d gate | d up) from da [R, F] and gu [R, 2F].
B200_API int b200_quant_swiglu_bwd_mxfp8(const void* da, long long ldda, const void* gu, long long ldgu, int R, int F,
                                         void* q_row, void* sf_row, int row_tile, void* q_col, void* sf_col, int col_tile,
                                         void* stream) {
  if (R % 128 != 0 || F % 128 != 0 || R <= 0 || F <= 0)
    return b200::fail(712, "quant_swiglu_bwd: R=%d and F=%d must be multiples of 128", R, F);
  if (ldgu % 8 != 0 || ldda % 8 != 0 || (((uintptr_t)gu | (uintptr_t)da) & 15) != 0)
    return b200::fail(713, "quant_swiglu_bwd: inputs must be 16-byte aligned");
  return launch_quant<2>(gu, ldgu, da, ldda, R, 2 * F, q_row, sf_row, row_tile, q_col, sf_col, col_tile, F, (cudaStream_t)stream,
                         "quant_swiglu_bwd_mxfp8");
}
