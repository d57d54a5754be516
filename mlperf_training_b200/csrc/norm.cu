// RMSNorm / LayerNorm forward and backward over rows of a [T, D] bf16 matrix (fp32 math).
//
// Forward keeps a row in registers (one 16-byte vector per thread per 2048 columns), so the
// activation is read once and written once.  Backward produces dx in one pass and the
// weight / bias gradients as per-CTA fp32 partial rows in scratch memory, which a second
// fixed-order kernel sums: no atomics, so runs are bit-reproducible.
//
// Covers the reference's norm family: generative_recommenders/ops/triton/triton_layer_norm.py
// (_weighted_layer_norm_fwd / _bwd_dx / _layer_norm_bwd_dwdb, RMSNorm fwd/bwd, SwishLayerNorm)
// and the Primus-Turbo RMSNorm selected by small_llm_pretraining/primus/conf/
// llama3.1_8B-pretrain-fp4.yaml:122-123.
#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int NT = 256;       // threads per CTA
constexpr int MAXV = 4;       // 16-byte vectors per thread kept in registers -> D <= 8192

B200_DEVICE float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float r = (l < NT / 32) ? red[l] : 0.f;
  r = warp_sum(r);
  return r;
}

B200_DEVICE void load8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
B200_DEVICE void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                       pack_bf16x2(f[6], f[7]));
  *reinterpret_cast<uint4*>(p) = u;
}

// mode: 0 = RMSNorm, 1 = LayerNorm.  act: 0 = none, 1 = swish (y = x * sigmoid(norm(x))).
// Optional residual input: h = x + res is normalised and also written to h_out.
template <int MODE>
__global__ void __launch_bounds__(NT)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out, float* __restrict__ mean_out,
                float* __restrict__ rstd_out, int T, int D, float eps, int act) {
  __shared__ float red[NT / 32];
  const int nvec = D / 8;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const __nv_bfloat16* xr = x + (long long)row * D;
    float v[MAXV][8];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int vi = threadIdx.x + i * NT;
      if (vi < nvec) {
        load8(xr + vi * 8, v[i]);
        if (res != nullptr) {
          float r8[8];
          load8(res + (long long)row * D + vi * 8, r8);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += r8[j];
          if (h_out != nullptr) {
            // round the sum to bf16 first so the normalised value matches what is stored
            store8(h_out + (long long)row * D + vi * 8, v[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16_rn(v[i][j]));
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) { s += v[i][j]; ss += v[i][j] * v[i][j]; }
      }
    }
    float mean = 0.f, rstd;
    if (MODE == 1) {
      mean = block_sum(s, red) / D;
      float var = 0.f;
#pragma unroll
      for (int i = 0; i < MAXV; ++i) {
        const int vi = threadIdx.x + i * NT;
        if (vi < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) { float d = v[i][j] - mean; var += d * d; }
        }
      }
      var = block_sum(var, red) / D;
      rstd = rsqrtf(var + eps);
    } else {
      ss = block_sum(ss, red) / D;
      rstd = rsqrtf(ss + eps);
    }
    if (threadIdx.x == 0) {
      if (rstd_out) rstd_out[row] = rstd;
      if (MODE == 1 && mean_out) mean_out[row] = mean;
    }
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int vi = threadIdx.x + i * NT;
      if (vi < nvec) {
        float w8[8], b8[8], o[8];
        if (w != nullptr) load8(w + vi * 8, w8);
        if (b != nullptr) load8(b + vi * 8, b8);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float n = (v[i][j] - mean) * rstd;
          if (w != nullptr) n *= w8[j];
          if (b != nullptr) n += b8[j];
          o[j] = act ? v[i][j] * (1.f / (1.f + __expf(-n))) : n;
        }
        store8(y + (long long)row * D + vi * 8, o);
      }
    }
  }
}

// dx for every row, plus per-CTA partial sums of dw (and db for LayerNorm) in `partial`
// laid out [gridDim.x][2][D] (dw row then db row).
template <int MODE, int ACT>
__global__ void __launch_bounds__(NT)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                float* __restrict__ partial, int T, int D) {
  __shared__ float red[NT / 32];
  const int nvec = D / 8;
  float dw_acc[MAXV][8], db_acc[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) { dw_acc[i][j] = 0.f; db_acc[i][j] = 0.f; }

  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const float rstd = rstd_in[row];
    const float mean = (MODE == 1) ? mean_in[row] : 0.f;
    float xh[MAXV][8], g[MAXV][8], direct[ACT ? MAXV : 1][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int vi = threadIdx.x + i * NT;
      if (vi < nvec) {
        float x8[8], d8[8], w8[8], b8[8];
        load8(x + (long long)row * D + vi * 8, x8);
        load8(dy + (long long)row * D + vi * 8, d8);
#pragma unroll
        for (int j = 0; j < 8; ++j) { w8[j] = 1.f; b8[j] = 0.f; }
        if (w != nullptr) load8(w + vi * 8, w8);
        if (ACT && b != nullptr) load8(b + vi * 8, b8);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xn = (x8[j] - mean) * rstd;
          float dn = d8[j];  // gradient w.r.t. the affine output n = xn * w + b
          if (ACT) {
            // y = x * sigmoid(n): through n the gradient is dy * x * s * (1 - s); the direct
            // path dy * s is added to dx after the row reductions
            const float n = xn * w8[j] + b8[j];
            const float sg = 1.f / (1.f + __expf(-n));
            dn = d8[j] * x8[j] * sg * (1.f - sg);
            direct[ACT ? i : 0][j] = d8[j] * sg;
          }
          dw_acc[i][j] += dn * xn;
          db_acc[i][j] += dn;
          const float gj = dn * w8[j];
          g[i][j] = gj;
          xh[i][j] = xn;
          s1 += gj * xn;
          s2 += gj;
        }
      }
    }
    s1 = block_sum(s1, red) / D;
    if (MODE == 1) s2 = block_sum(s2, red) / D; else s2 = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int vi = threadIdx.x + i * NT;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j] = rstd * (g[i][j] - xh[i][j] * s1 - s2);
          if (ACT) o[j] += direct[ACT ? i : 0][j];
        }
        if (dres != nullptr) {
          float r8[8];
          load8(dres + (long long)row * D + vi * 8, r8);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r8[j];
        }
        store8(dx + (long long)row * D + vi * 8, o);
      }
    }
  }
  if (partial != nullptr) {
    float* pw = partial + (long long)blockIdx.x * 2 * D;
    float* pb = pw + D;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int vi = threadIdx.x + i * NT;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { pw[vi * 8 + j] = dw_acc[i][j]; pb[vi * 8 + j] = db_acc[i][j]; }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Warp-per-row variants for D a multiple of 256 up to 4096: a lane owns the 16-byte vectors
// lane, lane + 32, ... of its row, all loads of a row are in flight together and the row
// reductions are warp shuffles (no block barrier).
// ---------------------------------------------------------------------------------------
constexpr int WMAXV = 16;

template <int MODE>
__global__ void __launch_bounds__(256)
norm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                     const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                     __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out, float* __restrict__ mean_out,
                     float* __restrict__ rstd_out, int T, int D, float eps, int act) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nv = D >> 8;  // vectors per lane
  for (int row = blockIdx.x * 8 + warp; row < T; row += gridDim.x * 8) {
    const long long base = (long long)row * D;
    uint4 xv[WMAXV];
#pragma unroll
    for (int i = 0; i < WMAXV; ++i)
      if (i < nv) xv[i] = *reinterpret_cast<const uint4*>(x + base + (lane + 32 * i) * 8);
    if (res != nullptr) {
#pragma unroll
      for (int i = 0; i < WMAXV; ++i)
        if (i < nv) {
          float a[8], r[8];
          load8(reinterpret_cast<const __nv_bfloat16*>(&xv[i]), a);
          load8(res + base + (lane + 32 * i) * 8, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) a[j] += r[j];
          xv[i] = make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]), pack_bf16x2(a[6], a[7]));
          if (h_out != nullptr) *reinterpret_cast<uint4*>(h_out + base + (lane + 32 * i) * 8) = xv[i];
        }
    }
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int i = 0; i < WMAXV; ++i)
      if (i < nv) {
        float a[8];
        load8(reinterpret_cast<const __nv_bfloat16*>(&xv[i]), a);
#pragma unroll
        for (int j = 0; j < 8; ++j) { s += a[j]; ss += a[j] * a[j]; }
      }
    float mean = 0.f, rstd;
    if (MODE == 1) {
      mean = warp_sum(s) / D;
      float var = 0.f;
#pragma unroll
      for (int i = 0; i < WMAXV; ++i)
        if (i < nv) {
          float a[8];
          load8(reinterpret_cast<const __nv_bfloat16*>(&xv[i]), a);
#pragma unroll
          for (int j = 0; j < 8; ++j) { const float d = a[j] - mean; var += d * d; }
        }
      rstd = rsqrtf(warp_sum(var) / D + eps);
    } else {
      rstd = rsqrtf(warp_sum(ss) / D + eps);
    }
    if (lane == 0) {
      if (rstd_out) rstd_out[row] = rstd;
      if (MODE == 1 && mean_out) mean_out[row] = mean;
    }
#pragma unroll
    for (int i = 0; i < WMAXV; ++i)
      if (i < nv) {
        const int c = (lane + 32 * i) * 8;
        float a[8], w8[8], b8[8], o[8];
        load8(reinterpret_cast<const __nv_bfloat16*>(&xv[i]), a);
        if (w != nullptr) load8(w + c, w8);
        if (b != nullptr) load8(b + c, b8);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float n = (a[j] - mean) * rstd;
          if (w != nullptr) n *= w8[j];
          if (b != nullptr) n += b8[j];
          o[j] = act ? a[j] * (1.f / (1.f + __expf(-n))) : n;
        }
        store8(y + base + c, o);
      }
  }
}

// dx per row; dw / db accumulated per warp in shared memory (fixed lane -> column mapping, no
// atomics), summed over the CTA's warps in order and written as one partial row per CTA.
template <int MODE, int ACT>
__global__ void __launch_bounds__(256)
norm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                     const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                     const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                     const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                     float* __restrict__ partial, int T, int D, int nwarps) {
  extern __shared__ float acc[];  // [nwarps][(MODE == 1 || ACT) ? 2 : 1][D]
  constexpr int NACC = (MODE == 1 || ACT) ? 2 : 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nv = D >> 8;
  float* my_w = acc + (long long)warp * NACC * D;
  float* my_b = my_w + D;
  if (warp < nwarps)
    for (int i = lane; i < NACC * D; i += 32) my_w[i] = 0.f;
  __syncwarp();
  if (warp < nwarps) {
    for (int row = blockIdx.x * nwarps + warp; row < T; row += gridDim.x * nwarps) {
      const long long base = (long long)row * D;
      const float rstd = rstd_in[row];
      const float mean = (MODE == 1) ? mean_in[row] : 0.f;
      uint4 xv[WMAXV], gv[WMAXV];
#pragma unroll
      for (int i = 0; i < WMAXV; ++i)
        if (i < nv) {
          xv[i] = *reinterpret_cast<const uint4*>(x + base + (lane + 32 * i) * 8);
          gv[i] = *reinterpret_cast<const uint4*>(dy + base + (lane + 32 * i) * 8);
        }
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int i = 0; i < WMAXV; ++i)
        if (i < nv) {
          const int c = (lane + 32 * i) * 8;
          float x8[8], d8[8], w8[8], b8[8];
          load8(reinterpret_cast<const __nv_bfloat16*>(&xv[i]), x8);
          load8(reinterpret_cast<const __nv_bfloat16*>(&gv[i]), d8);
#pragma unroll
          for (int j = 0; j < 8; ++j) { w8[j] = 1.f; b8[j] = 0.f; }
          if (w != nullptr) load8(w + c, w8);
          if (ACT && b != nullptr) load8(b + c, b8);
          float4 a0 = *reinterpret_cast<float4*>(my_w + c), a1 = *reinterpret_cast<float4*>(my_w + c + 4);
          float aw[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
          float ab[8];
          if (NACC == 2) {
            float4 b0 = *reinterpret_cast<float4*>(my_b + c), b1 = *reinterpret_cast<float4*>(my_b + c + 4);
            ab[0] = b0.x; ab[1] = b0.y; ab[2] = b0.z; ab[3] = b0.w; ab[4] = b1.x; ab[5] = b1.y; ab[6] = b1.z; ab[7] = b1.w;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float xn = (x8[j] - mean) * rstd;
            float dn = d8[j];
            if (ACT) {
              const float n = xn * w8[j] + b8[j];
              const float sg = 1.f / (1.f + __expf(-n));
              dn = d8[j] * x8[j] * sg * (1.f - sg);
            }
            aw[j] += dn * xn;
            if (NACC == 2) ab[j] += dn;
            const float gj = dn * w8[j];
            s1 += gj * xn;
            s2 += gj;
          }
          *reinterpret_cast<float4*>(my_w + c) = make_float4(aw[0], aw[1], aw[2], aw[3]);
          *reinterpret_cast<float4*>(my_w + c + 4) = make_float4(aw[4], aw[5], aw[6], aw[7]);
          if (NACC == 2) {
            *reinterpret_cast<float4*>(my_b + c) = make_float4(ab[0], ab[1], ab[2], ab[3]);
            *reinterpret_cast<float4*>(my_b + c + 4) = make_float4(ab[4], ab[5], ab[6], ab[7]);
          }
        }
      s1 = warp_sum(s1) / D;
      s2 = (MODE == 1) ? warp_sum(s2) / D : 0.f;
#pragma unroll
      for (int i = 0; i < WMAXV; ++i)
        if (i < nv) {
          const int c = (lane + 32 * i) * 8;
          float x8[8], d8[8], w8[8], b8[8], o[8];
          load8(reinterpret_cast<const __nv_bfloat16*>(&xv[i]), x8);
          load8(reinterpret_cast<const __nv_bfloat16*>(&gv[i]), d8);
#pragma unroll
          for (int j = 0; j < 8; ++j) { w8[j] = 1.f; b8[j] = 0.f; }
          if (w != nullptr) load8(w + c, w8);
          if (ACT && b != nullptr) load8(b + c, b8);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float xn = (x8[j] - mean) * rstd;
            float dn = d8[j], direct = 0.f;
            if (ACT) {
              const float n = xn * w8[j] + b8[j];
              const float sg = 1.f / (1.f + __expf(-n));
              dn = d8[j] * x8[j] * sg * (1.f - sg);
              direct = d8[j] * sg;
            }
            o[j] = rstd * (dn * w8[j] - xn * s1 - s2) + direct;
          }
          if (dres != nullptr) {
            float r8[8];
            load8(dres + base + c, r8);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] += r8[j];
          }
          store8(dx + base + c, o);
        }
    }
  }
  __syncthreads();
  if (partial != nullptr) {
    float* pw = partial + (long long)blockIdx.x * 2 * D;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      float sw = 0.f, sb = 0.f;
      for (int k = 0; k < nwarps; ++k) {
        sw += acc[(long long)k * NACC * D + c];
        if (NACC == 2) sb += acc[(long long)k * NACC * D + D + c];
      }
      pw[c] = sw;
      pw[D + c] = sb;
    }
  }
}

// out[c] (+)= sum_p partial[p][which][c], fixed order over p
__global__ void norm_bwd_reduce_kernel(const float* __restrict__ partial, int nparts, int D, float* __restrict__ dw,
                                       float* __restrict__ db, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float sw = 0.f, sb = 0.f;
  for (int p = 0; p < nparts; ++p) {
    sw += partial[(long long)p * 2 * D + c];
    sb += partial[(long long)p * 2 * D + D + c];
  }
  if (dw != nullptr) dw[c] = accumulate ? dw[c] + sw : sw;
  if (db != nullptr) db[c] = accumulate ? db[c] + sb : sb;
}

}  // namespace

// Number of fp32 elements of scratch needed by b200_norm_bwd for a [T, D] problem.
static bool warp_path(int D) { return D % 256 == 0 && D <= 4096; }

B200_API long long b200_norm_bwd_scratch_elems(int T, int D) {
  int grid = b200::sm_count() * 2;
  if (grid > T) grid = T;
  return (long long)grid * 2 * D;
}

// mode 0 RMSNorm / 1 LayerNorm.  res/h_out/b/mean/w may be null.  act=1: y = h * sigmoid(norm(h)).
B200_API int b200_norm_fwd(int mode, const void* x, const void* res, const void* w, const void* b, void* y,
                           void* h_out, float* mean, float* rstd, int T, int D, float eps, int act, void* stream) {
  if (D % 8 != 0 || D > NT * MAXV * 8) return b200::fail(300, "norm_fwd: D=%d must be a multiple of 8 and <= %d", D, NT * MAXV * 8);
  if (T <= 0) return 0;
  int grid = T < b200::sm_count() * 8 ? T : b200::sm_count() * 8;
  auto X = (const __nv_bfloat16*)x; auto R = (const __nv_bfloat16*)res; auto W = (const __nv_bfloat16*)w;
  auto B = (const __nv_bfloat16*)b; auto Y = (__nv_bfloat16*)y; auto H = (__nv_bfloat16*)h_out;
  if (warp_path(D)) {
    int wgrid = (T + 7) / 8;
    if (wgrid > b200::sm_count() * 8) wgrid = b200::sm_count() * 8;
    if (mode == 0) norm_fwd_warp_kernel<0><<<wgrid, 256, 0, (cudaStream_t)stream>>>(X, R, W, B, Y, H, mean, rstd, T, D, eps, act);
    else norm_fwd_warp_kernel<1><<<wgrid, 256, 0, (cudaStream_t)stream>>>(X, R, W, B, Y, H, mean, rstd, T, D, eps, act);
    b200::count_launch();
    return b200::check_launch("norm_fwd_warp");
  }
  if (mode == 0) norm_fwd_kernel<0><<<grid, NT, 0, (cudaStream_t)stream>>>(X, R, W, B, Y, H, mean, rstd, T, D, eps, act);
  else norm_fwd_kernel<1><<<grid, NT, 0, (cudaStream_t)stream>>>(X, R, W, B, Y, H, mean, rstd, T, D, eps, act);
  b200::count_launch();
  return b200::check_launch("norm_fwd");
}

// dx = d(norm)/dx (+ dres); dw/db fp32 [D] (written, or added to when accumulate != 0).
// `scratch` must hold b200_norm_bwd_scratch_elems(T, D) floats.
B200_API int b200_norm_bwd(int mode, const void* dy, const void* x, const void* w, const void* b, const float* mean,
                           const float* rstd, const void* dres, void* dx, float* dw, float* db, float* scratch,
                           int T, int D, int act, int accumulate, void* stream) {
  if (D % 8 != 0 || D > NT * MAXV * 8) return b200::fail(301, "norm_bwd: D=%d must be a multiple of 8 and <= %d", D, NT * MAXV * 8);
  if (T <= 0) return 0;
  int grid = b200::sm_count() * 2;
  if (grid > T) grid = T;
  auto DY = (const __nv_bfloat16*)dy; auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w;
  auto B = (const __nv_bfloat16*)b; auto DR = (const __nv_bfloat16*)dres; auto DX = (__nv_bfloat16*)dx;
  cudaStream_t st = (cudaStream_t)stream;
  if (warp_path(D)) {
    const int nacc = (mode == 1 || act) ? 2 : 1;
    int nwarps = (200 * 1024) / (D * 4 * nacc);
    if (nwarps > 8) nwarps = 8;
    const int smem = nwarps * nacc * D * 4;
    int wgrid = b200::sm_count();
    if (wgrid > grid) wgrid = grid;  // never more partial rows than the scratch holds
    static bool configured[64][4] = {{false}};
    int dev = 0;
    cudaGetDevice(&dev);
    const int variant = (mode ? 2 : 0) + (act ? 1 : 0);
    if (!configured[dev & 63][variant]) {
      cudaError_t e;
      if (variant == 0) e = cudaFuncSetAttribute(norm_bwd_warp_kernel<0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      else if (variant == 1) e = cudaFuncSetAttribute(norm_bwd_warp_kernel<0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      else if (variant == 2) e = cudaFuncSetAttribute(norm_bwd_warp_kernel<1, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      else e = cudaFuncSetAttribute(norm_bwd_warp_kernel<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (e != cudaSuccess) { cudaGetLastError(); return b200::fail(302, "norm_bwd: cannot raise shared memory: %s", cudaGetErrorString(e)); }
      configured[dev & 63][variant] = true;
    }
    if (variant == 0) norm_bwd_warp_kernel<0, 0><<<wgrid, 256, smem, st>>>(DY, X, W, B, mean, rstd, DR, DX, scratch, T, D, nwarps);
    else if (variant == 1) norm_bwd_warp_kernel<0, 1><<<wgrid, 256, smem, st>>>(DY, X, W, B, mean, rstd, DR, DX, scratch, T, D, nwarps);
    else if (variant == 2) norm_bwd_warp_kernel<1, 0><<<wgrid, 256, smem, st>>>(DY, X, W, B, mean, rstd, DR, DX, scratch, T, D, nwarps);
    else norm_bwd_warp_kernel<1, 1><<<wgrid, 256, smem, st>>>(DY, X, W, B, mean, rstd, DR, DX, scratch, T, D, nwarps);
    b200::count_launch();
    if (int r = b200::check_launch("norm_bwd_warp")) return r;
    if (scratch != nullptr && (dw != nullptr || db != nullptr)) {
      norm_bwd_reduce_kernel<<<(D + 255) / 256, 256, 0, st>>>(scratch, wgrid, D, dw, db, accumulate);
      b200::count_launch();
      return b200::check_launch("norm_bwd_reduce");
    }
    return 0;
  }
  if (mode == 0 && !act) norm_bwd_kernel<0, 0><<<grid, NT, 0, st>>>(DY, X, W, B, mean, rstd, DR, DX, scratch, T, D);
  else if (mode == 0) norm_bwd_kernel<0, 1><<<grid, NT, 0, st>>>(DY, X, W, B, mean, rstd, DR, DX, scratch, T, D);
  else if (!act) norm_bwd_kernel<1, 0><<<grid, NT, 0, st>>>(DY, X, W, B, mean, rstd, DR, DX, scratch, T, D);
  else norm_bwd_kernel<1, 1><<<grid, NT, 0, st>>>(DY, X, W, B, mean, rstd, DR, DX, scratch, T, D);
  b200::count_launch();
  if (int r = b200::check_launch("norm_bwd")) return r;
  if (scratch != nullptr && (dw != nullptr || db != nullptr)) {
    norm_bwd_reduce_kernel<<<(D + 255) / 256, 256, 0, (cudaStream_t)stream>>>(scratch, grid, D, dw, db, accumulate);
    b200::count_launch();
    return b200::check_launch("norm_bwd_reduce");
  }
  return 0;
}
