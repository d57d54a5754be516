// HSTU layer glue between the jagged attention and the output projection, one pass each way:
//
//   forward   u = silu(u_raw);  n = LayerNorm(attn) * w + b;  cat = [u | attn | u * n]        ([T, 3D] bf16)
//   backward  from dcat = [du' | da' | dy]:
//             du_raw = (du' + dy * n) * silu'(u_raw)
//             dattn  = da' + LayerNorm_bwd(dy * u)
//             dw    += sum_t (dy * u) * xhat,   db += sum_t dy * u
//
// u_raw is a column block of the fused uvqk projection (row pitch given), so the kernel reads it in
// place; du_raw is written with its own pitch so it can land inside the gradient of that projection.
// One warp owns a row (D a multiple of 256, at most 768: a lane keeps D/256 16-byte vectors of each
// operand in registers); the weight / bias gradients are kept per lane in registers over all rows the
// warp visits, summed over the CTA's warps in a fixed order and written as one partial row per CTA
// that a second kernel adds up: no atomics, bit-reproducible.
//
// Dropout of the concatenation (rate p, survivors scaled by 1 / (1 - p)) is part of both passes: the keep
// mask comes from a Philox stream keyed by (seed, row, lane), so backward regenerates it instead of
// reading a stored mask.
//
// Replaces the chain the reference fuses as "layer norm * u (+ dropout)" before the output linear
// (generative_recommenders/ops/triton/triton_hstu_linear.py: _ln_mul_dropout_fwd / _ln_mul_dropout_bwd,
// with concat_ux) and the SiLU of u (generative_recommenders/ops/hstu_compute.py: hstu_preprocess_and_attention).
#include <curand_kernel.h>

#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int GV = 3;   // vectors of 8 per lane -> D <= 768

B200_DEVICE void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
B200_DEVICE void st8(__nv_bfloat16* p, const float (&f)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                                            pack_bf16x2(f[6], f[7]));
}
B200_DEVICE float rbf(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// Keep masks of one row for this lane: bit (8 * s + j) of keep[i] covers element j of vector i in section s
// (0 = u, 1 = attn, 2 = y).  Forward and backward call this with the same (seed, row, lane) and get the same bits.
// Every 32-bit Philox word decides two elements: a 16-bit half is compared with thr = round(p * 65536), so the
// rate is p to within 2^-17.
template <int NV>
B200_DEVICE void draw_keep(unsigned (&keep)[NV], unsigned thr, unsigned long long seed, long long row, int lane) {
#pragma unroll
  for (int i = 0; i < NV; ++i) keep[i] = 0xffffffu;
  if (thr == 0) return;
  curandStatePhilox4_32_10_t st;
  curand_init(seed, (unsigned long long)row * 32 + lane, 0, &st);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    unsigned m = 0;
#pragma unroll
    for (int q = 0; q < 3; ++q) {
      const uint4 r = curand4(&st);
      const unsigned wv[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        m |= ((wv[k] & 0xffffu) >= thr ? 1u : 0u) << (8 * q + 2 * k);
        m |= ((wv[k] >> 16) >= thr ? 1u : 0u) << (8 * q + 2 * k + 1);
      }
    }
    keep[i] = m;
  }
}
B200_DEVICE void apply_keep(float (&f)[8], unsigned bits, float inv_keep) {
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = (bits >> j) & 1u ? f[j] * inv_keep : 0.f;
}

template <int NV>
__global__ void __launch_bounds__(256, 2)
gate_cat_fwd_kernel(const __nv_bfloat16* __restrict__ u_raw, long long ld_u, const __nv_bfloat16* __restrict__ attn,
                    const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                    __nv_bfloat16* __restrict__ cat, float* __restrict__ mean_out, float* __restrict__ rstd_out, int T,
                    float eps, float p, unsigned thr, unsigned long long seed) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int D = NV * 256;
  for (long long row = (long long)blockIdx.x * 8 + warp; row < T; row += (long long)gridDim.x * 8) {
    float a[NV][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        ld8(attn + row * D + (lane + 32 * i) * 8, a[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += a[i][j];
      }
    const float mean = warp_sum(s) / D;
    float var = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float d = a[i][j] - mean; var += d * d; }
      }
    const float rstd = rsqrtf(warp_sum(var) / D + eps);
    if (lane == 0) { mean_out[row] = mean; rstd_out[row] = rstd; }
    unsigned keep[NV];
    draw_keep<NV>(keep, thr, seed, row, lane);
    const float inv_keep = 1.f / (1.f - p);
    __nv_bfloat16* out = cat + row * 3 * D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (lane + 32 * i) * 8;
        float ur[8], w8[8], b8[8], u[8], y[8];
        ld8(u_raw + row * ld_u + c, ur);
        ld8(w + c, w8);
        ld8(b + c, b8);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          u[j] = rbf(ur[j] / (1.f + __expf(-ur[j])));
          const float n = rbf((a[i][j] - mean) * rstd * w8[j] + b8[j]);
          y[j] = u[j] * n;
        }
        if (thr != 0) {
          apply_keep(u, keep[i], inv_keep);
          apply_keep(a[i], keep[i] >> 8, inv_keep);
          apply_keep(y, keep[i] >> 16, inv_keep);
        }
        st8(out + c, u);
        st8(out + D + c, a[i]);
        st8(out + 2 * D + c, y);
      }
  }
}

template <int NV>
__global__ void __launch_bounds__(256, 2)
gate_cat_bwd_kernel(const __nv_bfloat16* __restrict__ dcat, const __nv_bfloat16* __restrict__ u_raw, long long ld_u,
                    const __nv_bfloat16* __restrict__ attn, const __nv_bfloat16* __restrict__ w,
                    const __nv_bfloat16* __restrict__ b, const float* __restrict__ mean_in,
                    const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ du_raw, long long ld_du,
                    __nv_bfloat16* __restrict__ dattn, float* __restrict__ partial, int T, float p, unsigned thr,
                    unsigned long long seed) {
  extern __shared__ float acc[];   // [8 warps][2][D]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int D = NV * 256;
  float gw[NV][8], gb[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) { gw[i][j] = 0.f; gb[i][j] = 0.f; }
  for (long long row = (long long)blockIdx.x * 8 + warp; row < T; row += (long long)gridDim.x * 8) {
    const float mean = mean_in[row], rstd = rstd_in[row];
    unsigned keep[NV];
    draw_keep<NV>(keep, thr, seed, row, lane);
    const float inv_keep = 1.f / (1.f - p);
    const __nv_bfloat16* dc = dcat + row * 3 * D;
    float xn[NV][8], g[NV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (lane + 32 * i) * 8;
        float ur[8], a8[8], w8[8], b8[8], dy[8], du[8], o[8];
        ld8(u_raw + row * ld_u + c, ur);
        ld8(attn + row * D + c, a8);
        ld8(w + c, w8);
        ld8(b + c, b8);
        ld8(dc + 2 * D + c, dy);
        ld8(dc + c, du);
        if (thr != 0) {
          apply_keep(du, keep[i], inv_keep);
          apply_keep(dy, keep[i] >> 16, inv_keep);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float sg = 1.f / (1.f + __expf(-ur[j]));
          const float u = rbf(ur[j] * sg);
          xn[i][j] = (a8[j] - mean) * rstd;
          const float n = rbf(xn[i][j] * w8[j] + b8[j]);
          const float dn = dy[j] * u;
          gw[i][j] += dn * xn[i][j];
          gb[i][j] += dn;
          g[i][j] = dn * w8[j];
          s1 += g[i][j] * xn[i][j];
          s2 += g[i][j];
          o[j] = (du[j] + dy[j] * n) * (sg * (1.f + ur[j] * (1.f - sg)));
        }
        st8(du_raw + row * ld_du + c, o);
      }
    s1 = warp_sum(s1) / D;
    s2 = warp_sum(s2) / D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (lane + 32 * i) * 8;
        float da[8], o[8];
        ld8(dc + D + c, da);
        if (thr != 0) apply_keep(da, keep[i] >> 8, inv_keep);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = da[j] + rstd * (g[i][j] - xn[i][j] * s1 - s2);
        st8(dattn + row * D + c, o);
      }
  }
  float* mine = acc + (long long)warp * 2 * D;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
      const int c = (lane + 32 * i) * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) { mine[c + j] = gw[i][j]; mine[D + c + j] = gb[i][j]; }
    }
  __syncthreads();
  float* pw = partial + (long long)blockIdx.x * 2 * D;
  for (int c = threadIdx.x; c < 2 * D; c += 256) {
    float sum = 0.f;
    for (int k = 0; k < 8; ++k) sum += acc[(long long)k * 2 * D + c];
    pw[c] = sum;
  }
}

__global__ void gate_cat_reduce_kernel(const float* __restrict__ partial, int nparts, int D, float* __restrict__ dw,
                                       float* __restrict__ db, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float sw = 0.f, sb = 0.f;
  for (int p = 0; p < nparts; ++p) {
    sw += partial[(long long)p * 2 * D + c];
    sb += partial[(long long)p * 2 * D + D + c];
  }
  dw[c] = accumulate ? dw[c] + sw : sw;
  db[c] = accumulate ? db[c] + sb : sb;
}

int gate_grid(int T) {
  int grid = (T + 7) / 8;
  const int cap = b200::sm_count() * 2;   // two resident CTAs per SM
  return grid < cap ? (grid < 1 ? 1 : grid) : cap;
}

bool gate_ok(int D, long long ld_u) { return D % 256 == 0 && D >= 256 && D <= 256 * GV && ld_u % 8 == 0; }

}  // namespace

// fp32 scratch elements b200_hstu_gate_cat_bwd needs for T rows of width D.
B200_API long long b200_hstu_gate_cat_scratch_elems(int T, int D) { return (long long)gate_grid(T) * 2 * D; }

// cat[T, 3D] = dropout([silu(u_raw) | attn | silu(u_raw) * LayerNorm(attn)], p);  mean / rstd [T] fp32 are kept for
// backward, which must be given the same p and seed.
B200_API int b200_hstu_gate_cat_fwd(const void* u_raw, long long ld_u, const void* attn, const void* w, const void* b,
                                    void* cat, float* mean, float* rstd, int T, int D, float eps, float p,
                                    unsigned long long seed, void* stream) {
  if (!(p >= 0.f && p < 1.f)) return b200::fail(902, "hstu_gate_cat_fwd: dropout rate %f outside [0, 1)", (double)p);
  if (!gate_ok(D, ld_u)) return b200::fail(900, "hstu_gate_cat_fwd: D=%d must be 256, 512 or 768 and the pitch %lld a multiple of 8", D, ld_u);
  if (T <= 0) return 0;
  const unsigned thr = (unsigned)lrintf(p * 65536.f);
  const float pe = (float)thr / 65536.f;   // the rate the 16-bit comparison realises
  auto U = (const __nv_bfloat16*)u_raw; auto A = (const __nv_bfloat16*)attn; auto W = (const __nv_bfloat16*)w;
  auto B = (const __nv_bfloat16*)b; auto C = (__nv_bfloat16*)cat;
  const int grid = gate_grid(T);
  cudaStream_t st = (cudaStream_t)stream;
  if (D == 256) gate_cat_fwd_kernel<1><<<grid, 256, 0, st>>>(U, ld_u, A, W, B, C, mean, rstd, T, eps, pe, thr, seed);
  else if (D == 512) gate_cat_fwd_kernel<2><<<grid, 256, 0, st>>>(U, ld_u, A, W, B, C, mean, rstd, T, eps, pe, thr, seed);
  else gate_cat_fwd_kernel<3><<<grid, 256, 0, st>>>(U, ld_u, A, W, B, C, mean, rstd, T, eps, pe, thr, seed);
  b200::count_launch();
  return b200::check_launch("hstu_gate_cat_fwd");
}

// du_raw (row pitch ld_du) and dattn [T, D] from dcat [T, 3D]; dw / db fp32 [D] written, or added to when
// accumulate != 0.  scratch: b200_hstu_gate_cat_scratch_elems(T, D) floats.
B200_API int b200_hstu_gate_cat_bwd(const void* dcat, const void* u_raw, long long ld_u, const void* attn, const void* w,
                                    const void* b, const float* mean, const float* rstd, void* du_raw, long long ld_du,
                                    void* dattn, float* dw, float* db, float* scratch, int T, int D, int accumulate,
                                    float p, unsigned long long seed, void* stream) {
  if (!(p >= 0.f && p < 1.f)) return b200::fail(902, "hstu_gate_cat_bwd: dropout rate %f outside [0, 1)", (double)p);
  if (!gate_ok(D, ld_u) || ld_du % 8 != 0)
    return b200::fail(901, "hstu_gate_cat_bwd: D=%d must be 256, 512 or 768 and the pitches %lld / %lld multiples of 8", D, ld_u, ld_du);
  if (T <= 0) return 0;
  const int grid = gate_grid(T);
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned thr = (unsigned)lrintf(p * 65536.f);
  const float pe = (float)thr / 65536.f;
  auto DC = (const __nv_bfloat16*)dcat; auto U = (const __nv_bfloat16*)u_raw; auto A = (const __nv_bfloat16*)attn;
  auto W = (const __nv_bfloat16*)w; auto B = (const __nv_bfloat16*)b; auto DU = (__nv_bfloat16*)du_raw; auto DA = (__nv_bfloat16*)dattn;
  const size_t smem = 8 * 2 * D * sizeof(float);
  if (D == 256) gate_cat_bwd_kernel<1><<<grid, 256, smem, st>>>(DC, U, ld_u, A, W, B, mean, rstd, DU, ld_du, DA, scratch, T, pe, thr, seed);
  else if (D == 512) gate_cat_bwd_kernel<2><<<grid, 256, smem, st>>>(DC, U, ld_u, A, W, B, mean, rstd, DU, ld_du, DA, scratch, T, pe, thr, seed);
  else gate_cat_bwd_kernel<3><<<grid, 256, smem, st>>>(DC, U, ld_u, A, W, B, mean, rstd, DU, ld_du, DA, scratch, T, pe, thr, seed);
  b200::count_launch();
  if (int r = b200::check_launch("hstu_gate_cat_bwd")) return r;
  gate_cat_reduce_kernel<<<(D + 255) / 256, 256, 0, st>>>(scratch, grid, D, dw, db, accumulate);
  b200::count_launch();
  return b200::check_launch("hstu_gate_cat_reduce");
}
