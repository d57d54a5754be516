// Glue kernels of the MMDiT (FLUX.1) blocks: the AdaLN modulation and the gated residual, each one pass
// forward and one pass (+ a per-sample column reduction) backward.
//
//   ln_modulate      y[t, :] = LayerNorm(x[t, :]) * (1 + scale[b, :]) + shift[b, :]        (no affine, b = t / S)
//   gate_residual    out[t, :] = res[t, :] + y[t, :] * gate[b, :]
//
// Backward:
//   ln_modulate_bwd      dx (row-wise LayerNorm backward of g = dy * (1 + scale))
//   modulate_param_bwd   dscale[b, :] = sum_s dy * xhat,  dshift[b, :] = sum_s dy          (column reduction per sample)
//   gate_bwd             dy = dout * gate[b, :];  dgate[b, :] = sum_s dout * y             (same reduction kernel shape)
//
// They replace chains of element-wise torch ops (LayerNorm, multiply, add, broadcast) and stand for the
// reference's fused diffusion glue, which it obtains from per-block torch.compile and Primus fusions
// (flux1/primus/config_common.sh:84-150).
#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int MAXV = 16;   // 8-element vectors per lane: D <= 32 * 8 * 16 = 4096

// one warp per row
__global__ void __launch_bounds__(256)
ln_modulate_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ shift,
                       const __nv_bfloat16* __restrict__ scale, long long ld_mod, __nv_bfloat16* __restrict__ y,
                       float* __restrict__ mean_out, float* __restrict__ rstd_out, int T, int D, int S, float eps) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= T) return;
  const int lane = threadIdx.x & 31;
  const int nv = D / 256;                         // vectors of 8 per lane
  const uint4* xr = reinterpret_cast<const uint4*>(x + (long long)row * D);
  float v[MAXV][8];
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    if (j < nv) {
      const uint4 u = xr[j * 32 + lane];
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      v[j][0] = a.x; v[j][1] = a.y; v[j][2] = b.x; v[j][3] = b.y; v[j][4] = c.x; v[j][5] = c.y; v[j][6] = d.x; v[j][7] = d.y;
#pragma unroll
      for (int i = 0; i < 8; ++i) sum += v[j][i];
    }
  }
  const float mean = warp_sum(sum) / D;
  float sq = 0.f;
#pragma unroll
  for (int j = 0; j < MAXV; ++j)
    if (j < nv)
#pragma unroll
      for (int i = 0; i < 8; ++i) { const float d = v[j][i] - mean; sq += d * d; }
  const float rstd = rsqrtf(warp_sum(sq) / D + eps);
  if (lane == 0) { mean_out[row] = mean; rstd_out[row] = rstd; }
  const long long b = row / S;
  const uint4* sh = reinterpret_cast<const uint4*>(shift + b * ld_mod);
  const uint4* sc = reinterpret_cast<const uint4*>(scale + b * ld_mod);
  uint4* yr = reinterpret_cast<uint4*>(y + (long long)row * D);
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    if (j < nv) {
      const uint4 us = sh[j * 32 + lane], uc = sc[j * 32 + lane];
      const float2 s0 = unpack_bf16x2(us.x), s1 = unpack_bf16x2(us.y), s2 = unpack_bf16x2(us.z), s3 = unpack_bf16x2(us.w);
      const float2 c0 = unpack_bf16x2(uc.x), c1 = unpack_bf16x2(uc.y), c2 = unpack_bf16x2(uc.z), c3 = unpack_bf16x2(uc.w);
      const float s[8] = {s0.x, s0.y, s1.x, s1.y, s2.x, s2.y, s3.x, s3.y};
      const float c[8] = {c0.x, c0.y, c1.x, c1.y, c2.x, c2.y, c3.x, c3.y};
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = (v[j][i] - mean) * rstd * (1.f + c[i]) + s[i];
      yr[j * 32 + lane] = make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]), pack_bf16x2(o[6], o[7]));
    }
  }
}

__global__ void __launch_bounds__(256)
ln_modulate_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                       const __nv_bfloat16* __restrict__ scale, long long ld_mod, const float* __restrict__ mean_in,
                       const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx, int T, int D, int S) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= T) return;
  const int lane = threadIdx.x & 31;
  const int nv = D / 256;
  const float mean = mean_in[row], rstd = rstd_in[row];
  const long long b = row / S;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (long long)row * D);
  const uint4* gr = reinterpret_cast<const uint4*>(dy + (long long)row * D);
  const uint4* sc = reinterpret_cast<const uint4*>(scale + b * ld_mod);
  // two passes over the row (the second one hits L1 / L2): keeps the kernel at a few dozen registers
  auto load = [&](int j, float (&xh)[8], float (&g)[8]) {
    const uint4 ux = xr[j * 32 + lane], ug = gr[j * 32 + lane], uc = sc[j * 32 + lane];
    const float2 x0 = unpack_bf16x2(ux.x), x1 = unpack_bf16x2(ux.y), x2 = unpack_bf16x2(ux.z), x3 = unpack_bf16x2(ux.w);
    const float2 g0 = unpack_bf16x2(ug.x), g1 = unpack_bf16x2(ug.y), g2 = unpack_bf16x2(ug.z), g3 = unpack_bf16x2(ug.w);
    const float2 c0 = unpack_bf16x2(uc.x), c1 = unpack_bf16x2(uc.y), c2 = unpack_bf16x2(uc.z), c3 = unpack_bf16x2(uc.w);
    const float xv[8] = {x0.x, x0.y, x1.x, x1.y, x2.x, x2.y, x3.x, x3.y};
    const float gv[8] = {g0.x, g0.y, g1.x, g1.y, g2.x, g2.y, g3.x, g3.y};
    const float cv[8] = {c0.x, c0.y, c1.x, c1.y, c2.x, c2.y, c3.x, c3.y};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      xh[i] = (xv[i] - mean) * rstd;
      g[i] = gv[i] * (1.f + cv[i]);
    }
  };
  float s1 = 0.f, s2 = 0.f;
  for (int j = 0; j < nv; ++j) {
    float xh[8], g[8];
    load(j, xh, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) { s1 += g[i]; s2 += g[i] * xh[i]; }
  }
  s1 = warp_sum(s1) / D;
  s2 = warp_sum(s2) / D;
  uint4* dr = reinterpret_cast<uint4*>(dx + (long long)row * D);
  for (int j = 0; j < nv; ++j) {
    float xh[8], g[8], o[8];
    load(j, xh, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = rstd * (g[i] - s1 - xh[i] * s2);
    dr[j * 32 + lane] = make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]), pack_bf16x2(o[6], o[7]));
  }
}

// Per-sample column sums over the S rows of sample b = blockIdx.y; a thread owns 2 adjacent columns.
//   MODE 0 (modulation):  out_a[b, c] = sum_s dy * xhat   (xhat from x, mean, rstd),  out_b[b, c] = sum_s dy
//   MODE 1 (gate):        out_a[b, c] = sum_s dy * x      (x is the gated branch y),  out_b unused
template <int MODE>
__global__ void __launch_bounds__(128)
sample_colsum_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                     const float* __restrict__ mean_in, const float* __restrict__ rstd_in, float* __restrict__ out_a,
                     float* __restrict__ out_b, int D, int S) {
  const int c = (blockIdx.x * 128 + threadIdx.x) * 2;
  if (c >= D) return;
  const long long b = blockIdx.y;
  float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
  for (int s = 0; s < S; ++s) {
    const long long row = b * S + s;
    const float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dy + row * D + c));
    float2 xv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(x + row * D + c));
    if (MODE == 0) {
      const float m = mean_in[row], r = rstd_in[row];
      xv.x = (xv.x - m) * r; xv.y = (xv.y - m) * r;
      b0 += g.x; b1 += g.y;
    }
    a0 += g.x * xv.x; a1 += g.y * xv.y;
  }
  out_a[b * D + c] = a0; out_a[b * D + c + 1] = a1;
  if (MODE == 0) { out_b[b * D + c] = b0; out_b[b * D + c + 1] = b1; }
}

// out = res + y * gate[b]   (BWD = 0)    |    dy = dout * gate[b]   (BWD = 1, res unused)
template <int BWD>
__global__ void __launch_bounds__(256)
gate_kernel(const __nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ gate,
            long long ld_mod, __nv_bfloat16* __restrict__ out, long long n8, int D8, int S) {
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n8; i += (long long)gridDim.x * 256) {
    const long long row = i / D8;
    const int cv = (int)(i - row * D8);
    const long long b = row / S;
    const uint4 uy = reinterpret_cast<const uint4*>(y)[i];
    const uint4 ug = *reinterpret_cast<const uint4*>(gate + b * ld_mod + cv * 8);
    const float2 y0 = unpack_bf16x2(uy.x), y1 = unpack_bf16x2(uy.y), y2 = unpack_bf16x2(uy.z), y3 = unpack_bf16x2(uy.w);
    const float2 g0 = unpack_bf16x2(ug.x), g1 = unpack_bf16x2(ug.y), g2 = unpack_bf16x2(ug.z), g3 = unpack_bf16x2(ug.w);
    float o[8] = {y0.x * g0.x, y0.y * g0.y, y1.x * g1.x, y1.y * g1.y, y2.x * g2.x, y2.y * g2.y, y3.x * g3.x, y3.y * g3.y};
    if (!BWD) {
      const uint4 ur = reinterpret_cast<const uint4*>(res)[i];
      const float2 r0 = unpack_bf16x2(ur.x), r1 = unpack_bf16x2(ur.y), r2 = unpack_bf16x2(ur.z), r3 = unpack_bf16x2(ur.w);
      o[0] += r0.x; o[1] += r0.y; o[2] += r1.x; o[3] += r1.y; o[4] += r2.x; o[5] += r2.y; o[6] += r3.x; o[7] += r3.y;
    }
    reinterpret_cast<uint4*>(out)[i] = make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]), pack_bf16x2(o[6], o[7]));
  }
}

int check_shapes(const char* what, int T, int D, int S, long long ld_mod, const void* a, const void* b) {
  if (T <= 0 || S <= 0 || T % S != 0) return b200::fail(1500, "%s: T=%d must be a positive multiple of S=%d", what, T, S);
  if (D % 256 != 0 || D > 256 * MAXV) return b200::fail(1501, "%s: D=%d must be a multiple of 256 up to %d", what, D, 256 * MAXV);
  if (ld_mod % 8 != 0 || (((uintptr_t)a | (uintptr_t)b) & 15) != 0)
    return b200::fail(1502, "%s: modulation vectors must be 16-byte aligned with a pitch that is a multiple of 8", what);
  return 0;
}

}  // namespace

// x, y: bf16 [T, D]; shift / scale: bf16 rows of pitch ld_mod (sample b at row b); mean / rstd: fp32 [T].
B200_API int b200_ln_modulate_fwd(const void* x, const void* shift, const void* scale, long long ld_mod, void* y, float* mean,
                                  float* rstd, int T, int D, int S, float eps, void* stream) {
  if (int r = check_shapes("ln_modulate_fwd", T, D, S, ld_mod, shift, scale)) return r;
  ln_modulate_fwd_kernel<<<(T + 7) / 8, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)shift, (const __nv_bfloat16*)scale, ld_mod, (__nv_bfloat16*)y, mean, rstd,
      T, D, S, eps);
  b200::count_launch();
  return b200::check_launch("ln_modulate_fwd");
}

// dx: bf16 [T, D]; dscale / dshift: fp32 [T / S, D].
B200_API int b200_ln_modulate_bwd(const void* dy, const void* x, const void* scale, long long ld_mod, const float* mean,
                                  const float* rstd, void* dx, float* dscale, float* dshift, int T, int D, int S, void* stream) {
  if (int r = check_shapes("ln_modulate_bwd", T, D, S, ld_mod, scale, scale)) return r;
  ln_modulate_bwd_kernel<<<(T + 7) / 8, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)scale, ld_mod, mean, rstd, (__nv_bfloat16*)dx, T, D, S);
  sample_colsum_kernel<0><<<dim3((D / 2 + 127) / 128, T / S), 128, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, mean, rstd, dscale, dshift, D, S);
  b200::count_launch(2);
  return b200::check_launch("ln_modulate_bwd");
}

// out = res + y * gate[b]
B200_API int b200_gate_residual_fwd(const void* res, const void* y, const void* gate, long long ld_mod, void* out, int T, int D,
                                    int S, void* stream) {
  if (int r = check_shapes("gate_residual_fwd", T, D, S, ld_mod, gate, gate)) return r;
  const long long n8 = (long long)T * D / 8;
  const int grid = (int)((n8 + 255) / 256 < 148 * 16 ? (n8 + 255) / 256 : 148 * 16);
  gate_kernel<0><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)res, (const __nv_bfloat16*)y,
                                                         (const __nv_bfloat16*)gate, ld_mod, (__nv_bfloat16*)out, n8, D / 8, S);
  b200::count_launch();
  return b200::check_launch("gate_residual_fwd");
}

// dy = dout * gate[b];  dgate[b, :] = sum_s dout * y   (fp32 [T / S, D])
B200_API int b200_gate_residual_bwd(const void* dout, const void* y, const void* gate, long long ld_mod, void* dy, float* dgate,
                                    int T, int D, int S, void* stream) {
  if (int r = check_shapes("gate_residual_bwd", T, D, S, ld_mod, gate, gate)) return r;
  const long long n8 = (long long)T * D / 8;
  const int grid = (int)((n8 + 255) / 256 < 148 * 16 ? (n8 + 255) / 256 : 148 * 16);
  gate_kernel<1><<<grid, 256, 0, (cudaStream_t)stream>>>(nullptr, (const __nv_bfloat16*)dout, (const __nv_bfloat16*)gate, ld_mod,
                                                         (__nv_bfloat16*)dy, n8, D / 8, S);
  sample_colsum_kernel<1><<<dim3((D / 2 + 127) / 128, T / S), 128, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dout, (const __nv_bfloat16*)y, nullptr, nullptr, dgate, nullptr, D, S);
  b200::count_launch(2);
  return b200::check_launch("gate_residual_bwd");
}
