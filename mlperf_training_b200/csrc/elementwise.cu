// Bandwidth-bound elementwise kernels (bf16 storage, fp32 math, 16-byte accesses):
// rotary embedding on a packed QKV buffer, SwiGLU / GELU and their backward, embedding row
// gather and its scatter-add backward, bf16 residual add, fp32 accumulate.
//
// Reference counterparts: the fused single-QKV RoPE and fused SwiGLU selected by
// small_llm_pretraining/primus/conf/llama3.1_8B-pretrain-fp4.yaml:62,122-123 (Primus-Turbo),
// generative_recommenders/ops/triton/triton_swiglu.py (_swiglu_fwd_kernel) and the dedup-expand
// row gather of generative_recommenders/dlrm_v4/train/ec_expand_gather.py.
#include "common.cuh"
#include "runtime.h"

namespace {

B200_DEVICE void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
B200_DEVICE void st8(__nv_bfloat16* p, const float (&f)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                            pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

// ---------------------------------------------------------------------------------------
// RoPE ("rotate-half" convention: pairs are (i, i + hd/2)), in place on rows of
// [T, row_stride] holding n_rot_heads heads of size hd starting at column col0.
// cos/sin tables are fp32 [S, hd/2]; position of token t is pos[t] if given, else t % S.
// sign = +1 forward, -1 backward (transpose of the rotation).
// ---------------------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ buf, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, const int* __restrict__ pos, long long T, int S,
                            long long row_stride, int col0, int n_heads, int hd, float sign) {
  const int half = hd / 2;
  const int vec_per_head = half / 8;  // each work item rotates 8 pairs
  const long long total = T * n_heads * vec_per_head;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_head);
    const long long r = i / vec_per_head;
    const int h = (int)(r % n_heads);
    const long long t = r / n_heads;
    const int p = pos ? pos[t] : (int)(t % S);
    __nv_bfloat16* base = buf + t * row_stride + col0 + h * hd + v * 8;
    float x1[8], x2[8], o1[8], o2[8];
    ld8(base, x1);
    ld8(base + half, x2);
    const float4* c4 = reinterpret_cast<const float4*>(cos_t + (long long)p * half + v * 8);
    const float4* s4 = reinterpret_cast<const float4*>(sin_t + (long long)p * half + v * 8);
    float c[8], s[8];
    float4 ca = c4[0], cb = c4[1], sa = s4[0], sb = s4[1];
    c[0] = ca.x; c[1] = ca.y; c[2] = ca.z; c[3] = ca.w; c[4] = cb.x; c[5] = cb.y; c[6] = cb.z; c[7] = cb.w;
    s[0] = sa.x; s[1] = sa.y; s[2] = sa.z; s[3] = sa.w; s[4] = sb.x; s[5] = sb.y; s[6] = sb.z; s[7] = sb.w;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sj = s[j] * sign;
      o1[j] = x1[j] * c[j] - x2[j] * sj;
      o2[j] = x2[j] * c[j] + x1[j] * sj;
    }
    st8(base, o1);
    st8(base + half, o2);
  }
}

// ---------------------------------------------------------------------------------------
// SwiGLU: a[t, f] = silu(gu[t, f]) * gu[t, F + f]  (gate columns first, up columns second)
// ---------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ a, long long T,
                                  int F) {
  const int vpr = F / 8;
  const long long total = T * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpr;
    const int v = (int)(i % vpr);
    float g[8], u[8], o[8];
    ld8(gu + t * 2 * F + v * 8, g);
    ld8(gu + t * 2 * F + F + v * 8, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    st8(a + t * F + v * 8, o);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ da, const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int F) {
  const int vpr = F / 8;
  const long long total = T * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpr;
    const int v = (int)(i % vpr);
    float g[8], u[8], d[8], dg[8], du[8];
    ld8(gu + t * 2 * F + v * 8, g);
    ld8(gu + t * 2 * F + F + v * 8, u);
    ld8(da + t * F + v * 8, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sg;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * sg * (1.f + g[j] * (1.f - sg));
    }
    st8(dgu + t * 2 * F + v * 8, dg);
    st8(dgu + t * 2 * F + F + v * 8, du);
  }
}

// GELU (tanh approximation), used by the MMDiT MLPs
B200_DEVICE float gelu_tanh(float x) {
  const float k = 0.7978845608028654f;
  return 0.5f * x * (1.f + tanhf(k * (x + 0.044715f * x * x * x)));
}
B200_DEVICE float gelu_tanh_grad(float x) {
  const float k = 0.7978845608028654f;
  const float th = tanhf(k * (x + 0.044715f * x * x * x));
  return 0.5f * (1.f + th) + 0.5f * x * (1.f - th * th) * k * (1.f + 3.f * 0.044715f * x * x);
}
__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float a[8], o[8];
    ld8(x + i * 8, a);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = gelu_tanh(a[j]);
    st8(y + i * 8, o);
  }
}
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                __nv_bfloat16* __restrict__ dx, long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float a[8], d[8], o[8];
    ld8(x + i * 8, a);
    ld8(dy + i * 8, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = d[j] * gelu_tanh_grad(a[j]);
    st8(dx + i * 8, o);
  }
}

// ---------------------------------------------------------------------------------------
// Embedding gather: out[t, :] = table[ids[t], :] (bf16, D % 8 == 0); ids < 0 give zero rows.
// ---------------------------------------------------------------------------------------
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ table, const long long* __restrict__ ids,
                                   __nv_bfloat16* __restrict__ out, long long T, int D, long long rows, int* status) {
  const int vpr = D / 8;
  const long long total = T * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpr;
    const int v = (int)(i % vpr);
    const long long id = ids[t];
    uint4 u = make_uint4(0, 0, 0, 0);
    if (id >= 0 && id < rows) u = *reinterpret_cast<const uint4*>(table + id * D + v * 8);
    else if (v == 0) B200_BOUNDS_REPORT(status, 401);
    *reinterpret_cast<uint4*>(out + t * D + v * 8) = u;
  }
}
// grad_table[ids[t], :] += dy[t, :]  (fp32 atomics; used for the vocabulary embedding)
__global__ void scatter_add_rows_kernel(const __nv_bfloat16* __restrict__ dy, const long long* __restrict__ ids,
                                        float* __restrict__ grad, long long T, int D, long long rows, int* status) {
  const int vpr = D / 8;
  const long long total = T * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpr;
    const int v = (int)(i % vpr);
    const long long id = ids[t];
    if (id < 0 || id >= rows) {
      if (v == 0) B200_BOUNDS_REPORT(status, 402);
      continue;
    }
    float d[8];
    ld8(dy + t * D + v * 8, d);
    float* g = grad + id * D + v * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(g + j, d[j]);
  }
}

// y = a + b (bf16)
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ y, long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float x[8], z[8];
    ld8(a + i * 8, x);
    ld8(b + i * 8, z);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += z[j];
    st8(y + i * 8, x);
  }
}
// acc(fp32) += src(bf16)
__global__ void accum_f32_bf16_kernel(float* __restrict__ acc, const __nv_bfloat16* __restrict__ src, long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float x[8];
    ld8(src + i * 8, x);
    float4* a4 = reinterpret_cast<float4*>(acc + i * 8);
    float4 p = a4[0], q = a4[1];
    p.x += x[0]; p.y += x[1]; p.z += x[2]; p.w += x[3];
    q.x += x[4]; q.y += x[5]; q.z += x[6]; q.w += x[7];
    a4[0] = p; a4[1] = q;
  }
}

inline int grid_for(long long work, int threads) {
  long long g = (work + threads - 1) / threads;
  long long cap = (long long)b200::sm_count() * 16;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace

B200_API int b200_rope(void* buf, const float* cos_t, const float* sin_t, const int* pos, long long T, int S,
                       long long row_stride, int col0, int n_heads, int hd, int backward, void* stream) {
  if (hd % 16 != 0 || row_stride % 8 != 0 || col0 % 8 != 0)
    return b200::fail(400, "rope: head dim %d must be a multiple of 16, stride/offset multiples of 8", hd);
  const long long work = T * n_heads * (hd / 16);
  if (work == 0) return 0;
  rope_kernel<<<grid_for(work, 256), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)buf, cos_t, sin_t, pos, T, S,
                                                                     row_stride, col0, n_heads, hd,
                                                                     backward ? -1.f : 1.f);
  b200::count_launch();
  return b200::check_launch("rope");
}
B200_API int b200_swiglu_fwd(const void* gu, void* a, long long T, int F, void* stream) {
  if (F % 8 != 0) return b200::fail(401, "swiglu: F=%d must be a multiple of 8", F);
  if (T == 0) return 0;
  swiglu_fwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gu,
                                                                                 (__nv_bfloat16*)a, T, F);
  b200::count_launch();
  return b200::check_launch("swiglu_fwd");
}
B200_API int b200_swiglu_bwd(const void* da, const void* gu, void* dgu, long long T, int F, void* stream) {
  if (F % 8 != 0) return b200::fail(401, "swiglu: F=%d must be a multiple of 8", F);
  if (T == 0) return 0;
  swiglu_bwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)da, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, T, F);
  b200::count_launch();
  return b200::check_launch("swiglu_bwd");
}
B200_API int b200_gelu_fwd(const void* x, void* y, long long n, void* stream) {
  if (n % 8 != 0) return b200::fail(402, "gelu: n=%lld must be a multiple of 8", n);
  if (n == 0) return 0;
  gelu_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n / 8);
  b200::count_launch();
  return b200::check_launch("gelu_fwd");
}
B200_API int b200_gelu_bwd(const void* dy, const void* x, void* dx, long long n, void* stream) {
  if (n % 8 != 0) return b200::fail(402, "gelu: n=%lld must be a multiple of 8", n);
  if (n == 0) return 0;
  gelu_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                                         (__nv_bfloat16*)dx, n / 8);
  b200::count_launch();
  return b200::check_launch("gelu_bwd");
}
B200_API int b200_gather_rows(const void* table, const long long* ids, void* out, long long T, int D, long long rows,
                              void* stream) {
  if (D % 8 != 0) return b200::fail(403, "gather_rows: D=%d must be a multiple of 8", D);
  if (T == 0) return 0;
  gather_rows_kernel<<<grid_for(T * (D / 8), 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)table, ids,
                                                                                  (__nv_bfloat16*)out, T, D, rows, b200::status_ptr());
  b200::count_launch();
  return b200::check_launch("gather_rows");
}
B200_API int b200_scatter_add_rows(const void* dy, const long long* ids, float* grad, long long T, int D,
                                   long long rows, void* stream) {
  if (D % 8 != 0) return b200::fail(403, "scatter_add_rows: D=%d must be a multiple of 8", D);
  if (T == 0) return 0;
  scatter_add_rows_kernel<<<grid_for(T * (D / 8), 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dy, ids,
                                                                                       grad, T, D, rows, b200::status_ptr());
  b200::count_launch();
  return b200::check_launch("scatter_add_rows");
}
B200_API int b200_add_bf16(const void* a, const void* b, void* y, long long n, void* stream) {
  if (n % 8 != 0) return b200::fail(404, "add_bf16: n=%lld must be a multiple of 8", n);
  if (n == 0) return 0;
  add_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                                         (__nv_bfloat16*)y, n / 8);
  b200::count_launch();
  return b200::check_launch("add_bf16");
}
B200_API int b200_accum_f32_bf16(float* acc, const void* src, long long n, void* stream) {
  if (n % 8 != 0) return b200::fail(405, "accum: n=%lld must be a multiple of 8", n);
  if (n == 0) return 0;
  accum_f32_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(acc, (const __nv_bfloat16*)src, n / 8);
  b200::count_launch();
  return b200::check_launch("accum_f32_bf16");
}
