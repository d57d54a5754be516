// Fused vocabulary cross-entropy (forward + in-place logits gradient) and the fused AdamW /
// gradient-norm kernels.
//
// Cross-entropy: one CTA per token row; an online max / sum pass over the bf16 logits, then a
// second pass that overwrites the logits with (softmax - onehot) * grad_scale, so the [T, V]
// probability tensor is never materialised in fp32.  Stands in for the TE fused parallel
// cross-entropy the reference selects (small_llm_pretraining/primus/conf/
// llama3.1_8B-pretrain-fp4.yaml:104-105).
//
// AdamW: one launch over a flat parameter buffer (bf16 or fp32 weights, fp32 or bf16 gradient,
// fp32 moments), global-norm clip coefficient folded in from a device scalar so no host read
// sits between the norm and the update; the counterpart of the reference's single-launch dense
// Adam (generative_recommenders/ops/triton/dense_adam_fused.py) and of Primus' fused Adam with
// clip + bf16 write-back (small_llm_moe_pretraining/primus/config_MI355X_1x8x1_tp1pp1ep1_gbs32.sh:49-56).
#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int CE_NT = 512;

B200_DEVICE void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
B200_DEVICE void st8(__nv_bfloat16* p, const float (&f)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                            pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

__global__ void __launch_bounds__(CE_NT)
cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                     float* __restrict__ loss, float* __restrict__ lse_out, long long ld, int V, float grad_scale,
                     int write_grad, long long ignore_index) {
  __shared__ float red_m[CE_NT / 32], red_s[CE_NT / 32];
  __shared__ float sh_m, sh_lse;
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const int nvec = V / 8;
  float m = -INFINITY, s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += CE_NT) {
    float x[8];
    ld8(lr + v * 8, x);
    float mx = x[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) mx = fmaxf(mx, x[j]);
    const float nm = fmaxf(m, mx);
    float add = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) add += __expf(x[j] - nm);
    s = s * __expf(m - nm) + add;
    m = nm;
  }
  // combine (m, s) pairs across the CTA
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    m = nm;
  }
  if (l == 0) { red_m[w] = m; red_s[w] = s; }
  __syncthreads();
  if (w == 0) {
    m = (l < CE_NT / 32) ? red_m[l] : -INFINITY;
    s = (l < CE_NT / 32) ? red_s[l] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const float os = __shfl_xor_sync(0xffffffffu, s, o);
      const float nm = fmaxf(m, om);
      s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
      m = nm;
    }
    if (l == 0) { sh_m = m; sh_lse = m + __logf(s); }
  }
  __syncthreads();
  const float lse = sh_lse;
  const long long label = labels[row];
  const bool valid = (label != ignore_index) && label >= 0 && label < V;
  if (threadIdx.x == 0) {
    loss[row] = valid ? (lse - __bfloat162float(lr[label])) : 0.f;
    if (lse_out) lse_out[row] = lse;
  }
  if (!write_grad) return;
  __syncthreads();  // the label logit was read above before any thread overwrites it
  const float gs = valid ? grad_scale : 0.f;
  for (int v = threadIdx.x; v < nvec; v += CE_NT) {
    float x[8], g[8];
    ld8(lr + v * 8, x);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(x[j] - lse);
      if (valid && (long long)(v * 8 + j) == label) p -= 1.f;
      g[j] = p * gs;
    }
    st8(lr + v * 8, g);
  }
}

// ---------------------------------------------------------------------------------------
// sum of squares of a flat gradient buffer -> per-CTA partials -> fixed-order final sum
// ---------------------------------------------------------------------------------------
template <typename G>
__global__ void __launch_bounds__(256)
sumsq_partial_kernel(const G* __restrict__ g, long long n, float* __restrict__ partial) {
  __shared__ float red[8];
  float acc = 0.f;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
    float v;
    if constexpr (sizeof(G) == 2) v = __bfloat162float(g[i]); else v = g[i];
    acc += v * v;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    r = warp_sum(r);
    if (threadIdx.x == 0) partial[blockIdx.x] = r;
  }
}
// out[0] (+)= sum(partial); one CTA
__global__ void sumsq_final_kernel(const float* __restrict__ partial, int n, float* __restrict__ out, int accumulate) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += partial[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    r = warp_sum(r);
    if (threadIdx.x == 0) out[0] = accumulate ? out[0] + r : r;
  }
}

// ---------------------------------------------------------------------------------------
// AdamW over a flat buffer.  P: bf16 or fp32 weights; G: bf16 or fp32 grads; M: fp32 or bf16 moments
// (bf16 moments halve the optimizer state; the update itself is computed in fp32).
// If `master` is non-null it holds fp32 master weights and `p` receives the bf16 copy.
// clip: if sumsq != null, grads are scaled by min(1, max_norm / (sqrt(*sumsq) + 1e-6)).
// ---------------------------------------------------------------------------------------
struct AdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale, max_norm;
};
template <typename T> B200_DEVICE float to_f32(T x) {
  if constexpr (sizeof(T) == 2) return __bfloat162float(x); else return x;
}
template <typename T> B200_DEVICE T from_f32(float x) {
  if constexpr (sizeof(T) == 2) return __float2bfloat16_rn(x); else return x;
}
template <typename P, typename G, typename M>
__global__ void __launch_bounds__(256)
adamw_kernel(P* __restrict__ p, float* __restrict__ master, const G* __restrict__ g, M* __restrict__ m,
             M* __restrict__ v, long long n, AdamArgs a, const float* __restrict__ sumsq, int zero_grad,
             G* __restrict__ g_mut) {
  float scale = a.grad_scale;
  if (sumsq != nullptr && a.max_norm > 0.f) {
    const float norm = sqrtf(*sumsq) * a.grad_scale;
    const float c = a.max_norm / (norm + 1e-6f);
    if (c < 1.f) scale *= c;
  }
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
    float gv;
    if constexpr (sizeof(G) == 2) gv = __bfloat162float(g[i]); else gv = g[i];
    gv *= scale;
    float w;
    if (master != nullptr) w = master[i];
    else if constexpr (sizeof(P) == 2) w = __bfloat162float(p[i]);
    else w = p[i];
    const float mi = a.beta1 * to_f32<M>(m[i]) + (1.f - a.beta1) * gv;
    const float vi = a.beta2 * to_f32<M>(v[i]) + (1.f - a.beta2) * gv * gv;
    m[i] = from_f32<M>(mi);
    v[i] = from_f32<M>(vi);
    const float mhat = mi / a.bc1;
    const float vhat = vi / a.bc2;
    w = w * (1.f - a.lr * a.wd) - a.lr * mhat / (sqrtf(vhat) + a.eps);
    if (master != nullptr) master[i] = w;
    if constexpr (sizeof(P) == 2) p[i] = __float2bfloat16_rn(w); else p[i] = w;
    if (zero_grad) {
      if constexpr (sizeof(G) == 2) g_mut[i] = __float2bfloat16_rn(0.f); else g_mut[i] = 0.f;
    }
  }
}

// four elements per thread per iteration with 8 / 16-byte accesses (all segments of the flat
// optimizer buffers are 8-element aligned, so this is the path every training step takes)
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static B200_DEVICE void load(const float* p, float (&f)[4]) { float4 v = *reinterpret_cast<const float4*>(p); f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
  static B200_DEVICE void store(float* p, const float (&f)[4]) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Vec4<__nv_bfloat16> {
  static B200_DEVICE void load(const __nv_bfloat16* p, float (&f)[4]) {
    uint2 v = *reinterpret_cast<const uint2*>(p);
    float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  }
  static B200_DEVICE void store(__nv_bfloat16* p, const float (&f)[4]) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]));
  }
};
template <typename P, typename G, typename M>
__global__ void __launch_bounds__(256)
adamw_vec4_kernel(P* __restrict__ p, float* __restrict__ master, G* __restrict__ g, M* __restrict__ m,
                  M* __restrict__ v, long long n4, AdamArgs a, const float* __restrict__ sumsq, int zero_grad) {
  float scale = a.grad_scale;
  if (sumsq != nullptr && a.max_norm > 0.f) {
    const float norm = sqrtf(*sumsq) * a.grad_scale;
    const float c = a.max_norm / (norm + 1e-6f);
    if (c < 1.f) scale *= c;
  }
  const float inv_bc1 = 1.f / a.bc1, inv_bc2 = 1.f / a.bc2, decay = 1.f - a.lr * a.wd;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n4; i += (long long)gridDim.x * 256) {
    const long long o = i * 4;
    float gv[4], w[4], mi[4], vi[4];
    Vec4<G>::load(g + o, gv);
    if (master != nullptr) Vec4<float>::load(master + o, w); else Vec4<P>::load(p + o, w);
    Vec4<M>::load(m + o, mi);
    Vec4<M>::load(v + o, vi);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = gv[j] * scale;
      mi[j] = a.beta1 * mi[j] + (1.f - a.beta1) * gj;
      vi[j] = a.beta2 * vi[j] + (1.f - a.beta2) * gj * gj;
      w[j] = w[j] * decay - a.lr * (mi[j] * inv_bc1) / (sqrtf(vi[j] * inv_bc2) + a.eps);
      gv[j] = 0.f;
    }
    Vec4<M>::store(m + o, mi);
    Vec4<M>::store(v + o, vi);
    if (master != nullptr) Vec4<float>::store(master + o, w);
    Vec4<P>::store(p + o, w);
    if (zero_grad) Vec4<G>::store(g + o, gv);
  }
}

}  // namespace

B200_API int b200_cross_entropy(void* logits, const long long* labels, float* loss, float* lse, long long T,
                                long long ld, int V, float grad_scale, int write_grad, long long ignore_index,
                                void* stream) {
  if (V % 8 != 0 || ld % 8 != 0) return b200::fail(500, "cross_entropy: V=%d and pitch %lld must be multiples of 8", V, ld);
  if (T == 0) return 0;
  cross_entropy_kernel<<<(unsigned)T, CE_NT, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)logits, labels, loss, lse, ld, V,
                                                                        grad_scale, write_grad, ignore_index);
  b200::count_launch();
  return b200::check_launch("cross_entropy");
}

// Number of fp32 scratch elements b200_sumsq needs.
B200_API int b200_sumsq_scratch_elems() { return b200::sm_count() * 4; }

// out[0] (+)= sum(g^2).  g_is_bf16 selects the gradient type.  scratch: b200_sumsq_scratch_elems() floats.
B200_API int b200_sumsq(const void* g, long long n, int g_is_bf16, float* scratch, float* out, int accumulate,
                        void* stream) {
  int grid = b200::sm_count() * 4;
  if ((long long)grid * 256 > n) grid = (int)((n + 255) / 256);
  if (grid < 1) grid = 1;
  if (g_is_bf16) sumsq_partial_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)g, n, scratch);
  else sumsq_partial_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((const float*)g, n, scratch);
  sumsq_final_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(scratch, grid, out, accumulate);
  b200::count_launch(2);
  return b200::check_launch("sumsq");
}

template <typename M>
static int launch_adamw(void* p, int p_is_bf16, float* master, void* g, int g_is_bf16, M* m, M* v, long long n, float lr,
                        float beta1, float beta2, float eps, float wd, int step, float grad_scale, const float* sumsq,
                        float max_norm, int zero_grad, void* stream) {
  if (n == 0) return 0;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = wd;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2 = 1.f - powf(beta2, (float)step);
  a.grad_scale = grad_scale; a.max_norm = max_norm;
  using bf = __nv_bfloat16;
  cudaStream_t st = (cudaStream_t)stream;
  const long long cap = (long long)b200::sm_count() * 16;
  const uintptr_t all = (uintptr_t)p | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v | (uintptr_t)master;
  if ((all & 15) == 0 && (n & 3) == 0) {
    const long long n4 = n / 4, g4 = (n4 + 255) / 256;
    const int grid4 = (int)(g4 < cap ? g4 : cap);
    if (p_is_bf16 && g_is_bf16) adamw_vec4_kernel<bf, bf, M><<<grid4, 256, 0, st>>>((bf*)p, master, (bf*)g, m, v, n4, a, sumsq, zero_grad);
    else if (p_is_bf16) adamw_vec4_kernel<bf, float, M><<<grid4, 256, 0, st>>>((bf*)p, master, (float*)g, m, v, n4, a, sumsq, zero_grad);
    else if (g_is_bf16) adamw_vec4_kernel<float, bf, M><<<grid4, 256, 0, st>>>((float*)p, master, (bf*)g, m, v, n4, a, sumsq, zero_grad);
    else adamw_vec4_kernel<float, float, M><<<grid4, 256, 0, st>>>((float*)p, master, (float*)g, m, v, n4, a, sumsq, zero_grad);
    b200::count_launch();
    return b200::check_launch("adamw");
  }
  const long long g64 = (n + 255) / 256;
  const int grid = (int)(g64 < cap ? g64 : cap);
  if (p_is_bf16 && g_is_bf16) adamw_kernel<bf, bf, M><<<grid, 256, 0, st>>>((bf*)p, master, (const bf*)g, m, v, n, a, sumsq, zero_grad, (bf*)g);
  else if (p_is_bf16) adamw_kernel<bf, float, M><<<grid, 256, 0, st>>>((bf*)p, master, (const float*)g, m, v, n, a, sumsq, zero_grad, (float*)g);
  else if (g_is_bf16) adamw_kernel<float, bf, M><<<grid, 256, 0, st>>>((float*)p, master, (const bf*)g, m, v, n, a, sumsq, zero_grad, (bf*)g);
  else adamw_kernel<float, float, M><<<grid, 256, 0, st>>>((float*)p, master, (const float*)g, m, v, n, a, sumsq, zero_grad, (float*)g);
  b200::count_launch();
  return b200::check_launch("adamw");
}

B200_API int b200_adamw(void* p, int p_is_bf16, float* master, void* g, int g_is_bf16, float* m, float* v,
                        long long n, float lr, float beta1, float beta2, float eps, float wd, int step,
                        float grad_scale, const float* sumsq, float max_norm, int zero_grad, void* stream) {
  return launch_adamw<float>(p, p_is_bf16, master, g, g_is_bf16, m, v, n, lr, beta1, beta2, eps, wd, step, grad_scale, sumsq,
                             max_norm, zero_grad, stream);
}

// The same step with both moments stored in bf16.
B200_API int b200_adamw_bf16m(void* p, int p_is_bf16, float* master, void* g, int g_is_bf16, void* m, void* v,
                              long long n, float lr, float beta1, float beta2, float eps, float wd, int step,
                              float grad_scale, const float* sumsq, float max_norm, int zero_grad, void* stream) {
  return launch_adamw<__nv_bfloat16>(p, p_is_bf16, master, g, g_is_bf16, (__nv_bfloat16*)m, (__nv_bfloat16*)v, n, lr, beta1,
                                     beta2, eps, wd, step, grad_scale, sumsq, max_norm, zero_grad, stream);
}
