// ZeRO / FSDP step kernels over NVLink peer memory (symmetric buffers: every rank holds the full
// fp32 gradient buffer and the full bf16 parameter buffer of a bucket at the same offsets).
//
//   zero_reduce_scatter : the owner of a shard reads that shard from every rank's gradient buffer
//                         (P2P loads over NVLink, fixed rank order -> deterministic sum), scales by
//                         1/W, keeps the fp32 result locally and emits per-CTA partial sums of squares
//                         for clipping.  The gradient buffers are NOT cleared here: clearing the peers'
//                         copies would send as many bytes out over NVLink as the reduction reads in;
//                         every rank clears its own buffer locally after the step's last barrier.
//   zero_adamw_all_gather : AdamW on the local shard (clip coefficient from a device scalar) and
//                         the updated bf16 parameters stored straight into EVERY rank's parameter
//                         buffer (P2P stores): update and all-gather are one pass over the shard.
//
// NVLS variants (zero_reduce_scatter_mc, zero_adamw_all_gather_mc): when the symmetric buffers are bound to
// an NVLink multicast object, the owner reads its shard once through the multicast address with
// multimem.ld_reduce (the NVSwitch adds the W copies and returns one stream of bytes) and writes the
// updated parameters once with multimem.st (the switch delivers them to every rank): the same two
// kernels with the loops over ranks replaced by one switch-side operation, 1/W of the peer traffic at
// the owner's port.  mc_all_gather / mc_reduce_scatter_acc are the bare collectives of the sharded-
// parameter (ZeRO-3) mode: gather a bucket's parameter shards into a window, reduce a gradient window
// into the owner's fp32 shard accumulator.
//
// Together they replace reduce-scatter -> cast/scale -> AdamW -> all-gather, i.e. the Megatron
// distributed-optimizer path with copy-engine parameter gather that the reference configures
// (small_llm_pretraining/primus/config_MI355X_1x8x1.sh:104-105 rccl_sdma backends,
// llama3.1_8B-pretrain-fp4.yaml:55-61,101).  Cross-rank ordering (gradients final before the
// reduce, parameters landed before the next forward) is the caller's barrier on the same stream.
#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int MAXW = 16;

struct Ptrs {
  void* p[MAXW];
};

__global__ void __launch_bounds__(256)
zero_reduce_scatter_kernel(Ptrs grads, int W, int rank, long long lo, long long n4, float scale,
                           float* __restrict__ out, float* __restrict__ partial_sumsq, int clear_peers) {
  __shared__ float red[8];
  float acc = 0.f;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n4; i += (long long)gridDim.x * 256) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < W; ++r) {
      float4* src = reinterpret_cast<float4*>(reinterpret_cast<float*>(grads.p[r]) + lo) + i;
      const float4 g = *src;
      s.x += g.x; s.y += g.y; s.z += g.z; s.w += g.w;
      if (clear_peers && r != rank) *src = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    reinterpret_cast<float4*>(out)[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    r = warp_sum(r);
    if (threadIdx.x == 0 && partial_sumsq != nullptr) partial_sumsq[blockIdx.x] = r;
  }
}

struct AdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale, max_norm;
};

__global__ void __launch_bounds__(256)
zero_adamw_all_gather_kernel(Ptrs params, int W, int rank, long long lo, long long n4, float* __restrict__ g,
                             float* __restrict__ m, float* __restrict__ v, float* __restrict__ master, AdamArgs a,
                             const float* __restrict__ sumsq, int zero_grad) {
  float scale = a.grad_scale;
  if (sumsq != nullptr && a.max_norm > 0.f) {
    const float norm = sqrtf(*sumsq) * a.grad_scale;
    const float c = a.max_norm / (norm + 1e-6f);
    if (c < 1.f) scale *= c;
  }
  const float inv_bc1 = 1.f / a.bc1, inv_bc2 = 1.f / a.bc2, decay = 1.f - a.lr * a.wd;
  __nv_bfloat16* mine = reinterpret_cast<__nv_bfloat16*>(params.p[rank]) + lo;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n4; i += (long long)gridDim.x * 256) {
    const float4 gv = reinterpret_cast<float4*>(g)[i];
    float4 mi = reinterpret_cast<float4*>(m)[i], vi = reinterpret_cast<float4*>(v)[i];
    float w[4];
    if (master != nullptr) {
      const float4 mw = reinterpret_cast<float4*>(master)[i];
      w[0] = mw.x; w[1] = mw.y; w[2] = mw.z; w[3] = mw.w;
    } else {
      const uint2 pw = reinterpret_cast<const uint2*>(mine)[i];
      const float2 a0 = unpack_bf16x2(pw.x), a1 = unpack_bf16x2(pw.y);
      w[0] = a0.x; w[1] = a0.y; w[2] = a1.x; w[3] = a1.y;
    }
    const float gg[4] = {gv.x * scale, gv.y * scale, gv.z * scale, gv.w * scale};
    float mm[4] = {mi.x, mi.y, mi.z, mi.w}, vv[4] = {vi.x, vi.y, vi.z, vi.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gg[j];
      vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gg[j] * gg[j];
      w[j] = w[j] * decay - a.lr * (mm[j] * inv_bc1) / (sqrtf(vv[j] * inv_bc2) + a.eps);
    }
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (master != nullptr) reinterpret_cast<float4*>(master)[i] = make_float4(w[0], w[1], w[2], w[3]);
    if (zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    const uint2 packed = make_uint2(pack_bf16x2(w[0], w[1]), pack_bf16x2(w[2], w[3]));
    // the all-gather: the same 8 bytes to every rank's parameter buffer, own copy included
    for (int r = 0; r < W; ++r)
      reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + lo)[i] = packed;
  }
}

// ---- multicast (NVLS) forms -------------------------------------------------------------------
B200_DEVICE float4 mc_ld_reduce_f32x4(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
B200_DEVICE void mc_st_b32x4(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// out[i] (=|+=) scale * sum over ranks of grad[lo + i], through the multicast address of the gradient buffers
__global__ void __launch_bounds__(256)
zero_reduce_scatter_mc_kernel(const float* __restrict__ mc_grads, long long lo, long long n4, float scale,
                              float* __restrict__ out, int accumulate, float* __restrict__ partial_sumsq) {
  __shared__ float red[8];
  float acc = 0.f;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n4; i += (long long)gridDim.x * 256) {
    float4 s = mc_ld_reduce_f32x4(mc_grads + lo + 4 * i);
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    if (accumulate) {
      const float4 o = reinterpret_cast<const float4*>(out)[i];
      s.x += o.x; s.y += o.y; s.z += o.z; s.w += o.w;
    }
    reinterpret_cast<float4*>(out)[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    r = warp_sum(r);
    if (threadIdx.x == 0 && partial_sumsq != nullptr) partial_sumsq[blockIdx.x] = r;
  }
}

// every rank's window[lo .. lo + n) = this rank's shard (16 bytes per store through the multicast address)
__global__ void __launch_bounds__(256)
mc_all_gather_kernel(const uint4* __restrict__ shard, uint4* __restrict__ mc_dst, long long n16) {
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n16; i += (long long)gridDim.x * 256)
    mc_st_b32x4(mc_dst + i, shard[i]);
}

// AdamW on the local shard; updated bf16 parameters leave once through the multicast address of the
// parameter buffers (local_params: this rank's own copy of the shard, read when there is no fp32 master)
__global__ void __launch_bounds__(256)
zero_adamw_all_gather_mc_kernel(__nv_bfloat16* __restrict__ mc_params, const __nv_bfloat16* __restrict__ local_params,
                                long long n8, float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                                float* __restrict__ master, AdamArgs a, const float* __restrict__ sumsq, int zero_grad) {
  float scale = a.grad_scale;
  if (sumsq != nullptr && a.max_norm > 0.f) {
    const float norm = sqrtf(*sumsq) * a.grad_scale;
    const float c = a.max_norm / (norm + 1e-6f);
    if (c < 1.f) scale *= c;
  }
  const float inv_bc1 = 1.f / a.bc1, inv_bc2 = 1.f / a.bc2, decay = 1.f - a.lr * a.wd;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n8; i += (long long)gridDim.x * 256) {
    float w[8], gg[8], mm[8], vv[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float4 gv = reinterpret_cast<const float4*>(g)[2 * i + h];
      const float4 mi = reinterpret_cast<const float4*>(m)[2 * i + h], vi = reinterpret_cast<const float4*>(v)[2 * i + h];
      gg[4 * h] = gv.x * scale; gg[4 * h + 1] = gv.y * scale; gg[4 * h + 2] = gv.z * scale; gg[4 * h + 3] = gv.w * scale;
      mm[4 * h] = mi.x; mm[4 * h + 1] = mi.y; mm[4 * h + 2] = mi.z; mm[4 * h + 3] = mi.w;
      vv[4 * h] = vi.x; vv[4 * h + 1] = vi.y; vv[4 * h + 2] = vi.z; vv[4 * h + 3] = vi.w;
      if (master != nullptr) {
        const float4 mw = reinterpret_cast<const float4*>(master)[2 * i + h];
        w[4 * h] = mw.x; w[4 * h + 1] = mw.y; w[4 * h + 2] = mw.z; w[4 * h + 3] = mw.w;
      }
    }
    if (master == nullptr) {
      const uint4 pw = reinterpret_cast<const uint4*>(local_params)[i];
      const float2 a0 = unpack_bf16x2(pw.x), a1 = unpack_bf16x2(pw.y), a2 = unpack_bf16x2(pw.z), a3 = unpack_bf16x2(pw.w);
      w[0] = a0.x; w[1] = a0.y; w[2] = a1.x; w[3] = a1.y; w[4] = a2.x; w[5] = a2.y; w[6] = a3.x; w[7] = a3.y;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gg[j];
      vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gg[j] * gg[j];
      w[j] = w[j] * decay - a.lr * (mm[j] * inv_bc1) / (sqrtf(vv[j] * inv_bc2) + a.eps);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      reinterpret_cast<float4*>(m)[2 * i + h] = make_float4(mm[4 * h], mm[4 * h + 1], mm[4 * h + 2], mm[4 * h + 3]);
      reinterpret_cast<float4*>(v)[2 * i + h] = make_float4(vv[4 * h], vv[4 * h + 1], vv[4 * h + 2], vv[4 * h + 3]);
      if (master != nullptr)
        reinterpret_cast<float4*>(master)[2 * i + h] = make_float4(w[4 * h], w[4 * h + 1], w[4 * h + 2], w[4 * h + 3]);
      if (zero_grad) reinterpret_cast<float4*>(g)[2 * i + h] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    mc_st_b32x4(reinterpret_cast<uint4*>(mc_params) + i,
                make_uint4(pack_bf16x2(w[0], w[1]), pack_bf16x2(w[2], w[3]), pack_bf16x2(w[4], w[5]), pack_bf16x2(w[6], w[7])));
  }
}

}  // namespace

// mc_grads: multicast address of the bucket's fp32 gradient buffers (same offsets on every rank); the
// shard [lo, lo + n) is reduced in the switch into `out` (n fp32, local; += when accumulate).
B200_API int b200_zero_reduce_scatter_mc(const float* mc_grads, long long lo, long long n, float scale, float* out,
                                         int accumulate, float* partial_sumsq, void* stream) {
  if (mc_grads == nullptr) return b200::fail(1102, "zero_reduce_scatter_mc: no multicast address");
  if ((n & 3) || (lo & 3)) return b200::fail(1101, "zero_reduce_scatter_mc: shard bounds must be multiples of 4 elements");
  const int grid = b200::sm_count() * 4;
  if (partial_sumsq != nullptr) cudaMemsetAsync(partial_sumsq, 0, grid * sizeof(float), (cudaStream_t)stream);
  if (n == 0) return 0;
  zero_reduce_scatter_mc_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(mc_grads, lo, n / 4, scale, out, accumulate ? 1 : 0,
                                                                        partial_sumsq);
  b200::count_launch();
  return b200::check_launch("zero_reduce_scatter_mc");
}

// shard: n_bytes of this rank's data; mc_dst: multicast address of the destination window at this rank's offset.
B200_API int b200_mc_all_gather(const void* shard, void* mc_dst, long long n_bytes, void* stream) {
  if (mc_dst == nullptr) return b200::fail(1102, "mc_all_gather: no multicast address");
  if ((n_bytes & 15) || ((uintptr_t)shard & 15) || ((uintptr_t)mc_dst & 15))
    return b200::fail(1103, "mc_all_gather: shard size and addresses must be multiples of 16 bytes");
  if (n_bytes == 0) return 0;
  mc_all_gather_kernel<<<b200::sm_count() * 2, 256, 0, (cudaStream_t)stream>>>((const uint4*)shard, (uint4*)mc_dst, n_bytes / 16);
  b200::count_launch();
  return b200::check_launch("mc_all_gather");
}

// mc_params: multicast address of the bf16 parameter buffers at the shard's offset; local_params: this
// rank's copy of the shard; g/m/v/master: local shard (n elements, n a multiple of 8).
B200_API int b200_zero_adamw_all_gather_mc(void* mc_params, const void* local_params, long long n, float* g, float* m,
                                           float* v, float* master, float lr, float beta1, float beta2, float eps, float wd,
                                           int step, float grad_scale, const float* sumsq, float max_norm, int zero_grad,
                                           void* stream) {
  if (mc_params == nullptr) return b200::fail(1102, "zero_adamw_all_gather_mc: no multicast address");
  if ((n & 7) || ((uintptr_t)mc_params & 15) || ((uintptr_t)local_params & 15))
    return b200::fail(1101, "zero_adamw_all_gather_mc: shard bounds must be multiples of 8 elements");
  if (n == 0) return 0;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = wd;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2 = 1.f - powf(beta2, (float)step);
  a.grad_scale = grad_scale; a.max_norm = max_norm;
  zero_adamw_all_gather_mc_kernel<<<b200::sm_count() * 4, 256, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)mc_params, (const __nv_bfloat16*)local_params, n / 8, g, m, v, master, a, sumsq, zero_grad);
  b200::count_launch();
  return b200::check_launch("zero_adamw_all_gather_mc");
}

B200_API int b200_zero_grid() { return b200::sm_count() * 4; }

// grad_ptrs[r]: base of rank r's full fp32 gradient buffer of the bucket; the shard [lo, lo + n) is
// reduced into `out` (n fp32, local).  partial_sumsq needs b200_zero_grid() floats (may be null).
B200_API int b200_zero_reduce_scatter(const unsigned long long* grad_ptrs, int W, int rank, long long lo, long long n,
                                      float scale, float* out, float* partial_sumsq, void* stream) {
  if (W > MAXW) return b200::fail(1100, "zero_reduce_scatter: world %d exceeds %d", W, MAXW);
  if ((n & 3) || (lo & 3)) return b200::fail(1101, "zero_reduce_scatter: shard bounds must be multiples of 4 elements");
  Ptrs ptrs{};
  for (int r = 0; r < W; ++r) ptrs.p[r] = reinterpret_cast<void*>(grad_ptrs[r]);
  const int grid = b200::sm_count() * 4;
  if (partial_sumsq != nullptr) cudaMemsetAsync(partial_sumsq, 0, grid * sizeof(float), (cudaStream_t)stream);
  zero_reduce_scatter_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(ptrs, W, rank, lo, n / 4, scale, out, partial_sumsq, 0);
  b200::count_launch();
  return b200::check_launch("zero_reduce_scatter");
}

// param_ptrs[r]: base of rank r's full bf16 parameter buffer; g/m/v/master: local shard (n elements).
B200_API int b200_zero_adamw_all_gather(const unsigned long long* param_ptrs, int W, int rank, long long lo, long long n,
                                        float* g, float* m, float* v, float* master, float lr, float beta1, float beta2,
                                        float eps, float wd, int step, float grad_scale, const float* sumsq,
                                        float max_norm, int zero_grad, void* stream) {
  if (W > MAXW) return b200::fail(1100, "zero_adamw_all_gather: world %d exceeds %d", W, MAXW);
  if ((n & 3) || (lo & 3)) return b200::fail(1101, "zero_adamw_all_gather: shard bounds must be multiples of 4 elements");
  if (n == 0) return 0;
  Ptrs ptrs{};
  for (int r = 0; r < W; ++r) ptrs.p[r] = reinterpret_cast<void*>(param_ptrs[r]);
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = wd;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2 = 1.f - powf(beta2, (float)step);
  a.grad_scale = grad_scale; a.max_norm = max_norm;
  const int grid = b200::sm_count() * 4;
  zero_adamw_all_gather_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(ptrs, W, rank, lo, n / 4, g, m, v, master, a,
                                                                      sumsq, zero_grad);
  b200::count_launch();
  return b200::check_launch("zero_adamw_all_gather");
}
