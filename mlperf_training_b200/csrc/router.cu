// MoE router kernels: fp32 top-k with softmax over the selected logits ("softmax after top-k",
// no auxiliary loss, no capacity: small_llm_moe_pretraining/primus/conf/
// gpt_oss_20B-MXFP4-deosc-mlperf-pretrain.yaml:115-118,130-167), per-expert token counts, and the
// stable counting-sort permutation that groups (token, slot) pairs by expert with every expert's
// segment padded to a multiple of 128 rows (the GEMM's M tile) - all on the device, no host read.
#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int MAX_E = 256;
constexpr int MAX_K = 8;

// one thread per token
__global__ void router_topk_kernel(const float* __restrict__ logits, int T, int E, int K, int* __restrict__ idx,
                                   float* __restrict__ w, int* __restrict__ counts) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const float* row = logits + (long long)t * E;
  int sel[MAX_K];
  float val[MAX_K];
  unsigned long long used_lo = 0, used_hi = 0, used_2 = 0, used_3 = 0;
  for (int j = 0; j < K; ++j) {
    float best = -INFINITY;
    int bi = 0;
    for (int e = 0; e < E; ++e) {
      const unsigned long long bit = 1ull << (e & 63);
      const unsigned long long u = (e < 64) ? used_lo : (e < 128) ? used_hi : (e < 192) ? used_2 : used_3;
      if (u & bit) continue;
      const float v = row[e];
      if (v > best || (v == best && false)) { best = v; bi = e; }
    }
    sel[j] = bi;
    val[j] = best;
    const unsigned long long bit = 1ull << (bi & 63);
    if (bi < 64) used_lo |= bit; else if (bi < 128) used_hi |= bit; else if (bi < 192) used_2 |= bit; else used_3 |= bit;
  }
  float m = val[0], s = 0.f;
  for (int j = 0; j < K; ++j) { val[j] = __expf(val[j] - m); s += val[j]; }
  for (int j = 0; j < K; ++j) {
    idx[(long long)t * K + j] = sel[j];
    w[(long long)t * K + j] = val[j] / s;
    if (counts != nullptr) atomicAdd(&counts[sel[j]], 1);
  }
}

// Single-CTA planner: padded segment offsets from counts.  seg[e] = first row of expert e in the
// permuted buffer, seg[E] = total padded rows; tile_expert[i] = expert of 128-row tile i (or -1).
__global__ void router_plan_kernel(const int* __restrict__ counts, int E, int pad, int* __restrict__ seg,
                                   int* __restrict__ tile_expert, int max_tiles) {
  __shared__ int s_seg[MAX_E + 1];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      s_seg[e] = acc;
      acc += (counts[e] + pad - 1) / pad * pad;
    }
    s_seg[E] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) seg[e] = s_seg[e];
  for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) {
    const int row = i * pad;
    int ex = -1;
    for (int e = 0; e < E; ++e)
      if (row >= s_seg[e] && row < s_seg[e + 1]) { ex = e; break; }
    tile_expert[i] = ex;
  }
}

// Stable ranks: position of pair p = (t, j) inside its expert = number of earlier pairs (in
// flattened order) routed to the same expert.  One CTA per expert scans the flattened index list.
__global__ void router_rank_kernel(const int* __restrict__ idx, int n, const int* __restrict__ seg,
                                   int* __restrict__ dest) {
  const int e = blockIdx.x;
  __shared__ int warp_tot[32];
  __shared__ int base;
  if (threadIdx.x == 0) base = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int start = 0; start < n; start += blockDim.x) {
    const int p = start + threadIdx.x;
    const int hit = (p < n && idx[p] == e) ? 1 : 0;
    const unsigned ballot = __ballot_sync(0xffffffffu, hit);
    const int before = __popc(ballot & ((1u << lane) - 1));
    if (lane == 0) warp_tot[warp] = __popc(ballot);
    __syncthreads();
    int woff = 0;
    for (int i = 0; i < warp; ++i) woff += warp_tot[i];
    if (hit) dest[p] = seg[e] + base + woff + before;
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int i = 0; i < nw; ++i) tot += warp_tot[i];
      base += tot;
    }
    __syncthreads();
  }
}

// x_perm[dest[p], :] = x[p / K, :] (rows not written stay zero: the caller clears the buffer),
// optional per-row probability copy prob_perm[dest[p]] = w[p]
__global__ void permute_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ dest, int n, int K,
                                    int D, __nv_bfloat16* __restrict__ out, const float* __restrict__ w,
                                    float* __restrict__ w_out) {
  const int vpr = D / 8;
  const long long total = (long long)n * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int p = (int)(i / vpr), v = (int)(i % vpr);
    const int d = dest[p];
    *reinterpret_cast<uint4*>(out + (long long)d * D + v * 8) =
        *reinterpret_cast<const uint4*>(x + (long long)(p / K) * D + v * 8);
    if (v == 0 && w != nullptr) w_out[d] = w[p];
  }
}

// y[t, :] = sum_j scale_j * y_perm[dest[t*K + j], :]   (scale = 1 when w is null)
__global__ void unpermute_sum_kernel(const __nv_bfloat16* __restrict__ yp, const int* __restrict__ dest,
                                     const float* __restrict__ w, int T, int K, int D,
                                     __nv_bfloat16* __restrict__ y) {
  const int vpr = D / 8;
  const long long total = (long long)T * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / vpr), v = (int)(i % vpr);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < K; ++j) {
      const int d = dest[t * K + j];
      const float s = w ? w[t * K + j] : 1.f;
      const uint4 u = *reinterpret_cast<const uint4*>(yp + (long long)d * D + v * 8);
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), e = unpack_bf16x2(u.w);
      acc[0] += s * a.x; acc[1] += s * a.y; acc[2] += s * b.x; acc[3] += s * b.y;
      acc[4] += s * c.x; acc[5] += s * c.y; acc[6] += s * e.x; acc[7] += s * e.y;
    }
    *reinterpret_cast<uint4*>(y + (long long)t * D + v * 8) =
        make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                   pack_bf16x2(acc[6], acc[7]));
  }
}

// Backward of unpermute_sum, one warp per (token, slot) pair p:
//   gyp[dest[p], :] = w[p] * gy[p / K, :]        (rows no pair maps to keep their previous content)
//   gw[p]           = <gy[p / K, :], yp[dest[p], :]>
__global__ void unpermute_bwd_kernel(const __nv_bfloat16* __restrict__ gy, const __nv_bfloat16* __restrict__ yp,
                                     const int* __restrict__ dest, const float* __restrict__ w, long long pairs, int K,
                                     int D, __nv_bfloat16* __restrict__ gyp, float* __restrict__ gw) {
  const long long p = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (p >= pairs) return;
  const long long t = p / K;
  const long long row = dest[p];
  const float s = w ? w[p] : 1.f;
  const __nv_bfloat16* g = gy + t * D;
  const __nv_bfloat16* y = yp + row * D;
  __nv_bfloat16* o = gyp + row * D;
  float dot = 0.f;
  for (int v = lane; v < D / 8; v += 32) {
    const uint4 a = *reinterpret_cast<const uint4*>(g + v * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(y + v * 8);
    const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
    const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z), b3 = unpack_bf16x2(b.w);
    dot += a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y + a2.x * b2.x + a2.y * b2.y + a3.x * b3.x + a3.y * b3.y;
    *reinterpret_cast<uint4*>(o + v * 8) =
        make_uint4(pack_bf16x2(s * a0.x, s * a0.y), pack_bf16x2(s * a1.x, s * a1.y), pack_bf16x2(s * a2.x, s * a2.y),
                   pack_bf16x2(s * a3.x, s * a3.y));
  }
  dot = warp_sum(dot);
  if (lane == 0 && gw != nullptr) gw[p] = dot;
}

// rows of tiles that belong to no expert (tile_expert < 0) are cleared; 128 rows per tile
__global__ void zero_dead_tiles_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ tile_expert, int D) {
  const int tile = blockIdx.x;
  if (tile_expert[tile] >= 0) return;
  uint4* p = reinterpret_cast<uint4*>(buf + (long long)tile * 128 * D);
  const int n = 128 * D / 8;
  for (int i = threadIdx.x; i < n; i += blockDim.x) p[i] = make_uint4(0, 0, 0, 0);
}

}  // namespace

B200_API int b200_unpermute_bwd(const void* gy, const void* yp, const int* dest, const float* w, long long pairs, int K,
                                int D, void* gyp, float* gw, void* stream) {
  if (D % 8 != 0) return b200::fail(904, "unpermute_bwd: D=%d must be a multiple of 8", D);
  if (pairs <= 0) return 0;
  const long long threads = pairs * 32;
  unpermute_bwd_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gy, (const __nv_bfloat16*)yp, dest, w, pairs, K, D, (__nv_bfloat16*)gyp, gw);
  b200::count_launch();
  return b200::check_launch("unpermute_bwd");
}

B200_API int b200_zero_dead_tiles(void* buf, const int* tile_expert, int n_tiles, int D, void* stream) {
  if (D % 8 != 0) return b200::fail(905, "zero_dead_tiles: D=%d must be a multiple of 8", D);
  if (n_tiles <= 0) return 0;
  zero_dead_tiles_kernel<<<n_tiles, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)buf, tile_expert, D);
  b200::count_launch();
  return b200::check_launch("zero_dead_tiles");
}

B200_API int b200_router_topk(const float* logits, int T, int E, int K, int* idx, float* w, int* counts, void* stream) {
  if (E > MAX_E || K > MAX_K || K > E) return b200::fail(900, "router_topk: E=%d (max %d), K=%d (max %d)", E, MAX_E, K, MAX_K);
  if (T == 0) return 0;
  router_topk_kernel<<<(T + 127) / 128, 128, 0, (cudaStream_t)stream>>>(logits, T, E, K, idx, w, counts);
  b200::count_launch();
  return b200::check_launch("router_topk");
}

// counts [E] -> seg [E+1] (padded to `pad` rows), tile_expert [max_tiles], dest [n] (n = T*K pairs)
B200_API int b200_router_plan(const int* counts, const int* idx, int n, int E, int pad, int* seg, int* tile_expert,
                              int max_tiles, int* dest, void* stream) {
  if (E > MAX_E) return b200::fail(901, "router_plan: E=%d exceeds %d", E, MAX_E);
  router_plan_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(counts, E, pad, seg, tile_expert, max_tiles);
  router_rank_kernel<<<E, 1024, 0, (cudaStream_t)stream>>>(idx, n, seg, dest);
  b200::count_launch(2);
  return b200::check_launch("router_plan");
}

B200_API int b200_permute_rows(const void* x, const int* dest, int n, int K, int D, void* out, const float* w,
                               float* w_out, void* stream) {
  if (D % 8 != 0) return b200::fail(902, "permute_rows: D=%d must be a multiple of 8", D);
  if (n == 0) return 0;
  long long work = (long long)n * (D / 8);
  int grid = (int)((work + 255) / 256 < (long long)b200::sm_count() * 16 ? (work + 255) / 256 : (long long)b200::sm_count() * 16);
  permute_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, dest, n, K, D, (__nv_bfloat16*)out, w, w_out);
  b200::count_launch();
  return b200::check_launch("permute_rows");
}

B200_API int b200_unpermute_sum(const void* yp, const int* dest, const float* w, int T, int K, int D, void* y,
                                void* stream) {
  if (D % 8 != 0) return b200::fail(903, "unpermute_sum: D=%d must be a multiple of 8", D);
  if (T == 0) return 0;
  long long work = (long long)T * (D / 8);
  int grid = (int)((work + 255) / 256 < (long long)b200::sm_count() * 16 ? (work + 255) / 256 : (long long)b200::sm_count() * 16);
  unpermute_sum_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)yp, dest, w, T, K, D, (__nv_bfloat16*)y);
  b200::count_launch();
  return b200::check_launch("unpermute_sum");
}
