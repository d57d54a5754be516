// Jagged HSTU attention forward for sm_100a (pointwise SiLU attention, no softmax):
//
//   O[i] = sum_j  silu(alpha * q_i . k_j) / N * mask(i, j) * v_j        per (sequence, head)
//
// over variable-length sequences stored back to back ([L, H, D] with row offsets), N the static
// maximum sequence length.  Because there is no running maximum or normaliser, key tiles are
// independent and nothing is saved for the backward pass.
//
// Mask (positions inside a sequence; C contextual tokens first, the last n_targets are targets):
//   id(p) = clamp(p - C + 1, 0, max_id),  max_id = len - n_targets - max(C - 1, 0)
//   visible(i, j) = j < len and (i == j or id(i) > id(j) or (id(i) == 0 and j < len - n_targets))
// i.e. causal over the history, every target sees the whole history and itself but no other
// target, contextual rows see the whole history.
//
// Same engine as attention_fwd.cu: one CTA per (sequence, head, pair of 128-query tiles), TMA
// loads, S = Q K^T and O += P V on tcgen05 with accumulators in TMEM, P written back into the S
// columns as bf16 and consumed from TMEM, ping-pong over the two query tiles.  The grid is sized
// by the maximum length; blocks past their sequence's end exit immediately.
//
// FP8 variant (head dim 128): Q, K, V arrive as e4m3 codes with one dequantisation factor per tensor,
// S = Q K^T and O += P V run as kind::f8f6f4 MMAs (twice the bf16 rate, half the operand bytes), and the
// activation silu(alpha s) is written back to the S columns as e4m3 (four keys per 32-bit column, the
// 1 / N factor and V's factor applied to O in the epilogue so that P keeps e4m3's range).  V stays in
// its row layout [keys][head dim] and is consumed as an MN-major operand.  This is the forward of the
// reference's production path (generative_recommenders/ops/flydsl/hstu_fwd.py:150, e4m3 forward).
//
// Math oracle: generative_recommenders/ops/pytorch/pt_hstu_attention.py:33-84,130-187; the
// reference's production kernels are generative_recommenders/ops/flydsl/hstu_fwd.py and
// generative_recommenders/ops/triton/triton_hstu_attention.py (_hstu_attn_fwd).
#include <cuda_fp8.h>

#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int NTHREADS = 320;  // warps 0-3 / 4-7: tile 0 / 1 activation + epilogue; warp 8: TMA; warp 9: MMA

struct HstuParams {
  int max_len;              // N: static maximum sequence length (the 1/N factor and the grid size)
  int H;
  int contextual;           // C
  float alpha;              // 1 / sqrt(d_qk)
  const int* offsets;       // [B + 1] row offsets of the sequences
  const int* num_targets;   // [B] or null
  __nv_bfloat16* out;       // [L, H, HD]
  long long out_row;        // elements between consecutive rows of out
  const float* inv_q;       // FP8 variant: dequantisation factors of Q, K, V (device scalars)
  const float* inv_k;
  const float* inv_v;
  int* status;
};

B200_DEVICE uint32_t pack4_e4m3(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

B200_DEVICE float tanh_approx(float x) {
  float y;
  asm volatile("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int HD, bool F8>
struct Smem {
  static constexpr int ES = F8 ? 1 : 2;               // bytes per operand element
  static constexpr int Q_TILE = BQ * HD * ES;
  static constexpr int KV_BYTES = BKV * HD * ES;
  static constexpr int TOTAL = 2 * Q_TILE + 4 * KV_BYTES + 1024 + 256;
};

template <int HD, bool F8>
__global__ void __launch_bounds__(NTHREADS, 1)
hstu_attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV,
                const HstuParams p) {
  using SM = Smem<HD, F8>;
  constexpr int EPB = 128 / SM::ES;   // elements per 128-byte block of a head row
  constexpr int NB = HD / EPB;        // 128-byte blocks per head row
  static_assert(!F8 || HD == 128, "the 8-bit variant is built for head dim 128");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                       // two tiles
  uint8_t* sK = sQ + 2 * SM::Q_TILE;        // two stages
  uint8_t* sV = sK + 2 * SM::KV_BYTES;      // two stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * SM::KV_BYTES);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // 2 (per query tile)
  uint64_t* p_full = bars + 11;     // 2 (per query tile, 4 arrivals)
  uint64_t* o_done = bars + 13;     // 2 (per query tile)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_pairs = (p.max_len + 2 * BQ - 1) / (2 * BQ);
  const int pair = num_pairs - 1 - (int)blockIdx.x;  // heaviest (latest) query tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int row_base = p.offsets[b];
  const int len = p.offsets[b + 1] - row_base;
  const int q0 = pair * 2 * BQ;
  if (q0 >= len) return;  // grid is sized by the maximum length: blocks past this sequence leave at once
  const int n_tgt = p.num_targets ? p.num_targets[b] : 0;
  const int ctx = p.contextual;
  const int hist_end = len - n_tgt;                   // first target position
  const int max_id = hist_end - (ctx > 0 ? ctx - 1 : 0);

  const int j_max = (len + BKV - 1) / BKV - 1;
  const int j_lo = 0;
  int n_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qt0 = q0 + t * BQ;
    int j_hi = (qt0 + BQ - 1) / BKV;
    if (ctx > 0 && qt0 < ctx) j_hi = j_max;           // contextual rows see every history column
    if (j_hi > j_max) j_hi = j_max;
    n_t[t] = (qt0 < len) ? (j_hi - j_lo + 1) : 0;
  }
  const int n_max = n_t[0] > n_t[1] ? n_t[0] : n_t[1];

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4); mbar_init(&o_done[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) { tmem_alloc(tmem_holder, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;


  if (warp == 8) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && n_max > 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, 2 * SM::Q_TILE);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int i = 0; i < NB; ++i)
          tma_load_3d(sQ + t * SM::Q_TILE + i * (BQ * 128), &tmQ, q_full, i * EPB, h, row_base + q0 + t * BQ);
      bool ok = true;
      for (int n = 0; n < n_max && ok; ++n) {
        const int j = j_lo + n, st = n & 1;
        const uint32_t ph = (n >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, 40)) { ok = false; break; }
        mbar_expect_tx(&k_full[st], SM::KV_BYTES);
#pragma unroll
        for (int i = 0; i < NB; ++i)
          tma_load_3d(sK + st * SM::KV_BYTES + i * (BKV * 128), &tmK, &k_full[st], i * EPB, h, row_base + j * BKV);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status, 41)) { ok = false; break; }
        mbar_expect_tx(&v_full[st], SM::KV_BYTES);
#pragma unroll
        for (int i = 0; i < NB; ++i)
          tma_load_3d(sV + st * SM::KV_BYTES + i * (BKV * 128), &tmV, &v_full[st], i * EPB, h, row_base + j * BKV);
      }
    }
  } else if (warp == 9) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && n_max > 0) {
      // formats: bf16 (code 1 of kind::f16) or e4m3 (code 0 of kind::f8f6f4)
      const uint32_t idesc_s = umma_idesc(F8 ? 0 : 1, F8 ? 0 : 1, 0, 0, BQ, BKV);  // Q (K-major) x K (K-major)
      const uint32_t idesc_o = umma_idesc(F8 ? 0 : 1, F8 ? 0 : 1, 0, 1, BQ, HD);   // P (TMEM)    x V (MN-major)
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 50);
      int k_ready = -1, v_ready = -1;  // last key tile index whose full barrier has been observed
      // S_t(n) = Q_t K(n)^T into the S columns of tile t
      auto issue_s = [&](int t, int n) -> bool {
        const int st = n & 1;
        if (k_ready < n) {
          if (!mbar_wait(&k_full[st], (n >> 1) & 1, abort_flag, p.status, 51)) return false;
          k_ready = n;
        }
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ + t * SM::Q_TILE), ka = smem_u32(sK + st * SM::KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < HD * SM::ES / 32; ++kk) {       // one MMA consumes 32 bytes of the head row
          const uint32_t o = (kk / 4) * (BQ * 128) + (kk % 4) * 32;
          if constexpr (F8)
            tc_mma_f8_ss(tmem_base + t * 128, umma_desc_sw128(qa + o, 16, 1024), umma_desc_sw128(ka + o, 16, 1024),
                         idesc_s, kk > 0 ? 1u : 0u);
          else
            tc_mma_f16_ss(tmem_base + t * 128, umma_desc_sw128(qa + o, 16, 1024), umma_desc_sw128(ka + o, 16, 1024),
                          idesc_s, kk > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[t]);
        // the last tile that reads K(n) frees its stage
        const bool last_user = (t == 1) || !(n < n_t[1]);
        if (last_user) tc_commit(&k_empty[st]);
        return true;
      };
      for (int t = 0; t < 2 && ok; ++t)
        if (n_t[t] > 0) ok = issue_s(t, 0);
      for (int n = 0; n < n_max && ok; ++n) {
        const int st = n & 1;
        for (int t = 0; t < 2 && ok; ++t) {
          if (n >= n_t[t]) continue;
          if (!mbar_wait(&p_full[t], n & 1, abort_flag, p.status, 53)) { ok = false; break; }
          if (v_ready < n) {
            if (!mbar_wait(&v_full[st], (n >> 1) & 1, abort_flag, p.status, 54)) { ok = false; break; }
            v_ready = n;
          }
          tc_fence_after();
          const uint32_t va = smem_u32(sV + st * SM::KV_BYTES);
          if constexpr (F8) {
#pragma unroll
            for (int kk = 0; kk < BKV / 32; ++kk) {
              // A = P_t in TMEM: 32 e4m3 keys = 8 columns per step; B = V: 32 key rows of 128 bytes (one block: HD = 128)
              tc_mma_f8_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + kk * 8,
                           umma_desc_sw128(va + kk * (32 * 128), BKV * 128, 1024), idesc_o, (n > 0 || kk > 0) ? 1u : 0u);
            }
          } else {
#pragma unroll
            for (int kk = 0; kk < BKV / 16; ++kk) {
              // A = P_t in TMEM: 16 bf16 keys = 8 columns per step; B = V: 16 key rows of 128 bytes
              tc_mma_f16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + kk * 8,
                            umma_desc_sw128(va + kk * (16 * 128), BKV * 128, 1024), idesc_o, (n > 0 || kk > 0) ? 1u : 0u);
            }
          }
          tc_commit(&o_done[t]);
          const bool last_user = (t == 1) || !(n < n_t[1]);
          if (last_user) tc_commit(&v_empty[st]);
          if (n + 1 < n_t[t]) ok = issue_s(t, n + 1);
        }
      }
    }
  } else if (warp < 8) {
    // ------------------------------ SiLU activation + epilogue (one warpgroup per query tile) ------
    const int t = warp >> 2;
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int qt0 = q0 + t * BQ;
    const int q_pos = qt0 + r;
    const uint32_t lane_base = uint32_t(q * 32) << 16;
    const uint32_t ts = tmem_base + lane_base + t * 128;
    const uint32_t to = tmem_base + lane_base + 256 + t * 128;
    const int my_n = n_t[t];
    const int q_id = min(max(q_pos - ctx + (ctx > 0 ? 1 : 0), 0), max_id);
    const bool plain = (n_tgt == 0 && ctx == 0);
    // 8-bit: S carries the factors of Q and K; P is stored without 1 / N (e4m3 range), O takes it with V's factor
    const float half_alpha = F8 ? 0.5f * p.alpha * (*p.inv_q) * (*p.inv_k) : 0.5f * p.alpha;
    const float inv_n = F8 ? 1.0f : 1.0f / (float)p.max_len;
    const float out_scale = F8 ? (*p.inv_v) / (float)p.max_len : 1.0f;
    bool ok = true;
    for (int n = 0; n < my_n && ok; ++n) {
      const int kv0 = (j_lo + n) * BKV;
      if (!mbar_wait(&s_full[t], n & 1, abort_flag, p.status, 170)) { ok = false; break; }
      tc_fence_after();
      // tiles strictly below the diagonal and inside the sequence need no element mask
      // (with targets / contextual tokens: ids grow with the position, so every pair of the tile is visible when its
      // first query is later than its last key)
      const int first_q_id = min(max(qt0 - ctx + (ctx > 0 ? 1 : 0), 0), max_id);
      const int last_k_id = min(max(kv0 + BKV - 1 - ctx + (ctx > 0 ? 1 : 0), 0), max_id);
      const bool inside = (kv0 + BKV <= len) && (qt0 + BQ <= len);
      const bool need_mask = plain ? ((kv0 + BKV - 1 > qt0) || !inside) : !(inside && first_q_id > last_k_id);
#pragma unroll 1
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(ts + c * 32, v);
        tc_wait_ld();
        uint32_t pk[16];
        float xf[F8 ? 32 : 1];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          // silu(a x) / N = (a x / 2)(1 + tanh(a x / 2)) / N
          const float h0 = __uint_as_float(v[2 * i]) * half_alpha, h1 = __uint_as_float(v[2 * i + 1]) * half_alpha;
          float x0 = h0 * (1.f + tanh_approx(h0)) * inv_n, x1 = h1 * (1.f + tanh_approx(h1)) * inv_n;
          if (need_mask) {
            const int kp = kv0 + c * 32 + 2 * i;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int kpe = kp + e;
              bool vis;
              if (plain) vis = kpe <= q_pos;
              else {
                const int k_id = min(max(kpe - ctx + (ctx > 0 ? 1 : 0), 0), max_id);
                vis = (kpe == q_pos) || (q_id > k_id) || (ctx > 0 && q_id == 0 && kpe < hist_end);
              }
              vis = vis && kpe < len && q_pos < len;
              if (!vis) { if (e == 0) x0 = 0.f; else x1 = 0.f; }
            }
          }
          if constexpr (F8) {
            xf[2 * i] = x0; xf[2 * i + 1] = x1;
          } else {
            pk[i] = pack_bf16x2(x0, x1);
          }
        }
        if constexpr (F8) {
          uint32_t p8[8];                                  // keys 4 j .. 4 j + 3 of the chunk in column j
#pragma unroll
          for (int j = 0; j < 8; ++j) p8[j] = pack4_e4m3(xf[4 * j], xf[4 * j + 1], xf[4 * j + 2], xf[4 * j + 3]);
          tmem_st_32x32b_x8(ts + c * 8, p8);
        } else {
          tmem_st_32x32b_x16(ts + c * 16, pk);
        }
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
    }
    // ------------------------------ epilogue: guarded row stores (rows past the sequence end are not written)
    if (ok && my_n > 0) ok = mbar_wait(&o_done[t], (my_n - 1) & 1, abort_flag, p.status, 171);
    if (ok && my_n > 0) {
      tc_fence_after();
      __nv_bfloat16* orow = p.out + (long long)(row_base + q_pos) * p.out_row + h * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(to + c * 32, v);
        tc_wait_ld();
        if (q_pos < len) {
#pragma unroll
          for (int g = 0; g < 4; ++g)
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = make_uint4(
                pack_bf16x2(__uint_as_float(v[8 * g]) * out_scale, __uint_as_float(v[8 * g + 1]) * out_scale),
                pack_bf16x2(__uint_as_float(v[8 * g + 2]) * out_scale, __uint_as_float(v[8 * g + 3]) * out_scale),
                pack_bf16x2(__uint_as_float(v[8 * g + 4]) * out_scale, __uint_as_float(v[8 * g + 5]) * out_scale),
                pack_bf16x2(__uint_as_float(v[8 * g + 6]) * out_scale, __uint_as_float(v[8 * g + 7]) * out_scale));
        }
      }
    }
  }

  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <int HD, bool F8>
int launch_hstu_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const HstuParams& p, int B,
                    cudaStream_t stream) {
  using SM = Smem<HD, F8>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(hstu_attn_fwd_kernel<HD, F8>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL);
    if (e != cudaSuccess) { cudaGetLastError(); return b200::fail(1201, "hstu_attn_fwd: cannot set %d bytes of shared memory: %s", SM::TOTAL, cudaGetErrorString(e)); }
    configured[dev & 63] = true;
  }
  dim3 grid((p.max_len + 2 * BQ - 1) / (2 * BQ), p.H, B);
  hstu_attn_fwd_kernel<HD, F8><<<grid, NTHREADS, SM::TOTAL, stream>>>(tq, tk, tv, p);
  b200::count_launch();
  return b200::check_launch("hstu_attn_fwd");
}

}  // namespace

// q / k / v: jagged [L, H, HD] bf16 views (row pitches in elements, heads contiguous inside a row);
// out: [L, H, HD].  offsets: int32 [B + 1] on the device; num_targets: int32 [B] or null.
B200_API int b200_hstu_attn_fwd(const void* q, const void* k, const void* v, void* out, const int* offsets,
                                const int* num_targets, int B, long long L, int H, int HD, int max_len, int contextual,
                                long long q_row, long long k_row, long long v_row, long long out_row, float alpha,
                                void* stream) {
  if (HD != 64 && HD != 128) return b200::fail(1200, "hstu_attn_fwd: head dim %d not supported (64 or 128)", HD);
  if (L == 0 || B == 0) return 0;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = b200::make_tmap_3d(&tq, b200::DT_BF16, q, HD, H, L, (uint64_t)HD * 2, (uint64_t)q_row * 2, 64, 1, BQ, b200::SWZ_128))) return r;
  if ((r = b200::make_tmap_3d(&tk, b200::DT_BF16, k, HD, H, L, (uint64_t)HD * 2, (uint64_t)k_row * 2, 64, 1, BKV, b200::SWZ_128))) return r;
  if ((r = b200::make_tmap_3d(&tv, b200::DT_BF16, v, HD, H, L, (uint64_t)HD * 2, (uint64_t)v_row * 2, 64, 1, BKV, b200::SWZ_128))) return r;
  HstuParams p;
  p.max_len = max_len; p.H = H; p.contextual = contextual; p.alpha = alpha;
  p.offsets = offsets; p.num_targets = num_targets;
  p.out = (__nv_bfloat16*)out; p.out_row = out_row;
  p.inv_q = p.inv_k = p.inv_v = nullptr;
  p.status = b200::status_ptr();
  if (HD == 128) return launch_hstu_fwd<128, false>(tq, tk, tv, p, B, (cudaStream_t)stream);
  return launch_hstu_fwd<64, false>(tq, tk, tv, p, B, (cudaStream_t)stream);
}

// The same on 8-bit operands: q / k / v hold e4m3 codes (jagged [L, H, 128] views, row pitches in bytes), value =
// code * (*inv_x) with the factors read on the device; out [L, H, 128] bf16.
B200_API int b200_hstu_attn_fwd_fp8(const void* q, const void* k, const void* v, void* out, const int* offsets,
                                    const int* num_targets, int B, long long L, int H, int HD, int max_len, int contextual,
                                    long long q_row, long long k_row, long long v_row, long long out_row, float alpha,
                                    const float* inv_q, const float* inv_k, const float* inv_v, void* stream) {
  if (HD != 128) return b200::fail(1202, "hstu_attn_fwd_fp8: head dim %d not supported (128)", HD);
  if (L == 0 || B == 0) return 0;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = b200::make_tmap_3d(&tq, b200::DT_U8, q, HD, H, L, (uint64_t)HD, (uint64_t)q_row, 128, 1, BQ, b200::SWZ_128))) return r;
  if ((r = b200::make_tmap_3d(&tk, b200::DT_U8, k, HD, H, L, (uint64_t)HD, (uint64_t)k_row, 128, 1, BKV, b200::SWZ_128))) return r;
  if ((r = b200::make_tmap_3d(&tv, b200::DT_U8, v, HD, H, L, (uint64_t)HD, (uint64_t)v_row, 128, 1, BKV, b200::SWZ_128))) return r;
  HstuParams p;
  p.max_len = max_len; p.H = H; p.contextual = contextual; p.alpha = alpha;
  p.offsets = offsets; p.num_targets = num_targets;
  p.out = (__nv_bfloat16*)out; p.out_row = out_row;
  p.inv_q = inv_q; p.inv_k = inv_k; p.inv_v = inv_v;
  p.status = b200::status_ptr();
  return launch_hstu_fwd<128, true>(tq, tk, tv, p, B, (cudaStream_t)stream);
}
