// Flash-attention forward for sm_100a: S = Q K^T and O += P V on tcgen05 tensor cores with the
// accumulators in TMEM, Q/K/V tiles brought in by TMA, online softmax in registers.
//
//   causal / non-causal, GQA (Hq a multiple of Hkv), sliding window, learned per-head sink
//   logits (an extra softmax column without a value), head_dim 64 or 128, bf16 in / bf16 out,
//   fp32 log-sum-exp saved for the backward pass.
//
// One CTA per (batch, head, pair of 128-query tiles); 320 threads:
//   warp 8      TMA producer (both Q tiles once, K/V double buffered, shared by the two tiles)
//   warp 9      MMA issuer, ping-pong over the two query tiles:
//                 S0(0) S1(0) | PV0(n) S0(n+1) PV1(n) S1(n+1) | ...
//               so the tensor core works on one tile while the other tile's softmax runs
//   warps 0-3   softmax of tile 0 (one query row per thread)
//   warps 4-7   softmax of tile 1
// TMEM (512 columns): S0 | S1 | O0 | O1.  The bf16 probabilities P overwrite the first half of
// their own S columns (tcgen05.st) and feed the second GEMM straight from TMEM (A operand in
// TMEM), so P never touches shared memory.  O is rescaled lazily: only when the running row
// maximum grew by more than 2^8.  A quarter of the exponentials run as a polynomial on the FMA
// pipe to relieve the MUFU unit.
//
// Stands in for the attention kernels the reference selects by config: Primus-Turbo / AITER /
// CK flash attention (small_llm_pretraining/primus/conf/llama3.1_8B-pretrain-fp4.yaml:117,125)
// and the sink / sliding-window attention of the GPT-OSS config
// (small_llm_moe_pretraining/primus/conf/gpt_oss_20B-MXFP4-deosc-mlperf-pretrain.yaml:125-127).
#include "common.cuh"
#include "runtime.h"

namespace {

#ifndef B200_ATTN_FWD_POLY
#define B200_ATTN_FWD_POLY 3
#endif
constexpr int POLY = B200_ATTN_FWD_POLY;  // pairs with (i & POLY) == POLY take the FMA-pipe polynomial: 3 = a quarter, 1 = half
constexpr int BQ = 128;   // query rows per tile (two tiles per CTA)
constexpr int BKV = 128;  // keys per tile
constexpr int NTHREADS = 320;  // warps 0-3 / 4-7: softmax of tile 0 / 1; warp 8: TMA; warp 9: MMA

struct FwdParams {
  int B, Hq, Hkv, Sq, Skv;
  int causal;       // 1: key position <= query position (+ Skv - Sq offset)
  int window;       // > 0: query attends to keys with q_pos - k_pos < window
  float scale_log2; // softmax scale * log2(e)
  const float* sink;  // [Hq] learned sink logits (natural-log domain, unscaled) or null
  float* lse;         // [B, Hq, Sq] natural-log log-sum-exp of the scaled scores
  int* status;
};

B200_DEVICE void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
B200_DEVICE void tma_store_4d(const CUtensorMap* map, const void* src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
               "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

template <int HD>
struct Smem {
  static constexpr int Q_TILE = BQ * HD * 2;
  static constexpr int KV_BYTES = BKV * HD * 2;
  static constexpr int TOTAL = 2 * Q_TILE + 4 * KV_BYTES + 1024 + 256;
};

template <int HD>
__global__ void __launch_bounds__(NTHREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                const FwdParams p) {
  using SM = Smem<HD>;
  constexpr int NB = HD / 64;  // 64-column (128-byte) blocks per head row
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
  const int num_pairs = (p.Sq + 2 * BQ - 1) / (2 * BQ);
  const int pair = num_pairs - 1 - (int)blockIdx.x;  // heaviest (latest) query tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = pair * 2 * BQ;
  const int off = p.Skv - p.Sq;  // causal diagonal offset (0 for self-attention)

  // key-tile range: a common first tile, a per-query-tile last tile
  const int j_max = (p.Skv + BKV - 1) / BKV - 1;
  int j_lo = 0;
  if (p.window > 0) {
    const int first = q0 + off - p.window + 1;
    if (first > 0) j_lo = first / BKV;
  }
  int n_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qt0 = q0 + t * BQ;
    int j_hi = j_max;
    if (p.causal) {
      const int last = (qt0 + BQ - 1 + off) / BKV;
      if (last < j_hi) j_hi = last;
    }
    n_t[t] = (qt0 < p.Sq && j_hi >= j_lo) ? (j_hi - j_lo + 1) : 0;
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
          tma_load_4d(sQ + t * SM::Q_TILE + i * (BQ * 128), &tmQ, q_full, i * 64, h, q0 + t * BQ, b);
      bool ok = true;
      for (int n = 0; n < n_max && ok; ++n) {
        const int j = j_lo + n, st = n & 1;
        const uint32_t ph = (n >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, 40)) { ok = false; break; }
        mbar_expect_tx(&k_full[st], SM::KV_BYTES);
#pragma unroll
        for (int i = 0; i < NB; ++i)
          tma_load_4d(sK + st * SM::KV_BYTES + i * (BKV * 128), &tmK, &k_full[st], i * 64, hk, j * BKV, b);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status, 41)) { ok = false; break; }
        mbar_expect_tx(&v_full[st], SM::KV_BYTES);
#pragma unroll
        for (int i = 0; i < NB; ++i)
          tma_load_4d(sV + st * SM::KV_BYTES + i * (BKV * 128), &tmV, &v_full[st], i * 64, hk, j * BKV, b);
      }
    }
  } else if (warp == 9) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && n_max > 0) {
      const uint32_t idesc_s = umma_idesc(1, 1, 0, 0, BQ, BKV);  // Q (K-major) x K (K-major)
      const uint32_t idesc_o = umma_idesc(1, 1, 0, 1, BQ, HD);   // P (TMEM)    x V (MN-major)
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
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t o = (kk / 4) * (BQ * 128) + (kk % 4) * 32;
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
#pragma unroll
          for (int kk = 0; kk < BKV / 16; ++kk) {
            // A = P_t in TMEM: 16 bf16 keys = 8 columns per step; B = V: 16 key rows of 128 bytes
            tc_mma_f16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + kk * 8,
                          umma_desc_sw128(va + kk * (16 * 128), BKV * 128, 1024), idesc_o, (n > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&o_done[t]);
          const bool last_user = (t == 1) || !(n < n_t[1]);
          if (last_user) tc_commit(&v_empty[st]);
          if (n + 1 < n_t[t]) ok = issue_s(t, n + 1);
        }
      }
    }
  } else if (warp < 8) {
    // ------------------------------ softmax + epilogue (one warpgroup per query tile) --------------
    const int t = warp >> 2;
    const int q = warp & 3;
    const int r = q * 32 + lane;           // row inside the query tile
    const int qt0 = q0 + t * BQ;
    const int q_pos = qt0 + r;
    const uint32_t lane_base = uint32_t(q * 32) << 16;
    const uint32_t ts = tmem_base + lane_base + t * 128;        // S / P columns of this tile
    const uint32_t to = tmem_base + lane_base + 256 + t * 128;  // O columns of this tile
    const int my_n = n_t[t];
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int n = 0; n < my_n && ok; ++n) {
      const int kv0 = (j_lo + n) * BKV;
      if (!mbar_wait(&s_full[t], n & 1, abort_flag, p.status, 60)) { ok = false; break; }
      tc_fence_after();
      const bool need_mask = (kv0 + BKV > p.Skv) || (p.causal && kv0 + BKV - 1 > qt0 + off) ||
                             (p.window > 0 && kv0 < qt0 + BQ - 1 + off - p.window + 1);
      const int hi = p.causal ? min(q_pos + off, p.Skv - 1) : p.Skv - 1;         // last visible key
      const int lo = p.window > 0 ? q_pos + off - p.window + 1 : 0;              // first visible key
      // the whole score row (128 fp32) comes into registers with one TMEM round trip
      uint32_t v[BKV];
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) tmem_ld_32x32b_x32(ts + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
      tc_wait_ld();
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < BKV; ++i) {
          const int kp = kv0 + i;
          if (kp > hi || kp < lo) v[i] = 0xff800000u;  // -inf
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < BKV; i += 4) {
        mx4[0] = fmaxf(mx4[0], __uint_as_float(v[i]));
        mx4[1] = fmaxf(mx4[1], __uint_as_float(v[i + 1]));
        mx4[2] = fmaxf(mx4[2], __uint_as_float(v[i + 2]));
        mx4[3] = fmaxf(mx4[3], __uint_as_float(v[i + 3]));
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx *= p.scale_log2;  // -inf stays -inf (scale > 0)
      // lazy rescale: move the reference maximum only when it grew by more than 2^8
      const bool grow = (mx > m_ref + 8.f) || (m_ref == -INFINITY && mx > -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_ref, mx);
        const float alpha = (m_ref == -INFINITY) ? 0.f : ex2_approx(m_ref - m_new);
        m_ref = m_new;
        l *= alpha;
        if (n > 0) {
          // O_t must be complete (P V of the previous key tile) before it is rescaled
          if (!mbar_wait(&o_done[t], (n - 1) & 1, abort_flag, p.status, 61)) { ok = false; break; }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(to + c * 32, o);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32b_x32(to + c * 32, o);
          }
          tc_wait_st();
        }
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      // P = exp2(S * scale - m) as bf16 pairs over the first half of the S columns; every fourth
      // pair takes the polynomial path (FMA pipe), the rest the MUFU path; -inf gives 0 on both
      float2 rs2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
      const float2 nm2 = make_float2(-m_use, -m_use);
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int e = c * 32 + 2 * i;
          const float2 a = ffma2(make_float2(__uint_as_float(v[e]), __uint_as_float(v[e + 1])), sc2, nm2);
          float2 x;
          if ((i & POLY) == POLY) x = ex2_poly2(a);
          else x = make_float2(ex2_approx(a.x), ex2_approx(a.y));
          rs2[i & 1] = fadd2(rs2[i & 1], x);
          pk[i] = pack_bf16x2(x.x, x.y);
        }
        tmem_st_32x32b_x16(ts + c * 16, pk);
      }
      const float rs = (rs2[0].x + rs2[0].y) + (rs2[1].x + rs2[1].y);
      l += rs;
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
    }
    // ------------------------------ epilogue ------------------------------
    if (ok && my_n > 0) ok = mbar_wait(&o_done[t], (my_n - 1) & 1, abort_flag, p.status, 62);
    if (ok && my_n > 0) {
      tc_fence_after();
      if (p.sink != nullptr) {
        const float sk = p.sink[h] * 1.4426950408889634f;
        if (m_ref == -INFINITY) { m_ref = sk; l = 1.f; }
        else l += ex2_approx(sk - m_ref);
      }
      const float inv = l > 0.f ? 1.f / l : 0.f;
      uint8_t* stage = sQ + t * SM::Q_TILE;  // the Q tile is dead after the last S MMA: reuse as O staging
      uint8_t* orow = stage + r * 128;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(to + c * 32, v);
        tc_wait_ld();
        uint8_t* blk = orow + (c / 2) * (BQ * 128);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int chunk = (c & 1) * 4 + g;
          uint4 u = make_uint4(
              pack_bf16x2(__uint_as_float(v[8 * g]) * inv, __uint_as_float(v[8 * g + 1]) * inv),
              pack_bf16x2(__uint_as_float(v[8 * g + 2]) * inv, __uint_as_float(v[8 * g + 3]) * inv),
              pack_bf16x2(__uint_as_float(v[8 * g + 4]) * inv, __uint_as_float(v[8 * g + 5]) * inv),
              pack_bf16x2(__uint_as_float(v[8 * g + 6]) * inv, __uint_as_float(v[8 * g + 7]) * inv));
          *reinterpret_cast<uint4*>(blk + ((chunk ^ (r & 7)) << 4)) = u;
        }
      }
      if (q_pos < p.Sq && p.lse != nullptr)
        p.lse[((long long)b * p.Hq + h) * p.Sq + q_pos] =
            (l > 0.f) ? (m_ref + log2f(l)) * 0.6931471805599453f : -INFINITY;
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && qt0 + q * 32 < p.Sq) {
#pragma unroll
        for (int i = 0; i < NB; ++i)
          tma_store_4d(&tmO, stage + i * (BQ * 128) + q * 32 * 128, i * 64, h, qt0 + q * 32, b);
        tma_store_commit();
        tma_store_wait_all<0>();
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

// tensor [B][S][H][HD] view with arbitrary row pitch: dims (inner to outer) {HD, H, S, B}
int make_qkv_map(CUtensorMap* m, const void* ptr, int HD, int H, int S, int B, long long row_stride,
                 long long batch_stride, int box_rows) {
  return b200::make_tmap_4d(m, b200::DT_BF16, ptr, HD, H, S, B, (uint64_t)HD * 2, (uint64_t)row_stride * 2,
                            (uint64_t)batch_stride * 2, 64, 1, box_rows, 1, b200::SWZ_128);
}

template <int HD>
int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to,
               const FwdParams& p, cudaStream_t stream) {
  using SM = Smem<HD>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL);
    if (e != cudaSuccess) cudaGetLastError();  // clear the sticky error before reporting
    if (e != cudaSuccess) return b200::fail(601, "attn_fwd: cannot set %d bytes of shared memory: %s", SM::TOTAL,
                                            cudaGetErrorString(e));
    configured[dev & 63] = true;
  }
  dim3 grid((p.Sq + 2 * BQ - 1) / (2 * BQ), p.Hq, p.B);
  attn_fwd_kernel<HD><<<grid, NTHREADS, SM::TOTAL, stream>>>(tq, tk, tv, to, p);
  b200::count_launch();
  return b200::check_launch("attn_fwd");
}

}  // namespace

// q: [B, Sq, Hq, HD], k/v: [B, Skv, Hkv, HD], o: [B, Sq, Hq, HD]; each with its own row pitch
// (elements between consecutive tokens) and batch pitch, heads contiguous inside a token row.
B200_API int b200_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const float* sink,
                           int B, int Sq, int Skv, int Hq, int Hkv, int HD, long long q_row, long long k_row,
                           long long v_row, long long o_row, long long q_batch, long long k_batch,
                           long long v_batch, long long o_batch, float scale, int causal, int window,
                           void* stream) {
  if (HD != 64 && HD != 128) return b200::fail(600, "attn_fwd: head dim %d not supported (64 or 128)", HD);
  if (Hq % Hkv != 0) return b200::fail(600, "attn_fwd: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
  if (causal && Skv < Sq) return b200::fail(600, "attn_fwd: causal needs Skv >= Sq");
  CUtensorMap tq, tk, tv, to;
  int r;
  if ((r = make_qkv_map(&tq, q, HD, Hq, Sq, B, q_row, q_batch, BQ))) return r;
  if ((r = make_qkv_map(&tk, k, HD, Hkv, Skv, B, k_row, k_batch, BKV))) return r;
  if ((r = make_qkv_map(&tv, v, HD, Hkv, Skv, B, v_row, v_batch, BKV))) return r;
  if ((r = make_qkv_map(&to, o, HD, Hq, Sq, B, o_row, o_batch, 32))) return r;
  FwdParams p;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq; p.Skv = Skv;
  p.causal = causal; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.sink = sink; p.lse = lse;
  p.status = b200::status_ptr();
  if (HD == 128) return launch_fwd<128>(tq, tk, tv, to, p, (cudaStream_t)stream);
  return launch_fwd<64>(tq, tk, tv, to, p, (cudaStream_t)stream);
}
