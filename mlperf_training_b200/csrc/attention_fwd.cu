// Flash-attention forward for sm_100a: S = Q K^T and O += P V on tcgen05 tensor cores with the
// accumulators in TMEM, Q/K/V tiles brought in by TMA, online softmax in registers.
//
//   causal / non-causal, GQA (Hq a multiple of Hkv), sliding window, learned per-head sink
//   logits (an extra softmax column without a value), head_dim 64 or 128, bf16 in / bf16 out,
//   fp32 log-sum-exp saved for the backward pass.
//
// One CTA per (batch, head, 128-query tile); 192 threads:
//   warp 0     TMA producer (Q once, K/V double buffered)
//   warp 1     MMA issuer: S[j+1] = Q K[j+1]^T is issued before P[j] V[j], so the next score
//              tile is computed while the softmax warps work on the current one
//   warps 2-5  softmax (one query row per thread), lazy rescale of O in TMEM, epilogue
// TMEM: S double buffered (2 x 128 columns) + O (HD columns).
//
// Stands in for the attention kernels the reference selects by config: Primus-Turbo / AITER /
// CK flash attention (small_llm_pretraining/primus/conf/llama3.1_8B-pretrain-fp4.yaml:117,125)
// and the sink / sliding-window attention of the GPT-OSS config
// (small_llm_moe_pretraining/primus/conf/gpt_oss_20B-MXFP4-deosc-mlperf-pretrain.yaml:125-127).
#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int BQ = 128;   // query rows per CTA
constexpr int BKV = 128;  // keys per tile
constexpr int NTHREADS = 192;

struct FwdParams {
  int B, Hq, Hkv, Sq, Skv;
  int causal;       // 1: key position <= query position (+ Skv - Sq offset)
  int window;       // > 0: query attends to keys with q_pos - k_pos < window
  float scale_log2; // softmax scale * log2(e)
  const float* sink;  // [Hq] learned sink logits (natural-log domain, unscaled) or null
  float* lse;         // [B, Hq, Sq] natural-log log-sum-exp of the scaled scores
  int* status;
};

B200_DEVICE float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

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
  static constexpr int Q_BYTES = BQ * HD * 2;
  static constexpr int KV_BYTES = BKV * HD * 2;
  static constexpr int P_BYTES = BQ * BKV * 2;
  static constexpr int O_STAGE = BQ * HD * 2;  // reuses the P buffer (HD <= BKV)
  static constexpr int TOTAL = Q_BYTES + 4 * KV_BYTES + P_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 512;
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
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + SM::Q_BYTES;
  uint8_t* sV = sK + 2 * SM::KV_BYTES;
  uint8_t* sP = sV + 2 * SM::KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + SM::P_BYTES);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // 2
  uint64_t* s_empty = bars + 11;    // 2
  uint64_t* p_full = bars + 13;     // 1
  uint64_t* o_done = bars + 14;     // 1
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_qt = (p.Sq + BQ - 1) / BQ;
  const int qt = num_qt - 1 - (int)blockIdx.x;  // heaviest (latest) query tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qt * BQ;
  const int off = p.Skv - p.Sq;  // causal diagonal offset (0 for self-attention)

  // key-tile range visited by this query tile
  int j_hi = (p.Skv + BKV - 1) / BKV - 1;
  if (p.causal) {
    int last = (q0 + BQ - 1 + off) / BKV;
    if (last < j_hi) j_hi = last;
  }
  int j_lo = 0;
  if (p.window > 0) {
    int first = q0 + off - p.window + 1;
    if (first > 0) j_lo = first / BKV;
  }
  const int n_tiles = j_hi - j_lo + 1;  // >= 1 whenever the query tile has any visible key

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_holder, SM::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_S = tmem_base;        // 2 x 128 columns
  const uint32_t tmem_O = tmem_base + 256;  // HD columns

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, SM::Q_BYTES);
#pragma unroll
      for (int i = 0; i < NB; ++i) tma_load_4d(sQ + i * (BQ * 128), &tmQ, q_full, i * 64, h, q0, b);
      bool ok = true;
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int j = j_lo + t, st = t & 1;
        const uint32_t ph = (t >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, 40)) { ok = false; break; }
        mbar_expect_tx(&k_full[st], SM::KV_BYTES);
#pragma unroll
        for (int i = 0; i < NB; ++i) tma_load_4d(sK + st * SM::KV_BYTES + i * (BKV * 128), &tmK, &k_full[st], i * 64, hk, j * BKV, b);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status, 41)) { ok = false; break; }
        mbar_expect_tx(&v_full[st], SM::KV_BYTES);
#pragma unroll
        for (int i = 0; i < NB; ++i) tma_load_4d(sV + st * SM::KV_BYTES + i * (BKV * 128), &tmV, &v_full[st], i * 64, hk, j * BKV, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      const uint32_t idesc_s = umma_idesc(1, 1, 0, 0, BQ, BKV);  // Q (K-major) x K (K-major)
      const uint32_t idesc_o = umma_idesc(1, 1, 0, 1, BQ, HD);   // P (K-major) x V (MN-major)
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 50);
      auto issue_s = [&](int t) -> bool {
        const int st = t & 1;
        const uint32_t ph = (t >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph, abort_flag, p.status, 51)) return false;
        if (!mbar_wait(&s_empty[st], ph ^ 1, abort_flag, p.status, 52)) return false;
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + st * SM::KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t o = (kk / 4) * (BQ * 128) + (kk % 4) * 32;
          tc_mma_f16_ss(tmem_S + st * BKV, umma_desc_sw128(qa + o, 16, 1024), umma_desc_sw128(ka + o, 16, 1024),
                        idesc_s, kk > 0 ? 1u : 0u);
        }
        tc_commit(&k_empty[st]);
        tc_commit(&s_full[st]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (t + 1 < n_tiles) { if (!issue_s(t + 1)) { ok = false; break; } }
        const int st = t & 1;
        const uint32_t ph = (t >> 1) & 1;
        if (!mbar_wait(p_full, t & 1, abort_flag, p.status, 53)) { ok = false; break; }
        if (!mbar_wait(&v_full[st], ph, abort_flag, p.status, 54)) { ok = false; break; }
        tc_fence_after();
        const uint32_t pa = smem_u32(sP), va = smem_u32(sV + st * SM::KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint32_t po = (kk / 4) * (BQ * 128) + (kk % 4) * 32;   // P: K-major, 64-key blocks
          const uint32_t vo = kk * (16 * 128);                          // V: 16 key rows of 128 bytes
          tc_mma_f16_ss(tmem_O, umma_desc_sw128(pa + po, 16, 1024), umma_desc_sw128(va + vo, BKV * 128, 1024),
                        idesc_o, (t > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&v_empty[st]);
        tc_commit(o_done);
      }
    }
  } else {
    // ------------------------------ softmax + epilogue ------------------------------
    const int q = warp & 3;
    const int r = q * 32 + lane;           // row inside the query tile
    const int q_pos = q0 + r;
    const uint32_t lane_base = uint32_t(q * 32) << 16;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = n_tiles > 0;
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int j = j_lo + t, st = t & 1;
      const uint32_t ph = (t >> 1) & 1;
      if (!mbar_wait(&s_full[st], ph, abort_flag, p.status, 60)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = j * BKV;
      // does this tile need element masks?
      const bool need_mask = (kv0 + BKV > p.Skv) || (p.causal && kv0 + BKV - 1 > q0 + off) ||
                             (p.window > 0 && kv0 < q0 + BQ - 1 + off - p.window + 1);
      const int hi = p.causal ? min(q_pos + off, p.Skv - 1) : p.Skv - 1;         // last visible key
      const int lo = p.window > 0 ? q_pos + off - p.window + 1 : 0;              // first visible key
      const uint32_t ts = tmem_S + lane_base + st * BKV;
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(ts + c * 32, v);
        tc_wait_ld();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kp = kv0 + c * 32 + i;
            if (kp <= hi && kp >= lo) mx = fmaxf(mx, __uint_as_float(v[i]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(v[i]));
        }
      }
      mx *= p.scale_log2;  // -inf stays -inf (scale > 0)
      // lazy rescale: move the reference maximum only when it grew by more than 2^8
      float alpha = 1.f;
      const bool grow = (mx > m_ref + 8.f) || (m_ref == -INFINITY && mx > -INFINITY);
      const bool warp_grow = __any_sync(0xffffffffu, grow);
      // P of the previous tile must have been consumed (and O complete) before P is overwritten
      if (t > 0) {
        if (!mbar_wait(o_done, (t - 1) & 1, abort_flag, p.status, 61)) { ok = false; break; }
        tc_fence_after();
      }
      if (warp_grow) {
        const float m_new = fmaxf(m_ref, mx);
        alpha = (m_ref == -INFINITY) ? 0.f : ex2(m_ref - m_new);
        m_ref = m_new;
        l *= alpha;
        if (t > 0) {
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(tmem_O + lane_base + c * 32, v);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32b_x32(tmem_O + lane_base + c * 32, v);
          }
          tc_wait_st();
        }
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      // pass 2: P = exp2(S * scale - m), row sum, bf16 into swizzled shared memory
      float rs = 0.f;
      uint8_t* prow = sP + r * 128;
#pragma unroll 1
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(ts + c * 32, v);
        tc_wait_ld();
        float e[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = ex2(__uint_as_float(v[i]) * p.scale_log2 - m_use);
          if (need_mask) {
            const int kp = kv0 + c * 32 + i;
            if (kp > hi || kp < lo) x = 0.f;
          }
          e[i] = x;
          rs += x;
        }
        uint8_t* blk = prow + (c / 2) * (BQ * 128);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int chunk = (c & 1) * 4 + g;
          uint4 u = make_uint4(pack_bf16x2(e[8 * g], e[8 * g + 1]), pack_bf16x2(e[8 * g + 2], e[8 * g + 3]),
                               pack_bf16x2(e[8 * g + 4], e[8 * g + 5]), pack_bf16x2(e[8 * g + 6], e[8 * g + 7]));
          *reinterpret_cast<uint4*>(blk + ((chunk ^ (r & 7)) << 4)) = u;
        }
      }
      l += rs;
      // S buffer free for the MMA warp; P ready for the tensor core
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s_empty[st]); mbar_arrive(p_full); }
    }
    // ------------------------------ epilogue ------------------------------
    if (ok) ok = mbar_wait(o_done, (n_tiles - 1) & 1, abort_flag, p.status, 62);
    if (ok) {
      tc_fence_after();
      if (p.sink != nullptr) {
        const float sk = p.sink[h] * 1.4426950408889634f;
        if (m_ref == -INFINITY) { m_ref = sk; l = 1.f; }
        else l += ex2(sk - m_ref);
      }
      const float inv = l > 0.f ? 1.f / l : 0.f;
      uint8_t* orow = sP + r * 128;  // P buffer reused as O staging: HD/64 blocks of [128][64]
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_O + lane_base + c * 32, v);
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
      if (lane == 0 && q0 + q * 32 < p.Sq) {
#pragma unroll
        for (int i = 0; i < NB; ++i)
          tma_store_4d(&tmO, sP + i * (BQ * 128) + q * 32 * 128, i * 64, h, q0 + q * 32, b);
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
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, SM::TMEM_COLS); }
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
    if (e != cudaSuccess) return b200::fail(601, "attn_fwd: cannot set %d bytes of shared memory: %s", SM::TOTAL,
                                            cudaGetErrorString(e));
    configured[dev & 63] = true;
  }
  dim3 grid((p.Sq + BQ - 1) / BQ, p.Hq, p.B);
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
