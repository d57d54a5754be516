// Flash-attention backward for sm_100a.  One CTA owns one (batch, kv-head, 128-key tile) and
// loops over the query heads of its GQA group and over the query tiles that see those keys:
//
//   S  = Q K^T            dP = dO V^T                   (tcgen05, accumulators in TMEM)
//   P  = exp2(S*c - lse)  dS = P * (dP - delta) * scale (softmax warps, registers)
//   dQ = dS K   (TMEM -> fp32 TMA reduce-add into a global fp32 dQ buffer)
//   dV += P^T dO          dK += dS^T Q                  (stay in TMEM for the whole CTA)
//
// P and dS are written once to shared memory as [query][key] bf16 tiles and read by the tensor
// core both key-contiguous (for dQ) and as MN-major operands (P^T, dS^T) through the UMMA
// descriptor, so no transposed copies are made.  dK / dV leave as bf16 through TMA stores.
//
// 320 threads: warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 workers.  Two workers share a
// TMEM lane quarter (32 query rows): each computes P / dS for half of the 128 key columns, then
// drains half of the dQ columns (TMEM -> registers, accumulator released, registers -> fp32 TMA
// reduce-add while the next S / dP GEMMs run).  A quarter of the exponentials is evaluated with a
// polynomial on the FMA pipe: 128 x 128 exp2 per tile would otherwise cost 1024 cycles of the
// 16-per-clock special-function unit alone.  TMEM (512 columns): S/dQ | dP | dK | dV.
//
// The reference takes this kernel from Primus-Turbo / AITER / CK (config knobs
// llama2_sft/primus/config_MI355X_1x8x1.sh:35-39); there is no in-tree counterpart.
#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int NTHREADS = 320;
constexpr int STG = 4096;  // dQ staging chunk: 32 rows x 32 fp32
#ifndef B200_ATTN_BWD_POLY
#define B200_ATTN_BWD_POLY 6
#endif
constexpr int POLY = B200_ATTN_BWD_POLY;   // pairs with (i & POLY) == POLY take the FMA-pipe polynomial: 6 = a quarter, 2 = half

struct BwdParams {
  int B, Hq, Hkv, Sq, Skv;
  int causal, window;
  float scale, scale_log2;
  const float* lse;    // [B, Hq, Sq]
  const float* delta;  // [B, Hq, Sq]  rowsum(dO * O)
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
B200_DEVICE void tma_reduce_add_4d(const CUtensorMap* map, const void* src, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
      "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

template <int HD>
struct Smem {
  static constexpr int T_BYTES = 128 * HD * 2;        // K, V, Q, dO tiles
  static constexpr int PS_BYTES = BQ * BKV * 2;       // P, dS tiles
  static constexpr int STG_BYTES = 4 * 2 * STG;
  static constexpr int TOTAL = 4 * T_BYTES + 2 * PS_BYTES + STG_BYTES + 1024 + 256;
};

template <int HD>
__global__ void __launch_bounds__(NTHREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const __grid_constant__ CUtensorMap tmdQ, const __grid_constant__ CUtensorMap tmdK,
                const __grid_constant__ CUtensorMap tmdV, const BwdParams p) {
  using SM = Smem<HD>;
  constexpr int NB = HD / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + SM::T_BYTES;
  uint8_t* sQ = sV + SM::T_BYTES;
  uint8_t* sdO = sQ + SM::T_BYTES;
  uint8_t* sP = sdO + SM::T_BYTES;
  uint8_t* sdS = sP + SM::PS_BYTES;
  uint8_t* sStg = sdS + SM::PS_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStg + SM::STG_BYTES);
  uint64_t* kv_full = bars + 0;     // K and V landed
  uint64_t* qdo_full = bars + 1;    // Q_i and dO_i landed
  uint64_t* qdo_empty = bars + 2;   // MMAs reading Q_i / dO_i / P / dS finished
  uint64_t* sdp_full = bars + 3;    // S and dP complete in TMEM
  uint64_t* pds_full = bars + 4;    // P and dS written to shared memory (4 arrivals)
  uint64_t* dq_full = bars + 5;     // dQ tile complete in TMEM
  uint64_t* dq_drained = bars + 6;  // dQ tile copied out of TMEM (4 arrivals)
  uint64_t* acc_done = bars + 7;    // every MMA of this CTA finished
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kt = (p.Skv + BKV - 1) / BKV;
  const int jt = blockIdx.x;  // key tile; early tiles see the most queries and are scheduled first
  const int hk = blockIdx.y, b = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  const int kv0 = jt * BKV;
  const int off = p.Skv - p.Sq;
  const int num_qt = (p.Sq + BQ - 1) / BQ;
  // query tiles that see at least one key of this tile
  int i_lo = 0, i_hi = num_qt - 1;
  if (p.causal) {
    int first_q = kv0 - off;  // first query position that sees key kv0
    if (first_q > 0) i_lo = first_q / BQ;
  }
  if (p.window > 0) {
    int last_q = kv0 + BKV - 1 + p.window - 1 - off;  // last query that still sees the tile's last key
    if (last_q / BQ < i_hi) i_hi = last_q / BQ;
  }
  const int n_q = (i_hi >= i_lo) ? (i_hi - i_lo + 1) : 0;
  const int n_iter = n_q * group;
  (void)num_kt;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1); mbar_init(qdo_full, 1); mbar_init(qdo_empty, 1); mbar_init(sdp_full, 1);
    mbar_init(pds_full, 8); mbar_init(dq_full, 1); mbar_init(dq_drained, 8); mbar_init(acc_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_holder, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tm_S = tmem_base;          // S, later dQ (128 columns)
  const uint32_t tm_dP = tmem_base + 128;
  const uint32_t tm_dK = tmem_base + 256;
  const uint32_t tm_dV = tmem_base + 384;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmdO);
      mbar_expect_tx(kv_full, 2 * SM::T_BYTES);
#pragma unroll
      for (int i = 0; i < NB; ++i) {
        tma_load_4d(sK + i * (BKV * 128), &tmK, kv_full, i * 64, hk, kv0, b);
        tma_load_4d(sV + i * (BKV * 128), &tmV, kv_full, i * 64, hk, kv0, b);
      }
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int h = hk * group + it / n_q;
        const int q0 = (i_lo + it % n_q) * BQ;
        if (!mbar_wait(qdo_empty, (it & 1) ^ 1, abort_flag, p.status, 70)) { ok = false; break; }
        mbar_expect_tx(qdo_full, 2 * SM::T_BYTES);
#pragma unroll
        for (int i = 0; i < NB; ++i) {
          tma_load_4d(sQ + i * (BQ * 128), &tmQ, qdo_full, i * 64, h, q0, b);
          tma_load_4d(sdO + i * (BQ * 128), &tmdO, qdo_full, i * 64, h, q0, b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && n_iter > 0) {
      const uint32_t id_kk = umma_idesc(1, 1, 0, 0, 128, 128);   // S = Q K^T, dP = dO V^T (both K-major)
      const uint32_t id_dq = umma_idesc(1, 1, 0, 1, 128, HD);    // dQ = dS (K-major) x K (MN-major)
      const uint32_t id_tt = umma_idesc(1, 1, 1, 1, 128, HD);    // dV = P^T dO, dK = dS^T Q (both MN-major)
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), adO = smem_u32(sdO);
      const uint32_t aP = smem_u32(sP), adS = smem_u32(sdS);
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, 80);
      for (int it = 0; it < n_iter && ok; ++it) {
        const uint32_t ph = it & 1;
        if (!mbar_wait(qdo_full, ph, abort_flag, p.status, 81)) { ok = false; break; }
        tc_fence_after();
        // S = Q K^T ; dP = dO V^T   (contraction over the head dim, both operands K-major)
        // dP first: its accumulator was read by the workers long ago, so these MMAs run while the workers
        // still drain dQ of the previous iteration out of the S / dQ columns
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t o = (kk / 4) * (128 * 128) + (kk % 4) * 32;
          tc_mma_f16_ss(tm_dP, umma_desc_sw128(adO + o, 16, 1024), umma_desc_sw128(aV + o, 16, 1024), id_kk, kk > 0);
        }
        if (it > 0 && !mbar_wait(dq_drained, (it - 1) & 1, abort_flag, p.status, 82)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t o = (kk / 4) * (128 * 128) + (kk % 4) * 32;
          tc_mma_f16_ss(tm_S, umma_desc_sw128(aQ + o, 16, 1024), umma_desc_sw128(aK + o, 16, 1024), id_kk, kk > 0);
        }
        tc_commit(sdp_full);
        if (!mbar_wait(pds_full, ph, abort_flag, p.status, 83)) { ok = false; break; }
        tc_fence_after();
        // dV += P^T dO ; dK += dS^T Q : contraction over queries, both operands MN-major
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk) {
          const uint32_t o = kk * (16 * 128);
          tc_mma_f16_ss(tm_dV, umma_desc_sw128(aP + o, 128 * 128, 1024), umma_desc_sw128(adO + o, 128 * 128, 1024),
                        id_tt, (it > 0 || kk > 0));
        }
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk) {
          const uint32_t o = kk * (16 * 128);
          tc_mma_f16_ss(tm_dK, umma_desc_sw128(adS + o, 128 * 128, 1024), umma_desc_sw128(aQ + o, 128 * 128, 1024),
                        id_tt, (it > 0 || kk > 0));
        }
        tc_commit(qdo_empty);  // Q_i / dO_i may be overwritten: the next tiles load during the dQ GEMM
        // dQ = dS K : A = dS [q][key] K-major, B = K [key][d] MN-major (contraction over keys)
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint32_t ao = (kk / 4) * (128 * 128) + (kk % 4) * 32;
          const uint32_t bo = kk * (16 * 128);
          tc_mma_f16_ss(tm_S, umma_desc_sw128(adS + ao, 16, 1024), umma_desc_sw128(aK + bo, 128 * 128, 1024), id_dq,
                        kk > 0);
        }
        tc_commit(dq_full);    // also: P / dS shared-memory tiles are free again
      }
      if (ok) tc_commit(acc_done);
    }
  } else {
    // ------------------------------ workers: P / dS, then dQ drain ------------------------------
    const int q = warp & 3;                   // TMEM lane quarter
    const int half = (warp - 2) >> 2;         // which half of the key columns / of the dQ columns
    const int r = q * 32 + lane;
    const uint32_t lane_base = uint32_t(q * 32) << 16;
    uint8_t* stg = sStg + (warp - 2) * STG;   // one staging buffer per worker
    constexpr int CH = HD / 64;               // dQ chunks (32 columns) per worker
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int h = hk * group + it / n_q;
      const int q0 = (i_lo + it % n_q) * BQ;
      const int q_pos = q0 + r;
      float lse2 = 0.f, dl = 0.f;
      bool row_ok = q_pos < p.Sq;
      if (row_ok) {
        const long long idx = ((long long)b * p.Hq + h) * p.Sq + q_pos;
        lse2 = p.lse[idx] * 1.4426950408889634f;
        dl = p.delta[idx];
        if (lse2 == -INFINITY) row_ok = false;  // row without any visible key
      }
      const bool need_mask = (kv0 + BKV > p.Skv) || (p.causal && kv0 + BKV - 1 > q0 + off) ||
                             (p.window > 0 && kv0 < q0 + BQ - 1 + off - p.window + 1) || (q0 + BQ > p.Sq) ||
                             __any_sync(0xffffffffu, !row_ok);
      const int hi = p.causal ? min(q_pos + off, p.Skv - 1) : p.Skv - 1;
      const int lo = p.window > 0 ? q_pos + off - p.window + 1 : 0;
      if (!mbar_wait(sdp_full, it & 1, abort_flag, p.status, 90)) { ok = false; break; }
      tc_fence_after();
      // the P / dS tiles are free: this warp waited for dq_full of the previous iteration in its drain step
      uint8_t* prow = sP + r * 128;
      uint8_t* drow = sdS + r * 128;
#pragma unroll 1
      for (int c = half * 2; c < half * 2 + 2; ++c) {
        uint32_t s[32], d[32];
        tmem_ld_32x32b_x32(tm_S + lane_base + c * 32, s);
        tmem_ld_32x32b_x32(tm_dP + lane_base + c * 32, d);
        tc_wait_ld();
        float pv[32], dv[32];
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nl2 = make_float2(-lse2, -lse2);
        const float2 s2 = make_float2(p.scale, p.scale), nd2 = make_float2(-dl * p.scale, -dl * p.scale);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 a = ffma2(make_float2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), sc2, nl2);
          float2 e;
          if ((i & POLY) == POLY) e = ex2_poly2(a);
          else e = make_float2(ex2_approx(a.x), ex2_approx(a.y));
          float p0 = e.x, p1 = e.y;
          if (need_mask) {
            const int kp = kv0 + c * 32 + i;
            if (!row_ok || kp > hi || kp < lo) p0 = 0.f;
            if (!row_ok || kp + 1 > hi || kp + 1 < lo) p1 = 0.f;
          }
          const float2 t2 = ffma2(make_float2(__uint_as_float(d[i]), __uint_as_float(d[i + 1])), s2, nd2);
          const float2 g2 = fmul2(make_float2(p0, p1), t2);
          pv[i] = p0; pv[i + 1] = p1;
          dv[i] = g2.x; dv[i + 1] = g2.y;
        }
        uint8_t* pb = prow + (c / 2) * (BQ * 128);
        uint8_t* db = drow + (c / 2) * (BQ * 128);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int sw = (((c & 1) * 4 + g) ^ (r & 7)) << 4;
          *reinterpret_cast<uint4*>(pb + sw) =
              make_uint4(pack_bf16x2(pv[8 * g], pv[8 * g + 1]), pack_bf16x2(pv[8 * g + 2], pv[8 * g + 3]),
                         pack_bf16x2(pv[8 * g + 4], pv[8 * g + 5]), pack_bf16x2(pv[8 * g + 6], pv[8 * g + 7]));
          *reinterpret_cast<uint4*>(db + sw) =
              make_uint4(pack_bf16x2(dv[8 * g], dv[8 * g + 1]), pack_bf16x2(dv[8 * g + 2], dv[8 * g + 3]),
                         pack_bf16x2(dv[8 * g + 4], dv[8 * g + 5]), pack_bf16x2(dv[8 * g + 6], dv[8 * g + 7]));
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      // ---- dQ drain: this worker's half of the head dim ----
      if (!mbar_wait(dq_full, it & 1, abort_flag, p.status, 95)) { ok = false; break; }
      tc_fence_after();
      uint32_t v[CH][32];
#pragma unroll
      for (int cc = 0; cc < CH; ++cc) tmem_ld_32x32b_x32(tm_S + lane_base + (half * CH + cc) * 32, v[cc]);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_drained);      // the accumulator may be overwritten by the next S
#pragma unroll
      for (int cc = 0; cc < CH; ++cc) {
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
        uint8_t* sb = stg + lane * 128;
#pragma unroll
        for (int g = 0; g < 8; ++g)
          *reinterpret_cast<uint4*>(sb + ((g ^ (lane & 7)) << 4)) =
              make_uint4(v[cc][4 * g], v[cc][4 * g + 1], v[cc][4 * g + 2], v[cc][4 * g + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (q0 + q * 32 < p.Sq) tma_reduce_add_4d(&tmdQ, stg, (half * CH + cc) * 32, h, q0 + q * 32, b);
          tma_store_commit();
        }
      }
    }
    // ------------------------------ dK / dV epilogue ------------------------------
    // workers of half 0 write dK (staged in the P tile), those of half 1 write dV (staged in the dS tile)
    if (ok && n_iter > 0) ok = mbar_wait(acc_done, 0, abort_flag, p.status, 92);
    if (ok) {
      tc_fence_after();
      uint8_t* tile = (half == 0) ? sP : sdS;
      uint8_t* dst = tile + r * 128;
      const uint32_t src = (half == 0 ? tm_dK : tm_dV) + lane_base;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        if (n_iter > 0) { tmem_ld_32x32b_x32(src + c * 32, v); tc_wait_ld(); }
        else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        uint8_t* blk = dst + (c / 2) * (BKV * 128);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int sw = (((c & 1) * 4 + g) ^ (r & 7)) << 4;
          *reinterpret_cast<uint4*>(blk + sw) = make_uint4(
              pack_bf16x2(__uint_as_float(v[8 * g]), __uint_as_float(v[8 * g + 1])),
              pack_bf16x2(__uint_as_float(v[8 * g + 2]), __uint_as_float(v[8 * g + 3])),
              pack_bf16x2(__uint_as_float(v[8 * g + 4]), __uint_as_float(v[8 * g + 5])),
              pack_bf16x2(__uint_as_float(v[8 * g + 6]), __uint_as_float(v[8 * g + 7])));
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && kv0 + q * 32 < p.Skv) {
#pragma unroll
        for (int i = 0; i < NB; ++i)
          tma_store_4d(half == 0 ? &tmdK : &tmdV, tile + i * (BKV * 128) + q * 32 * 128, i * 64, hk, kv0 + q * 32, b);
        tma_store_commit();
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// delta[b, h, s] = sum_d O[b, s, h, d] * dO[b, s, h, d]; one warp per (token, head)
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, int B, int S, int H, int HD, long long o_row,
                                  long long do_row, long long o_batch, long long do_batch) {
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * S * H;
  if (w >= total) return;
  const int h = (int)(w % H);
  const long long t = w / H;
  const int s = (int)(t % S);
  const int b = (int)(t / S);
  const __nv_bfloat16* op = o + b * o_batch + (long long)s * o_row + h * HD;
  const __nv_bfloat16* dp = dout + b * do_batch + (long long)s * do_row + h * HD;
  float acc = 0.f;
  for (int d = lane * 2; d < HD; d += 64) {
    float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(op + d));
    float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dp + d));
    acc += a.x * g.x + a.y * g.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) delta[((long long)b * H + h) * S + s] = acc;
}

int qkv_map(CUtensorMap* m, const void* ptr, int HD, int H, int S, int B, long long row, long long batch, int box_rows) {
  return b200::make_tmap_4d(m, b200::DT_BF16, ptr, HD, H, S, B, (uint64_t)HD * 2, (uint64_t)row * 2,
                            (uint64_t)batch * 2, 64, 1, box_rows, 1, b200::SWZ_128);
}

template <int HD>
int launch_bwd(const CUtensorMap* m, const BwdParams& p, cudaStream_t stream) {
  using SM = Smem<HD>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL);
    if (e != cudaSuccess) cudaGetLastError();  // clear the sticky error before reporting
    if (e != cudaSuccess) return b200::fail(611, "attn_bwd: cannot set %d bytes of shared memory: %s", SM::TOTAL,
                                            cudaGetErrorString(e));
    configured[dev & 63] = true;
  }
  dim3 grid((p.Skv + BKV - 1) / BKV, p.Hkv, p.B);
  attn_bwd_kernel<HD><<<grid, NTHREADS, SM::TOTAL, stream>>>(m[0], m[1], m[2], m[3], m[4], m[5], m[6], p);
  b200::count_launch();
  return b200::check_launch("attn_bwd");
}

}  // namespace

// delta = rowsum(O * dO), [B, H, S] fp32
B200_API int b200_attn_delta(const void* o, const void* dout, float* delta, int B, int S, int H, int HD,
                             long long o_row, long long do_row, long long o_batch, long long do_batch, void* stream) {
  const long long warps = (long long)B * S * H;
  if (warps == 0) return 0;
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  attn_delta_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, B, S, H, HD, o_row, do_row, o_batch, do_batch);
  b200::count_launch();
  return b200::check_launch("attn_delta");
}

// dq_acc: fp32 [B, Sq, Hq, HD] contiguous, zero-initialised by the caller (reduce-add target).
// dk / dv: bf16 [B, Skv, Hkv, HD] with their own pitches.
B200_API int b200_attn_bwd(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                           const float* delta, float* dq_acc, void* dk, void* dv, int B, int Sq, int Skv, int Hq,
                           int Hkv, int HD, long long q_row, long long k_row, long long v_row, long long do_row,
                           long long dk_row, long long dv_row, long long q_batch, long long k_batch,
                           long long v_batch, long long do_batch, long long dk_batch, long long dv_batch,
                           float scale, int causal, int window, void* stream) {
  if (HD != 64 && HD != 128) return b200::fail(610, "attn_bwd: head dim %d not supported (64 or 128)", HD);
  if (Hq % Hkv != 0) return b200::fail(610, "attn_bwd: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
  CUtensorMap m[7];
  int r;
  if ((r = qkv_map(&m[0], q, HD, Hq, Sq, B, q_row, q_batch, BQ))) return r;
  if ((r = qkv_map(&m[1], k, HD, Hkv, Skv, B, k_row, k_batch, BKV))) return r;
  if ((r = qkv_map(&m[2], v, HD, Hkv, Skv, B, v_row, v_batch, BKV))) return r;
  if ((r = qkv_map(&m[3], dout, HD, Hq, Sq, B, do_row, do_batch, BQ))) return r;
  if ((r = b200::make_tmap_4d(&m[4], b200::DT_F32, dq_acc, HD, Hq, Sq, B, (uint64_t)HD * 4, (uint64_t)Hq * HD * 4,
                              (uint64_t)Sq * Hq * HD * 4, 32, 1, 32, 1, b200::SWZ_128)))
    return r;
  if ((r = qkv_map(&m[5], dk, HD, Hkv, Skv, B, dk_row, dk_batch, 32))) return r;
  if ((r = qkv_map(&m[6], dv, HD, Hkv, Skv, B, dv_row, dv_batch, 32))) return r;
  BwdParams p;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq; p.Skv = Skv;
  p.causal = causal; p.window = window;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = lse; p.delta = delta;
  p.status = b200::status_ptr();
  if (HD == 128) return launch_bwd<128>(m, p, (cudaStream_t)stream);
  return launch_bwd<64>(m, p, (cudaStream_t)stream);
}
