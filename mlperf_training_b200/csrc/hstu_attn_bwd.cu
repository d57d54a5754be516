// Jagged HSTU attention backward for sm_100a.  With P = silu(alpha S) / N * mask and S = Q K^T:
//
//   dV += P^T dO      dP = dO V^T      dS = dP * silu'(alpha S) * alpha / N * mask
//   dQ  = dS K        dK += dS^T Q
//
// One CTA per (sequence, head, 128-key tile) loops over the query tiles that see those keys; same
// engine as attention_bwd.cu (TMA loads, five tcgen05 GEMMs with dK / dV resident in TMEM, P and
// dS as bf16 shared-memory tiles read both K-major and MN-major, dQ leaving through fp32 TMA
// reduce-add).  No row statistics are needed, so nothing but Q, K, V, dO is read.
// Mask and jagged layout as in hstu_attn_fwd.cu.
//
// Math oracle: autograd of generative_recommenders/ops/pytorch/pt_hstu_attention.py:130-187; the
// reference's production kernels are generative_recommenders/ops/flydsl/hstu_bwd_dkdv.py and
// generative_recommenders/ops/triton/triton_hstu_attention.py (_hstu_attn_bwd).
#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int NTHREADS = 320;
constexpr int STG = 4096;

struct HstuBwdParams {
  int max_len, H, contextual;
  float alpha;
  const int* offsets;
  const int* num_targets;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  long long dk_row, dv_row;
  int* status;
};

B200_DEVICE float tanh_approx(float x) {
  float y;
  asm volatile("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
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
hstu_attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const __grid_constant__ CUtensorMap tmdQ, const HstuBwdParams p) {
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
  const int jt = blockIdx.x;  // key tile; early tiles see the most queries and are scheduled first
  const int hk = blockIdx.y, b = blockIdx.z;
  const int row_base = p.offsets[b];
  const int len = p.offsets[b + 1] - row_base;
  const int kv0 = jt * BKV;
  if (kv0 >= len) return;     // grid is sized by the maximum length
  const int n_tgt = p.num_targets ? p.num_targets[b] : 0;
  const int ctx = p.contextual;
  const int hist_end = len - n_tgt;
  const int max_id = hist_end - (ctx > 0 ? ctx - 1 : 0);
  // query tiles that see at least one key of this tile: the causal range, plus tile 0 when it
  // holds contextual rows (they see every history column)
  const int i_lo = kv0 / BQ, i_hi = (len - 1) / BQ;
  const int extra = (ctx > 0 && i_lo > 0) ? 1 : 0;
  const int n_q = (i_hi - i_lo + 1) + extra;
  const int n_iter = n_q;
  auto q_tile = [&](int it) { return (extra && it == 0) ? 0 : i_lo + it - extra; };

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
        tma_load_3d(sK + i * (BKV * 128), &tmK, kv_full, i * 64, hk, row_base + kv0);
        tma_load_3d(sV + i * (BKV * 128), &tmV, kv_full, i * 64, hk, row_base + kv0);
      }
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int h = hk;
        const int q0 = q_tile(it) * BQ;
        if (!mbar_wait(qdo_empty, (it & 1) ^ 1, abort_flag, p.status, 70)) { ok = false; break; }
        mbar_expect_tx(qdo_full, 2 * SM::T_BYTES);
#pragma unroll
        for (int i = 0; i < NB; ++i) {
          tma_load_3d(sQ + i * (BQ * 128), &tmQ, qdo_full, i * 64, h, row_base + q0);
          tma_load_3d(sdO + i * (BQ * 128), &tmdO, qdo_full, i * 64, h, row_base + q0);
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
    // ------------------------------ workers (warps 2-9): P / dS, then dQ drain ------------------------------
    // Two workers share a TMEM lane quarter: each handles half of the key columns, then half of the
    // dQ columns (registers, accumulator released, fp32 TMA reduce-add while the next GEMMs run).
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = q * 32 + lane;
    const uint32_t lane_base = uint32_t(q * 32) << 16;
    uint8_t* stg = sStg + (warp - 2) * STG;
    constexpr int CH = HD / 64;
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int h = hk;
      const int q0 = q_tile(it) * BQ;
      const int q_pos = q0 + r;
      const bool row_ok = q_pos < len;
      const int q_id = min(max(q_pos - ctx + (ctx > 0 ? 1 : 0), 0), max_id);
      const bool plain = (n_tgt == 0 && ctx == 0);
      // a tile whose every (query, key) pair is visible needs no element mask: ids grow with the position, so it
      // is enough that the tile's first query is later than its last key, and that both tiles lie inside the sequence
      const int first_q_id = min(max(q0 - ctx + (ctx > 0 ? 1 : 0), 0), max_id);
      const int last_k_id = min(max(kv0 + BKV - 1 - ctx + (ctx > 0 ? 1 : 0), 0), max_id);
      const bool inside = (kv0 + BKV <= len) && (q0 + BQ <= len);
      const bool need_mask = plain ? ((kv0 + BKV - 1 > q0) || !inside) : !(inside && first_q_id > last_k_id);
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
        const float ha = 0.5f * p.alpha, inv_n = 1.0f / (float)p.max_len, an = p.alpha * inv_n;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          // P = silu(a s) / N ; dS = dP * silu'(a s) * a / N   (sig = (1 + tanh(a s / 2)) / 2)
          const float hx = __uint_as_float(s[i]) * ha;
          const float sig = 0.5f * (1.f + tanh_approx(hx));
          const float x = 2.f * hx;
          float p0 = x * sig * inv_n;
          float g0 = __uint_as_float(d[i]) * sig * (1.f + x * (1.f - sig)) * an;
          if (need_mask) {
            const int kp = kv0 + c * 32 + i;
            bool vis;
            if (plain) vis = kp <= q_pos;
            else {
              const int k_id = min(max(kp - ctx + (ctx > 0 ? 1 : 0), 0), max_id);
              vis = (kp == q_pos) || (q_id > k_id) || (ctx > 0 && q_id == 0 && kp < hist_end);
            }
            if (!(vis && kp < len && row_ok)) { p0 = 0.f; g0 = 0.f; }
          }
          pv[i] = p0;
          dv[i] = g0;
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
      if (lane == 0) mbar_arrive(dq_drained);
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
          if (q0 + q * 32 < len) tma_reduce_add_3d(&tmdQ, stg, (half * CH + cc) * 32, h, row_base + q0 + q * 32);
          tma_store_commit();
        }
      }
    }
    // ------------------------------ dK / dV epilogue ------------------------------
    // workers of half 0 write dK, those of half 1 write dV; guarded row stores: rows past the
    // sequence end belong to the next sequence
    if (ok && n_iter > 0) ok = mbar_wait(acc_done, 0, abort_flag, p.status, 92);
    if (ok) {
      tc_fence_after();
      const int k_pos = kv0 + r;
      __nv_bfloat16* dst = (half == 0 ? p.dk : p.dv) + (long long)(row_base + k_pos) * (half == 0 ? p.dk_row : p.dv_row) + hk * HD;
      const uint32_t src = (half == 0 ? tm_dK : tm_dV) + lane_base;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(src + c * 32, v);
        tc_wait_ld();
        if (k_pos < len) {
#pragma unroll
          for (int g = 0; g < 4; ++g)
            *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = make_uint4(
                pack_bf16x2(__uint_as_float(v[8 * g]), __uint_as_float(v[8 * g + 1])),
                pack_bf16x2(__uint_as_float(v[8 * g + 2]), __uint_as_float(v[8 * g + 3])),
                pack_bf16x2(__uint_as_float(v[8 * g + 4]), __uint_as_float(v[8 * g + 5])),
                pack_bf16x2(__uint_as_float(v[8 * g + 6]), __uint_as_float(v[8 * g + 7])));
        }
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

template <int HD>
int launch_hstu_bwd(const CUtensorMap* m, const HstuBwdParams& p, int B, cudaStream_t stream) {
  using SM = Smem<HD>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(hstu_attn_bwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL);
    if (e != cudaSuccess) { cudaGetLastError(); return b200::fail(1211, "hstu_attn_bwd: cannot set %d bytes of shared memory: %s", SM::TOTAL, cudaGetErrorString(e)); }
    configured[dev & 63] = true;
  }
  dim3 grid((p.max_len + BKV - 1) / BKV, p.H, B);
  hstu_attn_bwd_kernel<HD><<<grid, NTHREADS, SM::TOTAL, stream>>>(m[0], m[1], m[2], m[3], m[4], p);
  b200::count_launch();
  return b200::check_launch("hstu_attn_bwd");
}

}  // namespace

// q / k / v / dout: jagged [L, H, HD] bf16 views; dq_acc: fp32 [L, H, HD] contiguous, zeroed by the
// caller (reduce-add target); dk / dv: bf16 [L, H, HD] views (every valid row is written).
B200_API int b200_hstu_attn_bwd(const void* q, const void* k, const void* v, const void* dout, float* dq_acc, void* dk,
                                void* dv, const int* offsets, const int* num_targets, int B, long long L, int H, int HD,
                                int max_len, int contextual, long long q_row, long long k_row, long long v_row,
                                long long do_row, long long dk_row, long long dv_row, float alpha, void* stream) {
  if (HD != 64 && HD != 128) return b200::fail(1210, "hstu_attn_bwd: head dim %d not supported (64 or 128)", HD);
  if (L == 0 || B == 0) return 0;
  CUtensorMap m[5];
  int r;
  auto mk = [&](CUtensorMap* t, const void* ptr, long long row, int box) {
    return b200::make_tmap_3d(t, b200::DT_BF16, ptr, HD, H, L, (uint64_t)HD * 2, (uint64_t)row * 2, 64, 1, box, b200::SWZ_128);
  };
  if ((r = mk(&m[0], q, q_row, BQ))) return r;
  if ((r = mk(&m[1], k, k_row, BKV))) return r;
  if ((r = mk(&m[2], v, v_row, BKV))) return r;
  if ((r = mk(&m[3], dout, do_row, BQ))) return r;
  if ((r = b200::make_tmap_3d(&m[4], b200::DT_F32, dq_acc, HD, H, L, (uint64_t)HD * 4, (uint64_t)H * HD * 4, 32, 1, 32, b200::SWZ_128))) return r;
  HstuBwdParams p;
  p.max_len = max_len; p.H = H; p.contextual = contextual; p.alpha = alpha;
  p.offsets = offsets; p.num_targets = num_targets;
  p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv; p.dk_row = dk_row; p.dv_row = dv_row;
  p.status = b200::status_ptr();
  if (HD == 128) return launch_hstu_bwd<128>(m, p, B, (cudaStream_t)stream);
  return launch_hstu_bwd<64>(m, p, B, (cudaStream_t)stream);
}
