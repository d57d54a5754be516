// Grouped (per-expert) bf16 GEMMs of the MoE layer as single persistent launches driven by a
// device-resident plan - no host read of the routing result anywhere.
//
// Rows of the permuted activation buffer are grouped by expert; every expert's segment starts at
// a multiple of 128 rows (router.cu pads), so a 128-row tile never straddles two experts.
//
//   mode 1 (forward, dgrad)  D[r, :] = A[r, :] * op(B[e(r)])^T   for the rows r of each tile;
//                            B is a 3-D tensor [E][..][..], the expert of tile i is tile_expert[i]
//                            (-1 = tile beyond the last segment: skipped by all roles)
//   mode 2 (wgrad)           D[e] (+)= A[seg[e]:seg[e+1], :]^T * B[seg[e]:seg[e+1], :]
//                            the contraction runs over the expert's rows; D is [E][M][N]
//
// Same roles, pipeline and epilogue as gemm_bf16.cu.  The reference gets this from Primus-Turbo's
// grouped GEMM / fused grouped MLP (small_llm_moe_pretraining/primus/conf/
// gpt_oss_20B-MXFP4-deosc-mlperf-pretrain.yaml:186-222).
#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int EPI_WARPS = 4;
constexpr int STG_BYTES = 4096;
constexpr int A_STAGE = BM * BK * 2;
constexpr int B_STAGE = BN * BK * 2;
constexpr int STAGES = 4;
constexpr int EPI_BYTES = EPI_WARPS * 2 * STG_BYTES;
constexpr int SMEM = STAGES * (A_STAGE + B_STAGE) + EPI_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 2 * BN;

struct Params {
  int M, N, K;            // mode 1: M = rows of the padded buffer; mode 2: M, N = per-expert output, K unused
  int mode, E;
  int a_mn_major, b_mn_major;
  int out_f32, accumulate;
  const int* tile_expert; // mode 1: [ceil(M / 128)]
  const int* seg;         // mode 2: [E + 1] padded row offsets
  float alpha;
  int* status;
};

struct Tile {
  int mb, nb, e, row0, nkb;
  bool valid;
};

B200_DEVICE Tile tile_info(int t, int num_m, int num_n, const Params& p) {
  Tile ti;
  if (p.mode == 1) {
    ti.nb = t / num_m;       // m fastest: consecutive CTAs share one expert's weight tile in L2
    ti.mb = t - ti.nb * num_m;
    ti.e = p.tile_expert[ti.mb];
    ti.row0 = 0;
    ti.nkb = (p.K + BK - 1) / BK;
    ti.valid = ti.e >= 0;
  } else {
    const int per = num_m * num_n;
    ti.e = t / per;
    const int r = t - ti.e * per;
    ti.nb = r / num_m;
    ti.mb = r - ti.nb * num_m;
    ti.row0 = p.seg[ti.e];
    ti.nkb = (p.seg[ti.e + 1] - ti.row0) / BK;
    ti.valid = ti.nkb > 0;
  }
  return ti;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_grouped_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmD, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + STAGES * A_STAGE;
  uint8_t* sE = sB + STAGES * B_STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sE + EPI_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = (p.mode == 1 ? 1 : p.E) * num_m * num_n;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], EPI_WARPS); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Tile ti = tile_info(t, num_m, num_n, p);
        if (!ti.valid) continue;
        const int m0 = ti.mb * BM, n0 = ti.nb * BN;
        for (int kb = 0; kb < ti.nkb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, 140)) { ok = false; break; }
          mbar_expect_tx(&full[stage], A_STAGE + B_STAGE);
          uint8_t* a_dst = sA + stage * A_STAGE;
          uint8_t* b_dst = sB + stage * B_STAGE;
          const int k0 = ti.row0 + kb * BK;
          if (!p.a_mn_major) {
            tma_load_2d(a_dst, &tmA, &full[stage], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * (BK * 128), &tmA, &full[stage], m0 + 64 * j, k0);
          }
          if (p.mode == 1) {
            if (!p.b_mn_major) {
              tma_load_3d(b_dst, &tmB, &full[stage], k0, n0, ti.e);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_3d(b_dst + j * (BK * 128), &tmB, &full[stage], n0 + 64 * j, k0, ti.e);
            }
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * (BK * 128), &tmB, &full[stage], n0 + 64 * j, k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(1, 1, p.a_mn_major, p.b_mn_major, BM, BN);
      const uint32_t a_lbo = p.a_mn_major ? BK * 128 : 16;
      const uint32_t b_lbo = p.b_mn_major ? BK * 128 : 16;
      const uint32_t a_kstep = p.a_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      const uint32_t b_kstep = p.b_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Tile ti = tile_info(t, num_m, num_n, p);
        if (!ti.valid) continue;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ++it;
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag, p.status, 150)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < ti.nkb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, 151)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * A_STAGE);
          const uint32_t b_addr = smem_u32(sB + stage * B_STAGE);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t ad = umma_desc_sw128(a_addr + kk * a_kstep, a_lbo, 1024);
            const uint64_t bd = umma_desc_sw128(b_addr + kk * b_kstep, b_lbo, 1024);
            tc_mma_f16_ss(d_tmem, ad, bd, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&tfull[acc]);
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;
    const int ew = warp - 2;
    uint8_t* stg = sE + ew * 2 * STG_BYTES;
    int buf = 0;
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const Tile ti = tile_info(t, num_m, num_n, p);
      if (!ti.valid) continue;
      const int m0 = ti.mb * BM, n0 = ti.nb * BN;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ++it;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag, p.status, 160)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        tc_wait_ld();
        const int col0 = n0 + c * 32;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        if (p.out_f32) {
          uint8_t* sb = stg + buf * STG_BYTES + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(sb + ((j ^ (lane & 7)) << 4)) =
                make_uint4(__float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]), __float_as_uint(v[4 * j + 2]),
                           __float_as_uint(v[4 * j + 3]));
        } else {
          uint8_t* sb = stg + buf * STG_BYTES + lane * 64;   // dense 64-byte rows, 64-byte swizzle
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(sb + ((j ^ ((lane >> 1) & 3)) << 4)) =
                make_uint4(pack_bf16x2(v[8 * j], v[8 * j + 1]), pack_bf16x2(v[8 * j + 2], v[8 * j + 3]),
                           pack_bf16x2(v[8 * j + 4], v[8 * j + 5]), pack_bf16x2(v[8 * j + 6], v[8 * j + 7]));
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (col0 < p.N && m0 + q * 32 < p.M) {
            if (p.mode == 1) {
              if (p.accumulate) tma_reduce_add_2d(&tmD, stg + buf * STG_BYTES, col0, m0 + q * 32);
              else tma_store_2d(&tmD, stg + buf * STG_BYTES, col0, m0 + q * 32);
            } else {
              if (p.accumulate) tma_reduce_add_3d(&tmD, stg + buf * STG_BYTES, col0, m0 + q * 32, ti.e);
              else tma_store_3d(&tmD, stg + buf * STG_BYTES, col0, m0 + q * 32, ti.e);
            }
          }
          tma_store_commit();
        }
        buf ^= 1;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD, const Params& p, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) { cudaGetLastError(); return b200::fail(1001, "gemm_grouped: cannot set %d bytes of shared memory: %s", SMEM, cudaGetErrorString(e)); }
    configured[dev & 63] = true;
  }
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  const long long tiles = (long long)(p.mode == 1 ? 1 : p.E) * num_m * num_n;
  const int grid = tiles < b200::sm_count() ? (int)tiles : b200::sm_count();
  gemm_grouped_kernel<<<grid, NUM_THREADS, SMEM, stream>>>(tmA, tmB, tmD, p);
  b200::count_launch();
  return b200::check_launch("gemm_grouped");
}

}  // namespace

// Forward / dgrad over the padded, expert-grouped row buffer:
//   d[r, :] = alpha * a[r, :] @ op(b[e(r)])^T,  e(r) = tile_expert[r / 128]
// a: [rows, K] bf16; b: [E, N, K] (b_mn_major = 0) or [E, K, N] (b_mn_major = 1); d: [rows, N].
B200_API int b200_gemm_grouped_rows(const void* a, const void* b, void* d, const int* tile_expert, int rows, int N, int K,
                                    int E, long long lda, long long ldd, int b_mn_major, int out_f32, float alpha,
                                    void* stream) {
  if (rows % 128 != 0) return b200::fail(1010, "gemm_grouped_rows: rows=%d must be a multiple of 128", rows);
  CUtensorMap tmA, tmB, tmD;
  int r;
  if ((r = b200::make_tmap_2d(&tmA, b200::DT_BF16, a, K, rows, lda * 2, BK, BM, b200::SWZ_128))) return r;
  if (!b_mn_major) r = b200::make_tmap_3d(&tmB, b200::DT_BF16, b, K, N, E, (uint64_t)K * 2, (uint64_t)N * K * 2, BK, BN, 1, b200::SWZ_128);
  else r = b200::make_tmap_3d(&tmB, b200::DT_BF16, b, N, K, E, (uint64_t)N * 2, (uint64_t)N * K * 2, 64, BK, 1, b200::SWZ_128);
  if (r) return r;
  if (out_f32) r = b200::make_tmap_2d(&tmD, b200::DT_F32, d, N, rows, ldd * 4, 32, 32, b200::SWZ_128);
  else r = b200::make_tmap_2d(&tmD, b200::DT_BF16, d, N, rows, ldd * 2, 32, 32, b200::SWZ_64);
  if (r) return r;
  Params p{};
  p.M = rows; p.N = N; p.K = K; p.mode = 1; p.E = E;
  p.a_mn_major = 0; p.b_mn_major = b_mn_major ? 1 : 0;
  p.out_f32 = out_f32 ? 1 : 0; p.accumulate = 0;
  p.tile_expert = tile_expert; p.seg = nullptr;
  p.alpha = alpha; p.status = b200::status_ptr();
  return launch(tmA, tmB, tmD, p, (cudaStream_t)stream);
}

// Weight gradient: d[e] (+)= alpha * a[seg[e]:seg[e+1], :]^T @ b[seg[e]:seg[e+1], :]
// a: [rows, M] (dy), b: [rows, N] (x), d: [E, M, N] bf16 or fp32.  With accumulate == 0 the caller must
// have cleared d (experts without rows are skipped).
B200_API int b200_gemm_grouped_wgrad(const void* a, const void* b, void* d, const int* seg, int rows, int M, int N, int E,
                                     long long lda, long long ldb, int out_f32, int accumulate, float alpha,
                                     void* stream) {
  CUtensorMap tmA, tmB, tmD;
  int r;
  if ((r = b200::make_tmap_2d(&tmA, b200::DT_BF16, a, M, rows, lda * 2, 64, BK, b200::SWZ_128))) return r;
  if ((r = b200::make_tmap_2d(&tmB, b200::DT_BF16, b, N, rows, ldb * 2, 64, BK, b200::SWZ_128))) return r;
  if (out_f32) r = b200::make_tmap_3d(&tmD, b200::DT_F32, d, N, M, E, (uint64_t)N * 4, (uint64_t)M * N * 4, 32, 32, 1, b200::SWZ_128);
  else r = b200::make_tmap_3d(&tmD, b200::DT_BF16, d, N, M, E, (uint64_t)N * 2, (uint64_t)M * N * 2, 32, 32, 1, b200::SWZ_64);
  if (r) return r;
  Params p{};
  p.M = M; p.N = N; p.K = 0; p.mode = 2; p.E = E;
  p.a_mn_major = 1; p.b_mn_major = 1;
  p.out_f32 = out_f32 ? 1 : 0; p.accumulate = accumulate ? 1 : 0;
  p.tile_expert = nullptr; p.seg = seg;
  p.alpha = alpha; p.status = b200::status_ptr();
  return launch(tmA, tmB, tmD, p, (cudaStream_t)stream);
}
