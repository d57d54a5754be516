// Persistent warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory (128B swizzle) ->
// tcgen05.mma (accumulators in TMEM, double buffered) -> tcgen05.ld epilogue -> TMA store.
//
//   D[M,N] (=|+=) op(A)[M,K] * op(B)[N,K]^T (+ bias[N]) (+ residual[M,N])
//
// A and B are each given either K-major (row-major [rows][K], the nn.Linear layout) or
// MN-major (row-major [K][rows]); the tensor core reads both straight from shared memory, so
// forward (x W^T), dgrad (dy W) and wgrad (dy^T x) need no transposed copies.
//
// Roles (192 threads, one CTA per SM, static round-robin tile schedule with grouped raster):
//   warp 0     TMA producer           (one elected lane)
//   warp 1     tcgen05.mma issuer     (one lane) + TMEM allocation
//   warps 2-5  epilogue               (TMEM lanes 32*(warp%4) .. +31)
//
// Takes the place of the reference's library GEMM calls (hipBLASLt through torch.addmm,
// generative_recommenders/ops/hstu_compute.py:122-126) and of its hand-written MFMA GEMMs
// (generative_recommenders/ops/hip/k512_fp8_gemm.cu, k1536_fp8_addmm.cu) at bf16 precision.
#include <cstdlib>

#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;            // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int EPI_WARPS = 4;
constexpr int STG_BYTES = 4096;   // one epilogue staging buffer: 32 rows x 128 bytes

template <int BN>
struct Cfg {
  static constexpr int A_STAGE = BM * BK * 2;
  static constexpr int B_STAGE = BN * BK * 2;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int EPI_BYTES = EPI_WARPS * 2 * STG_BYTES;
  static constexpr int SMEM = STAGES * (A_STAGE + B_STAGE) + EPI_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int TMEM_COLS = 2 * BN;  // double-buffered fp32 accumulator
};

struct Params {
  int M, N, K;
  int a_mn_major, b_mn_major;
  int out_f32;        // 0: bf16 output, 1: fp32 output
  int accumulate;     // 0: store, 1: reduce-add into D
  int group_m;        // raster group height in tiles
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldr] or null
  long long ldr;
  float alpha;        // scale applied to the accumulator before bias/residual
  int* status;
};

B200_DEVICE void tile_coords(int t, int num_m, int num_n, int group_m, int& mb, int& nb) {
  int in_group = group_m * num_n;
  int g = t / in_group;
  int first_m = g * group_m;
  int gsz = min(num_m - first_m, group_m);
  int r = t - g * in_group;
  mb = first_m + (r % gsz);
  nb = r / gsz;
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmD, const Params p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + C::STAGES * C::A_STAGE;
  uint8_t* sE = sB + C::STAGES * C::B_STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sE + C::EPI_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + C::STAGES;
  uint64_t* tfull = bars + 2 * C::STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], EPI_WARPS); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, C::TMEM_COLS);
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
        int mb, nb; tile_coords(t, num_m, num_n, p.group_m, mb, nb);
        const int m0 = mb * BM, n0 = nb * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, 10)) { ok = false; break; }
          mbar_expect_tx(&full[stage], C::A_STAGE + C::B_STAGE);
          uint8_t* a_dst = sA + stage * C::A_STAGE;
          uint8_t* b_dst = sB + stage * C::B_STAGE;
          const int k0 = kb * BK;
          if (!p.a_mn_major) {
            tma_load_2d(a_dst, &tmA, &full[stage], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * (BK * 128), &tmA, &full[stage], m0 + 64 * j, k0);
          }
          if (!p.b_mn_major) {
            tma_load_2d(b_dst, &tmB, &full[stage], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * (BK * 128), &tmB, &full[stage], n0 + 64 * j, k0);
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
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
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag, p.status, 20)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, 21)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * C::A_STAGE);
          const uint32_t b_addr = smem_u32(sB + stage * C::B_STAGE);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t ad = umma_desc_sw128(a_addr + kk * a_kstep, a_lbo, 1024);
            const uint64_t bd = umma_desc_sw128(b_addr + kk * b_kstep, b_lbo, 1024);
            tc_mma_f16_ss(d_tmem, ad, bd, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&empty[stage]);  // frees the smem stage once these MMAs have read it
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&tfull[acc]);  // accumulator complete
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;                 // TMEM lane quarter owned by this warp
    const int ew = warp - 2;                // staging slot
    uint8_t* stg = sE + ew * 2 * STG_BYTES;
    int buf = 0;
    int it = 0;
    bool ok = true;
    const bool vec_res = p.residual != nullptr && (p.ldr % 8 == 0) && (p.N % 8 == 0) &&
                         ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0);
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      int mb, nb; tile_coords(t, num_m, num_n, p.group_m, mb, nb);
      const int m0 = mb * BM, n0 = nb * BN;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag, p.status, 30)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;   // global row of this thread
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
        if (p.bias != nullptr) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (col0 + i < p.N) v[i] += __bfloat162float(p.bias[col0 + i]);
        }
        if (p.residual != nullptr && row < p.M) {
          const __nv_bfloat16* rp = p.residual + (long long)row * p.ldr + col0;
          if (vec_res) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (col0 + j * 8 < p.N) {
                uint4 u = *reinterpret_cast<const uint4*>(rp + j * 8);
                float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
                v[j * 8 + 0] += f0.x; v[j * 8 + 1] += f0.y; v[j * 8 + 2] += f1.x; v[j * 8 + 3] += f1.y;
                v[j * 8 + 4] += f2.x; v[j * 8 + 5] += f2.y; v[j * 8 + 6] += f3.x; v[j * 8 + 7] += f3.y;
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) v[i] += __bfloat162float(rp[i]);
          }
        }
        if (p.out_f32) {
          // one staging buffer = 32 rows x 32 fp32 (128 bytes per row)
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
          uint8_t* sb = stg + buf * STG_BYTES + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 u = make_uint4(__float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]),
                                 __float_as_uint(v[4 * j + 2]), __float_as_uint(v[4 * j + 3]));
            *reinterpret_cast<uint4*>(sb + ((j ^ (lane & 7)) << 4)) = u;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (col0 < p.N && m0 + q * 32 < p.M) {
              if (p.accumulate) tma_reduce_add_2d(&tmD, stg + buf * STG_BYTES, col0, m0 + q * 32);
              else tma_store_2d(&tmD, stg + buf * STG_BYTES, col0, m0 + q * 32);
            }
            tma_store_commit();
          }
          buf ^= 1;
        } else {
          // one staging buffer = 32 rows x 64 bf16; two 32-column chunks fill it
          const int half = c & 1;
          if (half == 0) {
            if (lane == 0) tma_store_wait_read<1>();
            __syncwarp();
          }
          uint8_t* sb = stg + buf * STG_BYTES + lane * 128;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 u = make_uint4(pack_bf16x2(v[8 * j], v[8 * j + 1]), pack_bf16x2(v[8 * j + 2], v[8 * j + 3]),
                                 pack_bf16x2(v[8 * j + 4], v[8 * j + 5]), pack_bf16x2(v[8 * j + 6], v[8 * j + 7]));
            const int chunk = half * 4 + j;
            *reinterpret_cast<uint4*>(sb + ((chunk ^ (lane & 7)) << 4)) = u;
          }
          if (half == 1) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              const int cs = col0 - 32;
              if (cs < p.N && m0 + q * 32 < p.M) {
                if (p.accumulate) tma_reduce_add_2d(&tmD, stg + buf * STG_BYTES, cs, m0 + q * 32);
                else tma_store_2d(&tmD, stg + buf * STG_BYTES, cs, m0 + q * 32);
              }
              tma_store_commit();
            }
            buf ^= 1;
          }
        }
      }
      // all TMEM reads of this accumulator are complete (tc_wait_ld above): hand it back
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  // ------------------------------ teardown ------------------------------
  if (*abort_flag) {
    // let copies that are still in flight land before shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

template <int BN>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD, const Params& p,
           cudaStream_t stream) {
  using C = Cfg<BN>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) cudaGetLastError();  // clear the sticky error before reporting
    if (e != cudaSuccess) return b200::fail(201, "gemm_bf16: cannot set %d bytes of shared memory: %s", C::SMEM,
                                            cudaGetErrorString(e));
    configured[dev & 63] = true;
  }
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  const int tiles = num_m * num_n;
  const int grid = tiles < b200::sm_count() ? tiles : b200::sm_count();
  gemm_bf16_kernel<BN><<<grid, NUM_THREADS, C::SMEM, stream>>>(tmA, tmB, tmD, p);
  b200::count_launch();
  return b200::check_launch("gemm_bf16");
}

// Height (in tiles) of a raster group: consecutive CTAs work on `group_m` row tiles of one column tile, so the
// column's B tile is shared in L2 while the group's A rows stay resident (B200_GEMM_GROUP_M overrides).
static int raster_group_m() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B200_GEMM_GROUP_M");
    v = (e && atoi(e) > 0) ? atoi(e) : 16;
  }
  return v;
}

}  // namespace

// D[M,N] (=|+=) alpha * A * B^T (+ bias) (+ residual)
//   a: K-major [M, lda] (a_mn_major = 0) or MN-major [K, lda] (a_mn_major = 1); same for b with N.
//   lda / ldb / ldd / ldr are row pitches in elements.  out_f32 selects fp32 D.  accumulate != 0 adds into D.
B200_API int b200_gemm_bf16(const void* a, const void* b, void* d, int M, int N, int K, long long lda,
                            long long ldb, long long ldd, int a_mn_major, int b_mn_major, int out_f32,
                            int accumulate, const void* bias, const void* residual, long long ldr, float alpha,
                            void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return b200::fail(210, "gemm_bf16: empty problem %d x %d x %d", M, N, K);
  const int BN = (N > 128) ? 256 : 128;
  CUtensorMap tmA, tmB, tmD;
  int r;
  if (!a_mn_major) r = b200::make_tmap_2d(&tmA, b200::DT_BF16, a, K, M, lda * 2, BK, BM, b200::SWZ_128);
  else r = b200::make_tmap_2d(&tmA, b200::DT_BF16, a, M, K, lda * 2, 64, BK, b200::SWZ_128);
  if (r) return r;
  if (!b_mn_major) r = b200::make_tmap_2d(&tmB, b200::DT_BF16, b, K, N, ldb * 2, BK, BN, b200::SWZ_128);
  else r = b200::make_tmap_2d(&tmB, b200::DT_BF16, b, N, K, ldb * 2, 64, BK, b200::SWZ_128);
  if (r) return r;
  if (out_f32) r = b200::make_tmap_2d(&tmD, b200::DT_F32, d, N, M, ldd * 4, 32, 32, b200::SWZ_128);
  else r = b200::make_tmap_2d(&tmD, b200::DT_BF16, d, N, M, ldd * 2, 64, 32, b200::SWZ_128);
  if (r) return r;
  Params p;
  p.M = M; p.N = N; p.K = K;
  p.a_mn_major = a_mn_major ? 1 : 0; p.b_mn_major = b_mn_major ? 1 : 0;
  p.out_f32 = out_f32 ? 1 : 0; p.accumulate = accumulate ? 1 : 0;
  p.group_m = raster_group_m();
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.alpha = alpha;
  p.status = b200::status_ptr();
  if (BN == 256) return launch<256>(tmA, tmB, tmD, p, (cudaStream_t)stream);
  return launch<128>(tmA, tmB, tmD, p, (cudaStream_t)stream);
}
