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
#include "gemm_core.cuh"
#include "runtime.h"

namespace {

using gemmcore::tile_coords;

constexpr int BM = 128;
constexpr int BK = 64;            // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = gemmcore::NUM_THREADS;
constexpr int EPI_WARPS = gemmcore::EPI_WARPS;
constexpr int STG_BYTES = gemmcore::STG_BYTES;   // one epilogue staging buffer: 32 rows x 128 bytes

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
  int group_m;        // raster group height in tiles
  gemmcore::EpiArgs epi = {};
  int* status;
};

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
    uint8_t* stg = sE + (warp - 2) * 2 * STG_BYTES;
    int buf = 0;
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      int mb, nb; tile_coords(t, num_m, num_n, p.group_m, mb, nb);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag, p.status, 30)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
      gemmcore::epilogue_drain<BN, true>(&tmD, &tmD, p.epi, t_row, mb * BM + q * 32, nb * BN, stg, buf, lane);
      // all TMEM reads of this accumulator are complete: hand it back
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

}  // namespace

// One CTA pair per 256 x BN tile (gemm_core.cuh).
template <int BN>
static int run_pair(const void* a, const void* b, void* d, int M, int N, int K, long long lda, long long ldb,
                    long long ldd, int a_mn_major, int b_mn_major, const gemmcore::EpiArgs& epi, cudaStream_t stream) {
  using namespace gemmcore;
  CUtensorMap tmA, tmB, tmD;
  int r;
  if (!a_mn_major) r = b200::make_tmap_2d(&tmA, b200::DT_BF16, a, K, M, lda * 2, BK, 128, b200::SWZ_128);
  else r = b200::make_tmap_2d(&tmA, b200::DT_BF16, a, M, K, lda * 2, 64, BK, b200::SWZ_128);
  if (r) return r;
  if (!b_mn_major) r = b200::make_tmap_2d(&tmB, b200::DT_BF16, b, K, N, ldb * 2, BK, BN / 2, b200::SWZ_128);
  else r = b200::make_tmap_2d(&tmB, b200::DT_BF16, b, N, K, ldb * 2, 64, BK, b200::SWZ_128);
  if (r) return r;
  CUtensorMap tmDt;
  if ((r = make_out_tmap<BN>(&tmD, &tmDt, d, M, N, ldd, epi.out_f32))) return r;
  PairParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major;
  p.a_fmt = 0; p.b_fmt = 0;
  p.group_m = raster_group_m() > 1 ? raster_group_m() / 2 : 1;
  p.epi = epi;
  p.status = b200::status_ptr();
  return launch_pair<KIND_BF16, BN, 1>(tmA, tmB, tmA, tmB, tmD, tmDt, p, stream, "gemm_bf16(pair)");
}

// D[M,N] (=|+=) alpha * A * B^T (+ bias) (+ residual)
//   a: K-major [M, lda] (a_mn_major = 0) or MN-major [K, lda] (a_mn_major = 1); same for b with N.
//   lda / ldb / ldd / ldr are row pitches in elements.  out_f32 selects fp32 D.  accumulate != 0 adds into D.
B200_API int b200_gemm_bf16(const void* a, const void* b, void* d, int M, int N, int K, long long lda,
                            long long ldb, long long ldd, int a_mn_major, int b_mn_major, int out_f32,
                            int accumulate, const void* bias, const void* residual, long long ldr, float alpha,
                            void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return b200::fail(210, "gemm_bf16: empty problem %d x %d x %d", M, N, K);
  const int BN = (N > 128) ? 256 : 128;
  gemmcore::EpiArgs epi = {};
  epi.M = M; epi.N = N;
  epi.out_f32 = out_f32 ? 1 : 0; epi.accumulate = accumulate ? 1 : 0;
  epi.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  epi.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  epi.ldr = ldr;
  epi.alpha = alpha;
  if (M > 128 && gemmcore::pair_enabled()) {
    if (BN == 256) return run_pair<256>(a, b, d, M, N, K, lda, ldb, ldd, a_mn_major ? 1 : 0, b_mn_major ? 1 : 0, epi,
                                        (cudaStream_t)stream);
    return run_pair<128>(a, b, d, M, N, K, lda, ldb, ldd, a_mn_major ? 1 : 0, b_mn_major ? 1 : 0, epi,
                         (cudaStream_t)stream);
  }
  CUtensorMap tmA, tmB, tmD, tmDt;
  int r;
  if (!a_mn_major) r = b200::make_tmap_2d(&tmA, b200::DT_BF16, a, K, M, lda * 2, BK, BM, b200::SWZ_128);
  else r = b200::make_tmap_2d(&tmA, b200::DT_BF16, a, M, K, lda * 2, 64, BK, b200::SWZ_128);
  if (r) return r;
  if (!b_mn_major) r = b200::make_tmap_2d(&tmB, b200::DT_BF16, b, K, N, ldb * 2, BK, BN, b200::SWZ_128);
  else r = b200::make_tmap_2d(&tmB, b200::DT_BF16, b, N, K, ldb * 2, 64, BK, b200::SWZ_128);
  if (r) return r;
  r = (BN == 256) ? gemmcore::make_out_tmap<256>(&tmD, &tmDt, d, M, N, ldd, out_f32)
                  : gemmcore::make_out_tmap<128>(&tmD, &tmDt, d, M, N, ldd, out_f32);
  if (r) return r;
  Params p;
  p.M = M; p.N = N; p.K = K;
  p.a_mn_major = a_mn_major ? 1 : 0; p.b_mn_major = b_mn_major ? 1 : 0;
  p.group_m = gemmcore::raster_group_m();
  p.epi = epi;
  p.status = b200::status_ptr();
  if (BN == 256) return launch<256>(tmA, tmB, tmD, p, (cudaStream_t)stream);
  return launch<128>(tmA, tmB, tmD, p, (cudaStream_t)stream);
}
