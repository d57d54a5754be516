// Persistent warp-specialised MXFP8 block-scaled GEMM for sm_100a:
//
//   D[M,N] (=|+=) alpha * (A_q * 2^sfa)[M,K] * (B_q * 2^sfb)[N,K]^T (+ bias[N]) (+ residual[M,N])
//
// A_q / B_q are e4m3 codes, K-major; sfa / sfb hold one UE8M0 scale per 32 contraction elements in
// the atom layout written by quant_mxfp8.cu (tile rows = 128 for A, = BN for B; BN = 208 for N > 128).
//
// Two kernels share that contract:
//   * problems taller than 128 rows run gemmcore::gemm_pair_kernel (gemm_core.cuh): CTA pairs on
//     256 x 208 tiles with tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale, two 128-byte K blocks
//     per pipeline stage, scales written to TMEM by four forwarding warps (tcgen05.st), one
//     tcgen05.commit per stage;
//   * M <= 128 runs the one-CTA kernel of this file: per 128-wide K stage the TMA producer brings the
//     two code tiles (128B-swizzled) and the scale atoms (plain bulk copies), the MMA warp forwards
//     the atoms to TMEM with tcgen05.cp and issues four MMAs of K = 32, selecting the scale byte
//     through the instruction descriptor.
// Accumulators are double buffered in TMEM; BN = 208 keeps 2 x 208 accumulator columns + the scale
// sets inside the 512 columns.
//
// Replaces the reference's block-scaled GEMM providers: Primus-Turbo FlyDSL / AITER a4w4 kernels
// (llama2_sft/primus/a4w4_tuned_gemms.csv) and the in-tree scaled-MFMA GEMMs
// (generative_recommenders/ops/hip/k512_mx6_gemm.cu) at MXFP8 precision.
#include <cstdlib>

#include "common.cuh"
#include "gemm_core.cuh"
#include "runtime.h"

namespace {

using gemmcore::tile_coords;

constexpr int BM = 128;
constexpr int BK = 128;           // 128 e4m3 = 128 bytes = one swizzle row = 4 scale columns
constexpr int UMMA_K = 32;
constexpr int NUM_THREADS = gemmcore::NUM_THREADS;
constexpr int EPI_WARPS = gemmcore::EPI_WARPS;
constexpr int STG_BYTES = gemmcore::STG_BYTES;

template <int BN>
struct Cfg {
  static constexpr int A_STAGE = BM * BK;
  static constexpr int B_STAGE = BN * BK;
  static constexpr int B_ATOMS = (BN + 127) / 128;
  static constexpr int SFA_STAGE = 512;
  static constexpr int SFB_STAGE = 512 * B_ATOMS;
  static constexpr int STAGE = A_STAGE + B_STAGE + SFA_STAGE + SFB_STAGE;
  static constexpr int STAGES = (BN > 128) ? 4 : 5;
  static constexpr int EPI_BYTES = EPI_WARPS * 2 * STG_BYTES;
  static constexpr int SMEM = STAGES * STAGE + EPI_BYTES + 1024 + 256;
  static constexpr int SF_COL = 2 * BN;        // first TMEM column of the scale area
  // The scale columns are multi-buffered: tcgen05.cp of k block i+1 must not wait for the MMAs of k
  // block i to finish reading theirs (cp and mma execute in order on the tensor pipe).
  static constexpr int SF_SET_COLS = 4 + 4 * B_ATOMS;
  static constexpr int SF_SETS = 4;
  static constexpr int TMEM_COLS = (2 * BN + SF_SETS * SF_SET_COLS) <= 256 ? 256 : 512;
  static_assert(2 * BN + SF_SETS * SF_SET_COLS <= 512, "accumulators and scale sets exceed tensor memory");
};

struct Params {
  int M, N, K;
  int group_m;
  const uint8_t* sfa;
  const uint8_t* sfb;
  gemmcore::EpiArgs epi = {};
  int* status;
};

B200_DEVICE void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmDt, const Params p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + C::STAGES * C::A_STAGE;
  uint8_t* sSFA = sB + C::STAGES * C::B_STAGE;
  uint8_t* sSFB = sSFA + C::STAGES * C::SFA_STAGE;
  uint8_t* sE = sSFB + C::STAGES * C::SFB_STAGE;
  sE = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(sE) + 1023) & ~uintptr_t(1023));
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
  const int num_kb = p.K / BK;

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
        const uint8_t* sfa_t = p.sfa + (long long)mb * num_kb * 512;
        const uint8_t* sfb_t = p.sfb + (long long)nb * num_kb * C::SFB_STAGE;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, 110)) { ok = false; break; }
          mbar_expect_tx(&full[stage], C::STAGE);
          tma_load_2d(sA + stage * C::A_STAGE, &tmA, &full[stage], kb * BK, mb * BM);
          tma_load_2d(sB + stage * C::B_STAGE, &tmB, &full[stage], kb * BK, nb * BN);
          bulk_load(sSFA + stage * C::SFA_STAGE, sfa_t + (long long)kb * 512, C::SFA_STAGE, &full[stage]);
          bulk_load(sSFB + stage * C::SFB_STAGE, sfb_t + (long long)kb * C::SFB_STAGE, C::SFB_STAGE, &full[stage]);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t idesc0 = umma_idesc_mx(0, 0, 0, 0, BM, BN);
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      uint32_t sf_set = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag, p.status, 120)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, 121)) { ok = false; break; }
          tc_fence_after();
          const uint32_t t_sfa = tmem_base + C::SF_COL + sf_set * C::SF_SET_COLS;
          const uint32_t t_sfb = t_sfa + 4;
          sf_set = (sf_set + 1) % C::SF_SETS;
          // scale atoms: shared memory -> TMEM (32 rows x 16 bytes each, replicated to the 4 lane quarters)
          tc_cp_32x128b_warpx4(t_sfa, umma_desc_noswz(smem_u32(sSFA + stage * C::SFA_STAGE), 0, 128));
#pragma unroll
          for (int a = 0; a < C::B_ATOMS; ++a)
            tc_cp_32x128b_warpx4(t_sfb + 4 * a, umma_desc_noswz(smem_u32(sSFB + stage * C::SFB_STAGE + a * 512), 0, 128));
          const uint32_t a_addr = smem_u32(sA + stage * C::A_STAGE);
          const uint32_t b_addr = smem_u32(sB + stage * C::B_STAGE);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t ad = umma_desc_sw128(a_addr + kk * UMMA_K, 16, 1024);
            const uint64_t bd = umma_desc_sw128(b_addr + kk * UMMA_K, 16, 1024);
            // scale byte kk of every 32-bit scale column: a_sf_id bits [29,31), b_sf_id bits [4,6)
            const uint32_t idesc = idesc0 | ((uint32_t)kk << 29) | ((uint32_t)kk << 4);
            tc_mma_mxf8_ss(d_tmem, ad, bd, idesc, (kb > 0 || kk > 0) ? 1u : 0u, t_sfa, t_sfb);
          }
          tc_commit(&empty[stage]);
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&tfull[acc]);
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;
    uint8_t* stg = sE + (warp - 2) * 2 * STG_BYTES;
    int buf = 0;
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      int mb, nb; tile_coords(t, num_m, num_n, p.group_m, mb, nb);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag, p.status, 130)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
      gemmcore::epilogue_drain<BN, (BN % 64 == 0)>(&tmD, &tmDt, p.epi, t_row, mb * BM + q * 32, nb * BN, stg, buf, lane);
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
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

template <int BN>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD, const CUtensorMap& tmDt,
           const Params& p, cudaStream_t stream) {
  using C = Cfg<BN>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_mxfp8_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) { cudaGetLastError(); }
    if (e != cudaSuccess) return b200::fail(801, "gemm_mxfp8: cannot set %d bytes of shared memory: %s", C::SMEM,
                                            cudaGetErrorString(e));
    configured[dev & 63] = true;
  }
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  const int tiles = num_m * num_n;
  const int grid = tiles < b200::sm_count() ? tiles : b200::sm_count();
  gemm_mxfp8_kernel<BN><<<grid, NUM_THREADS, C::SMEM, stream>>>(tmA, tmB, tmD, tmDt, p);
  b200::count_launch();
  return b200::check_launch("gemm_mxfp8");
}

}  // namespace

// N tile the kernel will use for an output width N (the B operand's scales must be laid out with
// this tile height by the quantiser).
// 208 columns fill tensor memory (2 x 208 accumulator columns + 6 scale sets of 16 columns = 512);
// B200_MXFP8_BN=128|208 forces one choice.
static int pick_bn(int N) {
  if (N <= 128) return 128;
  static int forced = -1;
  if (forced < 0) {
    const char* e = getenv("B200_MXFP8_BN");
    forced = e ? atoi(e) : 0;
  }
  if (forced == 128 || forced == 208) return forced;
  return 208;
}
B200_API int b200_gemm_mxfp8_bn(int N) { return pick_bn(N); }

// One CTA pair per 256 x BN tile (gemm_core.cuh); KSUB = 128-byte K blocks per pipeline stage
// (B200_MXFP8_KSUB=1|2).
template <int BN>
static int run_pair(const void* a_q, const void* sfa, const void* b_q, const void* sfb, void* d, int M, int N, int K,
                    long long lda, long long ldb, long long ldd, const gemmcore::EpiArgs& epi, cudaStream_t stream) {
  using namespace gemmcore;
  static int ksub = -1;
  if (ksub < 0) {
    const char* e = getenv("B200_MXFP8_KSUB");
    ksub = (e && atoi(e) == 1) ? 1 : 2;
  }
  CUtensorMap tmA, tmB, tmSFA, tmSFB, tmD;
  int r;
  if ((r = b200::make_tmap_2d(&tmA, b200::DT_U8, a_q, K, M, lda, 128, 128, b200::SWZ_128))) return r;
  if ((r = b200::make_tmap_2d(&tmB, b200::DT_U8, b_q, K, N, ldb, 128, BN / 2, b200::SWZ_128))) return r;
  // scale atoms (512 bytes) as rows of 128 int32: [row tile][k group] for A, [column tile][k group][atom] for B
  const int kg = K / 128, atoms = (BN + 127) / 128;
  const long long a_rows = (long long)((M + 127) / 128) * kg;
  const long long b_rows = (long long)((N + BN - 1) / BN) * kg * atoms;
  if ((r = b200::make_tmap_2d(&tmSFA, b200::DT_I32, sfa, 128, a_rows, 512, 128, ksub, b200::SWZ_NONE))) return r;
  if ((r = b200::make_tmap_2d(&tmSFB, b200::DT_I32, sfb, 128, b_rows, 512, 128, ksub * atoms, b200::SWZ_NONE))) return r;
  CUtensorMap tmDt;
  if ((r = make_out_tmap<BN>(&tmD, &tmDt, d, M, N, ldd, epi.out_f32))) return r;
  PairParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.a_mn_major = 0; p.b_mn_major = 0;
  p.a_fmt = 0; p.b_fmt = 0;
  p.group_m = raster_group_m() > 1 ? raster_group_m() / 2 : 1;
  p.epi = epi;
  p.status = b200::status_ptr();
  if (ksub == 2) return launch_pair<KIND_MXFP8, BN, 2>(tmA, tmB, tmSFA, tmSFB, tmD, tmDt, p, stream, "gemm_mxfp8(pair)");
  return launch_pair<KIND_MXFP8, BN, 1>(tmA, tmB, tmSFA, tmSFB, tmD, tmDt, p, stream, "gemm_mxfp8(pair)");
}

// a_q [M, K] / b_q [N, K] e4m3 (row pitches lda / ldb in bytes), sfa / sfb scale atoms
// (tile rows 128 for A, b200_gemm_mxfp8_bn(N) for B).  K must be a multiple of 128.
B200_API int b200_gemm_mxfp8(const void* a_q, const void* sfa, const void* b_q, const void* sfb, void* d, int M, int N,
                             int K, long long lda, long long ldb, long long ldd, int out_f32, int accumulate,
                             const void* bias, const void* residual, long long ldr, float alpha, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return b200::fail(810, "gemm_mxfp8: empty problem %d x %d x %d", M, N, K);
  if (K % BK != 0) return b200::fail(811, "gemm_mxfp8: K=%d must be a multiple of %d", K, BK);
  const int BN = pick_bn(N);
  gemmcore::EpiArgs epi = {};
  epi.M = M; epi.N = N;
  epi.out_f32 = out_f32 ? 1 : 0; epi.accumulate = accumulate ? 1 : 0;
  epi.bias = (const __nv_bfloat16*)bias;
  epi.residual = (const __nv_bfloat16*)residual;
  epi.ldr = ldr;
  epi.alpha = alpha;
  if (M > 128 && gemmcore::pair_enabled()) {
    if (BN == 208) return run_pair<208>(a_q, sfa, b_q, sfb, d, M, N, K, lda, ldb, ldd, epi, (cudaStream_t)stream);
    return run_pair<128>(a_q, sfa, b_q, sfb, d, M, N, K, lda, ldb, ldd, epi, (cudaStream_t)stream);
  }
  CUtensorMap tmA, tmB, tmD, tmDt;
  int r;
  if ((r = b200::make_tmap_2d(&tmA, b200::DT_U8, a_q, K, M, lda, BK, BM, b200::SWZ_128))) return r;
  if ((r = b200::make_tmap_2d(&tmB, b200::DT_U8, b_q, K, N, ldb, BK, BN, b200::SWZ_128))) return r;
  r = (BN == 208) ? gemmcore::make_out_tmap<208>(&tmD, &tmDt, d, M, N, ldd, out_f32)
                  : gemmcore::make_out_tmap<128>(&tmD, &tmDt, d, M, N, ldd, out_f32);
  if (r) return r;
  Params p;
  p.M = M; p.N = N; p.K = K;
  p.group_m = gemmcore::raster_group_m();
  p.sfa = (const uint8_t*)sfa; p.sfb = (const uint8_t*)sfb;
  p.epi = epi;
  p.status = b200::status_ptr();
  if (BN == 208) return launch<208>(tmA, tmB, tmD, tmDt, p, (cudaStream_t)stream);
  return launch<128>(tmA, tmB, tmD, tmDt, p, (cudaStream_t)stream);
}
