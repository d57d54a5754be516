// Per-tensor FP8 GEMM for sm_100a (tcgen05.mma.cta_group::2.kind::f8f6f4, CTA pairs on 256 x 256 tiles):
//
//   D[M,N] (=|+=) (scale_a^-1 * scale_b^-1) * A_q[M,K] * B_q[N,K]^T (+ bias[N]) (+ residual[M,N])
//
// A_q / B_q are e4m3 or e5m2 codes (each operand its own format), K-major; the two per-tensor
// dequantisation factors are device scalars read by the epilogue, so the host never waits for an
// amax.  The mainloop, pipeline and epilogue are gemmcore::gemm_pair_kernel (gemm_core.cuh) - the
// bf16 kernel with one-byte elements (128 contraction elements per 128-byte stage row, K = 32 per MMA).
//
// Counterpart of the reference's per-tensor FP8 GEMMs (hipBLASLt scaled matmul and the hand-written
// MFMA kernels generative_recommenders/ops/hip/k512_fp8_gemm.cu, k1536_fp8_addmm.cu).
#include "common.cuh"
#include "gemm_core.cuh"
#include "runtime.h"

// a_q [M, K] / b_q [N, K] fp8 codes (row pitches lda / ldb in bytes); a_e5m2 / b_e5m2 select the format;
// inv_scale_a / inv_scale_b: device floats (may be null = 1).  M > 128; K a multiple of 16.
B200_API int b200_gemm_fp8(const void* a_q, const void* b_q, void* d, int M, int N, int K, long long lda, long long ldb,
                           long long ldd, int a_e5m2, int b_e5m2, const float* inv_scale_a, const float* inv_scale_b,
                           int out_f32, int accumulate, const void* bias, const void* residual, long long ldr, float alpha,
                           void* stream) {
  using namespace gemmcore;
  if (M <= 128 || N <= 0 || K <= 0) return b200::fail(830, "gemm_fp8: needs M > 128 (got %d x %d x %d)", M, N, K);
  if (K % 16 != 0) return b200::fail(831, "gemm_fp8: K=%d must be a multiple of 16", K);
  EpiArgs epi = {};
  epi.M = M; epi.N = N;
  epi.out_f32 = out_f32 ? 1 : 0; epi.accumulate = accumulate ? 1 : 0;
  epi.bias = (const __nv_bfloat16*)bias;
  epi.residual = (const __nv_bfloat16*)residual;
  epi.ldr = ldr;
  epi.alpha = alpha;
  epi.alpha_a = inv_scale_a; epi.alpha_b = inv_scale_b;
  PairParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.a_mn_major = 0; p.b_mn_major = 0;
  p.a_fmt = a_e5m2 ? 1 : 0; p.b_fmt = b_e5m2 ? 1 : 0;
  p.group_m = raster_group_m() > 1 ? raster_group_m() / 2 : 1;
  p.epi = epi;
  p.status = b200::status_ptr();
  CUtensorMap tmA, tmB, tmD, tmDt;
  int r;
  if ((r = b200::make_tmap_2d(&tmA, b200::DT_U8, a_q, K, M, lda, 128, 128, b200::SWZ_128))) return r;
  if (N > 128) {
    if ((r = b200::make_tmap_2d(&tmB, b200::DT_U8, b_q, K, N, ldb, 128, 128, b200::SWZ_128))) return r;
    if ((r = make_out_tmap<256>(&tmD, &tmDt, d, M, N, ldd, epi.out_f32))) return r;
    return launch_pair<KIND_FP8, 256, 1>(tmA, tmB, tmA, tmB, tmD, tmDt, p, (cudaStream_t)stream, "gemm_fp8");
  }
  if ((r = b200::make_tmap_2d(&tmB, b200::DT_U8, b_q, K, N, ldb, 128, 64, b200::SWZ_128))) return r;
  if ((r = make_out_tmap<128>(&tmD, &tmDt, d, M, N, ldd, epi.out_f32))) return r;
  return launch_pair<KIND_FP8, 128, 1>(tmA, tmB, tmA, tmB, tmD, tmDt, p, (cudaStream_t)stream, "gemm_fp8");
}
