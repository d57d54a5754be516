// Grouped (per-expert) MXFP8 GEMMs of the MoE layer on the CTA-pair tcgen05 core (gemm_core.cuh):
// e4m3 codes with one UE8M0 scale per 32 contraction elements, block-scaled MMAs, one persistent
// launch per GEMM driven by the device-resident dispatch plan (no host read of the routing result).
//
//   rows   (forward, dgrad)  D[r, :] = A[r, :] * W[e(r)]^T      A: the padded row buffer (expert segments
//                            start at multiples of 256 rows), W: the experts' matrices stacked [(E * N), K]
//   wgrad                    D[e] += Y^T[:, seg_e] * X^T[:, seg_e]^T   both operands are the column-wise
//                            (transposed) quantised copies, so the contraction over an expert's rows is K-major
//
// The reference gets this stage from its grouped GEMM / fused grouped MLP with MX-scaled operands
// (small_llm_moe_pretraining/primus/conf/gpt_oss_20B-MXFP4-deosc-mlperf-pretrain.yaml:130-167,186-222).
#include "gemm_core.cuh"

namespace {

using namespace gemmcore;

// N tile: a column tile must not straddle two experts of the stacked weight, so it has to divide N.
int grouped_bn(int N) {
  if (N % 192 == 0) return 192;
  if (N % 128 == 0) return 128;
  return 0;
}

template <int BN>
int run_grouped(const void* a_q, const void* sfa, const void* b_q, const void* sfb, void* d, const PairParams& p0,
                long long a_rows_total, long long b_rows_total, long long d_rows_total, long long lda, long long ldb,
                long long ldd, cudaStream_t stream, const char* what) {
  CUtensorMap tmA, tmB, tmSFA, tmSFB, tmD, tmDt;
  int r;
  const int K = p0.K;
  if ((r = b200::make_tmap_2d(&tmA, b200::DT_U8, a_q, K, a_rows_total, lda, 128, 128, b200::SWZ_128))) return r;
  if ((r = b200::make_tmap_2d(&tmB, b200::DT_U8, b_q, K, b_rows_total, ldb, 128, BN / 2, b200::SWZ_128))) return r;
  const int kg = (K + 127) / 128, atoms = (BN + 127) / 128;
  const long long sfa_rows = ((a_rows_total + 127) / 128) * kg;
  const long long sfb_rows = (b_rows_total / BN) * kg * atoms;
  if ((r = b200::make_tmap_2d(&tmSFA, b200::DT_I32, sfa, 128, sfa_rows, 512, 128, 2, b200::SWZ_NONE))) return r;
  if ((r = b200::make_tmap_2d(&tmSFB, b200::DT_I32, sfb, 128, sfb_rows, 512, 128, 2 * atoms, b200::SWZ_NONE))) return r;
  if ((r = make_out_tmap<BN>(&tmD, &tmDt, d, (int)d_rows_total, p0.N, ldd, p0.epi.out_f32))) return r;
  return launch_pair<KIND_MXFP8, BN, 2>(tmA, tmB, tmSFA, tmSFB, tmD, tmDt, p0, stream, what);
}

}  // namespace

// N tile the grouped kernels use for per-expert output width N (0: no tile divides N - use the bf16 path).
// The B operand's scales must be laid out with this tile height by the quantiser.
B200_API int b200_gemm_grouped_mx_bn(int N) { return grouped_bn(N); }

// a_q [rows, K] e4m3 (pitch lda bytes) with scale atoms sfa (tile rows 128); b_q [(E * N), K] (pitch ldb) with
// scale atoms sfb (tile rows b200_gemm_grouped_mx_bn(N)); d [rows, N] bf16 or fp32 (pitch ldd elements);
// tile_expert [rows / 256] on the device.  rows must be a multiple of 256, K of 32.
B200_API int b200_gemm_grouped_mx_rows(const void* a_q, const void* sfa, const void* b_q, const void* sfb, void* d,
                                       const int* tile_expert, int rows, int N, int K, int E, long long lda, long long ldb,
                                       long long ldd, int out_f32, float alpha, void* stream) {
  const int BN = grouped_bn(N);
  if (rows <= 0 || rows % 256 != 0 || K <= 0 || K % 32 != 0 || E <= 0 || BN == 0)
    return b200::fail(830, "gemm_grouped_mx_rows: rows=%d (x256) N=%d (x128 or x192) K=%d (x32) E=%d", rows, N, K, E);
  PairParams p = {};
  p.grp.mode = 1; p.grp.E = E; p.grp.tile_expert = tile_expert;
  p.M = rows; p.N = N; p.K = K;
  p.group_m = 16;               // 16 row tiles (4096 rows) stay in L2 while their experts' weight tiles stream once
  p.epi.M = rows; p.epi.N = N;
  p.epi.out_f32 = out_f32 ? 1 : 0;
  p.epi.alpha = alpha;
  p.status = b200::status_ptr();
  if (BN == 192)
    return run_grouped<192>(a_q, sfa, b_q, sfb, d, p, rows, (long long)E * N, rows, lda, ldb, ldd, (cudaStream_t)stream,
                            "gemm_grouped_mx_rows");
  return run_grouped<128>(a_q, sfa, b_q, sfb, d, p, rows, (long long)E * N, rows, lda, ldb, ldd, (cudaStream_t)stream,
                          "gemm_grouped_mx_rows");
}

// a_q [M, T] / b_q [N, T]: column-wise quantised copies (contraction over the T rows of the padded buffer; pitches
// lda / ldb bytes; scale tiles 128 / b200_gemm_grouped_mx_bn(N)); seg [E + 1] padded segment offsets (multiples of
// 256) on the device; d [E, M, N] contiguous, bf16 or fp32.  M must be a multiple of 32.
B200_API int b200_gemm_grouped_mx_wgrad(const void* a_q, const void* sfa, const void* b_q, const void* sfb, void* d,
                                        const int* seg, int T, int M, int N, int E, long long lda, long long ldb, int out_f32,
                                        int accumulate, float alpha, void* stream) {
  const int BN = grouped_bn(N);
  if (T <= 0 || T % 256 != 0 || M <= 0 || M % 32 != 0 || E <= 0 || BN == 0)
    return b200::fail(831, "gemm_grouped_mx_wgrad: T=%d (x256) M=%d (x32) N=%d (x128 or x192) E=%d", T, M, N, E);
  PairParams p = {};
  p.grp.mode = 2; p.grp.E = E; p.grp.seg = seg;
  p.M = M; p.N = N; p.K = T;
  p.group_m = 1;
  p.epi.M = M; p.epi.N = N;
  p.epi.out_f32 = out_f32 ? 1 : 0;
  p.epi.accumulate = accumulate ? 1 : 0;
  p.epi.alpha = alpha;
  p.status = b200::status_ptr();
  if (BN == 192)
    return run_grouped<192>(a_q, sfa, b_q, sfb, d, p, M, N, (long long)E * M, lda, ldb, N, (cudaStream_t)stream,
                            "gemm_grouped_mx_wgrad");
  return run_grouped<128>(a_q, sfa, b_q, sfb, d, p, M, N, (long long)E * M, lda, ldb, N, (cudaStream_t)stream,
                          "gemm_grouped_mx_wgrad");
}
