// All-gather -> GEMM over NVLink peer memory on the CTA-pair tcgen05 core (gemm_core.cuh): the tensor-parallel
// column linear with sequence-parallel input, D[T, N] = gather_rows(A)[T, K] * B^T, in ONE launch.  The first
// n_copy / 2 CTA pairs move the ranks' row blocks (tp_copy.cuh), the others are the persistent pair GEMM whose
// TMA producers wait per block; operands are bf16, or e4m3 / e5m2 codes with one factor per tensor (frozen base of
// a LoRA run: llama2_sft/primus/src/llama2_custom.py:1904-1910), in which case the blocks cross NVLink as codes.
// GEMM -> reduce-scatter (the row-parallel linear) runs on the same core: the epilogue warps store their tiles into
// the owners' staging buffers and the launch's reduce pairs sum them (tp_reduce.cuh).  The reduction-dimension
// gather (weight gradients) stays in gemm_tp.cu.
#include "gemm_core.cuh"

using namespace gemmcore;

// Raster group height in 256-row tiles (B200_TP_RS_GROUP_M / B200_TP_AG_GROUP_M override the defaults).
static int env_int(const char* name, int dflt) {
  const char* e = getenv(name);
  return (e && atoi(e) > 0) ? atoi(e) : dflt;
}

// a: this rank's gather buffer [M = W * rows_per, K] (own block written; row pitch lda: elements for bf16, bytes for
// 8-bit codes), b [N, K], d [M, N] bf16.  fp8 = 0: bf16 operands; fp8 = 1: codes with formats a_e5m2 / b_e5m2 and
// device factors inv_a / inv_b.  peer_ptrs[c]: rank c's gather buffer; chunk_bytes: bytes of one rank block;
// chunk_flags: W ints, zero at launch (copy_mode 1: this rank's entry of flag_ptrs[], peer-writable, zeroed on every
// rank before the cross-rank barrier that precedes the launch).  rows_per must be a multiple of 256.
B200_API int b200_gemm_tp_gather_pair(const void* a, const void* b, void* d, int M, int N, int K, long long lda,
                                      long long ldb, long long ldd, int fp8, int a_e5m2, int b_e5m2, const float* inv_a,
                                      const float* inv_b, float alpha, const unsigned long long* peer_ptrs, int W, int rank,
                                      void* gbuf_local, long long chunk_bytes, int rows_per, int* chunk_flags, int n_copy,
                                      int copy_mode, const unsigned long long* flag_ptrs, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return b200::fail(1530, "gemm_tp_gather_pair: empty problem %d x %d x %d", M, N, K);
  if (W < 1 || W > TP_MAXW || rank < 0 || rank >= W) return b200::fail(1531, "gemm_tp_gather_pair: bad world %d / rank %d", W, rank);
  if (rows_per % 256 != 0 || (long long)rows_per * W != M)
    return b200::fail(1532, "gemm_tp_gather_pair: needs M = W * rows_per with rows_per %% 256 == 0 (M=%d rows_per=%d)", M, rows_per);
  if (chunk_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(gbuf_local) & 15))
    return b200::fail(1533, "gemm_tp_gather_pair: blocks must be 16-byte aligned and sized");
  PairParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.a_fmt = a_e5m2 ? 1 : 0; p.b_fmt = b_e5m2 ? 1 : 0;
  p.group_m = env_int("B200_TP_AG_GROUP_M", 8);
  p.epi.M = M; p.epi.N = N;
  p.epi.alpha = alpha;
  p.epi.alpha_a = fp8 ? inv_a : nullptr;
  p.epi.alpha_b = fp8 ? inv_b : nullptr;
  p.status = b200::status_ptr();
  TpGather& t = p.tp;
  t.on = 1; t.W = W; t.rank = rank; t.rows_per = rows_per;
  t.n_aux = W > 1 ? ((n_copy > 0 ? n_copy : 8) + 1) / 2 : 0;
  t.copy_mode = (copy_mode == 1 && W > 1) ? 1 : 0;
  for (int c = 0; c < W; ++c) t.peer_src[c] = reinterpret_cast<const uint8_t*>(peer_ptrs[c]);
  t.gdst = reinterpret_cast<uint8_t*>(gbuf_local);
  t.chunk_bytes = chunk_bytes;
  const int piece = t.copy_mode == 1 ? tpcopy::PUSH_PIECE : tpcopy::COPY_PIECE;
  t.pieces_per_chunk = (int)((chunk_bytes + piece - 1) / piece);
  t.chunk_flag = chunk_flags;
  t.status = p.status;
  if (t.copy_mode == 1) {
    if (flag_ptrs == nullptr) return b200::fail(1534, "gemm_tp_gather_pair: push mode needs the peers' counter arrays");
    for (int c = 0; c < W; ++c) t.chunk_flag_peer[c] = reinterpret_cast<int*>(flag_ptrs[c]);
  }
  CUtensorMap tmA, tmB, tmD, tmDt;
  int r;
  cudaStream_t st = (cudaStream_t)stream;
  const bool wide = N > 128;
  if (fp8) {
    if ((r = b200::make_tmap_2d(&tmA, b200::DT_U8, a, K, M, lda, 128, 128, b200::SWZ_128))) return r;
    if ((r = b200::make_tmap_2d(&tmB, b200::DT_U8, b, K, N, ldb, 128, wide ? 128 : 64, b200::SWZ_128))) return r;
  } else {
    if ((r = b200::make_tmap_2d(&tmA, b200::DT_BF16, a, K, M, lda * 2, 64, 128, b200::SWZ_128))) return r;
    if ((r = b200::make_tmap_2d(&tmB, b200::DT_BF16, b, K, N, ldb * 2, 64, wide ? 128 : 64, b200::SWZ_128))) return r;
  }
  if (wide) {
    if ((r = make_out_tmap<256>(&tmD, &tmDt, d, M, N, ldd, 0))) return r;
    if (fp8) return launch_pair<KIND_FP8, 256, 1>(tmA, tmB, tmA, tmB, tmD, tmDt, p, st, "gemm_tp_gather_pair(fp8)");
    return launch_pair<KIND_BF16, 256, 1>(tmA, tmB, tmA, tmB, tmD, tmDt, p, st, "gemm_tp_gather_pair");
  }
  if ((r = make_out_tmap<128>(&tmD, &tmDt, d, M, N, ldd, 0))) return r;
  if (fp8) return launch_pair<KIND_FP8, 128, 1>(tmA, tmB, tmA, tmB, tmD, tmDt, p, st, "gemm_tp_gather_pair(fp8)");
  return launch_pair<KIND_BF16, 128, 1>(tmA, tmB, tmA, tmB, tmD, tmDt, p, st, "gemm_tp_gather_pair");
}

// GEMM -> reduce-scatter: P[M, N] = alpha * A * B^T is this rank's partial sum; rank o receives out[rows_per, N] = sum
// over ranks of P[o * rows_per .., :] (+ residual), bf16.  Operands as in b200_gemm_tp_gather_pair.
//   stage_ptrs[o]: rank o's staging buffer, W * rows_per * N bf16 (symmetric memory)
//   flag_ptrs[o] : rank o's counters, rows_per / 128 ints (symmetric memory), zero at launch on every rank
//   work_counter : one local int, zero at launch.  (n_red + 1) / 2 CTA pairs only reduce.
// M must be a multiple of W * 256, N of 8.
B200_API int b200_gemm_tp_rs_pair(const void* a, const void* b, int M, int N, int K, long long lda, long long ldb, int fp8,
                                  int a_e5m2, int b_e5m2, const float* inv_a, const float* inv_b, float alpha,
                                  const unsigned long long* stage_ptrs, const unsigned long long* flag_ptrs, int W, int rank,
                                  int* work_counter, void* out, long long ld_out, const void* residual, long long ld_res,
                                  int n_red, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return b200::fail(1540, "gemm_tp_rs_pair: empty problem %d x %d x %d", M, N, K);
  if (W < 1 || W > TP_MAXW || rank < 0 || rank >= W) return b200::fail(1541, "gemm_tp_rs_pair: bad world %d / rank %d", W, rank);
  if (M % (W * 256) != 0) return b200::fail(1542, "gemm_tp_rs_pair: M=%d must be a multiple of W * 256 = %d", M, W * 256);
  if (N % 8 != 0 || ld_out % 8 != 0 || (residual != nullptr && ld_res % 8 != 0))
    return b200::fail(1543, "gemm_tp_rs_pair: N and the output / residual pitches must be multiples of 8");
  const int rows_per = M / W;
  PairParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.a_fmt = a_e5m2 ? 1 : 0; p.b_fmt = b_e5m2 ? 1 : 0;
  p.group_m = env_int("B200_TP_RS_GROUP_M", W);   // one row tile of every owner per raster group: a row block completes early
  p.epi.M = M; p.epi.N = N;
  p.epi.alpha = alpha;
  p.epi.alpha_a = fp8 ? inv_a : nullptr;
  p.epi.alpha_b = fp8 ? inv_b : nullptr;
  p.status = b200::status_ptr();
  TpReduce& t = p.rs;
  t.on = 1; t.W = W; t.rank = rank; t.rows_per = rows_per; t.N = N;
  t.n_aux = ((n_red > 0 ? n_red : 8) + 1) / 2;
  OwnerMaps<TP_MAXW> om = {};
  int r;
  for (int o = 0; o < W; ++o) {
    t.stage_peer[o] = reinterpret_cast<uint8_t*>(stage_ptrs[o]);
    t.flag_peer[o] = reinterpret_cast<int*>(flag_ptrs[o]);
    if ((r = b200::make_tmap_2d(&om.m[o], b200::DT_BF16, t.stage_peer[o], N, (long long)W * rows_per, (long long)N * 2, 64, 32,
                                b200::SWZ_128))) return r;
  }
  t.work_counter = work_counter;
  t.rs_out = reinterpret_cast<__nv_bfloat16*>(out);
  t.ld_out = ld_out;
  t.rs_residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  t.ld_res = ld_res;
  t.status = p.status;
  CUtensorMap tmA, tmB;
  cudaStream_t st = (cudaStream_t)stream;
  const bool wide = N > 128;
  if (fp8) {
    if ((r = b200::make_tmap_2d(&tmA, b200::DT_U8, a, K, M, lda, 128, 128, b200::SWZ_128))) return r;
    if ((r = b200::make_tmap_2d(&tmB, b200::DT_U8, b, K, N, ldb, 128, wide ? 128 : 64, b200::SWZ_128))) return r;
  } else {
    if ((r = b200::make_tmap_2d(&tmA, b200::DT_BF16, a, K, M, lda * 2, 64, 128, b200::SWZ_128))) return r;
    if ((r = b200::make_tmap_2d(&tmB, b200::DT_BF16, b, K, N, ldb * 2, 64, wide ? 128 : 64, b200::SWZ_128))) return r;
  }
  const CUtensorMap& tmD = om.m[0];   // the plain output maps are not used by this mode
  if (wide) {
    if (fp8) return launch_pair<KIND_FP8, 256, 1, TP_MAXW>(tmA, tmB, tmA, tmB, tmD, tmD, p, st, "gemm_tp_rs_pair(fp8)", &om);
    return launch_pair<KIND_BF16, 256, 1, TP_MAXW>(tmA, tmB, tmA, tmB, tmD, tmD, p, st, "gemm_tp_rs_pair", &om);
  }
  if (fp8) return launch_pair<KIND_FP8, 128, 1, TP_MAXW>(tmA, tmB, tmA, tmB, tmD, tmD, p, st, "gemm_tp_rs_pair(fp8)", &om);
  return launch_pair<KIND_BF16, 128, 1, TP_MAXW>(tmA, tmB, tmA, tmB, tmD, tmD, p, st, "gemm_tp_rs_pair", &om);
}
