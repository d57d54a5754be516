// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (tcgen05; bf16 operands, or
// e4m3 / e5m2 operands with one dequantisation factor per tensor - the frozen-base linears of the LoRA
// fine-tuning recipe, llama2_sft/primus/src/llama2_custom.py:1904-1910 - whose gathered blocks then cross
// NVLink at one byte per element).
//
//   mode 1  all-gather -> GEMM (rows):  D[T, N] = gather_rows(A)[T, K] * B^T.  Every rank holds the
//           rows [r*T/W, (r+1)*T/W) of A in its copy of a symmetric buffer.  A few CTAs of the SAME
//           kernel pull the peers' row blocks into the local buffer with bulk async copies
//           (global(peer) -> shared -> global(local)) and publish one counter per peer block; the
//           TMA producer of every GEMM CTA waits on the counter of the block its tile needs.  Tiles
//           are visited own-block first, then peer rank+1, rank+2, ... - the order the copies land.
//   mode 2  all-gather -> GEMM (reduction dim):  the gathered dimension is K (weight gradients:
//           K = tokens).  Same copy CTAs; the producer starts its k loop at the local block and
//           waits per k block.
//   mode 3  GEMM -> reduce-scatter:  P = A * B^T is a partial sum [T, N]; rank o owns rows
//           [o*T/W, ...).  Epilogue warps store each bf16 tile straight into the OWNER's staging
//           buffer (slot of the sending rank) with peer stores and bump the owner's per-row-tile
//           counter; reduce work items (8 rows x N) are claimed from a queue by a few dedicated CTAs
//           and by the GEMM CTAs once their tiles are done: wait for the counter, sum the W slots
//           in fp32 (+ residual), write the bf16 result.  Tiles are ordered row-tile-major across
//           owners so row tile j of every owner completes while tile j+1 is being computed.
//
// The reference runs these as library collectives around library GEMMs (Megatron tensor / sequence
// parallel linears; the TransformerEngine userbuffer overlap is switched off in every shipped
// config: llama2_sft/primus/config_MI355X_1x8x1.sh:115-118).
//
// This file holds the one-CTA-per-tile kernels.  Row blocks that are multiples of 256 run modes 1 and 3 on the CTA-pair
// core instead (gemm_tp_pair.cu, gemm_core.cuh), with the same copy and reduce roles (tp_copy.cuh, tp_reduce.cuh); these
// kernels serve the remaining shapes and mode 2.
//
// Loads never use cluster multicast.  Every wait is bounded (2 s) and reports into the status block.
#include "common.cuh"
#include "runtime.h"
#include "tp_copy.cuh"
#include "tp_reduce.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int EPI_WARPS = 4;
constexpr int STG_BYTES = 4096;
constexpr int MAXW = 16;
using tpcopy::COPY_PIECE;
using tpcopy::COPY_STAGES;
using tpcopy::PUSH_PIECE;
using tpcopy::bulk_g2s;
using tpcopy::bulk_s2g;
using tpcopy::fence_proxy_async_all;
using tpcopy::red_release_gpu_add;
using tpcopy::red_release_sys_add;
using tpcopy::ld_cg_u4;
using tpreduce::RS_SPLIT;

template <int BN>
struct Cfg {
  static constexpr int A_STAGE = BM * BK * 2;
  static constexpr int B_STAGE = BN * BK * 2;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int EPI_BYTES = EPI_WARPS * 2 * STG_BYTES;
  static constexpr int SMEM = STAGES * (A_STAGE + B_STAGE) + EPI_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 2 * BN;
  static_assert(COPY_STAGES * COPY_PIECE + 1024 + 256 <= SMEM, "copy ring must fit the GEMM allocation");
};

struct OwnerMaps { CUtensorMap m[MAXW]; };   // mode 3: rank o's staging buffer viewed as [W * rows_per, N] bf16

struct Params {
  int M, N, K;
  int a_mn_major, b_mn_major;
  int out_f32, accumulate;
  int group_m;
  float alpha;
  int* status;
  // ---- 8-bit operands (K-major only): format codes 0 = e4m3, 1 = e5m2; factors are device scalars
  int fp8, a_fmt, b_fmt;
  const float* inv_a;
  const float* inv_b;
  // ---- tensor-parallel part
  int mode, W, rank;
  int rows_per;                    // rows (mode 1, 3) or k elements (mode 2) per rank block
  int n_aux;                       // copy CTAs (mode 1, 2) / dedicated reduce CTAs (mode 3): blockIdx < n_aux
  // gather
  const uint8_t* peer_src[MAXW];   // base of rank c's gather buffer (same layout everywhere)
  uint8_t* gdst;                   // local gather buffer
  long long chunk_bytes;           // bytes of one rank block (contiguous)
  int pieces_per_chunk;
  int* chunk_flag;                 // [W] counters of this rank, zero at launch (peer-writable memory in push mode)
  int copy_mode;                   // 0: pull the peers' blocks; 1: push the own block to every peer
  int* chunk_flag_peer[MAXW];      // push mode: rank d's chunk_flag array
  // reduce-scatter
  uint8_t* stage_peer[MAXW];       // rank o's staging buffer [W][rows_per][N] bf16
  int* flag_peer[MAXW];            // rank o's counters [rows_per / BM], zero at launch
  int* work_counter;               // local, zero at launch
  __nv_bfloat16* rs_out;
  long long ld_out;
  const __nv_bfloat16* rs_residual;
  long long ld_res;
};

// logical tile index -> (row tile, column tile) with the visiting order of the mode
B200_DEVICE void tile_coords(int t, int num_m, int num_n, const Params& p, int& mb, int& nb) {
  const int in_group = p.group_m * num_n;
  const int g = t / in_group;
  const int first_m = g * p.group_m;
  const int gsz = min(num_m - first_m, p.group_m);
  const int r = t - g * in_group;
  const int ml = first_m + (r % gsz);
  nb = r / gsz;
  if (p.mode == 1) {
    const int tpc = p.rows_per / BM;
    mb = ((p.rank + ml / tpc) % p.W) * tpc + (ml % tpc);
  } else if (p.mode == 3) {
    const int tpc = p.rows_per / BM;
    mb = ((p.rank + 1 + ml % p.W) % p.W) * tpc + ml / p.W;
  } else {
    mb = ml;
  }
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tp_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmD, const __grid_constant__ Params p,
               const __grid_constant__ OwnerMaps om) {
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
  volatile int* work_slot = abort_flag + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int bk = p.fp8 ? 2 * BK : BK;           // contraction elements per 128-byte k block
  const int num_kb = (p.K + bk - 1) / bk;

  // ---------------- auxiliary CTAs: no tensor memory, no GEMM barriers ----------------
  if ((int)blockIdx.x < p.n_aux) {
    if (p.mode == 3) tpreduce::reduce_cta(p, num_n, smem, bars, NUM_THREADS);
    else if (p.copy_mode == 1) tpcopy::copy_cta_push(p, (int)blockIdx.x, p.n_aux, NUM_THREADS);
    else tpcopy::copy_cta(p, (int)blockIdx.x, p.n_aux, smem, bars);
    return;
  }
  const int cta = blockIdx.x - p.n_aux;
  const int n_gemm = gridDim.x - p.n_aux;

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
      uint32_t ready = 1u << p.rank;          // rank blocks known to be in the local buffer
      const int kb_per = (p.mode == 2) ? p.rows_per / bk : 0;
      const int kb_start = (p.mode == 2) ? p.rank * kb_per : 0;
      auto need = [&](int c) -> bool {
        if (ready & (1u << c)) return true;
        if (!flag_wait_geq(p.chunk_flag + c, p.pieces_per_chunk, B200_WAIT_LIMIT_NS, p.status, 11)) {
          *abort_flag = 1;
          return false;
        }
        fence_proxy_async_all();              // the copies were written through the async proxy of another CTA
        ready |= 1u << c;
        return true;
      };
      for (int t = cta; t < num_tiles && ok; t += n_gemm) {
        int mb, nb; tile_coords(t, num_m, num_n, p, mb, nb);
        const int m0 = mb * BM, n0 = nb * BN;
        if (p.mode == 1 && !need(m0 / p.rows_per)) { ok = false; break; }
        for (int i = 0; i < num_kb; ++i) {
          int kb = i;
          if (p.mode == 2) {
            kb = kb_start + i;
            if (kb >= num_kb) kb -= num_kb;
            if (!need(kb / kb_per)) { ok = false; break; }
          }
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, 10)) { ok = false; break; }
          mbar_expect_tx(&full[stage], C::A_STAGE + C::B_STAGE);
          uint8_t* a_dst = sA + stage * C::A_STAGE;
          uint8_t* b_dst = sB + stage * C::B_STAGE;
          const int k0 = kb * bk;
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
      const uint32_t idesc = p.fp8 ? umma_idesc(p.a_fmt, p.b_fmt, 0, 0, BM, BN) : umma_idesc(1, 1, p.a_mn_major, p.b_mn_major, BM, BN);
      const uint32_t a_lbo = p.a_mn_major ? BK * 128 : 16;
      const uint32_t b_lbo = p.b_mn_major ? BK * 128 : 16;
      const uint32_t a_kstep = p.a_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      const uint32_t b_kstep = p.b_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += n_gemm, ++it) {
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
            if (p.fp8) tc_mma_f8_ss(d_tmem, ad, bd, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            else tc_mma_f16_ss(d_tmem, ad, bd, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
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
    const int ew = warp - 2;
    uint8_t* stg = sE + ew * 2 * STG_BYTES;
    float alpha = p.alpha;
    if (p.inv_a != nullptr) alpha *= *p.inv_a;       // dequantisation factors of 8-bit operands
    if (p.inv_b != nullptr) alpha *= *p.inv_b;
    int buf = 0;
    int it = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += n_gemm, ++it) {
      int mb, nb; tile_coords(t, num_m, num_n, p, mb, nb);
      const int m0 = mb * BM, n0 = nb * BN;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag, p.status, 30)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
      // mode 3: the tile goes into the owner's staging slot of this rank through the owner's tensor map
      const int owner = (p.mode == 3) ? m0 / p.rows_per : 0;
      const CUtensorMap* tmOut = (p.mode == 3) ? &om.m[owner] : &tmD;
      const int out_row0 = (p.mode == 3) ? p.rank * p.rows_per + (m0 - owner * p.rows_per) + q * 32 : m0 + q * 32;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        tc_wait_ld();
        const int col0 = n0 + c * 32;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * alpha;
        if (p.out_f32) {
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
                if (p.accumulate) tma_reduce_add_2d(tmOut, stg + buf * STG_BYTES, cs, out_row0);
                else tma_store_2d(tmOut, stg + buf * STG_BYTES, cs, out_row0);
              }
              tma_store_commit();
            }
            buf ^= 1;
          }
        }
      }
      // all TMEM reads of this accumulator are complete: hand it back before the (slow) publication
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (p.mode == 3 && lane == 0) {
        // the tile's bulk stores must be complete (not only read out of shared memory) before the
        // owner's counter is bumped
        tma_store_wait_all<0>();
        fence_proxy_async_all();
        __threadfence_system();
        red_release_sys_add(p.flag_peer[owner] + (m0 - owner * p.rows_per) / BM, 1);
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
    // tiles done: help with the reduction of the rows this rank owns.  All four warps enter (their
    // named barrier needs every one of them); after an abort the leader hands out no work.
    if (p.mode == 3) tpreduce::reduce_loop(p, num_n, threadIdx.x - 64, EPI_WARPS * 32, 1, work_slot, abort_flag);
  }

  // ------------------------------ teardown ------------------------------
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
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD, const Params& p, const OwnerMaps& om,
           int tiles, cudaStream_t stream) {
  using C = Cfg<BN>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tp_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return b200::fail(1501, "gemm_tp: cannot set %d bytes of shared memory: %s", C::SMEM, cudaGetErrorString(e));
    }
    configured[dev & 63] = true;
  }
  // every CTA must be resident at once (GEMM CTAs wait on the auxiliary CTAs): one CTA per SM at most
  const int sms = b200::sm_count();
  int n_gemm = sms - p.n_aux;
  if (tiles < n_gemm) n_gemm = tiles;
  if (n_gemm < 1) return b200::fail(1502, "gemm_tp: %d auxiliary CTAs leave no SM for the GEMM", p.n_aux);
  gemm_tp_kernel<BN><<<p.n_aux + n_gemm, NUM_THREADS, C::SMEM, stream>>>(tmA, tmB, tmD, p, om);
  b200::count_launch();
  return b200::check_launch("gemm_tp");
}

struct Fp8Args {                 // 8-bit operands: element = byte, pitches in bytes, K-major only
  int on, a_fmt, b_fmt;
  const float* inv_a;
  const float* inv_b;
};

int make_ab_maps(CUtensorMap* tmA, CUtensorMap* tmB, const void* a, const void* b, int M, int N, int K, long long lda,
                 long long ldb, int a_mn, int b_mn, int BN, bool fp8) {
  int r;
  if (fp8) {
    if ((r = b200::make_tmap_2d(tmA, b200::DT_U8, a, K, M, lda, 2 * BK, BM, b200::SWZ_128))) return r;
    return b200::make_tmap_2d(tmB, b200::DT_U8, b, K, N, ldb, 2 * BK, BN, b200::SWZ_128);
  }
  if (!a_mn) r = b200::make_tmap_2d(tmA, b200::DT_BF16, a, K, M, lda * 2, BK, BM, b200::SWZ_128);
  else r = b200::make_tmap_2d(tmA, b200::DT_BF16, a, M, K, lda * 2, 64, BK, b200::SWZ_128);
  if (r) return r;
  if (!b_mn) r = b200::make_tmap_2d(tmB, b200::DT_BF16, b, K, N, ldb * 2, BK, BN, b200::SWZ_128);
  else r = b200::make_tmap_2d(tmB, b200::DT_BF16, b, N, K, ldb * 2, 64, BK, b200::SWZ_128);
  return r;
}

}  // namespace

// All-gather -> GEMM.  `a`, `b`, `d` as in b200_gemm_bf16; the gathered operand lives in the local
// copy `gbuf_local` of a symmetric buffer whose copies on all ranks are `peer_ptrs[0..W)`; rank c's
// block is the byte range [c*chunk_bytes, (c+1)*chunk_bytes) and rank `rank` has already written its
// own block (all ranks: a cross-rank barrier between that write and this launch).
//   mode 1: the blocks are row blocks of A (rows_per rows each, M = W*rows_per, rows_per % 128 == 0)
//   mode 2: the blocks are k blocks (rows_per k-elements each, K = W*rows_per, rows_per % 64 == 0)
// chunk_flags: W ints, zero at launch.  n_copy CTAs do the copies: copy_mode 0 pulls the peers' blocks
// (chunk_flags may be ordinary local memory); copy_mode 1 pushes the own block to every peer, then
// chunk_flags must be this rank's entry of flag_ptrs[0..W) (peer-writable memory, zeroed on every rank
// before the cross-rank barrier that precedes the launch).
static int tp_gather_impl(const void* a, const void* b, void* d, int M, int N, int K, long long lda,
                          long long ldb, long long ldd, int a_mn_major, int b_mn_major, int out_f32,
                          int accumulate, float alpha, int mode, const unsigned long long* peer_ptrs, int W,
                          int rank, void* gbuf_local, long long chunk_bytes, int rows_per, int* chunk_flags,
                          int n_copy, int copy_mode, const unsigned long long* flag_ptrs, void* stream, const Fp8Args& f8) {
  if (f8.on && (a_mn_major || b_mn_major)) return b200::fail(1517, "gemm_tp_gather: 8-bit operands must be K-major");
  if (M <= 0 || N <= 0 || K <= 0) return b200::fail(1510, "gemm_tp_gather: empty problem %d x %d x %d", M, N, K);
  if (W < 1 || W > MAXW || rank < 0 || rank >= W) return b200::fail(1511, "gemm_tp_gather: bad world %d / rank %d", W, rank);
  if (mode == 1 && (rows_per % BM != 0 || (long long)rows_per * W != M))
    return b200::fail(1512, "gemm_tp_gather: mode 1 needs M = W * rows_per with rows_per %% 128 == 0 (M=%d rows_per=%d)", M, rows_per);
  if (mode == 2 && (rows_per % (f8.on ? 2 * BK : BK) != 0 || (long long)rows_per * W != K))
    return b200::fail(1513, "gemm_tp_gather: mode 2 needs K = W * rows_per with rows_per %% 64 == 0 (K=%d rows_per=%d)", K, rows_per);
  if (mode != 1 && mode != 2) return b200::fail(1514, "gemm_tp_gather: mode %d", mode);
  if (chunk_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(gbuf_local) & 15))
    return b200::fail(1515, "gemm_tp_gather: blocks must be 16-byte aligned and sized");
  const int BN = (N > 128) ? 256 : 128;
  CUtensorMap tmA, tmB, tmD;
  int r = make_ab_maps(&tmA, &tmB, a, b, M, N, K, lda, ldb, a_mn_major, b_mn_major, BN, f8.on != 0);
  if (r) return r;
  if (out_f32) r = b200::make_tmap_2d(&tmD, b200::DT_F32, d, N, M, ldd * 4, 32, 32, b200::SWZ_128);
  else r = b200::make_tmap_2d(&tmD, b200::DT_BF16, d, N, M, ldd * 2, 64, 32, b200::SWZ_128);
  if (r) return r;
  Params p{};
  p.M = M; p.N = N; p.K = K;
  p.a_mn_major = a_mn_major ? 1 : 0; p.b_mn_major = b_mn_major ? 1 : 0;
  p.out_f32 = out_f32 ? 1 : 0; p.accumulate = accumulate ? 1 : 0;
  p.group_m = 16; p.alpha = alpha; p.status = b200::status_ptr();
  p.fp8 = f8.on; p.a_fmt = f8.a_fmt; p.b_fmt = f8.b_fmt; p.inv_a = f8.inv_a; p.inv_b = f8.inv_b;
  p.mode = mode; p.W = W; p.rank = rank; p.rows_per = rows_per;
  p.n_aux = (W > 1) ? (n_copy > 0 ? n_copy : 8) : 0;
  for (int c = 0; c < W; ++c) p.peer_src[c] = reinterpret_cast<const uint8_t*>(peer_ptrs[c]);
  p.gdst = reinterpret_cast<uint8_t*>(gbuf_local);
  p.chunk_bytes = chunk_bytes;
  p.chunk_flag = chunk_flags;
  p.copy_mode = (copy_mode == 1 && W > 1) ? 1 : 0;
  const int piece = p.copy_mode == 1 ? PUSH_PIECE : COPY_PIECE;
  p.pieces_per_chunk = (int)((chunk_bytes + piece - 1) / piece);
  if (p.copy_mode == 1) {
    if (flag_ptrs == nullptr) return b200::fail(1516, "gemm_tp_gather: push mode needs the peers' counter arrays");
    for (int c = 0; c < W; ++c) p.chunk_flag_peer[c] = reinterpret_cast<int*>(flag_ptrs[c]);
  }
  static const OwnerMaps no_maps{};
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  if (BN == 256) return launch<256>(tmA, tmB, tmD, p, no_maps, tiles, (cudaStream_t)stream);
  return launch<128>(tmA, tmB, tmD, p, no_maps, tiles, (cudaStream_t)stream);
}

B200_API int b200_gemm_tp_gather(const void* a, const void* b, void* d, int M, int N, int K, long long lda,
                                 long long ldb, long long ldd, int a_mn_major, int b_mn_major, int out_f32,
                                 int accumulate, float alpha, int mode, const unsigned long long* peer_ptrs, int W,
                                 int rank, void* gbuf_local, long long chunk_bytes, int rows_per, int* chunk_flags,
                                 int n_copy, int copy_mode, const unsigned long long* flag_ptrs, void* stream) {
  return tp_gather_impl(a, b, d, M, N, K, lda, ldb, ldd, a_mn_major, b_mn_major, out_f32, accumulate, alpha, mode, peer_ptrs,
                        W, rank, gbuf_local, chunk_bytes, rows_per, chunk_flags, n_copy, copy_mode, flag_ptrs, stream,
                        Fp8Args{0, 0, 0, nullptr, nullptr});
}

// The same with 8-bit operands: a [M, K] / b [N, K] hold e4m3 (fmt 0) or e5m2 (fmt 1) codes, pitches in bytes,
// value = code * (*inv_scale) with the factors read on the device; the gathered blocks are codes as well, and
// every rank must have quantised its block with the same factor.
B200_API int b200_gemm_tp_gather_fp8(const void* a, const void* b, void* d, int M, int N, int K, long long lda,
                                     long long ldb, long long ldd, int a_e5m2, int b_e5m2, const float* inv_a,
                                     const float* inv_b, int out_f32, int accumulate, float alpha, int mode,
                                     const unsigned long long* peer_ptrs, int W, int rank, void* gbuf_local,
                                     long long chunk_bytes, int rows_per, int* chunk_flags, int n_copy, int copy_mode,
                                     const unsigned long long* flag_ptrs, void* stream) {
  return tp_gather_impl(a, b, d, M, N, K, lda, ldb, ldd, 0, 0, out_f32, accumulate, alpha, mode, peer_ptrs, W, rank,
                        gbuf_local, chunk_bytes, rows_per, chunk_flags, n_copy, copy_mode, flag_ptrs, stream,
                        Fp8Args{1, a_e5m2 ? 1 : 0, b_e5m2 ? 1 : 0, inv_a, inv_b});
}

// GEMM -> reduce-scatter.  P[M, N] = alpha * A * B^T is this rank's partial sum; rank o receives
// out[rows_per, N] = sum over ranks of P[o*rows_per .. , :] (+ residual), bf16.
//   stage_ptrs[o]: rank o's staging buffer, W * rows_per * N bf16 (symmetric memory)
//   flag_ptrs[o] : rank o's counters, rows_per / 128 ints (symmetric memory), zero at launch on every
//                  rank (zero them, then a cross-rank barrier, then launch)
//   work_counter : one local int, zero at launch.  n_red CTAs only reduce.
static int tp_rs_impl(const void* a, const void* b, int M, int N, int K, long long lda, long long ldb,
                      int a_mn_major, int b_mn_major, float alpha, const unsigned long long* stage_ptrs,
                      const unsigned long long* flag_ptrs, int W, int rank, int* work_counter, void* out,
                      long long ld_out, const void* residual, long long ld_res, int n_red, void* stream, const Fp8Args& f8) {
  if (f8.on && (a_mn_major || b_mn_major)) return b200::fail(1524, "gemm_tp_rs: 8-bit operands must be K-major");
  if (M <= 0 || N <= 0 || K <= 0) return b200::fail(1520, "gemm_tp_rs: empty problem %d x %d x %d", M, N, K);
  if (W < 1 || W > MAXW || rank < 0 || rank >= W) return b200::fail(1521, "gemm_tp_rs: bad world %d / rank %d", W, rank);
  if (M % (W * BM) != 0) return b200::fail(1522, "gemm_tp_rs: M=%d must be a multiple of W * 128 = %d", M, W * BM);
  if (N % 8 != 0 || ld_out % 8 != 0 || (residual != nullptr && ld_res % 8 != 0))
    return b200::fail(1523, "gemm_tp_rs: N and the output / residual pitches must be multiples of 8");
  const int BN = (N > 128) ? 256 : 128;
  const int rows_per = M / W;
  CUtensorMap tmA, tmB, tmD;
  int r = make_ab_maps(&tmA, &tmB, a, b, M, N, K, lda, ldb, a_mn_major, b_mn_major, BN, f8.on != 0);
  if (r) return r;
  r = b200::make_tmap_2d(&tmD, b200::DT_BF16, out, N, rows_per, ld_out * 2, 64, 32, b200::SWZ_128);   // not used by mode 3
  if (r) return r;
  Params p{};
  p.M = M; p.N = N; p.K = K;
  p.a_mn_major = a_mn_major ? 1 : 0; p.b_mn_major = b_mn_major ? 1 : 0;
  p.group_m = 16; p.alpha = alpha; p.status = b200::status_ptr();
  p.fp8 = f8.on; p.a_fmt = f8.a_fmt; p.b_fmt = f8.b_fmt; p.inv_a = f8.inv_a; p.inv_b = f8.inv_b;
  p.mode = 3; p.W = W; p.rank = rank; p.rows_per = rows_per;
  p.n_aux = n_red > 0 ? n_red : 8;
  for (int o = 0; o < W; ++o) {
    p.stage_peer[o] = reinterpret_cast<uint8_t*>(stage_ptrs[o]);
    p.flag_peer[o] = reinterpret_cast<int*>(flag_ptrs[o]);
  }
  p.work_counter = work_counter;
  p.rs_out = reinterpret_cast<__nv_bfloat16*>(out);
  p.ld_out = ld_out;
  p.rs_residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ld_res = ld_res;
  OwnerMaps om{};
  for (int o = 0; o < W; ++o) {
    r = b200::make_tmap_2d(&om.m[o], b200::DT_BF16, p.stage_peer[o], N, (long long)W * rows_per, (long long)N * 2, 64, 32,
                           b200::SWZ_128);
    if (r) return r;
  }
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  if (BN == 256) return launch<256>(tmA, tmB, tmD, p, om, tiles, (cudaStream_t)stream);
  return launch<128>(tmA, tmB, tmD, p, om, tiles, (cudaStream_t)stream);
}

B200_API int b200_gemm_tp_rs(const void* a, const void* b, int M, int N, int K, long long lda, long long ldb,
                             int a_mn_major, int b_mn_major, float alpha, const unsigned long long* stage_ptrs,
                             const unsigned long long* flag_ptrs, int W, int rank, int* work_counter, void* out,
                             long long ld_out, const void* residual, long long ld_res, int n_red, void* stream) {
  return tp_rs_impl(a, b, M, N, K, lda, ldb, a_mn_major, b_mn_major, alpha, stage_ptrs, flag_ptrs, W, rank, work_counter, out,
                    ld_out, residual, ld_res, n_red, stream, Fp8Args{0, 0, 0, nullptr, nullptr});
}

// The same with 8-bit operands (see b200_gemm_tp_gather_fp8); every rank may use its own factors, the partial sums
// travel as bf16.
B200_API int b200_gemm_tp_rs_fp8(const void* a, const void* b, int M, int N, int K, long long lda, long long ldb,
                                 int a_e5m2, int b_e5m2, const float* inv_a, const float* inv_b, float alpha,
                                 const unsigned long long* stage_ptrs, const unsigned long long* flag_ptrs, int W, int rank,
                                 int* work_counter, void* out, long long ld_out, const void* residual, long long ld_res,
                                 int n_red, void* stream) {
  return tp_rs_impl(a, b, M, N, K, lda, ldb, 0, 0, alpha, stage_ptrs, flag_ptrs, W, rank, work_counter, out, ld_out, residual,
                    ld_res, n_red, stream, Fp8Args{1, a_e5m2 ? 1 : 0, b_e5m2 ? 1 : 0, inv_a, inv_b});
}
