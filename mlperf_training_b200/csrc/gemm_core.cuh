// Shared roles of the tcgen05 GEMM kernels of this library.
//
//   * epilogue_drain<BN, WIDE>: one epilogue warp moves its 32 TMEM lanes x BN accumulator columns
//     through alpha / bias / residual to global memory with TMA stores (or TMA reduce-adds), used
//     by the dense bf16, MXFP8, grouped and tensor-parallel kernels alike.
//   * gemm_pair_kernel<KIND, BN, KSUB>: the persistent CTA-pair mainloop.  Two CTAs of a cluster
//     work on one 256 x BN output tile with tcgen05.mma.cta_group::2: each CTA stages its own 128
//     rows of A and its own BN/2 rows of B (its own TMA loads, no multicast), the leader CTA's
//     single MMA lane issues 256-row instructions that read both CTAs' shared memory, and each
//     CTA's TMEM receives the 128 x BN accumulator of its rows.  Compared with one CTA per
//     128 x BN tile this halves the B bytes staged and read per FLOP and halves the number of
//     tcgen05 instructions per FLOP.
//
// Pair protocol (leader = cluster rank 0):
//   full[s]   (leader's)  1 arrival (leader producer's expect_tx for the bytes of BOTH CTAs) +
//                         the completion bytes of both CTAs' TMA loads
//   empty[s]  (each CTA)  released by the leader's tcgen05.commit to both CTAs
//   tfull[a]  (each CTA)  accumulator a complete: leader's tcgen05.commit to both CTAs
//   tempty[a] (leader's)  2 x 4 arrivals: the epilogue warps of both CTAs have drained accumulator a
// MXFP8 only - the UE8M0 scales reach TMEM through four extra warps per CTA (one per TMEM lane
// quarter) that read the staged scale atoms from shared memory and write them with tcgen05.st, so
// that the tensor pipe carries nothing but MMAs (a tcgen05.cp per atom stalls the in-order pipe for
// about as long as an MMA):
//   sffull[s]  (each CTA)  this CTA's scale atoms of stage s have landed
//   sfrdy[s]   (leader's)  2 x 4 arrivals: the scale sets of stage s are in both CTAs' TMEM
// Every staged k block has its own scale set in TMEM (16 columns), so a set is rewritten only after
// the producer has seen empty[] of the stage's previous use: the forwarders need no signal from the
// MMAs, run as far ahead as the loads do, and the MMA lane issues exactly one tcgen05.commit per stage.
// The N tile of the MXFP8 kernels is 208 so that 2 accumulators + 6 scale sets fill the 512 columns.
// Every wait is bounded (common.cuh); the cluster barrier before exit keeps both CTAs' shared
// memory and barriers alive until the partner's last signal has landed.
//
// Tile schedulers on the same mainloop (tile_info):
//   * dense            grouped raster over (row tile, column tile)
//   * GroupArgs        MoE: rows grouped by expert with the stacked expert weights as B (forward, dgrad), or one
//                      contraction range per expert (weight gradients)
//   * TpGather         all-gather -> GEMM: the first CTA pairs of the launch copy the ranks' row blocks over NVLink
//                      (tp_copy.cuh), the producers wait per block and visit the blocks in arrival order
//   * TpReduce         GEMM -> reduce-scatter: tiles leave through the owners' tensor maps into their staging
//                      buffers, the first CTA pairs and - after their tiles - all epilogue warps reduce (tp_reduce.cuh)
#pragma once
#include <cstdlib>

#include "common.cuh"
#include "runtime.h"
#include "tp_copy.cuh"
#include "tp_reduce.cuh"

namespace gemmcore {

constexpr int EPI_WARPS = 4;
constexpr int STG_BYTES = 4096;   // one epilogue staging buffer (32 rows x 128 bytes)
constexpr int NUM_THREADS = 192;  // warp 0 TMA, warp 1 MMA + TMEM allocation, warps 2-5 epilogue

enum Kind : int { KIND_BF16 = 0, KIND_MXFP8 = 1, KIND_FP8 = 2 };   // FP8: e4m3 / e5m2 codes, one factor per tensor

struct EpiArgs {
  int M, N;
  int out_f32;                    // 0: bf16 output, 1: fp32 output
  int accumulate;                 // 0: store, 1: reduce-add into D
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldr] or null
  long long ldr;
  float alpha;                    // scale applied to the accumulator before bias / residual
  const float* alpha_a;           // optional device scalars multiplied into alpha (per-tensor dequantisation
  const float* alpha_b;           // factors of the FP8 operands)
};

// Grouped raster: consecutive tiles walk `group_m` row tiles of one column tile, so a column's B tile
// is shared in L2 while the group's A rows stay resident.
B200_DEVICE void tile_coords(int t, int num_m, int num_n, int group_m, int& mb, int& nb) {
  const int in_group = group_m * num_n;
  const int g = t / in_group;
  const int first_m = g * group_m;
  const int gsz = min(num_m - first_m, group_m);
  const int r = t - g * in_group;
  mb = first_m + (r % gsz);
  nb = r / gsz;
}

// Height (in tiles) of a raster group (B200_GEMM_GROUP_M overrides).
inline int raster_group_m() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B200_GEMM_GROUP_M");
    v = (e && atoi(e) > 0) ? atoi(e) : 16;
  }
  return v;
}

// Drains one accumulator (TMEM address t_row: this warp's lane quarter, first accumulator column)
// to D rows [row0, row0 + 32) x columns [n0, n0 + BN) (row0 is checked against e.M; `row_off` is added to
// the row coordinate of the stores: the first row of the tile's matrix inside a stacked output).  `stg` is
// this warp's pair of staging buffers, `buf` its running buffer index.  fp32 output and narrow bf16 output leave 32 columns per TMA
// store (tmD boxes: fp32 32 x 32 with 128-byte swizzle, bf16 32 x 32 with 64-byte swizzle); WIDE
// bf16 output (BN a multiple of 64) leaves 64 columns per store (box 64 x 32, 128-byte swizzle).
// A BN of 32 k + 16 ends with one 16-column store through tmTail (fp32: box 16 x 32 with 64-byte
// swizzle; bf16: box 16 x 32, dense 32-byte rows).
template <int BN, bool WIDE>
B200_DEVICE void epilogue_drain(const CUtensorMap* tmD, const CUtensorMap* tmTail, const EpiArgs& e, uint32_t t_row,
                                int row0, int n0, uint8_t* stg, int& buf, int lane, int row_off = 0) {
  static_assert(BN % 16 == 0, "accumulator width must be a multiple of 16 columns");
  static_assert(!WIDE || BN % 64 == 0, "64-column stores need BN to be a multiple of 64");
  const int row = row0 + lane;
  float alpha = e.alpha;
  if (e.alpha_a != nullptr) alpha *= *e.alpha_a;
  if (e.alpha_b != nullptr) alpha *= *e.alpha_b;
  const bool vec_res = e.residual != nullptr && (e.ldr % 8 == 0) && (e.N % 8 == 0) &&
                       ((reinterpret_cast<uintptr_t>(e.residual) & 15) == 0);
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {   // whole 32-column chunks
    uint32_t r[32];
    tmem_ld_32x32b_x32(t_row + c * 32, r);
    tc_wait_ld();
    const int col0 = n0 + c * 32;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * alpha;
    if (e.bias != nullptr) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < e.N) v[i] += __bfloat162float(e.bias[col0 + i]);
    }
    if (e.residual != nullptr && row < e.M) {
      const __nv_bfloat16* rp = e.residual + (long long)row * e.ldr + col0;
      if (vec_res) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (col0 + j * 8 < e.N) {
            const uint4 u = *reinterpret_cast<const uint4*>(rp + j * 8);
            const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
            v[j * 8 + 0] += f0.x; v[j * 8 + 1] += f0.y; v[j * 8 + 2] += f1.x; v[j * 8 + 3] += f1.y;
            v[j * 8 + 4] += f2.x; v[j * 8 + 5] += f2.y; v[j * 8 + 6] += f3.x; v[j * 8 + 7] += f3.y;
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (col0 + i < e.N) v[i] += __bfloat162float(rp[i]);
      }
    }
    if (e.out_f32) {
      // 32 rows x 32 fp32 (128 bytes per row), 128-byte swizzle
      if (lane == 0) tma_store_wait_read<1>();
      __syncwarp();
      uint8_t* sb = stg + buf * STG_BYTES + lane * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(sb + ((j ^ (lane & 7)) << 4)) =
            make_uint4(__float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]), __float_as_uint(v[4 * j + 2]),
                       __float_as_uint(v[4 * j + 3]));
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (col0 < e.N && row0 < e.M) {
          if (e.accumulate) tma_reduce_add_2d(tmD, stg + buf * STG_BYTES, col0, row0 + row_off);
          else tma_store_2d(tmD, stg + buf * STG_BYTES, col0, row0 + row_off);
        }
        tma_store_commit();
      }
      buf ^= 1;
    } else if (!WIDE) {
      // 32 rows x 32 bf16 = dense 64-byte rows, 64-byte swizzle (chunk ^= (row / 2) % 4)
      if (lane == 0) tma_store_wait_read<1>();
      __syncwarp();
      uint8_t* sb = stg + buf * STG_BYTES + lane * 64;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint4*>(sb + ((j ^ ((lane >> 1) & 3)) << 4)) =
            make_uint4(pack_bf16x2(v[8 * j], v[8 * j + 1]), pack_bf16x2(v[8 * j + 2], v[8 * j + 3]),
                       pack_bf16x2(v[8 * j + 4], v[8 * j + 5]), pack_bf16x2(v[8 * j + 6], v[8 * j + 7]));
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (col0 < e.N && row0 < e.M) {
          if (e.accumulate) tma_reduce_add_2d(tmD, stg + buf * STG_BYTES, col0, row0 + row_off);
          else tma_store_2d(tmD, stg + buf * STG_BYTES, col0, row0 + row_off);
        }
        tma_store_commit();
      }
      buf ^= 1;
    } else {
      // 32 rows x 64 bf16 (128 bytes per row): two 32-column chunks fill one staging buffer
      const int half = c & 1;
      if (half == 0) {
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
      }
      uint8_t* sb = stg + buf * STG_BYTES + lane * 128;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int chunk = half * 4 + j;
        *reinterpret_cast<uint4*>(sb + ((chunk ^ (lane & 7)) << 4)) =
            make_uint4(pack_bf16x2(v[8 * j], v[8 * j + 1]), pack_bf16x2(v[8 * j + 2], v[8 * j + 3]),
                       pack_bf16x2(v[8 * j + 4], v[8 * j + 5]), pack_bf16x2(v[8 * j + 6], v[8 * j + 7]));
      }
      if (half == 1) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int cs = col0 - 32;
          if (cs < e.N && row0 < e.M) {
            if (e.accumulate) tma_reduce_add_2d(tmD, stg + buf * STG_BYTES, cs, row0 + row_off);
            else tma_store_2d(tmD, stg + buf * STG_BYTES, cs, row0 + row_off);
          }
          tma_store_commit();
        }
        buf ^= 1;
      }
    }
  }
  if constexpr (BN % 32 == 16) {
    constexpr int c = BN / 32;
    uint32_t r[16];
    tmem_ld_32x32b_x16(t_row + c * 32, r);
    tc_wait_ld();
    const int col0 = n0 + c * 32;
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]) * alpha;
    if (e.bias != nullptr) {
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (col0 + i < e.N) v[i] += __bfloat162float(e.bias[col0 + i]);
    }
    if (e.residual != nullptr && row < e.M) {
      const __nv_bfloat16* rp = e.residual + (long long)row * e.ldr + col0;
      if (vec_res) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          if (col0 + j * 8 < e.N) {
            const uint4 u = *reinterpret_cast<const uint4*>(rp + j * 8);
            const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
            v[j * 8 + 0] += f0.x; v[j * 8 + 1] += f0.y; v[j * 8 + 2] += f1.x; v[j * 8 + 3] += f1.y;
            v[j * 8 + 4] += f2.x; v[j * 8 + 5] += f2.y; v[j * 8 + 6] += f3.x; v[j * 8 + 7] += f3.y;
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (col0 + i < e.N) v[i] += __bfloat162float(rp[i]);
      }
    }
    if (lane == 0) tma_store_wait_read<1>();
    __syncwarp();
    if (e.out_f32) {
      // 32 rows x 16 fp32 = 64-byte rows, 64-byte swizzle
      uint8_t* sb = stg + buf * STG_BYTES + lane * 64;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint4*>(sb + ((j ^ ((lane >> 1) & 3)) << 4)) =
            make_uint4(__float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]), __float_as_uint(v[4 * j + 2]),
                       __float_as_uint(v[4 * j + 3]));
    } else {
      // 32 rows x 16 bf16 = dense 32-byte rows
      uint8_t* sb = stg + buf * STG_BYTES + lane * 32;
#pragma unroll
      for (int j = 0; j < 2; ++j)
        *reinterpret_cast<uint4*>(sb + (j << 4)) =
            make_uint4(pack_bf16x2(v[8 * j], v[8 * j + 1]), pack_bf16x2(v[8 * j + 2], v[8 * j + 3]),
                       pack_bf16x2(v[8 * j + 4], v[8 * j + 5]), pack_bf16x2(v[8 * j + 6], v[8 * j + 7]));
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      if (col0 < e.N && row0 < e.M) {
        if (e.accumulate) tma_reduce_add_2d(tmTail, stg + buf * STG_BYTES, col0, row0 + row_off);
        else tma_store_2d(tmTail, stg + buf * STG_BYTES, col0, row0 + row_off);
      }
      tma_store_commit();
    }
    buf ^= 1;
  }
}

// Tensor map of D for epilogue_drain (ldd in elements).
template <int BN>
inline int make_out_tmap(CUtensorMap* tmD, CUtensorMap* tmTail, void* d, int M, int N, long long ldd, int out_f32) {
  int r;
  if (out_f32) r = b200::make_tmap_2d(tmD, b200::DT_F32, d, N, M, ldd * 4, 32, 32, b200::SWZ_128);
  else if (BN % 64 == 0) r = b200::make_tmap_2d(tmD, b200::DT_BF16, d, N, M, ldd * 2, 64, 32, b200::SWZ_128);
  else r = b200::make_tmap_2d(tmD, b200::DT_BF16, d, N, M, ldd * 2, 32, 32, b200::SWZ_64);
  if (r) return r;
  if (BN % 32 == 16) {
    if (out_f32) return b200::make_tmap_2d(tmTail, b200::DT_F32, d, N, M, ldd * 4, 16, 32, b200::SWZ_64);
    return b200::make_tmap_2d(tmTail, b200::DT_BF16, d, N, M, ldd * 2, 16, 32, b200::SWZ_NONE);
  }
  *tmTail = *tmD;
  return 0;
}

// ----------------------------------------------------------------------------------
// CTA-pair mainloop
// ----------------------------------------------------------------------------------
template <int KIND, int BN, int KSUB>
struct PairCfg {
  static constexpr bool MX = (KIND == KIND_MXFP8);
  static constexpr int THREADS = MX ? NUM_THREADS + 128 : NUM_THREADS;   // + 4 scale-forwarding warps
  static constexpr int BNH = BN / 2;              // B rows staged by each CTA
  static constexpr int A_SUB = 128 * 128;         // 128 rows x 128 bytes of K
  static constexpr int B_SUB = BNH * 128;
  static constexpr int B_ATOMS = (BN + 127) / 128;
  static constexpr int SFA_SUB = MX ? 512 : 0;
  static constexpr int SFB_SUB = MX ? 512 * B_ATOMS : 0;
  static constexpr int AB_STAGE = KSUB * (A_SUB + B_SUB);      // operand bytes landed per CTA per stage
  static constexpr int SF_STAGE = KSUB * (SFA_SUB + SFB_SUB);  // scale bytes landed per CTA per stage
  static constexpr int STAGE = AB_STAGE + SF_STAGE;
  static constexpr int EPI_BYTES = EPI_WARPS * 2 * STG_BYTES;
  static constexpr int SMEM_BUDGET = 232448 - 1024 - 1024 - 512 - EPI_BYTES;
  static constexpr int STAGES = SMEM_BUDGET / STAGE;
  static constexpr int SMEM = STAGES * STAGE + 1024 + 1024 + 512 + EPI_BYTES;
  static constexpr int SF_COL = 2 * BN;           // first TMEM column of the scale area
  static constexpr int SF_SET_COLS = 16;          // 4 columns of A scales, 4 per 128 rows of B, padding
  static constexpr int SF_SETS = STAGES * KSUB;   // one scale set per staged k block
  static constexpr int USED_COLS = 2 * BN + (MX ? SF_SETS * SF_SET_COLS : 0);
  static constexpr int TMEM_COLS = USED_COLS <= 256 ? 256 : 512;
  static constexpr int NUM_BARS = 2 * STAGES + 4 + (MX ? 2 * STAGES : 0);
  static_assert(4 + 4 * B_ATOMS <= SF_SET_COLS, "scale set too narrow");
  static_assert(USED_COLS <= 512, "accumulators and scale sets exceed tensor memory");
  static_assert(B_SUB % 1024 == 0, "B half tile must be whole swizzle atoms");
  static_assert(STAGES >= 2, "not enough shared memory for two stages");
  static_assert(NUM_BARS * 8 + 16 <= 512, "barrier block overflows its 512 bytes");
  static_assert(BN % 16 == 0 && BN <= 256, "N of a 256-row MMA must be a multiple of 16 up to 256");
};

// Grouped (per-expert) problems on the pair kernel, MXFP8 operands:
//   mode 1  D[r, :] = A[r, :] * B[e(r)]^T over a row buffer whose expert segments start at multiples of
//           256 rows; B is the experts' matrices stacked as [(E * N), K], its scale atoms were laid out
//           with N a multiple of the N tile (a tile never straddles two experts); tiles of 256 rows whose
//           tile_expert is negative (past the last segment) are skipped by every role
//   mode 2  D[e] (+)= A[:, seg[e]:seg[e+1]] * B[:, seg[e]:seg[e+1]]^T - the contraction runs over the
//           expert's rows of the (transposed, K-major) operands; D is the experts' [M, N] outputs stacked
//           as [(E * M), N]; an expert without rows is skipped (accumulate into a zeroed D)
struct GroupArgs {
  int mode;                       // 0: plain GEMM
  int E;
  const int* tile_expert;         // mode 1: [ceil(M / 256)]
  const int* seg;                 // mode 2: [E + 1], multiples of 256
};

struct TileInfo {
  int mb, nb, e, kb0, nkb;
  bool valid;
};

// All-gather -> GEMM inside one launch (tensor parallelism, sequence-parallel activations): the rows of A are
// gathered over W ranks.  Rank c's block is the byte range [c * chunk_bytes, (c + 1) * chunk_bytes) of a buffer
// that exists on every rank at peer_src[c] (this rank's copy: gdst); this rank has written its own block.  The
// first n_aux CTA pairs of the launch do nothing but move blocks over NVLink (tp_copy.cuh: pull the peers' blocks
// with bulk async copies, or push the own block to every peer with posted stores) and publish per-block counters;
// the TMA producers of the GEMM pairs visit the row tiles own-block first, then rank + 1, rank + 2, ... - the order
// in which the blocks land - and wait (bounded) on the counter of the block a tile needs.
constexpr int TP_MAXW = 16;
struct TpGather {
  int on;
  int W, rank;
  int rows_per;                    // rows of A per rank block (a multiple of 256)
  int n_aux;                       // CTA pairs that only copy
  int copy_mode;                   // 0: pull the peers' blocks; 1: push the own block to every peer
  const uint8_t* peer_src[TP_MAXW];
  uint8_t* gdst;
  long long chunk_bytes;
  int pieces_per_chunk;
  int* chunk_flag;                 // [W] counters of this rank, zero at launch (peer-writable memory in push mode)
  int* chunk_flag_peer[TP_MAXW];   // push mode: rank d's chunk_flag array
  int* status;
};

// GEMM -> reduce-scatter inside one launch (tensor parallelism, row-parallel linear): P = A * B^T is this rank's
// partial sum [M, N]; rank o owns rows [o * rows_per, (o + 1) * rows_per).  The epilogue warps store each bf16 tile
// into the owner's staging buffer (slot of the sending rank) through the owner's tensor map and bump the owner's
// per-128-row counter; the first n_aux CTA pairs and, once their tiles are done, the epilogue warps of the GEMM
// pairs reduce the rows this rank owns (tp_reduce.cuh).  Tiles are visited row-tile-major across owners, so that row
// tile j of every owner completes while tile j + 1 is being computed.
struct TpReduce {
  int on;
  int W, rank;
  int rows_per;                    // rows per owner (a multiple of 256)
  int n_aux;                       // CTA pairs that only reduce
  int N;
  uint8_t* stage_peer[TP_MAXW];    // rank o's staging buffer [W][rows_per][N] bf16
  int* flag_peer[TP_MAXW];         // rank o's counters [rows_per / 128], zero at launch
  int* work_counter;               // local, zero at launch
  __nv_bfloat16* rs_out;
  long long ld_out;
  const __nv_bfloat16* rs_residual;
  long long ld_res;
  int* status;
};

// Tensor maps of the owners' staging buffers ([W * rows_per, N] bf16, 64 x 32 boxes); one unused entry for the
// launches that do not reduce-scatter.
template <int NOWN>
struct OwnerMaps { CUtensorMap m[NOWN]; };

struct PairParams {
  GroupArgs grp;
  int M, N, K;                    // K in elements (bf16) or bytes (e4m3); mode 2: M, N per expert, K = all rows
  int a_mn_major, b_mn_major;     // bf16 only
  int a_fmt, b_fmt;               // FP8 only: 0 = e4m3, 1 = e5m2
  int group_m;
  EpiArgs epi;
  int* status;
  TpGather tp;
  TpReduce rs;
};

// Tile t of the launch: its row / column tile, expert and range of k stages (kb_elems = contraction
// elements per stage).
B200_DEVICE TileInfo tile_info(int t, int num_m, int num_n, int num_kb, int kb_elems, const PairParams& p) {
  TileInfo ti;
  ti.e = 0; ti.kb0 = 0; ti.nkb = num_kb; ti.valid = true;
  if (p.grp.mode == 2) {
    const int per = num_m * num_n;
    ti.e = t / per;
    const int r = t - ti.e * per;
    ti.nb = r / num_m;
    ti.mb = r - ti.nb * num_m;
    const int lo = p.grp.seg[ti.e], hi = p.grp.seg[ti.e + 1];
    ti.kb0 = lo / kb_elems;
    ti.nkb = (hi - lo) / kb_elems;
    ti.valid = ti.nkb > 0;
  } else {
    tile_coords(t, num_m, num_n, p.group_m, ti.mb, ti.nb);
    if (p.tp.on) {
      // own block first, then the blocks of rank + 1, rank + 2, ...: the order in which the gathered blocks arrive
      const int tpc = p.tp.rows_per / 256;
      ti.mb = ((p.tp.rank + ti.mb / tpc) % p.tp.W) * tpc + (ti.mb % tpc);
    }
    if (p.rs.on) {
      // row-tile-major across owners, starting with the next rank's rows
      const int tpc = p.rs.rows_per / 256;
      const int ml = ti.mb;
      ti.mb = ((p.rs.rank + 1 + ml % p.rs.W) % p.rs.W) * tpc + ml / p.rs.W;
    }
    if (p.grp.mode == 1) {
      ti.e = p.grp.tile_expert[ti.mb];
      ti.valid = ti.e >= 0;
    }
  }
  return ti;
}

template <int KIND, int BN, int KSUB, int NOWN = 1>
__global__ void __launch_bounds__(PairCfg<KIND, BN, KSUB>::THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
                 const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmDt,
                 const __grid_constant__ PairParams p, const __grid_constant__ OwnerMaps<NOWN> om) {
  using C = PairCfg<KIND, BN, KSUB>;
  constexpr bool MX = C::MX;
  constexpr bool F8 = (KIND == KIND_FP8);
  constexpr int KB_ELEMS = (MX || F8) ? 128 : 64; // contraction elements per 128-byte sub-block
  constexpr int UMMA_K_BYTES = 32;                // one MMA consumes 32 bytes of K per row
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + C::STAGES * KSUB * C::A_SUB;
  uint8_t* sSFA = sB + C::STAGES * KSUB * C::B_SUB;
  uint8_t* sSFB = sSFA + C::STAGES * KSUB * C::SFA_SUB;
  uint8_t* sE = sSFB + C::STAGES * KSUB * C::SFB_SUB;
  sE = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(sE) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(sE + C::EPI_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + C::STAGES;
  uint64_t* tfull = bars + 2 * C::STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* sffull = tempty + 2;                  // MX only: [STAGES]
  uint64_t* sfrdy = sffull + C::STAGES;           // MX only: [STAGES]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + C::NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  volatile int* work_slot = abort_flag + 1;       // reduce-scatter: the work item the epilogue warps share

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();        // 0 = leader of the pair
  // leading CTA pairs that only move gathered blocks / only reduce
  const int n_aux = p.tp.on ? p.tp.n_aux : (p.rs.on ? p.rs.n_aux : 0);
  const bool is_aux = (int)(blockIdx.x >> 1) < n_aux;
  const int pair_id = (int)(blockIdx.x >> 1) - n_aux;
  const int num_pairs = (int)(gridDim.x >> 1) - n_aux;
  const int num_m = (p.M + 255) / 256;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = (p.grp.mode == 2 ? p.grp.E : 1) * num_m * num_n;
  const int num_kb = (p.K + KB_ELEMS * KSUB - 1) / (KB_ELEMS * KSUB);
  const int num_kb128 = (p.K + KB_ELEMS - 1) / KB_ELEMS;   // 128-byte K blocks (scale groups of the MX layout)

  if (threadIdx.x == 0) {
    if (!is_aux) {                                // a copy CTA sets up its own barriers in the same words
      for (int i = 0; i < C::STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
      for (int i = 0; i < 2; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], 2 * EPI_WARPS); }
      if (MX) {
        for (int i = 0; i < C::STAGES; ++i) { mbar_init(&sffull[i], 1); mbar_init(&sfrdy[i], 8); }
      }
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1 && !is_aux) {
    tmem_alloc_pair(tmem_holder, C::TMEM_COLS);   // one warp of each CTA of the pair takes part
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                             // the partner's barriers are initialised before any remote signal
  tc_fence_after();
  const uint32_t tmem_base = is_aux ? 0u : *tmem_holder;

  if (is_aux) {
    // ------------------------------ copy CTAs of the all-gather ------------------------------
    if constexpr (!MX) {                          // (the gathering launchers use the bf16 and per-tensor FP8 kinds)
      static_assert(tpcopy::COPY_STAGES * tpcopy::COPY_PIECE <= C::STAGES * C::STAGE, "copy ring must fit the operand stages");
      if (p.rs.on) tpreduce::reduce_cta(p.rs, num_n, smem, bars, C::THREADS);
      else if (p.tp.copy_mode == 1) tpcopy::copy_cta_push(p.tp, (int)blockIdx.x, 2 * n_aux, C::THREADS);
      else tpcopy::copy_cta(p.tp, (int)blockIdx.x, 2 * n_aux, smem, bars);
    }
  } else if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB);
      if (MX) { tma_prefetch_desc(&tmSFA); tma_prefetch_desc(&tmSFB); }
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      uint32_t ready = p.tp.on ? (1u << p.tp.rank) : 0xffffffffu;   // gathered blocks known to be in the local buffer
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
        const TileInfo ti = tile_info(t, num_m, num_n, num_kb, KB_ELEMS * KSUB, p);
        if (!ti.valid) continue;
        const int mb = ti.mb;
        const int nb = ti.nb + (p.grp.mode == 1 ? ti.e * num_n : 0);   // column tile inside the stacked B
        const int m0 = mb * 256 + (int)rank * 128;          // this CTA's rows of A
        const int n0 = ti.nb * BN + (int)rank * C::BNH + (p.grp.mode == 1 ? ti.e * p.N : 0);   // this CTA's rows of B
        if (p.tp.on) {
          const int c = (mb * 256) / p.tp.rows_per;             // rank block that holds this tile's rows of A
          if (!(ready & (1u << c))) {
            if (!flag_wait_geq(p.tp.chunk_flag + c, p.tp.pieces_per_chunk, B200_WAIT_LIMIT_NS, p.status, 311)) {
              *abort_flag = 1;
              ok = false;
              break;
            }
            tpcopy::fence_proxy_async_all();                    // the block was written through another CTA's (or GPU's) proxy
            ready |= 1u << c;
          }
        }
        for (int kb = ti.kb0; kb < ti.kb0 + ti.nkb; ++kb) {
          if (!mbar_wait_spin(&empty[stage], phase ^ 1, abort_flag, p.status, 310)) { ok = false; break; }
          const uint32_t bar = mapa_u32(smem_u32(&full[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full[stage], 2 * C::AB_STAGE);
          if (MX) {
            // scale atoms first (the forwarding warps turn them into TMEM contents while the operand tiles
            // are still in flight), as rows of 128 int32, the stage's KSUB k groups in one box each
            // (consecutive k groups of a tile are adjacent in the atom layout): A's atoms of this CTA's 128
            // rows, B's atoms of the whole N tile (each CTA's tensor core scales all N columns of its rows)
            mbar_expect_tx(&sffull[stage], C::SF_STAGE);
            const int kg = kb * KSUB;
            tma_load_2d(sSFA + stage * KSUB * C::SFA_SUB, &tmSFA, &sffull[stage], 0, (mb * 2 + (int)rank) * num_kb128 + kg);
            tma_load_2d(sSFB + stage * KSUB * C::SFB_SUB, &tmSFB, &sffull[stage], 0, (nb * num_kb128 + kg) * C::B_ATOMS);
          }
#pragma unroll
          for (int s = 0; s < KSUB; ++s) {
            uint8_t* a_dst = sA + (stage * KSUB + s) * C::A_SUB;
            uint8_t* b_dst = sB + (stage * KSUB + s) * C::B_SUB;
            const int k0 = (kb * KSUB + s) * KB_ELEMS;
            if (MX || F8 || !p.a_mn_major) {
              tma_load_2d_pair(a_dst, &tmA, bar, k0, m0);
            } else {
#pragma unroll
              for (int j = 0; j < 2; ++j) tma_load_2d_pair(a_dst + j * 8192, &tmA, bar, m0 + 64 * j, k0);
            }
            if (MX || F8 || !p.b_mn_major) {
              tma_load_2d_pair(b_dst, &tmB, bar, k0, n0);
            } else {
#pragma unroll
              for (int j = 0; j < C::BNH / 64; ++j) tma_load_2d_pair(b_dst + j * 8192, &tmB, bar, n0 + 64 * j, k0);
            }
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc0 = MX ? umma_idesc_mx(0, 0, 0, 0, 256, BN)
                              : F8 ? umma_idesc(p.a_fmt, p.b_fmt, 0, 0, 256, BN)
                                   : umma_idesc(1, 1, p.a_mn_major, p.b_mn_major, 256, BN);
      const bool a_mn = !MX && !F8 && p.a_mn_major, b_mn = !MX && !F8 && p.b_mn_major;
      const uint32_t a_lbo = a_mn ? 8192 : 16, b_lbo = b_mn ? 8192 : 16;
      // K advance per MMA: 32 bytes along a K-major row, or 16 rows of 128 bytes in an MN-major tile
      const uint32_t a_kstep = a_mn ? 16 * 128 : UMMA_K_BYTES;
      const uint32_t b_kstep = b_mn ? 16 * 128 : UMMA_K_BYTES;
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
        const TileInfo ti = tile_info(t, num_m, num_n, num_kb, KB_ELEMS * KSUB, p);
        if (!ti.valid) continue;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ++it;
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag, p.status, 320)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < ti.nkb && ok; ++kb) {
          if (!mbar_wait_spin(&full[stage], phase, abort_flag, p.status, 321)) { ok = false; break; }
          if (MX && !mbar_wait_spin(&sfrdy[stage], phase, abort_flag, p.status, 322)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int s = 0; s < KSUB; ++s) {
            const uint32_t a_addr = smem_u32(sA + (stage * KSUB + s) * C::A_SUB);
            const uint32_t b_addr = smem_u32(sB + (stage * KSUB + s) * C::B_SUB);
            uint32_t t_sfa = 0, t_sfb = 0;
            if (MX) {
              t_sfa = tmem_base + C::SF_COL + (uint32_t)(stage * KSUB + s) * C::SF_SET_COLS;
              t_sfb = t_sfa + 4;
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint64_t ad = umma_desc_sw128(a_addr + kk * a_kstep, a_lbo, 1024);
              const uint64_t bd = umma_desc_sw128(b_addr + kk * b_kstep, b_lbo, 1024);
              const uint32_t accum = (kb > 0 || s > 0 || kk > 0) ? 1u : 0u;
              if (MX) {
                // scale byte kk of every 32-bit scale column: a_sf_id bits [29,31), b_sf_id bits [4,6)
                tc_mma_mxf8_ss_pair(d_tmem, ad, bd, idesc0 | ((uint32_t)kk << 29) | ((uint32_t)kk << 4), accum, t_sfa, t_sfb);
              } else if (F8) {
                tc_mma_f8_ss_pair(d_tmem, ad, bd, idesc0, accum);
              } else {
                tc_mma_f16_ss_pair(d_tmem, ad, bd, idesc0, accum);
              }
            }
          }
          tc_commit_pair(&empty[stage], 3);       // both CTAs may refill the stage once these MMAs have read it
          if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit_pair(&tfull[acc], 3);   // accumulator complete in both CTAs' TMEM
      }
    }
  } else if (warp < 2 + EPI_WARPS) {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    const int q = warp & 3;                       // TMEM lane quarter owned by this warp
    uint8_t* stg = sE + (warp - 2) * 2 * STG_BYTES;
    const uint32_t tempty_leader0 = mapa_u32(smem_u32(&tempty[0]), 0);
    const uint32_t tempty_leader1 = mapa_u32(smem_u32(&tempty[1]), 0);
    int buf = 0;
    int it = 0;
    bool ok = true;
    for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
      const TileInfo ti = tile_info(t, num_m, num_n, num_kb, KB_ELEMS * KSUB, p);
      if (!ti.valid) continue;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ++it;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag, p.status, 330)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
      if (p.rs.on) {
        // the tile goes into the owner's staging slot of this rank, through the owner's tensor map; then the owner's
        // counter of these 128 rows learns that this warp's part has landed
        const int m0 = ti.mb * 256 + (int)rank * 128;
        const int owner = m0 / p.rs.rows_per;
        const CUtensorMap* tmo = &om.m[owner < NOWN ? owner : 0];
        epilogue_drain<BN, (BN % 64 == 0)>(tmo, tmo, p.epi, t_row, m0 + q * 32, ti.nb * BN, stg, buf, lane,
                                           (p.rs.rank - owner) * p.rs.rows_per);
        if (lane == 0) {
          tma_store_wait_all<0>();
          tpcopy::fence_proxy_async_all();
          __threadfence_system();
          tpcopy::red_release_sys_add(p.rs.flag_peer[owner] + (m0 - owner * p.rs.rows_per) / 128, 1);
        }
      } else {
        epilogue_drain<BN, (BN % 64 == 0)>(&tmD, &tmDt, p.epi, t_row, ti.mb * 256 + (int)rank * 128 + q * 32, ti.nb * BN, stg, buf,
                                           lane, p.grp.mode == 2 ? ti.e * p.M : 0);
      }
      // all TMEM reads of this accumulator are complete (tcgen05.wait::ld inside): hand it back to the leader
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc ? tempty_leader1 : tempty_leader0);
    }
    if (lane == 0) tma_store_wait_all<0>();
    // tiles done: help with the reduction of the rows this rank owns.  All four warps enter (their named barrier
    // needs every one of them); after an abort the leader hands out no work.
    if (p.rs.on) tpreduce::reduce_loop(p.rs, num_n, (int)threadIdx.x - 64, EPI_WARPS * 32, 1, work_slot, abort_flag);
  } else if (MX) {
    // ------------------------------ scale forwarders (both CTAs, MXFP8) ------------------------------
    // Warp of TMEM lane quarter q: per k block, lane l reads the 16 bytes of each staged atom that hold
    // the scales of rows l, 32 + l, 64 + l, 96 + l (4 scale columns each) and writes them to its quarter
    // of the scale set with tcgen05.st; every quarter holds the same copy, as the MMA expects.
    const int q = warp & 3;
    const uint32_t lane_base = tmem_base + (uint32_t(q * 32) << 16) + C::SF_COL;
    const uint32_t rdy_leader0 = mapa_u32(smem_u32(&sfrdy[0]), 0);
    int stage = 0; uint32_t phase = 0;
    bool ok = true;
    for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
      const TileInfo ti = tile_info(t, num_m, num_n, num_kb, KB_ELEMS * KSUB, p);
      if (!ti.valid) continue;
      for (int kb = 0; kb < ti.nkb; ++kb) {
        // the atoms of this stage have landed; its scale sets are free, because the producer loaded the
        // stage only after the MMAs of its previous use had completed
        if (!mbar_wait_spin(&sffull[stage], phase, abort_flag, p.status, 340)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int s = 0; s < KSUB; ++s) {
          uint32_t r[16];
          const uint4 a4 = *reinterpret_cast<const uint4*>(sSFA + (stage * KSUB + s) * C::SFA_SUB + lane * 16);
          r[0] = a4.x; r[1] = a4.y; r[2] = a4.z; r[3] = a4.w;
#pragma unroll
          for (int a = 0; a < 2; ++a) {
            uint4 b4 = make_uint4(0u, 0u, 0u, 0u);
            if (a < C::B_ATOMS)
              b4 = *reinterpret_cast<const uint4*>(sSFB + (stage * KSUB + s) * C::SFB_SUB + a * 512 + lane * 16);
            r[4 + 4 * a] = b4.x; r[5 + 4 * a] = b4.y; r[6 + 4 * a] = b4.z; r[7 + 4 * a] = b4.w;
          }
          r[12] = r[13] = r[14] = r[15] = 0u;
          tmem_st_32x32b_x16(lane_base + (uint32_t)(stage * KSUB + s) * C::SF_SET_COLS, r);
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(rdy_leader0 + (uint32_t)stage * 8);
        if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
      }
    }
  }

  // ------------------------------ teardown ------------------------------
  if (!is_aux && *abort_flag) {                   // (a copy / reduce CTA reuses these words and waits for its own copies)
    // let copies that are still in flight land before shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                             // no signal to the partner is in flight past this point
  if (warp == 1 && !is_aux) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
  }
}

// Launches gemm_pair_kernel on as many CTA pairs as can be resident at once (a persistent grid must
// not exceed that: a pair that waits for SMs would start only after a resident pair finished all its
// tiles).  Returns 0, or a failure code with message.
template <int KIND, int BN, int KSUB, int NOWN = 1>
int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmSFA, const CUtensorMap& tmSFB,
                const CUtensorMap& tmD, const CUtensorMap& tmDt, const PairParams& p, cudaStream_t stream,
                const char* what, const OwnerMaps<NOWN>* owners = nullptr) {
  using C = PairCfg<KIND, BN, KSUB>;
  static int max_pairs[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  auto kern = gemm_pair_kernel<KIND, BN, KSUB, NOWN>;
  static const OwnerMaps<NOWN> no_owners = {};
  const OwnerMaps<NOWN>& om = owners != nullptr ? *owners : no_owners;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(C::THREADS, 1, 1);
  cfg.dynamicSmemBytes = C::SMEM;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (max_pairs[dev] == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return b200::fail(821, "%s: cannot set %d bytes of shared memory: %s", what, C::SMEM, cudaGetErrorString(e));
    }
    cfg.gridDim = dim3(2 * (b200::sm_count() / 2), 1, 1);
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess || n <= 0) {
      cudaGetLastError();
      return b200::fail(822, "%s: no resident CTA pair possible (%s)", what, cudaGetErrorString(e));
    }
    max_pairs[dev] = n;
  }
  const int num_m = (p.M + 255) / 256, num_n = (p.N + BN - 1) / BN;
  const int tiles = (p.grp.mode == 2 ? p.grp.E : 1) * num_m * num_n;
  // every CTA of a gathering launch must be resident at once: its GEMM pairs wait for its copy pairs
  const int n_aux = p.tp.on ? p.tp.n_aux : (p.rs.on ? p.rs.n_aux : 0);
  if (n_aux >= max_pairs[dev]) return b200::fail(823, "%s: %d copy pairs leave no SM for the GEMM", what, n_aux);
  const int room = max_pairs[dev] - n_aux;
  const int pairs = (tiles < room ? tiles : room) + n_aux;
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmSFA, tmSFB, tmD, tmDt, p, om);
  b200::count_launch();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return b200::fail(200, "%s: launch failed: %s", what, cudaGetErrorString(e));
  }
  return b200::check_launch(what);
}

// CTA pairs are the default for every problem taller than one 128-row tile; B200_GEMM_PAIR=0 keeps
// the one-CTA-per-tile kernels (A/B measurements).
inline bool pair_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B200_GEMM_PAIR");
    v = (e && atoi(e) == 0) ? 0 : 1;
  }
  return v != 0;
}

}  // namespace gemmcore
