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
// Loads never use cluster multicast.  Every wait is bounded (2 s) and reports into the status block.
#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int EPI_WARPS = 4;
constexpr int STG_BYTES = 4096;
constexpr int MAXW = 16;
constexpr int COPY_PIECE = 32768;     // bytes per bulk copy
constexpr int COPY_STAGES = 6;
constexpr int RS_SPLIT = 64;          // reduce work items per 128-row tile (2 rows each: a short tail)

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

B200_DEVICE void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
B200_DEVICE void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
B200_DEVICE void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
B200_DEVICE void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
B200_DEVICE void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
B200_DEVICE uint4 ld_cg_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

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

// ------------------------------ copy CTA (modes 1, 2) ------------------------------
// One thread drives a ring of bulk copies peer -> shared -> local and publishes a piece two
// stores after it was issued (its bulk group is then complete).
B200_DEVICE void copy_cta(const Params& p, uint8_t* smem, uint64_t* bars) {
  if (threadIdx.x != 0) return;
  for (int i = 0; i < COPY_STAGES; ++i) mbar_init(&bars[i], 1);
  mbar_fence_init();
  const int ppc = p.pieces_per_chunk;
  const int total = (p.W - 1) * ppc;
  const int mine = (total - (int)blockIdx.x + p.n_aux - 1) / p.n_aux;   // pieces blockIdx, blockIdx + n_aux, ...
  volatile int dummy_abort = 0;
  auto piece_of = [&](int i, int& chunk, long long& off, uint32_t& bytes) {
    const int g = blockIdx.x + i * p.n_aux;
    chunk = (p.rank + 1 + g / ppc) % p.W;
    off = (long long)(g % ppc) * COPY_PIECE;
    const long long left = p.chunk_bytes - off;
    bytes = (uint32_t)(left < COPY_PIECE ? left : COPY_PIECE);
  };
  auto issue_load = [&](int i) {
    int c; long long off; uint32_t bytes;
    piece_of(i, c, off, bytes);
    const int s = i % COPY_STAGES;
    mbar_expect_tx(&bars[s], bytes);
    bulk_g2s(smem + s * COPY_PIECE, p.peer_src[c] + (long long)c * p.chunk_bytes + off, bytes, &bars[s]);
  };
  auto publish = [&](int i) {
    int c; long long off; uint32_t bytes;
    piece_of(i, c, off, bytes);
    fence_proxy_async_all();
    red_release_gpu_add(p.chunk_flag + c, 1);
  };
  const int ahead = COPY_STAGES - 2;
  for (int i = 0; i < mine && i < ahead; ++i) issue_load(i);
  bool ok = true;
  for (int i = 0; i < mine; ++i) {
    const int s = i % COPY_STAGES;
    if (!mbar_wait(&bars[s], (i / COPY_STAGES) & 1, &dummy_abort, p.status, 40)) { ok = false; break; }
    int c; long long off; uint32_t bytes;
    piece_of(i, c, off, bytes);
    bulk_s2g(p.gdst + (long long)c * p.chunk_bytes + off, smem + s * COPY_PIECE, bytes);
    tma_store_commit();
    tma_store_wait_all<2>();                 // stores up to i-2 are complete
    if (i >= 2) publish(i - 2);
    if (i + ahead < mine) issue_load(i + ahead);   // stage (i-2) % STAGES: its store has completed
  }
  tma_store_wait_all<0>();
  if (ok) {
    if (mine >= 2) publish(mine - 2);
    if (mine >= 1) publish(mine - 1);
  } else {
    // loads that never completed may still land: give them time before shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
}

// Push variant: every thread of the CTA copies 16-byte vectors of this rank's block from local memory
// straight into every peer's buffer (plain posted stores: no round trip per piece), and one thread
// bumps the peers' counters after each PUSH_PIECE bytes, behind a system-scope fence.
constexpr int PUSH_PIECE = 262144;

B200_DEVICE void copy_cta_push(const Params& p) {
  // Work items are (destination, piece), destination-major: the rank that consumes this block first
  // (rank - 1: it visits its own block, then rank + 1's, ...) receives all of it first.
  const int ppc = (int)((p.chunk_bytes + PUSH_PIECE - 1) / PUSH_PIECE);
  const long long base = (long long)p.rank * p.chunk_bytes;
  const uint8_t* src = p.gdst + base;
  const int items = (p.W - 1) * ppc;
  for (int it = blockIdx.x; it < items; it += p.n_aux) {
    const int d = (p.rank - 1 - it / ppc + 2 * p.W) % p.W;
    const long long off = (long long)(it % ppc) * PUSH_PIECE;
    const long long left = p.chunk_bytes - off;
    const int nvec = (int)((left < PUSH_PIECE ? left : PUSH_PIECE) / 16);
    uint8_t* dst = const_cast<uint8_t*>(p.peer_src[d]) + base + off;
    constexpr int U = 16;
    for (int v0 = threadIdx.x; v0 < nvec; v0 += U * NUM_THREADS) {
      uint4 q[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = v0 + u * NUM_THREADS;
        if (v < nvec) q[u] = ld_cg_u4(src + off + (long long)v * 16);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = v0 + u * NUM_THREADS;
        if (v < nvec) *reinterpret_cast<uint4*>(dst + (long long)v * 16) = q[u];
      }
    }
    __threadfence_system();
    named_bar_sync(3, NUM_THREADS);
    if (threadIdx.x == 0) red_release_sys_add(p.chunk_flag_peer[d] + p.rank, 1);
  }
}

// ------------------------------ reduce work (mode 3) ------------------------------
// `nthreads` threads (a named barrier `bar_id` among them) claim items until the queue is empty.
B200_DEVICE void reduce_loop(const Params& p, int num_n, int tid, int nthreads, int bar_id, volatile int* slot,
                             volatile int* abort_flag) {
  const int tpc = p.rows_per / BM;
  const int items = tpc * RS_SPLIT;
  const int nvec = p.N / 8;
  const uint8_t* stage = p.stage_peer[p.rank];
  const int* flags = p.flag_peer[p.rank];
  while (true) {
    if (tid == 0) {
      int it = (abort_flag != nullptr && *abort_flag) ? items : atomicAdd(p.work_counter, 1);
      if (it < items) {
        const int want = p.W * num_n * EPI_WARPS;
        if (!flag_wait_geq(flags + it / RS_SPLIT, want, B200_WAIT_LIMIT_NS, p.status, 50)) it = items;  // give up
      }
      *slot = it;
    }
    named_bar_sync(bar_id, nthreads);
    const int it = *slot;
    named_bar_sync(bar_id, nthreads);      // everyone has read the slot before it is rewritten
    if (it >= items) break;
    const int row0 = (it / RS_SPLIT) * BM + (it % RS_SPLIT) * (BM / RS_SPLIT);
    constexpr int U = 4;                   // vectors per thread in flight per source
    const int total = (BM / RS_SPLIT) * nvec;
    for (int base = tid; base < total; base += U * nthreads) {
      float acc[U][8];
      long long off[U];
      bool live[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int idx = base + u * nthreads;
        live[u] = idx < total;
        const int row = row0 + (live[u] ? idx / nvec : 0);
        const int v = live[u] ? idx % nvec : 0;
        off[u] = (long long)row * p.N + v * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[u][i] = 0.f;
        if (p.rs_residual != nullptr && live[u]) {
          const uint4 q = *reinterpret_cast<const uint4*>(p.rs_residual + (long long)row * p.ld_res + v * 8);
          const float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y), f2 = unpack_bf16x2(q.z), f3 = unpack_bf16x2(q.w);
          acc[u][0] = f0.x; acc[u][1] = f0.y; acc[u][2] = f1.x; acc[u][3] = f1.y;
          acc[u][4] = f2.x; acc[u][5] = f2.y; acc[u][6] = f3.x; acc[u][7] = f3.y;
        }
      }
      for (int s2 = 0; s2 < p.W; ++s2) {
        uint4 q[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          q[u] = live[u] ? ld_cg_u4(stage + ((long long)s2 * p.rows_per * p.N + off[u]) * 2) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float2 f0 = unpack_bf16x2(q[u].x), f1 = unpack_bf16x2(q[u].y), f2 = unpack_bf16x2(q[u].z), f3 = unpack_bf16x2(q[u].w);
          acc[u][0] += f0.x; acc[u][1] += f0.y; acc[u][2] += f1.x; acc[u][3] += f1.y;
          acc[u][4] += f2.x; acc[u][5] += f2.y; acc[u][6] += f3.x; acc[u][7] += f3.y;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (!live[u]) continue;
        const int idx = base + u * nthreads;
        const int row = row0 + idx / nvec;
        const int v = idx % nvec;
        const uint4 o = make_uint4(pack_bf16x2(acc[u][0], acc[u][1]), pack_bf16x2(acc[u][2], acc[u][3]),
                                   pack_bf16x2(acc[u][4], acc[u][5]), pack_bf16x2(acc[u][6], acc[u][7]));
        *reinterpret_cast<uint4*>(p.rs_out + (long long)row * p.ld_out + v * 8) = o;
      }
    }
  }
}

// ------------------------------ dedicated reduce CTA (mode 3) ------------------------------
// Streams the W staged copies of each row segment into shared memory with bulk async copies (one
// thread keeps a 6-deep ring of 32 KB stages in flight), five consumer warps add them in fp32.
struct RedMeta { int row, c0, cols; };

B200_DEVICE void reduce_cta(const Params& p, int num_n, uint8_t* smem, uint64_t* bars) {
  constexpr int RST = COPY_STAGES;
  constexpr int CONSUMER_WARPS = NUM_THREADS / 32 - 1;
  uint64_t* full = bars;
  uint64_t* empty = bars + RST;
  RedMeta* meta = reinterpret_cast<RedMeta*>(bars + 2 * RST);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(meta + RST);
  if (threadIdx.x == 0) {
    for (int i = 0; i < RST; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], CONSUMER_WARPS); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int unit_cols = (COPY_PIECE / 2 / p.W) & ~7;
  if (unit_cols > p.N) unit_cols = p.N;
  const uint8_t* stage = p.stage_peer[p.rank];
  if (warp == 0) {
    if (lane != 0) return;
    const int tpc = p.rows_per / BM;
    const int items = tpc * RS_SPLIT;
    const int want = p.W * num_n * EPI_WARPS;
    const int* flags = p.flag_peer[p.rank];
    int st = 0; uint32_t ph = 0;
    bool ok = true;
    while (ok) {
      const int it = atomicAdd(p.work_counter, 1);
      if (it >= items) break;
      if (!flag_wait_geq(flags + it / RS_SPLIT, want, B200_WAIT_LIMIT_NS, p.status, 51)) break;
      fence_proxy_async_all();
      const int row0 = (it / RS_SPLIT) * BM + (it % RS_SPLIT) * (BM / RS_SPLIT);
      for (int r = 0; r < BM / RS_SPLIT && ok; ++r) {
        for (int c0 = 0; c0 < p.N; c0 += unit_cols) {
          if (!mbar_wait(&empty[st], ph ^ 1, abort_flag, p.status, 52)) { ok = false; break; }
          const int cols = min(unit_cols, p.N - c0);
          meta[st].row = row0 + r; meta[st].c0 = c0; meta[st].cols = cols;
          mbar_expect_tx(&full[st], (uint32_t)(p.W * cols * 2));
          for (int s2 = 0; s2 < p.W; ++s2)
            bulk_g2s(smem + st * COPY_PIECE + s2 * cols * 2,
                     stage + (((long long)s2 * p.rows_per + row0 + r) * p.N + c0) * 2, (uint32_t)(cols * 2), &full[st]);
          if (++st == RST) { st = 0; ph ^= 1; }
        }
      }
    }
    // sentinel: tells the consumers to leave
    if (mbar_wait(&empty[st], ph ^ 1, abort_flag, p.status, 53)) {
      meta[st].row = -1;
      mbar_arrive(&full[st]);
    }
    return;
  }
  int st = 0; uint32_t ph = 0;
  const int ctid = threadIdx.x - 32, cn = CONSUMER_WARPS * 32;
  while (true) {
    if (!mbar_wait(&full[st], ph, abort_flag, p.status, 54)) break;
    const RedMeta m = meta[st];
    if (m.row < 0) break;
    const uint8_t* sb = smem + st * COPY_PIECE;
    for (int v = ctid; v < m.cols / 8; v += cn) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      if (p.rs_residual != nullptr) {
        const uint4 q = *reinterpret_cast<const uint4*>(p.rs_residual + (long long)m.row * p.ld_res + m.c0 + v * 8);
        const float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y), f2 = unpack_bf16x2(q.z), f3 = unpack_bf16x2(q.w);
        acc[0] = f0.x; acc[1] = f0.y; acc[2] = f1.x; acc[3] = f1.y; acc[4] = f2.x; acc[5] = f2.y; acc[6] = f3.x; acc[7] = f3.y;
      }
      for (int s2 = 0; s2 < p.W; ++s2) {
        const uint4 q = *reinterpret_cast<const uint4*>(sb + s2 * m.cols * 2 + v * 16);
        const float2 f0 = unpack_bf16x2(q.x), f1 = unpack_bf16x2(q.y), f2 = unpack_bf16x2(q.z), f3 = unpack_bf16x2(q.w);
        acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y; acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
      }
      const uint4 o = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                                 pack_bf16x2(acc[6], acc[7]));
      *reinterpret_cast<uint4*>(p.rs_out + (long long)m.row * p.ld_out + m.c0 + v * 8) = o;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[st]);
    if (++st == RST) { st = 0; ph ^= 1; }
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
    if (p.mode == 3) reduce_cta(p, num_n, smem, bars);
    else if (p.copy_mode == 1) copy_cta_push(p);
    else copy_cta(p, smem, bars);
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
    if (p.mode == 3) reduce_loop(p, num_n, threadIdx.x - 64, EPI_WARPS * 32, 1, work_slot, abort_flag);
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
