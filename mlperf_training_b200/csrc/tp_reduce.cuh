// Reduce roles of the GEMM -> reduce-scatter kernels: every rank's epilogue stores its partial tile into the
// OWNER's staging buffer (slot of the sending rank) over NVLink and bumps the owner's per-128-row counter; the
// owner sums the W slots of its rows in fp32 (+ residual) and writes the bf16 result.  Reduce work items (a few rows
// x N) are claimed from a queue by dedicated CTAs of the SAME launch (streaming the slots through shared memory with
// bulk async copies) and by the GEMM CTAs' epilogue warps once their tiles are done.  Shared by the one-CTA-per-tile
// kernel (gemm_tp.cu) and the CTA-pair kernel (gemm_core.cuh).
//
// `P` provides: W, rank, rows_per, N, stage_peer[], flag_peer[], work_counter, rs_out, ld_out, rs_residual, ld_res,
// status.  Counters count (rank, column tile, epilogue warp) arrivals per 128 rows: `num_n` is the number of column
// tiles of the launching GEMM.
#pragma once
#include "common.cuh"
#include "tp_copy.cuh"

namespace tpreduce {

using tpcopy::COPY_PIECE;
using tpcopy::COPY_STAGES;
using tpcopy::bulk_g2s;
using tpcopy::fence_proxy_async_all;
using tpcopy::ld_cg_u4;
constexpr int BM = 128;               // rows per counter
constexpr int EPI_WARPS = 4;
constexpr int RS_SPLIT = 64;          // reduce work items per 128 rows (2 rows each: a short tail)

// `nthreads` threads (a named barrier `bar_id` among them) claim items until the queue is empty.
template <class P>
B200_DEVICE void reduce_loop(const P& p, int num_n, int tid, int nthreads, int bar_id, volatile int* slot,
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

template <class P>
B200_DEVICE void reduce_cta(const P& p, int num_n, uint8_t* smem, uint64_t* bars, int nthreads) {
  constexpr int RST = COPY_STAGES;
  const int CONSUMER_WARPS = nthreads / 32 - 1;
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

}  // namespace tpreduce
